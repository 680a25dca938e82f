// Host interface of the bf16 tensor-core update path (update_bf16.cu).
#pragma once
#include "umma.cuh"
#include "ppo_kernels.cuh"

namespace mrl {
namespace tc {

constexpr int H = 256;  // hidden width this path is specialised for

// True when the network / minibatch shape is covered by the tensor-core kernels.
bool supported(const mrl_net_spec* net, int batch);
// Bytes of device workspace State::init needs for minibatches of `batch` rows.
int64_t workspace_bytes(int batch, int hidden);
int max_splits();
int make_tensor_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                    uint64_t pitch_elems = 0);
// [32 rows x 32 columns] boxes with the 64-byte swizzle: the epilogue staging tiles of the row-tile kernel.
int make_box_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems = 0);

// Activation buffers, bf16 weight copies and TMA descriptors of one minibatch
// shape; shared by the actor and the critic, which run one after the other.
struct State {
    int batch;
    int* err;  // device word: 0, or the code of the first wait that gave up
    int hh, nb;  // hidden width (256 or 512) and its number of 256-wide blocks
    __nv_bfloat16 *h0, *h1, *g1, *g0, *w1, *w1t;   // activations [batch, hh]; W1 and W1^T as bf16 [hh, hh]
    float* part;
    CUtensorMap tm_h0[2], tm_g1[2], tm_h0_mn[2], tm_g1_mn[2];   // 256-wide column blocks of the activations
    CUtensorMap tm_w1t[2][2], tm_w1[2][2];                       // [row block][column block] of W1^T and W1
    CUtensorMap tm_h1_box[2], tm_g0_box[2], tm_h0_box[2];        // [32 x 32] epilogue staging boxes per column block
    // hh = 512: full-width views for the row-tile kernel with 128-wide output blocks and K = 512
    CUtensorMap tm_h0_full, tm_g1_full, tm_w1t_full, tm_w1_full, tm_h1_boxf, tm_g0_boxf, tm_h0_boxf;

    int init(void* workspace, int batch, int hidden, int* err_flag);
    // head_out [batch, out_dim] = logits / values (fp32).  convert = false reuses the bf16 copies of W1 made
    // by the previous call (same network, unchanged parameters).
    int forward(const mrl_net_spec* net, const float* params, const float* x, float* head_out, cudaStream_t st,
                bool convert = true);
    // grads [PARAM_SIZE] is overwritten (fp32, reference parameter order)
    int backward(const mrl_net_spec* net, const float* params, const float* x, const float* dout, float* grads,
                 cudaStream_t st);
};

// W1 fp32 [256, 256] -> bf16 row-major copy and bf16 transposed copy.
int convert_w1(const float* W1, __nv_bfloat16* w1, __nv_bfloat16* w1t, cudaStream_t st);

// ---- rollout policy step on tensor cores (rollout_bf16.cu) ----------------------
struct DeviceCountersFwd;  // (DeviceCounters lives in rollout.cuh)
struct PolicyStepArgs {
    const float* obs;
    const float* actor_params;
    const float* critic_params;
    int n, in_dim, num_actions, t, greedy;
    int act;          // trunk activation: 0 ReLU, 1 tanh
    int continuous;   // 1: Gaussian head (num_actions means; log_std follows b2), actions [n, num_actions]
    float* actions;
    float* values;
    float* r_obs; float* r_actions; float* r_log_probs; float* r_values;
    const void* counters;  // const DeviceCounters*
};

bool policy_supported(int in_dim, int num_actions, int hidden);
int64_t policy_workspace_bytes();

struct PolicyState {
    int* err;
    __nv_bfloat16* w1t[2];     // bf16 W1^T of actor and critic, refreshed once per rollout
    __nv_bfloat16* scratch_w1; // row-major bf16 copy (by-product of the conversion)
    CUtensorMap tm_w1t[2];
    int init(void* workspace, int* err_flag);
    // Converts the current W1 of both networks (call once per rollout, before step 0).
    int prepare(const float* actor_params, const float* critic_params, int in_dim, cudaStream_t st);
    // Actor + critic forward, sampling and pre-step store for rollout step a.t.
    int step(const PolicyStepArgs& a, cudaStream_t st);
};

}  // namespace tc
}  // namespace mrl
