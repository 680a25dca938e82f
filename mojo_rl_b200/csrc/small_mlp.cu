// Fused fp32 training step of the hidden-64 actor / critic MLPs (CartPole and
// Pendulum configs: 4-64-64-{2,1}, 3-64-64-{(1,log_std),1}).
//
// One kernel does what the reference spreads over ~20 launches per network and
// minibatch (Model.forward_gpu_ws, the PPO loss-gradient kernel,
// Model.backward_gpu_ws: deep_rl/model/sequential.mojo:537-865,
// deep_agents/ppo/ppo.mojo:285-378, :538-633, deep_agents/ppo/kernels.mojo:230-486):
// a block takes 128 minibatch rows at a time, keeps h0, h1 and their gradients
// in shared memory, and accumulates the weight gradients of its rows in
// registers; nothing but the observations, the per-row loss inputs and one
// partial gradient vector per block touches HBM.  The networks are far too
// small for tensor cores to matter and stay fp32 (CUDA-core FMA chains in the
// reference's summation order: bias first, k ascending), so the forward
// values are bit-identical to the layer-by-layer path.
//
// Reductions over rows are kept in double precision per block and summed
// over blocks in a fixed order (deterministic; not the serial order of the
// reference's kernels).  Compile with -fmad=false.
#include "env_cartpole.cuh"
#include "env_pendulum.cuh"
#include "ppo_kernels.cuh"
#include "rollout.cuh"
#include "small_mlp.cuh"

namespace mrl {
namespace small {

constexpr int H = 64, TM = 128, THREADS = 256, PITCH = 68, MAX_IN = 8, MAX_OUT = 4;

struct TrainArgs {
    const float* params;
    int in_dim, out_dim, act, mode;   // out_dim: actions / action dims / 1; act: 0 ReLU, 1 tanh
    const float* x;                   // [B, in_dim]
    const float* actions;             // [B] (discrete index) or [B, out_dim] (Gaussian)
    const float* adv;
    const float* ret;
    const float* old_lp;
    const float* old_v;
    int B;
    float clip_eps, entropy_coef, value_loss_coef;
    int clip_value;
    double* partial;      // [grid][pstride]: per-block gradient sums, parameter order, then the KL sum
    int pstride;
};

__device__ __forceinline__ float act_fwd(float v, int act) { return act == 0 ? (v > 0.0f ? v : 0.0f) : mrl_tanhf(v); }
// derivative applied to an upstream gradient, from the stored activation y
__device__ __forceinline__ float act_bwd(float g, float y, int act) {
    return act == 0 ? (y > 0.0f ? g : 0.0f) : g * (1.0f - y * y);
}

// dst[row][col0..col0+3] = epilogue(init + A[row][:] . W[:][col0..col0+3]) for the thread's eight rows
// rg, rg + 16, ..., rg + 112.  A: [TM][PITCH] in shared memory, W: [64][64] k-major in shared memory.
template <int ROWSTEP = 16, class Epi>
__device__ __forceinline__ void tile_gemm64(const float* __restrict__ A, const float* __restrict__ W, int rg, int c0,
                                            const float (&init)[4], Epi epi) {
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = init[j];
#pragma unroll 2
    for (int k = 0; k < H; k += 4) {
        float4 a[8], w[4];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float4*>(A + (rg + ROWSTEP * i) * PITCH + k);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) w[kk] = *reinterpret_cast<const float4*>(W + (k + kk) * H + c0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float av[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                acc[i][0] = fmaf(av[kk], w[kk].x, acc[i][0]);
                acc[i][1] = fmaf(av[kk], w[kk].y, acc[i][1]);
                acc[i][2] = fmaf(av[kk], w[kk].z, acc[i][2]);
                acc[i][3] = fmaf(av[kk], w[kk].w, acc[i][3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) epi(rg + ROWSTEP * i, c0, acc[i]);
}

__global__ void __launch_bounds__(THREADS, 1) fused_train_kernel(TrainArgs p) {
    extern __shared__ __align__(16) float smem[];
    float* W1s = smem;                    // [k][j]
    float* W1t = W1s + H * H;             // [j][k]: W1t[j * 64 + i] = W1[i][j]
    float* S0 = W1t + H * H;              // h0 [TM][PITCH]
    float* S1 = S0 + TM * PITCH;          // h1, later g0
    float* G1 = S1 + TM * PITCH;          // g1
    float* W0s = G1 + TM * PITCH;         // [MAX_IN][64]
    float* b0s = W0s + MAX_IN * H;
    float* b1s = b0s + H;
    float* W2s = b1s + H;                 // [64][MAX_OUT]
    float* b2s = W2s + H * MAX_OUT;       // [MAX_OUT]
    float* lss = b2s + MAX_OUT;           // log_std [MAX_OUT]
    float* xs = lss + MAX_OUT;            // [TM][MAX_IN]
    float* douts = xs + TM * MAX_IN;      // [TM][2 * MAX_OUT]
    __shared__ double kl_sm[32];

    const int tid = threadIdx.x;
    const int I = p.in_dim, O = p.out_dim, act = p.act;
    const bool gaussian = p.mode == ACTOR_GAUSSIAN;
    const float* W0 = p.params;
    const float* b0 = W0 + I * H;
    const float* W1 = b0 + H;
    const float* b1 = W1 + H * H;
    const float* W2 = b1 + H;
    const float* b2 = W2 + H * O;
    const float* ls = b2 + O;
    for (int i = tid; i < H * H; i += THREADS) {
        float w = W1[i];
        W1s[i] = w;
        W1t[(i % H) * H + i / H] = w;
    }
    for (int i = tid; i < MAX_IN * H; i += THREADS) W0s[i] = i < I * H ? W0[i] : 0.0f;
    for (int i = tid; i < H; i += THREADS) { b0s[i] = b0[i]; b1s[i] = b1[i]; }
    for (int i = tid; i < H * MAX_OUT; i += THREADS) {
        int k = i / MAX_OUT, o = i % MAX_OUT;
        W2s[i] = o < O ? W2[k * O + o] : 0.0f;
    }
    if (tid < MAX_OUT) {
        b2s[tid] = tid < O ? b2[tid] : 0.0f;
        float l = (gaussian && tid < O) ? ls[tid] : 0.0f;
        if (l < -5.0f) l = -5.0f;               // stochastic_actor.mojo:386-575: the output carries the clamped value
        else if (l > 2.0f) l = 2.0f;
        lss[tid] = l;
    }
    __syncthreads();

    const int rg = tid >> 4, c0 = (tid & 15) * 4;     // 8 x 4 output tile of the row-tile GEMMs
    const int wi0 = (tid >> 4) * 4, wj0 = (tid & 15) * 4;  // 4 x 4 tile of dW1
    double dW1[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dW1[i][j] = 0.0;
    double dW0a = 0.0, dW0b = 0.0;          // entries tid and tid + 256 of dW0 [I][64]
    double db0 = 0.0, db1 = 0.0;            // threads < 64
    double dW2 = 0.0;                       // entry (k = tid / 4, o = tid % 4)
    double db2 = 0.0, dls = 0.0;            // threads < MAX_OUT
    double kl_acc = 0.0;                    // threads < TM

    const int n_tiles = (p.B + TM - 1) / TM;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int row0 = tile * TM;
        for (int i = tid; i < TM * MAX_IN; i += THREADS) {
            int r = i / MAX_IN, k = i % MAX_IN;
            xs[i] = (row0 + r < p.B && k < I) ? p.x[(size_t)(row0 + r) * I + k] : 0.0f;
        }
        __syncthreads();
        // h0 = act(x W0 + b0)
        {
            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = b0s[c0 + j];
            for (int k = 0; k < I; ++k) {
                const float4 w = *reinterpret_cast<const float4*>(W0s + k * H + c0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float a = xs[(rg + 16 * i) * MAX_IN + k];
                    acc[i][0] = fmaf(a, w.x, acc[i][0]);
                    acc[i][1] = fmaf(a, w.y, acc[i][1]);
                    acc[i][2] = fmaf(a, w.z, acc[i][2]);
                    acc[i][3] = fmaf(a, w.w, acc[i][3]);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
                *reinterpret_cast<float4*>(S0 + (rg + 16 * i) * PITCH + c0) =
                    make_float4(act_fwd(acc[i][0], act), act_fwd(acc[i][1], act), act_fwd(acc[i][2], act),
                                act_fwd(acc[i][3], act));
        }
        __syncthreads();
        // h1 = act(h0 W1 + b1)
        {
            const float init[4] = {b1s[c0], b1s[c0 + 1], b1s[c0 + 2], b1s[c0 + 3]};
            tile_gemm64(S0, W1s, rg, c0, init, [&](int r, int c, const float (&v)[4]) {
                *reinterpret_cast<float4*>(S1 + r * PITCH + c) =
                    make_float4(act_fwd(v[0], act), act_fwd(v[1], act), act_fwd(v[2], act), act_fwd(v[3], act));
            });
        }
        __syncthreads();
        // head and loss gradient, one row per thread
        if (tid < TM) {
            const int r = tid, row = row0 + r;
            float dout[2 * MAX_OUT];
#pragma unroll
            for (int o = 0; o < 2 * MAX_OUT; ++o) dout[o] = 0.0f;
            if (row < p.B) {
                float out[2 * MAX_OUT];
#pragma unroll
                for (int o = 0; o < MAX_OUT; ++o) out[o] = b2s[o];
                for (int k = 0; k < H; ++k) {
                    const float hv = S1[r * PITCH + k];
                    const float4 w = *reinterpret_cast<const float4*>(W2s + k * MAX_OUT);
                    out[0] = fmaf(hv, w.x, out[0]);
                    out[1] = fmaf(hv, w.y, out[1]);
                    out[2] = fmaf(hv, w.z, out[2]);
                    out[3] = fmaf(hv, w.w, out[3]);
                }
                const float bdiv = (float)p.B;
                if (p.mode == ACTOR_DISCRETE) {
                    float klv;
                    actor_grad_one(out, O, p.old_lp[row], p.adv[row], (int)p.actions[row], p.clip_eps, p.entropy_coef,
                                   bdiv, dout, klv);
                    kl_acc += (double)klv;
                } else if (p.mode == ACTOR_GAUSSIAN) {
                    float row_out[2 * MAX_OUT], a[MAX_OUT], klv;
                    for (int o = 0; o < O; ++o) {
                        row_out[o] = out[o];
                        row_out[O + o] = lss[o];
                        a[o] = p.actions[(size_t)row * O + o];
                    }
                    continuous_actor_grad_one(row_out, O, p.old_lp[row], p.adv[row], a, p.clip_eps, p.entropy_coef,
                                              bdiv, dout, klv);
                    kl_acc += (double)klv;
                } else if (p.mode == CRITIC_DISCRETE) {
                    dout[0] = critic_grad_one(out[0], p.old_v ? p.old_v[row] : 0.0f, p.ret[row], p.value_loss_coef,
                                              p.clip_eps, p.clip_value, bdiv);
                } else {
                    dout[0] = continuous_critic_grad_one(out[0], p.old_v ? p.old_v[row] : 0.0f, p.ret[row], p.clip_eps,
                                                         p.clip_value, bdiv);
                }
            }
#pragma unroll
            for (int o = 0; o < 2 * MAX_OUT; ++o) douts[r * 2 * MAX_OUT + o] = dout[o];
        }
        __syncthreads();
        // g1 = (dout W2^T) * act'(h1); head gradients
        {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = rg + 16 * i;
                const float4 y = *reinterpret_cast<const float4*>(S1 + r * PITCH + c0);
                const float yv[4] = {y.x, y.y, y.z, y.w};
                float g[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float acc = 0.0f;
                    for (int o = 0; o < O; ++o) acc = fmaf(douts[r * 2 * MAX_OUT + o], W2s[(c0 + j) * MAX_OUT + o], acc);
                    g[j] = act_bwd(acc, yv[j], act);
                }
                *reinterpret_cast<float4*>(G1 + r * PITCH + c0) = make_float4(g[0], g[1], g[2], g[3]);
            }
            // dW2[k][o] += sum_r h1[r][k] dout[r][o]
            {
                const int k = tid >> 2, o = tid & 3;
                float acc = 0.0f;
                if (o < O)
                    for (int r = 0; r < TM; ++r) acc = fmaf(S1[r * PITCH + k], douts[r * 2 * MAX_OUT + o], acc);
                dW2 += (double)acc;
            }
            if (tid < MAX_OUT && tid < O) {
                float acc = 0.0f, accl = 0.0f;
                for (int r = 0; r < TM; ++r) {
                    acc += douts[r * 2 * MAX_OUT + tid];
                    if (gaussian) accl += douts[r * 2 * MAX_OUT + O + tid];
                }
                db2 += (double)acc;
                dls += (double)accl;
            }
        }
        __syncthreads();
        // dW1 += h0^T g1, db1 += sum g1
        {
            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
#pragma unroll 4
            for (int r = 0; r < TM; ++r) {
                const float4 a = *reinterpret_cast<const float4*>(S0 + r * PITCH + wi0);
                const float4 b = *reinterpret_cast<const float4*>(G1 + r * PITCH + wj0);
                const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) dW1[i][j] += (double)acc[i][j];
            if (tid < H) {
                float s = 0.0f;
                for (int r = 0; r < TM; ++r) s += G1[r * PITCH + tid];
                db1 += (double)s;
            }
        }
        // g0 = (g1 W1^T) * act'(h0), written over h1 (no longer needed: the head gradients above are done
        // before the barrier that precedes this block)
        {
            const float init[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            tile_gemm64(G1, W1t, rg, c0, init, [&](int r, int c, const float (&v)[4]) {
                const float4 y = *reinterpret_cast<const float4*>(S0 + r * PITCH + c);
                *reinterpret_cast<float4*>(S1 + r * PITCH + c) =
                    make_float4(act_bwd(v[0], y.x, act), act_bwd(v[1], y.y, act), act_bwd(v[2], y.z, act),
                                act_bwd(v[3], y.w, act));
            });
        }
        __syncthreads();
        // dW0 += x^T g0, db0 += sum g0
        {
            for (int e = tid, slot = 0; e < I * H; e += THREADS, ++slot) {
                const int k = e / H, i = e % H;
                float acc = 0.0f;
                for (int r = 0; r < TM; ++r) acc = fmaf(xs[r * MAX_IN + k], S1[r * PITCH + i], acc);
                if (slot == 0) dW0a += (double)acc; else dW0b += (double)acc;
            }
            if (tid < H) {
                float s = 0.0f;
                for (int r = 0; r < TM; ++r) s += S1[r * PITCH + tid];
                db0 += (double)s;
            }
        }
        __syncthreads();
    }

    // per-block partial sums, parameter order: W0 b0 W1 b1 W2 b2 [log_std], then the KL sum
    double* out = p.partial + (size_t)blockIdx.x * p.pstride;
    const int oW0 = 0, ob0 = I * H, oW1 = ob0 + H, ob1 = oW1 + H * H, oW2 = ob1 + H, ob2 = oW2 + H * O, ols = ob2 + O;
    if (tid < I * H) out[oW0 + tid] = dW0a;
    if (tid + THREADS < I * H) out[oW0 + tid + THREADS] = dW0b;
    if (tid < H) { out[ob0 + tid] = db0; out[ob1 + tid] = db1; }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) out[oW1 + (wi0 + i) * H + wj0 + j] = dW1[i][j];
    {
        const int k = tid >> 2, o = tid & 3;
        if (o < O) out[oW2 + k * O + o] = dW2;
    }
    if (tid < O) {
        out[ob2 + tid] = db2;
        if (gaussian) out[ols + tid] = dls;
    }
    kl_acc = block_sum(kl_acc, kl_sm);
    if (tid == 0) out[p.pstride - 1] = kl_acc;
}

// grads[i] = sum over blocks of partial[b][i] (b ascending); the KL sum goes to kl_out as fp32.
__global__ void reduce_partials_kernel(const double* __restrict__ partial, int nblocks, int pstride, int n_params,
                                       float* __restrict__ grads, float* __restrict__ kl_out) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_params) {
        double acc = 0.0;
        for (int b = 0; b < nblocks; ++b) acc += partial[(size_t)b * pstride + i];
        grads[i] = (float)acc;
    } else if (i == n_params && kl_out != nullptr) {
        double acc = 0.0;
        for (int b = 0; b < nblocks; ++b) acc += partial[(size_t)b * pstride + pstride - 1];
        kl_out[0] = (float)acc;
    }
}

// ---------------------------------------------------------------------------
// Persistent rollout of the hidden-64 configs: environments are independent and
// the parameters are fixed during a rollout, so one launch runs all T steps.  A
// block owns 32 environments; warps 0-1 evaluate the actor, warps 2-3 the critic
// (both weight sets stay in shared memory), then lanes of warp 0 sample, store
// the pre-step data, step their environment, do the episode bookkeeping and the
// selective reset, and write the next observation back to shared memory.
// Per step this is _sample_actions_kernel / _sample_continuous_actions_kernel,
// the store kernels, EnvType.step_kernel_gpu, the tracking kernels and
// selective_reset_kernel_gpu (ppo.mojo:2056-2285; ppo_continuous.mojo:2618-2836).
// ---------------------------------------------------------------------------
constexpr int RT = 32, RTHREADS = 128;

struct RolloutArgs {
    const float* actor_params;
    const float* critic_params;
    int in_dim, out_dim, act, gaussian, greedy;
    int T;
    float* logits_unused;
    float* actions;      // [n, act_w] (last step's)
    float* values;       // [n]
    float* r_obs; float* r_actions; float* r_log_probs; float* r_values;
    RolloutStepArgs env;  // t is set per step inside the kernel
};

struct NetSmem {
    float W1s[H * H];
    float W0s[MAX_IN * H];
    float b0s[H], b1s[H];
    float W2s[H * MAX_OUT];
    float b2s[MAX_OUT], lss[MAX_OUT];
    float S0[RT * PITCH], S1[RT * PITCH];
};

__device__ __forceinline__ void load_net(NetSmem& m, const float* params, int I, int O, bool gaussian, int lt, int nt) {
    const float* W0 = params;
    const float* b0 = W0 + I * H;
    const float* W1 = b0 + H;
    const float* b1 = W1 + H * H;
    const float* W2 = b1 + H;
    const float* b2 = W2 + H * O;
    const float* ls = b2 + O;
    for (int i = lt; i < H * H; i += nt) m.W1s[i] = W1[i];
    for (int i = lt; i < MAX_IN * H; i += nt) m.W0s[i] = i < I * H ? W0[i] : 0.0f;
    for (int i = lt; i < H; i += nt) { m.b0s[i] = b0[i]; m.b1s[i] = b1[i]; }
    for (int i = lt; i < H * MAX_OUT; i += nt) {
        int k = i / MAX_OUT, o = i % MAX_OUT;
        m.W2s[i] = o < O ? W2[k * O + o] : 0.0f;
    }
    if (lt < MAX_OUT) {
        m.b2s[lt] = lt < O ? b2[lt] : 0.0f;
        float l = (gaussian && lt < O) ? ls[lt] : 0.0f;
        if (l < -5.0f) l = -5.0f;
        else if (l > 2.0f) l = 2.0f;
        m.lss[lt] = l;
    }
}

template <int ENV>  // 0 CartPole, 1 Pendulum
__global__ void __launch_bounds__(RTHREADS, 1) fused_rollout_kernel(RolloutArgs p) {
    extern __shared__ __align__(16) unsigned char raw[];
    NetSmem* nets = reinterpret_cast<NetSmem*>(raw);                 // [2]
    float* xs = reinterpret_cast<float*>(raw + 2 * sizeof(NetSmem)); // [RT][MAX_IN]
    float* heads = xs + RT * MAX_IN;                                 // [RT][MAX_OUT + 1]: actor outputs, value
    constexpr int SS = ENV == 0 ? 4 : 8, OD = ENV == 0 ? 4 : 3;

    const int tid = threadIdx.x;
    const int net = tid >> 6, lt = tid & 63;      // network of this thread, thread index inside it
    const int I = p.in_dim, act = p.act, n = p.env.n;
    const int O = net == 0 ? p.out_dim : 1;
    NetSmem& m = nets[net];
    load_net(m, net == 0 ? p.actor_params : p.critic_params, I, O, net == 0 && p.gaussian, lt, 64);
    const int env0 = blockIdx.x * RT;
    const int env = env0 + tid;                   // environment of lanes 0..31 of warp 0
    const bool env_thread = tid < RT && env < n;
    float st[SS];
    float ep_r = 0.0f, ep_s = 0.0f;
    if (tid < RT) {
#pragma unroll
        for (int k = 0; k < MAX_IN; ++k) xs[tid * MAX_IN + k] = 0.0f;
    }
    if (env_thread) {
#pragma unroll
        for (int k = 0; k < SS; ++k) st[k] = p.env.states[(size_t)env * SS + k];
#pragma unroll
        for (int k = 0; k < OD; ++k) xs[tid * MAX_IN + k] = p.env.obs[(size_t)env * OD + k];
        ep_r = p.env.episode_rewards[env];
        ep_s = p.env.episode_steps[env];
    }
    __syncthreads();

    const int rg = lt >> 4, c0 = (lt & 15) * 4;   // rows rg, rg + 4, ..., rg + 28; columns c0..c0+3
    const long long total_steps0 = p.env.ctr->total_steps;
    for (int t = 0; t < p.T; ++t) {
        // h0 = act(x W0 + b0)
        {
            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = m.b0s[c0 + j];
            for (int k = 0; k < I; ++k) {
                const float4 w = *reinterpret_cast<const float4*>(m.W0s + k * H + c0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float a = xs[(rg + 4 * i) * MAX_IN + k];
                    acc[i][0] = fmaf(a, w.x, acc[i][0]);
                    acc[i][1] = fmaf(a, w.y, acc[i][1]);
                    acc[i][2] = fmaf(a, w.z, acc[i][2]);
                    acc[i][3] = fmaf(a, w.w, acc[i][3]);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
                *reinterpret_cast<float4*>(m.S0 + (rg + 4 * i) * PITCH + c0) =
                    make_float4(act_fwd(acc[i][0], act), act_fwd(acc[i][1], act), act_fwd(acc[i][2], act),
                                act_fwd(acc[i][3], act));
        }
        __syncthreads();
        {
            const float init[4] = {m.b1s[c0], m.b1s[c0 + 1], m.b1s[c0 + 2], m.b1s[c0 + 3]};
            tile_gemm64<4>(m.S0, m.W1s, rg, c0, init, [&](int r, int c, const float (&v)[4]) {
                *reinterpret_cast<float4*>(m.S1 + r * PITCH + c) =
                    make_float4(act_fwd(v[0], act), act_fwd(v[1], act), act_fwd(v[2], act), act_fwd(v[3], act));
            });
        }
        __syncthreads();
        // heads: first warp of each network, one row per lane
        if (lt < RT) {
            float out[MAX_OUT];
#pragma unroll
            for (int o = 0; o < MAX_OUT; ++o) out[o] = m.b2s[o];
            for (int k = 0; k < H; ++k) {
                const float hv = m.S1[lt * PITCH + k];
                const float4 w = *reinterpret_cast<const float4*>(m.W2s + k * MAX_OUT);
                out[0] = fmaf(hv, w.x, out[0]);
                out[1] = fmaf(hv, w.y, out[1]);
                out[2] = fmaf(hv, w.z, out[2]);
                out[3] = fmaf(hv, w.w, out[3]);
            }
            if (net == 0) {
#pragma unroll
                for (int o = 0; o < MAX_OUT; ++o) heads[lt * (MAX_OUT + 1) + o] = out[o];
            } else {
                heads[lt * (MAX_OUT + 1) + MAX_OUT] = out[0];
            }
        }
        __syncthreads();
        if (env_thread) {
            const unsigned long long ts = (unsigned long long)total_steps0 + (unsigned long long)t * (unsigned long long)n;
            const uint32_t seed = (uint32_t)(ts * 2654435761ull + (unsigned long long)t * 7919ull);
            const size_t off = (size_t)t * n + env;
            float a_out[MAX_OUT], lp;
            const int A = p.out_dim;
            if (p.gaussian) {
                float row[2 * MAX_OUT];
                for (int o = 0; o < A; ++o) { row[o] = heads[tid * (MAX_OUT + 1) + o]; row[A + o] = nets[0].lss[o]; }
                sample_continuous_one(row, A, seed, env, p.greedy, a_out, lp);
                for (int o = 0; o < A; ++o) p.r_actions[off * A + o] = a_out[o];
            } else {
                float row[MAX_OUT];
#pragma unroll
                for (int o = 0; o < MAX_OUT; ++o) row[o] = heads[tid * (MAX_OUT + 1) + o];
                sample_one(row, A, seed, env, p.greedy, a_out[0], lp);
                p.r_actions[off] = a_out[0];
            }
            const float value = heads[tid * (MAX_OUT + 1) + MAX_OUT];
            p.r_log_probs[off] = lp;
            p.r_values[off] = value;
#pragma unroll
            for (int k = 0; k < OD; ++k) p.r_obs[off * OD + k] = xs[tid * MAX_IN + k];
            // environment step, bookkeeping, selective reset
            RolloutStepArgs a = p.env;
            a.t = t;
            float reward, done;
            if (ENV == 0) {
                float s4[4] = {st[0], st[1], st[2], st[3]};
                bool d = cartpole::step(s4, (int)a_out[0]);
                reward = 1.0f;
                done = d ? 1.0f : 0.0f;
                st[0] = s4[0]; st[1] = s4[1]; st[2] = s4[2]; st[3] = s4[3];
            } else {
                float s8[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) s8[k] = st[k % SS];
                pendulum::step(s8, a_out[0], reward, done);
#pragma unroll
                for (int k = 0; k < SS; ++k) st[k] = s8[k];
            }
            a.r_rewards[off] = reward;
            a.r_dones[off] = done;
            ep_r = ep_r + reward;
            ep_s = ep_s + 1.0f;
            if (done > 0.5f) {
                unsigned long long slot = atomicAdd(&a.ctr->ring_head, 1ull);
                a.ring_returns[slot % EP_RING] = ep_r;
                a.ring_lengths[slot % EP_RING] = ep_s;
                atomicAdd(&a.ctr->completed_episodes, 1ull);
                atomicAdd(&a.ctr->sum_episode_reward, (double)ep_r);
                atomicAdd(&a.ctr->sum_episode_steps, (double)ep_s);
                ep_r = 0.0f;
                ep_s = 0.0f;
                const unsigned long long rs = auto_reset_seed(a);
                if (ENV == 0) {
                    float s4[4];
                    cartpole::reset(s4, (uint32_t)((unsigned long long)env * 2654435761ull + (uint32_t)rs));
                    st[0] = s4[0]; st[1] = s4[1]; st[2] = s4[2]; st[3] = s4[3];
                } else {
                    float s8[8];
                    pendulum::reset(s8, pendulum::combined_seed((float)rs, env));
#pragma unroll
                    for (int k = 0; k < SS; ++k) st[k] = s8[k];
                }
                done = 0.0f;   // both environments clear the flag in their selective reset
            }
            if (t == p.T - 1) {
                a.rewards[env] = reward;
                a.dones[env] = done;
                a.episode_rewards[env] = ep_r;
                a.episode_steps[env] = ep_s;
                p.values[env] = value;
                for (int o = 0; o < (p.gaussian ? A : 1); ++o) p.actions[(size_t)env * (p.gaussian ? A : 1) + o] = a_out[o];
#pragma unroll
                for (int k = 0; k < SS; ++k) a.states[(size_t)env * SS + k] = st[k];
#pragma unroll
                for (int k = 0; k < OD; ++k) a.obs[(size_t)env * OD + k] = st[k];
            }
#pragma unroll
            for (int k = 0; k < OD; ++k) xs[tid * MAX_IN + k] = st[k];
        }
        __syncthreads();
    }
}

constexpr int ROLLOUT_SMEM = 2 * (int)sizeof(NetSmem) + (RT * MAX_IN + RT * (MAX_OUT + 1)) * 4;

bool rollout_supported(int env_kind, const mrl_net_spec* actor, const mrl_net_spec* critic) {
    return (env_kind == MRL_ENV_CARTPOLE || env_kind == MRL_ENV_PENDULUM) && supported(actor) && supported(critic) &&
           critic->out_dim == 1;
}

int rollout(int env_kind, const mrl_net_spec* actor, const float* actor_params, const float* critic_params, int T,
            int greedy, float* actions, float* values, float* r_obs, float* r_actions, float* r_log_probs,
            float* r_values, const RolloutStepArgs& env, cudaStream_t st) {
    static bool attr_done = false;
    if (!attr_done) {
        MRL_CUDA_OK(cudaFuncSetAttribute(fused_rollout_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROLLOUT_SMEM));
        MRL_CUDA_OK(cudaFuncSetAttribute(fused_rollout_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROLLOUT_SMEM));
        attr_done = true;
    }
    RolloutArgs a{};
    a.actor_params = actor_params; a.critic_params = critic_params;
    a.in_dim = actor->in_dim; a.out_dim = actor->out_dim; a.act = actor->activation == MRL_ACT_RELU ? 0 : 1;
    a.gaussian = actor->head == MRL_HEAD_STOCHASTIC_ACTOR ? 1 : 0;
    a.greedy = greedy; a.T = T;
    a.actions = actions; a.values = values;
    a.r_obs = r_obs; a.r_actions = r_actions; a.r_log_probs = r_log_probs; a.r_values = r_values;
    a.env = env;
    const int grid = ceil_div(env.n, RT);
    if (env_kind == MRL_ENV_CARTPOLE) { MRL_LAUNCH(fused_rollout_kernel<0>, grid, RTHREADS, ROLLOUT_SMEM, st, a); }
    else { MRL_LAUNCH(fused_rollout_kernel<1>, grid, RTHREADS, ROLLOUT_SMEM, st, a); }
    return MRL_OK;
}

constexpr int SMEM_FLOATS = 2 * H * H + 3 * TM * PITCH + MAX_IN * H + 2 * H + H * MAX_OUT + 2 * MAX_OUT + TM * MAX_IN +
                            TM * 2 * MAX_OUT;
constexpr int SMEM_BYTES = SMEM_FLOATS * 4;

bool supported(const mrl_net_spec* net) {
    return net->hidden_dim == H && net->in_dim >= 1 && net->in_dim <= MAX_IN && net->out_dim >= 1 &&
           net->out_dim <= MAX_OUT;
}

int grid_blocks(int batch) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    int tiles = (batch + TM - 1) / TM;
    return tiles < sms ? tiles : sms;
}

int64_t partial_doubles(const mrl_net_spec* net, int batch, int param_size) {
    (void)net;
    return (int64_t)grid_blocks(batch) * (param_size + 1);
}

// Forward, loss gradient and backward of one network over one minibatch; grads receives the
// parameter gradients and kl_out (nullable) the sum of the per-row KL terms.
int train_step(const mrl_net_spec* net, int mode, const float* params, int param_size, const float* x,
               const float* actions, const float* adv, const float* ret, const float* old_lp, const float* old_v,
               int batch, float clip_eps, float entropy_coef, float value_loss_coef, int clip_value, double* partial,
               float* grads, float* kl_out, cudaStream_t st) {
    static bool attr_done = false;
    if (!attr_done) {
        MRL_CUDA_OK(cudaFuncSetAttribute(fused_train_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_done = true;
    }
    TrainArgs a{};
    a.params = params; a.in_dim = net->in_dim; a.out_dim = net->out_dim;
    a.act = net->activation == MRL_ACT_RELU ? 0 : 1;
    a.mode = mode;
    a.x = x; a.actions = actions; a.adv = adv; a.ret = ret; a.old_lp = old_lp; a.old_v = old_v;
    a.B = batch; a.clip_eps = clip_eps; a.entropy_coef = entropy_coef; a.value_loss_coef = value_loss_coef;
    a.clip_value = clip_value;
    a.partial = partial;
    a.pstride = param_size + 1;
    const int grid = grid_blocks(batch);
    MRL_LAUNCH(fused_train_kernel, grid, THREADS, SMEM_BYTES, st, a);
    MRL_LAUNCH(reduce_partials_kernel, ceil_div(param_size + 1, 128), 128, 0, st, partial, grid, a.pstride, param_size,
               grads, kl_out);
    return MRL_OK;
}

}  // namespace small
}  // namespace mrl

using namespace mrl;

extern "C" int64_t mrl_fused_train_scratch_doubles(const mrl_net_spec* net, int batch) {
    if (!net || batch <= 0 || !small::supported(net)) return -1;
    return small::partial_doubles(net, batch, mrl_net_param_size(net));
}

extern "C" int mrl_fused_train_step(const mrl_net_spec* net, int mode, int batch, const float* params,
                                    const float* obs, const float* actions, const float* advantages,
                                    const float* returns, const float* old_log_probs, const float* old_values,
                                    float clip_epsilon, float entropy_coef, float value_loss_coef, int clip_value,
                                    double* scratch, float* grads, float* kl_sum, void* stream) {
    MRL_CHECK_ARG(net && batch > 0 && params && obs && scratch && grads);
    MRL_CHECK_ARG(mode >= 0 && mode <= 3);
    if (!small::supported(net)) {
        set_error("the fused train step covers hidden_dim 64, in_dim <= 8, out_dim <= 4");
        return MRL_ERR_UNSUPPORTED;
    }
    const bool actor = mode == small::ACTOR_DISCRETE || mode == small::ACTOR_GAUSSIAN;
    MRL_CHECK_ARG((mode == small::ACTOR_GAUSSIAN) == (net->head == MRL_HEAD_STOCHASTIC_ACTOR));
    if (actor) MRL_CHECK_ARG(actions && advantages && old_log_probs);
    else MRL_CHECK_ARG(returns && net->out_dim == 1 && (!clip_value || old_values));
    return small::train_step(net, mode, params, mrl_net_param_size(net), obs, actions, advantages, returns,
                             old_log_probs, old_values, batch, clip_epsilon, entropy_coef, value_loss_coef, clip_value,
                             scratch, grads, kl_sum, as_stream(stream));
}
