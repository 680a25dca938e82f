// Per-sample device functions of the PPO kernels, shared by the stand-alone
// entry points and the fused phases.
#pragma once
#include "common.cuh"

namespace mrl {

constexpr int MAX_ACTIONS = 16;

// _sample_actions_kernel body (deep_agents/ppo/ppo.mojo:4064-4123): per-env
// xorshift32 stream seeded by seed ^ (i * 2654435761); inverse-CDF draw that
// falls through to action 0; log-prob = log(p + 1e-8).  greedy: first maximum
// of the softmax probabilities (ppo.mojo:1019-1022, core/utils/softmax.mojo).
__device__ __forceinline__ void sample_one(const float* __restrict__ l, int A, uint32_t seed, int i,
                                           int greedy, float& action_out, float& log_prob_out) {
    uint32_t rng = seed ^ ((uint32_t)i * 2654435761u);
    rng = xorshift32(rng);
    float max_logit = l[0];
    for (int a = 1; a < A; ++a) if (l[a] > max_logit) max_logit = l[a];
    float sum_exp = 0.0f;
    for (int a = 0; a < A; ++a) sum_exp = sum_exp + mrl_expf(l[a] - max_logit);
    int selected = 0;
    if (greedy) {
        float best = mrl_expf(l[0] - max_logit) / sum_exp;
        for (int a = 1; a < A; ++a) {
            float p = mrl_expf(l[a] - max_logit) / sum_exp;
            if (p > best) { best = p; selected = a; }
        }
    } else {
        float rand_val = xs_uniform(rng);
        float cumsum = 0.0f;
        for (int a = 0; a < A; ++a) {
            float prob = mrl_expf(l[a] - max_logit) / sum_exp;
            cumsum = cumsum + prob;
            if (rand_val < cumsum) { selected = a; break; }
        }
    }
    action_out = (float)selected;
    float sp = mrl_expf(l[selected] - max_logit) / sum_exp;
    log_prob_out = mrl_logf(sp + 1e-8f);
}

// ppo_actor_grad_with_kl_kernel body (ppo.mojo:285-378).
__device__ __forceinline__ void actor_grad_one(const float* __restrict__ l, int A, float old_log_prob,
                                               float advantage, int action, float clip_epsilon,
                                               float entropy_coef, float batch_div, float* g, float& kl) {
    float max_logit = l[0];
    for (int a = 1; a < A; ++a) if (l[a] > max_logit) max_logit = l[a];
    float sum_exp = 0.0f;
    for (int a = 0; a < A; ++a) sum_exp = sum_exp + mrl_expf(l[a] - max_logit);
    float probs[MAX_ACTIONS];
    float p_action = 0.0f;
    for (int a = 0; a < A; ++a) {
        probs[a] = mrl_expf(l[a] - max_logit) / sum_exp;
        if (a == action) p_action = probs[a];
    }
    float new_log_prob = mrl_logf(p_action + 1e-8f);
    kl = old_log_prob - new_log_prob;
    float ratio = mrl_expf(new_log_prob - old_log_prob);
    bool is_clipped = (ratio < 1.0f - clip_epsilon) || (ratio > 1.0f + clip_epsilon);
    for (int a = 0; a < A; ++a) {
        if (is_clipped) { g[a] = 0.0f; continue; }
        float d_log_prob = a == action ? 1.0f - probs[a] : -probs[a];
        float log_prob_ent = mrl_logf(probs[a] + 1e-8f);
        float d_entropy = -probs[a] * (1.0f + log_prob_ent);
        g[a] = (-advantage * ratio * d_log_prob - entropy_coef * d_entropy) / batch_div;
    }
}

// ppo_critic_grad_kernel / ppo_critic_grad_clipped_kernel bodies (ppo.mojo:538-633).
__device__ __forceinline__ float critic_grad_one(float v_new, float v_old, float ret, float value_loss_coef,
                                                 float clip_epsilon, int clip_value, float batch_div) {
    if (!clip_value) return 2.0f * value_loss_coef * (v_new - ret) / batch_div;
    float v_diff = v_new - v_old;
    float v_clipped;
    if (v_diff > clip_epsilon) v_clipped = v_old + clip_epsilon;
    else if (v_diff < -clip_epsilon) v_clipped = v_old - clip_epsilon;
    else v_clipped = v_new;
    float loss_unclipped = (v_new - ret) * (v_new - ret);
    float loss_clipped = (v_clipped - ret) * (v_clipped - ret);
    float grad;
    if (loss_unclipped > loss_clipped) grad = 2.0f * (v_new - ret);
    else if (v_diff > clip_epsilon || v_diff < -clip_epsilon) grad = 0.0f;
    else grad = 2.0f * (v_new - ret);
    return value_loss_coef * grad / batch_div;
}

// Host-side launchers shared with the fused agent (defined in ppo_kernels.cu / mlp.cu).
int normalize_advantages_impl(int64_t n, float* adv, double* stats2, cudaStream_t st);
int grad_clip_impl(int n, float* grads, float max_norm, double* sumsq, float* report, cudaStream_t st);
int mlp_forward_impl(const mrl_net_spec* net, int batch, const float* in, const float* params, float* out,
                     float* cache, float* workspace, cudaStream_t st);
int mlp_backward_impl(const mrl_net_spec* net, int batch, const float* grad_out, const float* params,
                      const float* cache, float* grad_in, float* grads, float* workspace, cudaStream_t st);
int64_t mlp_workspace_floats(const mrl_net_spec* n, int batch);

}  // namespace mrl
