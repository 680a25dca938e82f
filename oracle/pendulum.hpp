// CPU ORACLE - test infrastructure, not product code.
//
// fp32 restatement of PendulumV2's GPU path: envs/pendulum/pendulum_v2.mojo:300-604,
// constants.mojo:12-155.  Reset draws come from Philox (see physics2d.hpp:
// parity unpinned at that boundary).
#pragma once
#include "physics2d.hpp"

namespace oracle {
namespace pendulum {

// envs/pendulum/constants.mojo:98-109
constexpr double MAX_SPEED = 8.0, MAX_TORQUE = 2.0, DT = 0.05, G = 10.0, M = 1.0, L = 1.0;
constexpr int MAX_STEPS = 200;
constexpr int STATE_SIZE = 8, OBS_DIM = 3, ACTION_DIM = 1;
// layout: [cos, sin, theta_dot, theta, step_count, done, total_reward, last_torque]

// pendulum_v2.mojo:407-544
inline void step_all(float* states, const float* actions, float* rewards, float* dones, float* obs, int n) {
    const float max_speed = (float)MAX_SPEED, max_torque = (float)MAX_TORQUE, dt = (float)DT;
    const float g = (float)G, m = (float)M, l = (float)L, max_steps = (float)MAX_STEPS;
    for (int env = 0; env < n; ++env) {
        float* s = states + (size_t)env * STATE_SIZE;
        float theta = s[3], theta_dot = s[2], step_count = s[4], total_reward = s[6];
        float u = actions[env] * max_torque;
        if (u > max_torque) u = max_torque;
        else if (u < -max_torque) u = -max_torque;
        float sin_theta = mrl_sinf(theta);
        float theta_acc = (3.0f * g / (2.0f * l)) * sin_theta + (3.0f / (m * l * l)) * u;
        theta_dot = theta_dot + theta_acc * dt;
        theta = theta + theta_dot * dt;
        if (theta_dot > max_speed) theta_dot = max_speed;
        else if (theta_dot < -max_speed) theta_dot = -max_speed;
        const float PI = 3.14159265358979323846f;
        const float TWO_PI = PI * 2.0f;
        while (theta > PI) theta = theta - TWO_PI;
        while (theta < -PI) theta = theta + TWO_PI;
        step_count = step_count + 1.0f;
        float reward = -(theta * theta + 0.1f * theta_dot * theta_dot + 0.001f * u * u);
        total_reward = total_reward + reward;
        float is_done = step_count >= max_steps ? 1.0f : 0.0f;
        float sn, cs;
        mrl_sincosf(theta, &sn, &cs);
        s[0] = cs; s[1] = sn; s[2] = theta_dot; s[3] = theta;
        s[4] = step_count; s[5] = is_done; s[6] = total_reward; s[7] = u;
        rewards[env] = reward;
        dones[env] = is_done;
        obs[(size_t)env * 3 + 0] = cs; obs[(size_t)env * 3 + 1] = sn; obs[(size_t)env * 3 + 2] = theta_dot;
    }
}

// pendulum_v2.mojo:548-604
inline void reset_env(float* s, int64_t seed) {
    Philox rng((uint64_t)seed, 0);
    float r[4];
    rng.step_uniform(r);
    const float PI = 3.14159265358979323846f;
    float theta = (r[0] * 2.0f - 1.0f) * PI;
    float theta_dot = r[1] * 2.0f - 1.0f;
    for (int i = 0; i < STATE_SIZE; ++i) s[i] = 0.0f;
    float sn, cs;
    mrl_sincosf(theta, &sn, &cs);
    s[0] = cs; s[1] = sn; s[2] = theta_dot; s[3] = theta;
}

// pendulum_v2.mojo:330: Int(seed_f32) * 2654435761 + env * 12345 (env, not env + 1)
inline int64_t combined_seed(uint64_t rng_seed, int env) {
    float seed_f = (float)rng_seed;
    int64_t si = (int64_t)seed_f;
    return (int64_t)((uint64_t)si * 2654435761ull + (uint64_t)env * 12345ull);
}
inline void reset_all(float* states, int n, uint64_t rng_seed) {
    for (int i = 0; i < n; ++i) reset_env(states + (size_t)i * STATE_SIZE, combined_seed(rng_seed, i));
}
// pendulum_v2.mojo:381-392: resets where done > 0.5 and clears the flag
inline void selective_reset(float* states, float* dones, int n, uint64_t rng_seed) {
    for (int i = 0; i < n; ++i)
        if (dones[i] > 0.5f) {
            reset_env(states + (size_t)i * STATE_SIZE, combined_seed(rng_seed, i));
            dones[i] = 0.0f;
        }
}

}  // namespace pendulum
}  // namespace oracle
