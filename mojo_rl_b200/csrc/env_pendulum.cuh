// PendulumV2 GPU path of the reference (envs/pendulum/pendulum_v2.mojo:300-604,
// constants.mojo): state row [cos, sin, theta_dot, theta, step, done, total_reward, last_torque].
#pragma once
#include "common.cuh"

namespace mrl {
namespace pendulum {

constexpr double MAX_SPEED = 8.0, MAX_TORQUE = 2.0, DT = 0.05, G = 10.0, M = 1.0, L = 1.0;
constexpr int MAX_STEPS = 200;
constexpr int STATE_SIZE = 8, OBS_DIM = 3, ACTION_DIM = 1;

// One step on a row held in registers; pendulum_v2.mojo:407-544.
__device__ __forceinline__ void step(float (&s)[8], float raw_action, float& reward, float& done) {
    const float max_speed = (float)MAX_SPEED, max_torque = (float)MAX_TORQUE, dt = (float)DT;
    const float g = (float)G, m = (float)M, l = (float)L, max_steps = (float)MAX_STEPS;
    float theta = s[3], theta_dot = s[2], step_count = s[4], total_reward = s[6];
    float u = raw_action * max_torque;
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
    // the reference loops `while theta > PI`; |theta| grows by at most 0.4 per step, so a
    // bounded number of passes is equivalent and cannot spin on a non-finite angle
    for (int i = 0; i < 4 && theta > PI; ++i) theta = theta - TWO_PI;
    for (int i = 0; i < 4 && theta < -PI; ++i) theta = theta + TWO_PI;
    step_count = step_count + 1.0f;
    reward = -(theta * theta + 0.1f * theta_dot * theta_dot + 0.001f * u * u);
    total_reward = total_reward + reward;
    done = step_count >= max_steps ? 1.0f : 0.0f;
    float sn, cs;
    mrl_sincosf(theta, &sn, &cs);
    s[0] = cs; s[1] = sn; s[2] = theta_dot; s[3] = theta;
    s[4] = step_count; s[5] = done; s[6] = total_reward; s[7] = u;
}

// pendulum_v2.mojo:548-604
__device__ __forceinline__ void reset(float (&s)[8], int64_t seed) {
    Philox rng((uint64_t)seed, 0);
    float r[4];
    rng.step_uniform(r);
    const float PI = 3.14159265358979323846f;
    float theta = (r[0] * 2.0f - 1.0f) * PI;
    float theta_dot = r[1] * 2.0f - 1.0f;
    float sn, cs;
    mrl_sincosf(theta, &sn, &cs);
    s[0] = cs; s[1] = sn; s[2] = theta_dot; s[3] = theta;
    s[4] = 0.0f; s[5] = 0.0f; s[6] = 0.0f; s[7] = 0.0f;
}

// Int(seed_f32) * 2654435761 + env * 12345 (pendulum_v2.mojo:330, :387)
__host__ __device__ __forceinline__ int64_t combined_seed(float seed_f32, int env) {
    int64_t si = (int64_t)seed_f32;
    return (int64_t)((uint64_t)si * 2654435761ull + (uint64_t)env * 12345ull);
}

__device__ __forceinline__ void load_row(const float* __restrict__ p, float (&s)[8]) {
    float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    s[0] = a.x; s[1] = a.y; s[2] = a.z; s[3] = a.w; s[4] = b.x; s[5] = b.y; s[6] = b.z; s[7] = b.w;
}
__device__ __forceinline__ void store_row(float* __restrict__ p, const float (&s)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(s[0], s[1], s[2], s[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(s[4], s[5], s[6], s[7]);
}

}  // namespace pendulum
}  // namespace mrl
