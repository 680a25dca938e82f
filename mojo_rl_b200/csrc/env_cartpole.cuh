// CartPole GPU kernels of the reference (envs/cartpole.mojo:702-905, obs copy of
// the step wrapper :963-984): no step counter, reward 1.0 on every step.
#pragma once
#include "common.cuh"

namespace mrl {
namespace cartpole {

constexpr double GRAVITY = 9.8, CART_MASS = 1.0, POLE_MASS = 0.1, TOTAL_MASS = CART_MASS + POLE_MASS;
constexpr double POLE_HALF_LENGTH = 0.5, POLE_MASS_LENGTH = POLE_MASS * POLE_HALF_LENGTH;
constexpr double FORCE_MAG = 10.0, TAU = 0.02, X_THRESHOLD = 2.4, THETA_THRESHOLD = 0.2095;
constexpr int STATE_SIZE = 4, OBS_DIM = 4, NUM_ACTIONS = 2;

// One Euler step on (x, x_dot, theta, theta_dot); returns done.
__device__ __forceinline__ bool step(float (&s)[4], int action) {
    float force = action == 1 ? (float)FORCE_MAG : (float)(-FORCE_MAG);
    float sin_theta, cos_theta;
    mrl_sincosf(s[2], &sin_theta, &cos_theta);
    float temp = (force + (float)POLE_MASS_LENGTH * s[3] * s[3] * sin_theta) / (float)TOTAL_MASS;
    float theta_acc =
        ((float)GRAVITY * sin_theta - cos_theta * temp) /
        ((float)POLE_HALF_LENGTH *
         ((float)(4.0 / 3.0) - (float)POLE_MASS * cos_theta * cos_theta / (float)TOTAL_MASS));
    float x_acc = temp - (float)POLE_MASS_LENGTH * theta_acc * cos_theta / (float)TOTAL_MASS;
    float x = s[0], x_dot = s[1], theta = s[2], theta_dot = s[3];
    s[0] = x + (float)TAU * x_dot;
    s[1] = x_dot + (float)TAU * x_acc;
    s[2] = theta + (float)TAU * theta_dot;
    s[3] = theta_dot + (float)TAU * theta_acc;
    return (s[0] < (float)(-X_THRESHOLD)) || (s[0] > (float)X_THRESHOLD) ||
           (s[2] < (float)(-THETA_THRESHOLD)) || (s[2] > (float)THETA_THRESHOLD);
}

// cartpole.mojo:802-835 / :873-902: four xorshift32 draws in [-0.05, 0.05].
__device__ __forceinline__ void reset(float (&s)[4], uint32_t seed) {
    uint32_t rng = xorshift32(seed);
    s[0] = xs_range(rng, -0.05f, 0.05f);
    s[1] = xs_range(rng, -0.05f, 0.05f);
    s[2] = xs_range(rng, -0.05f, 0.05f);
    s[3] = xs_range(rng, -0.05f, 0.05f);
}

}  // namespace cartpole
}  // namespace mrl
