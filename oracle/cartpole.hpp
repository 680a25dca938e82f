// CPU ORACLE - test infrastructure, not product code.
//
// fp32 restatement of CartPole's GPU kernels, envs/cartpole.mojo:702-905 and
// the obs copy of its step wrapper (:963-984).  xorshift32 is fully specified
// in the reference (deep_rl/gpu/random.mojo:11-41), so reset states are
// reproducible end to end; cos/sin come from include/mrl_detmath.h.
#pragma once
#include "physics2d.hpp"

namespace oracle {
namespace cartpole {

// envs/cartpole.mojo:54-68
constexpr double GRAVITY = 9.8, CART_MASS = 1.0, POLE_MASS = 0.1, TOTAL_MASS = CART_MASS + POLE_MASS;
constexpr double POLE_HALF_LENGTH = 0.5, POLE_MASS_LENGTH = POLE_MASS * POLE_HALF_LENGTH;
constexpr double FORCE_MAG = 10.0, TAU = 0.02, X_THRESHOLD = 2.4, THETA_THRESHOLD = 0.2095;
constexpr int STATE_SIZE = 4, OBS_DIM = 4, NUM_ACTIONS = 2;

// envs/cartpole.mojo:702-781: no step counter, reward 1.0 on every step.
inline void step_all(float* states, const float* actions, float* rewards, float* dones, float* obs,
                     int n) {
    for (int i = 0; i < n; ++i) {
        float* s = states + (size_t)i * STATE_SIZE;
        float force = (int)actions[i] == 1 ? (float)FORCE_MAG : (float)(-FORCE_MAG);
        float sin_theta, cos_theta;
        mrl_sincosf(s[2], &sin_theta, &cos_theta);
        float temp = (force + (float)POLE_MASS_LENGTH * s[3] * s[3] * sin_theta) / (float)TOTAL_MASS;
        float theta_acc =
            ((float)GRAVITY * sin_theta - cos_theta * temp) /
            ((float)POLE_HALF_LENGTH *
             ((float)(4.0 / 3.0) - (float)POLE_MASS * cos_theta * cos_theta / (float)TOTAL_MASS));
        float x_acc = temp - (float)POLE_MASS_LENGTH * theta_acc * cos_theta / (float)TOTAL_MASS;
        s[0] += (float)TAU * s[1];
        s[1] += (float)TAU * x_acc;
        s[2] += (float)TAU * s[3];
        s[3] += (float)TAU * theta_acc;
        bool done = (s[0] < (float)(-X_THRESHOLD)) || (s[0] > (float)X_THRESHOLD) ||
                    (s[2] < (float)(-THETA_THRESHOLD)) || (s[2] > (float)THETA_THRESHOLD);
        rewards[i] = 1.0f;
        dones[i] = done ? 1.0f : 0.0f;
        for (int d = 0; d < OBS_DIM; ++d) obs[(size_t)i * OBS_DIM + d] = s[d];
    }
}

inline void reset_one(float* s, uint32_t seed) {
    uint32_t rng = xorshift32(seed);
    s[0] = random_range(rng, -0.05f, 0.05f);
    s[1] = random_range(rng, -0.05f, 0.05f);
    s[2] = random_range(rng, -0.05f, 0.05f);
    s[3] = random_range(rng, -0.05f, 0.05f);
}

// envs/cartpole.mojo:784-835: the seed argument of the trait method is ignored.
inline void reset_all(float* states, int n) {
    for (int i = 0; i < n; ++i)
        reset_one(states + (size_t)i * STATE_SIZE, (uint32_t)((uint64_t)i * 2654435761ull + 12345ull));
}

// envs/cartpole.mojo:838-905, :1085-1091: seed truncated to 32 bits; resets
// where done >= 0.5 (the test is `done < 0.5 -> return`) and clears the flag.
inline void selective_reset(float* states, float* dones, int n, uint64_t rng_seed) {
    uint32_t seed32 = (uint32_t)rng_seed;
    for (int i = 0; i < n; ++i) {
        if (dones[i] < 0.5f) continue;
        reset_one(states + (size_t)i * STATE_SIZE, (uint32_t)((uint64_t)i * 2654435761ull + seed32));
        dones[i] = 0.0f;
    }
}

}  // namespace cartpole
}  // namespace oracle
