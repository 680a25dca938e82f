// CPU ORACLE - test infrastructure, not product code.
//
// fp32 restatement of HalfCheetahPlanarV2's GPU path:
// envs/half_cheetah/cheetah_planar_v2.mojo:1039-1901, constants.mojo,
// physics2d/collision/flat_terrain.mojo:456-580.  Seven rectangles (torso and
// two three-segment legs) joined by six motorised, limited revolute joints on a
// flat ground at y = 0; five physics sub-steps per environment step.  Reset
// draws come from Philox (see physics2d.hpp: parity unpinned at that boundary).
#pragma once
#include "physics2d.hpp"

namespace oracle {
namespace cheetah {

constexpr Layout L = CHEETAH_LAYOUT;
constexpr int STATE_SIZE = L.state_size();  // 253
constexpr int OBS_DIM = 17, ACTION_DIM = 6, NUM_BODIES = 7, NUM_SHAPES = 7, MAX_CONTACTS = 14, MAX_JOINTS = 6;
constexpr int OBS_OFFSET = 0, BODIES_OFFSET = L.bodies_offset(), FORCES_OFFSET = L.forces_offset(),
              JOINTS_OFFSET = L.joints_offset(), JOINT_COUNT_OFFSET = L.joint_count_offset(),
              METADATA_OFFSET = L.metadata_offset();
constexpr int META_STEP_COUNT = 0, META_PREV_X = 1, META_DONE = 3, META_TOTAL_REWARD = 4;

// envs/half_cheetah/constants.mojo
constexpr double DT = 0.01, GRAVITY_X = 0.0, GRAVITY_Y = -9.81, FRICTION = 0.9, RESTITUTION = 0.0,
                 BAUMGARTE = 0.2, SLOP = 0.005;
constexpr int FRAME_SKIP = 5, VELOCITY_ITERATIONS = 4, POSITION_ITERATIONS = 2, MAX_STEPS = 1000;
constexpr double TORSO_LENGTH = 1.0, TORSO_RADIUS = 0.046, TORSO_MASS = 6.25, INIT_HEIGHT = 0.7;
// segments in body order 1..6: bthigh, bshin, bfoot, fthigh, fshin, ffoot
constexpr double SEG_LENGTH[6] = {0.145, 0.15, 0.094, 0.133, 0.106, 0.07};
constexpr double SEG_RADIUS[6] = {0.046, 0.046, 0.046, 0.046, 0.046, 0.046};
constexpr double SEG_MASS[6] = {1.0, 1.0, 1.0, 1.0, 1.0, 1.0};
constexpr double LIMIT_LOW[6] = {-0.52, -0.785, -0.4, -1.0, -1.2, -0.5};
constexpr double LIMIT_HIGH[6] = {1.05, 0.785, 0.785, 0.7, 0.87, 0.5};
constexpr double MAX_TORQUE = 1.0, CTRL_COST_WEIGHT = 0.1, FORWARD_REWARD_WEIGHT = 1.0, HEIGHT_BONUS_WEIGHT = 1.0,
                 TARGET_HEIGHT = 0.5, MIN_HEIGHT_FOR_BONUS = 0.1, GROUND_CONTACT_PENALTY = 0.5;
constexpr int BODY_BFOOT = 3, BODY_FFOOT = 6;

// _init_shapes_gpu, cheetah_planar_v2.mojo:1497-1573: [NUM_SHAPES][SHAPE_MAX_SIZE]
inline void init_shapes(float* shapes) {
    for (int i = 0; i < NUM_SHAPES * SHAPE_MAX_SIZE; ++i) shapes[i] = 0.0f;
    float half_len = (float)(TORSO_LENGTH / 2), half_h = (float)TORSO_RADIUS;
    float* s0 = shapes;
    s0[0] = (float)SHAPE_POLYGON; s0[1] = 4.0f;
    s0[2] = -half_len; s0[3] = -half_h; s0[4] = -half_len; s0[5] = half_h;
    s0[6] = half_len; s0[7] = half_h; s0[8] = half_len; s0[9] = -half_h;
    for (int k = 0; k < 6; ++k) {
        float* sh = shapes + (k + 1) * SHAPE_MAX_SIZE;
        float seg_len = (float)SEG_LENGTH[k] / 2.0f, seg_w = (float)SEG_RADIUS[k];
        sh[0] = (float)SHAPE_POLYGON; sh[1] = 4.0f;
        sh[2] = -seg_w; sh[3] = -seg_len; sh[4] = -seg_w; sh[5] = seg_len;
        sh[6] = seg_w; sh[7] = seg_len; sh[8] = seg_w; sh[9] = -seg_len;
    }
}

// _compute_obs_gpu, cheetah_planar_v2.mojo:1427-1494
inline void compute_obs(float* s) {
    auto body = [&](int b) { return s + BODIES_OFFSET + b * BODY_STATE_SIZE; };
    const float* t = body(0);
    float* o = s + OBS_OFFSET;
    o[0] = t[IDX_Y];
    o[1] = t[IDX_ANGLE];
    const int parent[6] = {0, 1, 2, 0, 4, 5};
    for (int k = 0; k < 6; ++k) {
        o[2 + k] = body(k + 1)[IDX_ANGLE] - body(parent[k])[IDX_ANGLE];
        o[11 + k] = body(k + 1)[IDX_OMEGA] - body(parent[k])[IDX_OMEGA];
    }
    o[8] = t[IDX_VX];
    o[9] = t[IDX_VY];
    o[10] = t[IDX_OMEGA];
}

// _reset_env_gpu, cheetah_planar_v2.mojo:1175-1234 (+ :1237-1424)
inline void reset_env(float* s, int64_t seed) {
    Philox rng((uint64_t)seed, 0);
    float r[4];
    rng.step_uniform(r);
    float init_x = 0.0f, init_y = (float)INIT_HEIGHT;
    float init_vx = (r[0] * 2.0f - 1.0f) * 0.1f;
    float init_vy = (r[1] * 2.0f - 1.0f) * 0.1f;
    auto set_body = [&](int b, float x, float y, float inv_mass, float inv_inertia) {
        float* p = s + BODIES_OFFSET + b * BODY_STATE_SIZE;
        p[IDX_X] = x; p[IDX_Y] = y; p[IDX_ANGLE] = 0.0f;
        p[IDX_VX] = init_vx; p[IDX_VY] = init_vy; p[IDX_OMEGA] = 0.0f;
        p[IDX_INV_MASS] = inv_mass; p[IDX_INV_INERTIA] = inv_inertia;
        p[IDX_SHAPE] = (float)b;
    };
    set_body(0, init_x, init_y, (float)(1.0 / TORSO_MASS),
             (float)(1.0 / (TORSO_MASS * TORSO_LENGTH * TORSO_LENGTH / 12.0)));
    float back_hip_x = init_x - (float)(TORSO_LENGTH / 2), front_hip_x = init_x + (float)(TORSO_LENGTH / 2);
    // the y offsets are compile-time Float64 sums rounded once to fp32
    const double yoff[6] = {SEG_LENGTH[0] / 2, SEG_LENGTH[0] + SEG_LENGTH[1] / 2,
                            SEG_LENGTH[0] + SEG_LENGTH[1] + SEG_LENGTH[2] / 2,
                            SEG_LENGTH[3] / 2, SEG_LENGTH[3] + SEG_LENGTH[4] / 2,
                            SEG_LENGTH[3] + SEG_LENGTH[4] + SEG_LENGTH[5] / 2};
    for (int k = 0; k < 6; ++k)
        set_body(k + 1, k < 3 ? back_hip_x : front_hip_x, init_y - (float)yoff[k], (float)(1.0 / SEG_MASS[k]),
                 (float)(12.0 / (SEG_MASS[k] * SEG_LENGTH[k] * SEG_LENGTH[k])));
    // joints: hip, knee, ankle per leg
    s[JOINT_COUNT_OFFSET] = 6.0f;
    const int body_a[6] = {0, 1, 2, 0, 4, 5};
    for (int j = 0; j < 6; ++j) {
        float* jt = s + JOINTS_OFFSET + j * JOINT_DATA_SIZE;
        float ax, ay;
        if (j == 0) { ax = (float)(-TORSO_LENGTH / 2); ay = 0.0f; }
        else if (j == 3) { ax = (float)(TORSO_LENGTH / 2); ay = 0.0f; }
        else { ax = 0.0f; ay = (float)(-SEG_LENGTH[j - 1] / 2); }
        jt[JOINT_TYPE] = (float)JOINT_REVOLUTE;
        jt[JOINT_BODY_A] = (float)body_a[j];
        jt[JOINT_BODY_B] = (float)(j + 1);
        jt[JOINT_ANCHOR_AX] = ax;
        jt[JOINT_ANCHOR_AY] = ay;
        jt[JOINT_ANCHOR_BX] = 0.0f;
        jt[JOINT_ANCHOR_BY] = (float)(SEG_LENGTH[j] / 2);
        jt[JOINT_REF_ANGLE] = 0.0f;
        jt[JOINT_LOWER_LIMIT] = (float)LIMIT_LOW[j];
        jt[JOINT_UPPER_LIMIT] = (float)LIMIT_HIGH[j];
        jt[JOINT_MAX_MOTOR_TORQUE] = (float)MAX_TORQUE;
        jt[JOINT_MOTOR_SPEED] = 0.0f;
        jt[JOINT_FLAGS] = (float)(JOINT_FLAG_LIMIT_ENABLED | JOINT_FLAG_MOTOR_ENABLED);
    }
    for (int b = 0; b < NUM_BODIES; ++b)
        for (int k = 0; k < 3; ++k) s[FORCES_OFFSET + b * 3 + k] = 0.0f;
    s[METADATA_OFFSET + META_STEP_COUNT] = 0.0f;
    s[METADATA_OFFSET + META_PREV_X] = init_x;
    s[METADATA_OFFSET + META_DONE] = 0.0f;
    s[METADATA_OFFSET + META_TOTAL_REWARD] = 0.0f;
    compute_obs(s);
}

// FlatTerrainCollision.detect_single_env, flat_terrain.mojo:456-580 (polygon branch
// and circle branch).  Returns the contact count.
inline int flat_terrain_detect(const float* s, const float* shapes, float ground_y, float* contacts) {
    int count = 0;
    for (int b = 0; b < NUM_BODIES; ++b) {
        const float* body = s + BODIES_OFFSET + b * BODY_STATE_SIZE;
        float bx = body[IDX_X], by = body[IDX_Y];
        const float* sh = shapes + (int)body[IDX_SHAPE] * SHAPE_MAX_SIZE;
        float sin_a, cos_a;
        mrl_sincosf(body[IDX_ANGLE], &sin_a, &cos_a);
        if ((int)sh[0] == SHAPE_POLYGON) {
            int n_verts = (int)sh[1];
            for (int v = 0; v < MAX_POLYGON_VERTS; ++v) {
                if (v >= n_verts) break;
                float lx = sh[2 + v * 2], ly = sh[3 + v * 2];
                float wx = bx + lx * cos_a - ly * sin_a;
                float wy = by + lx * sin_a + ly * cos_a;
                float pen = ground_y - wy;
                if (pen > 0.0f && count < MAX_CONTACTS) {
                    write_contact(contacts + count * CONTACT_DATA_SIZE, b, wx, wy, 0.0f, 1.0f, pen);
                    ++count;
                }
            }
        } else if ((int)sh[0] == SHAPE_CIRCLE) {
            float radius = sh[1], ox = sh[2], oy = sh[3];
            float cx = bx + ox * cos_a - oy * sin_a;
            float cy = by + ox * sin_a + oy * cos_a;
            float pen = ground_y - (cy - radius);
            if (pen > 0.0f && count < MAX_CONTACTS) {
                write_contact(contacts + count * CONTACT_DATA_SIZE, b, cx, cy - radius, 0.0f, 1.0f, pen);
                ++count;
            }
        }
    }
    return count;
}

// _step_env_gpu, cheetah_planar_v2.mojo:1671-1901
inline void step_env(float* s, const float* shapes, const float* action, float* reward_out, float* done_out) {
    const float dt = (float)DT, gx = (float)GRAVITY_X, gy = (float)GRAVITY_Y, friction = (float)FRICTION,
                restitution = (float)RESTITUTION, baumgarte = (float)BAUMGARTE, slop = (float)SLOP;
    float* torso = s + BODIES_OFFSET;
    float x_before = torso[IDX_X];
    for (int j = 0; j < 6; ++j) {
        float* jt = s + JOINTS_OFFSET + j * JOINT_DATA_SIZE;
        float a = action[j];
        if (a > 1.0f) a = 1.0f;
        else if (a < -1.0f) a = -1.0f;
        float motor_sign = a >= 0.0f ? 1.0f : -1.0f;
        jt[JOINT_MOTOR_SPEED] = motor_sign * 1000.0f;
        jt[JOINT_MAX_MOTOR_TORQUE] = (float)MAX_TORQUE * fabsf(a);
    }
    int joint_count = (int)s[JOINT_COUNT_OFFSET];
    float contacts[MAX_CONTACTS * CONTACT_DATA_SIZE];
    int contact_count = 0;
    for (int sub = 0; sub < FRAME_SKIP; ++sub) {
        integrate_velocities(s, NUM_BODIES, BODIES_OFFSET, FORCES_OFFSET, gx, gy, dt);
        contact_count = flat_terrain_detect(s, shapes, 0.0f, contacts);
        for (int it = 0; it < VELOCITY_ITERATIONS; ++it) {
            solve_velocity_contacts(s, BODIES_OFFSET, contacts, contact_count, friction, restitution);
            solve_velocity_joints(s, BODIES_OFFSET, JOINTS_OFFSET, MAX_JOINTS, joint_count, dt);
        }
        integrate_positions(s, NUM_BODIES, BODIES_OFFSET, dt);
        for (int it = 0; it < POSITION_ITERATIONS; ++it) {
            solve_position_contacts(s, BODIES_OFFSET, contacts, contact_count, baumgarte, slop);
            solve_position_joints(s, BODIES_OFFSET, JOINTS_OFFSET, MAX_JOINTS, joint_count, baumgarte, slop);
        }
        for (int b = 0; b < NUM_BODIES; ++b)
            for (int k = 0; k < 3; ++k) s[FORCES_OFFSET + b * 3 + k] = 0.0f;
    }
    float x_after = torso[IDX_X], torso_z = torso[IDX_Y];
    float forward_velocity = (x_after - x_before) / (dt * (float)FRAME_SKIP);
    float forward_reward = (float)FORWARD_REWARD_WEIGHT * forward_velocity;
    float ctrl_cost = 0.0f;
    for (int j = 0; j < 6; ++j) {
        float a = action[j];
        if (a > 1.0f) a = 1.0f;
        else if (a < -1.0f) a = -1.0f;
        ctrl_cost = ctrl_cost + a * a;
    }
    ctrl_cost = ctrl_cost * (float)CTRL_COST_WEIGHT;
    float height_bonus = 0.0f;
    if (torso_z > (float)MIN_HEIGHT_FOR_BONUS) {
        float eff = torso_z;
        if (eff > (float)TARGET_HEIGHT) eff = (float)TARGET_HEIGHT;
        height_bonus = (float)HEIGHT_BONUS_WEIGHT * eff;
    }
    // contacts of the last sub-step: every non-foot body vertex on the ground costs 0.5
    float ground_contact_penalty = 0.0f;
    for (int c = 0; c < contact_count; ++c) {
        int body_a = (int)contacts[c * CONTACT_DATA_SIZE + CONTACT_BODY_A];
        int body_b = (int)contacts[c * CONTACT_DATA_SIZE + CONTACT_BODY_B];
        if (body_b == -1 && body_a != BODY_BFOOT && body_a != BODY_FFOOT)
            ground_contact_penalty = ground_contact_penalty + (float)GROUND_CONTACT_PENALTY;
    }
    float reward = forward_reward - ctrl_cost + height_bonus - ground_contact_penalty;
    float step_count = s[METADATA_OFFSET + META_STEP_COUNT] + 1.0f;
    s[METADATA_OFFSET + META_STEP_COUNT] = step_count;
    float done = step_count >= (float)MAX_STEPS ? 1.0f : 0.0f;  // TERMINATE_WHEN_UNHEALTHY is False
    *reward_out = reward;
    *done_out = done;
    compute_obs(s);
}

inline void step_all(float* states, const float* actions, float* rewards, float* dones, float* obs, int n) {
    float shapes[NUM_SHAPES * SHAPE_MAX_SIZE];
    init_shapes(shapes);
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int env = 0; env < n; ++env) {
        float* s = states + (size_t)env * STATE_SIZE;
        step_env(s, shapes, actions + (size_t)env * ACTION_DIM, &rewards[env], &dones[env]);
        for (int d = 0; d < OBS_DIM; ++d) obs[(size_t)env * OBS_DIM + d] = s[OBS_OFFSET + d];
    }
}

// cheetah_planar_v2.mojo:1109, :1151: Int(seed_f32) * 2654435761 + (i + 1) * 12345
inline int64_t combined_seed(uint64_t rng_seed, int env) {
    float seed_f = (float)rng_seed;
    int64_t si = (int64_t)seed_f;
    return (int64_t)((uint64_t)si * 2654435761ull + (uint64_t)(env + 1) * 12345ull);
}
inline void reset_all(float* states, int n, uint64_t rng_seed) {
    for (int i = 0; i < n; ++i) reset_env(states + (size_t)i * STATE_SIZE, combined_seed(rng_seed, i));
}
// cheetah_planar_v2.mojo:1121-1167: resets where done > 0.5 and clears the flag
inline void selective_reset(float* states, float* dones, int n, uint64_t rng_seed) {
    for (int i = 0; i < n; ++i)
        if (dones[i] > 0.5f) {
            reset_env(states + (size_t)i * STATE_SIZE, combined_seed(rng_seed, i));
            dones[i] = 0.0f;
        }
}

}  // namespace cheetah
}  // namespace oracle
