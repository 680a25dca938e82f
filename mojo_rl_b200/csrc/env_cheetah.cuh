// Planar HalfCheetah (HalfCheetahPlanarV2) on the register-resident physics core.
// Reference: envs/half_cheetah/cheetah_planar_v2.mojo:1039-1901 (GPU path),
// envs/half_cheetah/constants.mojo, physics2d/collision/flat_terrain.mojo:456-580.
// Seven rectangles (torso + two legs of thigh, shin, foot), six motorised and
// limited revolute joints, flat ground at y = 0, five physics sub-steps per
// environment step.
#pragma once
#include "physics2d.cuh"

namespace mrl {
namespace cheetah {

using namespace phys;

constexpr double DT = 0.01, GRAVITY_X = 0.0, GRAVITY_Y = -9.81, FRICTION = 0.9, RESTITUTION = 0.0,
                 BAUMGARTE = 0.2, SLOP = 0.005;
constexpr int FRAME_SKIP = 5, VELOCITY_ITERATIONS = 4, POSITION_ITERATIONS = 2, MAX_STEPS = 1000;
constexpr double TORSO_LENGTH = 1.0, TORSO_RADIUS = 0.046, TORSO_MASS = 6.25, INIT_HEIGHT = 0.7;
constexpr double MAX_TORQUE = 1.0, CTRL_COST_WEIGHT = 0.1, FORWARD_REWARD_WEIGHT = 1.0, HEIGHT_BONUS_WEIGHT = 1.0,
                 TARGET_HEIGHT = 0.5, MIN_HEIGHT_FOR_BONUS = 0.1, GROUND_CONTACT_PENALTY = 0.5;
constexpr int BODY_BFOOT = 3, BODY_FFOOT = 6;

// physics2d/layout.mojo:290-299 (HalfCheetahLayout)
constexpr int NUM_BODIES = 7, MAX_CONTACTS = 14, MAX_JOINTS = 6, OBS_DIM = 17, ACTION_DIM = 6;
constexpr int BODIES_OFFSET = 17, FORCES_OFFSET = 108, JOINTS_OFFSET = 129, JOINT_COUNT_OFFSET = 231,
              EDGES_OFFSET = 232, EDGE_COUNT_OFFSET = 244, METADATA_OFFSET = 245, STATE_SIZE = 253;
constexpr int META_STEP_COUNT = 0, META_PREV_X = 1, META_DONE = 3, META_TOTAL_REWARD = 4;

// segments in body order 1..6: bthigh, bshin, bfoot, fthigh, fshin, ffoot
__host__ __device__ constexpr double seg_length(int k) {
    return k == 0 ? 0.145 : k == 1 ? 0.15 : k == 2 ? 0.094 : k == 3 ? 0.133 : k == 4 ? 0.106 : 0.07;
}
__host__ __device__ constexpr double seg_radius(int) { return 0.046; }
__host__ __device__ constexpr double seg_mass(int) { return 1.0; }
__host__ __device__ constexpr double limit_low(int j) {
    return j == 0 ? -0.52 : j == 1 ? -0.785 : j == 2 ? -0.4 : j == 3 ? -1.0 : j == 4 ? -1.2 : -0.5;
}
__host__ __device__ constexpr double limit_high(int j) {
    return j == 0 ? 1.05 : j == 1 ? 0.785 : j == 2 ? 0.785 : j == 3 ? 0.7 : j == 4 ? 0.87 : 0.5;
}

// Distance from the hip height down to the centre of segment k, summed in
// double precision in the order the reference writes it (:1256-1326).
__host__ __device__ constexpr double seg_center_drop(int k) {
    return k == 0 ? seg_length(0) / 2
         : k == 1 ? seg_length(0) + seg_length(1) / 2
         : k == 2 ? seg_length(0) + seg_length(1) + seg_length(2) / 2
         : k == 3 ? seg_length(3) / 2
         : k == 4 ? seg_length(3) + seg_length(4) / 2
                  : seg_length(3) + seg_length(4) + seg_length(5) / 2;
}

struct Traits {  // hip, knee, ankle per leg
    __host__ __device__ static constexpr int ja(int j) { return j == 0 ? 0 : j == 3 ? 0 : j; }
    __host__ __device__ static constexpr int jb(int j) { return j + 1; }
};

// Rectangle vertices of _init_shapes_gpu (cheetah_planar_v2.mojo:1497-1573); the shape of body b is b.
__device__ __forceinline__ void shape_vertex(int body, int v, float& lx, float& ly) {
    float hx, hy;
    if (body == 0) { hx = (float)(TORSO_LENGTH / 2); hy = (float)TORSO_RADIUS; }
    else { hx = (float)seg_radius(body - 1); hy = (float)seg_length(body - 1) / 2.0f; }
    lx = (v < 2) ? -hx : hx;
    ly = (v == 0 || v == 3) ? -hy : hy;
}

struct Env {
    Bodies<NUM_BODIES> b;
    JointParams jp[MAX_JOINTS];
    int n_joints;
};

__device__ __forceinline__ void load_row(const float* s, Env& e) {
#pragma unroll
    for (int i = 0; i < NUM_BODIES; ++i) {
        const float* body = s + BODIES_OFFSET + i * BODY_STATE_SIZE;
        e.b.x[i] = body[IDX_X]; e.b.y[i] = body[IDX_Y]; e.b.a[i] = body[IDX_ANGLE];
        e.b.vx[i] = body[IDX_VX]; e.b.vy[i] = body[IDX_VY]; e.b.w[i] = body[IDX_OMEGA];
        e.b.inv_m[i] = body[IDX_INV_MASS]; e.b.inv_i[i] = body[IDX_INV_INERTIA];
    }
#pragma unroll
    for (int j = 0; j < MAX_JOINTS; ++j) {
        const float* jt = s + JOINTS_OFFSET + j * JOINT_DATA_SIZE;
        e.jp[j].ax = jt[JOINT_ANCHOR_AX]; e.jp[j].ay = jt[JOINT_ANCHOR_AY];
        e.jp[j].bx = jt[JOINT_ANCHOR_BX]; e.jp[j].by = jt[JOINT_ANCHOR_BY];
        e.jp[j].ref = jt[JOINT_REF_ANGLE]; e.jp[j].lo = jt[JOINT_LOWER_LIMIT];
        e.jp[j].hi = jt[JOINT_UPPER_LIMIT]; e.jp[j].max_torque = jt[JOINT_MAX_MOTOR_TORQUE];
        e.jp[j].motor_speed = jt[JOINT_MOTOR_SPEED]; e.jp[j].stiffness = jt[JOINT_STIFFNESS];
        e.jp[j].damping = jt[JOINT_DAMPING]; e.jp[j].flags = (int)jt[JOINT_FLAGS];
    }
    e.n_joints = (int)s[JOINT_COUNT_OFFSET];
}

// _compute_obs_gpu, cheetah_planar_v2.mojo:1427-1494
__device__ __forceinline__ void compute_obs(const Bodies<NUM_BODIES>& b, float (&o)[OBS_DIM]) {
    o[0] = b.y[0];
    o[1] = b.a[0];
#pragma unroll
    for (int k = 0; k < 6; ++k) {
        const int child = k + 1, parent = Traits::ja(k);
        o[2 + k] = b.a[child] - b.a[parent];
        o[11 + k] = b.w[child] - b.w[parent];
    }
    o[8] = b.vx[0];
    o[9] = b.vy[0];
    o[10] = b.w[0];
}

// FlatTerrainCollision.detect_single_env (flat_terrain.mojo:456-580), polygon branch.
__device__ __forceinline__ void detect_flat(const Bodies<NUM_BODIES>& b, float ground_y,
                                            Contacts<MAX_CONTACTS>& c) {
    c.n = 0;
#pragma unroll
    for (int k = 0; k < MAX_CONTACTS; ++k) { c.nx[k] = 0.0f; c.ny[k] = 1.0f; }
#pragma unroll
    for (int body = 0; body < NUM_BODIES; ++body) {
        const float cos_a = b.cs[body], sin_a = b.sn[body];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            float lx, ly;
            shape_vertex(body, v, lx, ly);
            float wx = b.x[body] + lx * cos_a - ly * sin_a;
            float wy = b.y[body] + lx * sin_a + ly * cos_a;
            float penetration = ground_y - wy;
            if (penetration > 0.0f && c.n < MAX_CONTACTS) {
                const int s = c.n;
#pragma unroll
                for (int k = 0; k < MAX_CONTACTS; ++k)
                    if (k == s) { c.body[k] = body; c.px[k] = wx; c.py[k] = wy; c.depth[k] = penetration; }
                c.n = s + 1;
            }
        }
    }
}

// _step_env_gpu, cheetah_planar_v2.mojo:1671-1901.  s: the environment's row
// (shared or global memory); act: its six actions.
__device__ __forceinline__ void step_row(float* s, const float* __restrict__ act, float (&obs)[OBS_DIM],
                                         float& reward_out, float& done_out) {
    Env e;
    load_row(s, e);
    const float dt = (float)DT;
    const float x_before = e.b.x[0];
    float ctrl_cost = 0.0f;
#pragma unroll
    for (int j = 0; j < MAX_JOINTS; ++j) {
        float a = act[j];
        if (a > 1.0f) a = 1.0f;
        else if (a < -1.0f) a = -1.0f;
        const float motor_sign = a >= 0.0f ? 1.0f : -1.0f;
        e.jp[j].motor_speed = motor_sign * 1000.0f;
        e.jp[j].max_torque = (float)MAX_TORQUE * fabsf(a);
        s[JOINTS_OFFSET + j * JOINT_DATA_SIZE + JOINT_MOTOR_SPEED] = e.jp[j].motor_speed;
        s[JOINTS_OFFSET + j * JOINT_DATA_SIZE + JOINT_MAX_MOTOR_TORQUE] = e.jp[j].max_torque;
        ctrl_cost = ctrl_cost + a * a;
    }
    ctrl_cost = ctrl_cost * (float)CTRL_COST_WEIGHT;
    Contacts<MAX_CONTACTS> c;
#pragma unroll 1
    for (int sub = 0; sub < FRAME_SKIP; ++sub) {
        float fx[NUM_BODIES], fy[NUM_BODIES], tau[NUM_BODIES];
#pragma unroll
        for (int i = 0; i < NUM_BODIES; ++i) {  // the force slots are cleared after every sub-step
            fx[i] = sub == 0 ? s[FORCES_OFFSET + i * 3 + 0] : 0.0f;
            fy[i] = sub == 0 ? s[FORCES_OFFSET + i * 3 + 1] : 0.0f;
            tau[i] = sub == 0 ? s[FORCES_OFFSET + i * 3 + 2] : 0.0f;
        }
        integrate_velocities(e.b, fx, fy, tau, (float)GRAVITY_X, (float)GRAVITY_Y, dt);
        refresh_trig(e.b);
        detect_flat(e.b, 0.0f, c);
        ContactPre<MAX_CONTACTS> cp;
        prepare_contacts(e.b, c, cp);
        JointPre jpre[MAX_JOINTS];
        prepare_joints<Traits>(e.b, e.jp, jpre);
    #pragma unroll 1
    for (int it = 0; it < VELOCITY_ITERATIONS; ++it) {
            solve_velocity_contacts(e.b, c, cp, (float)FRICTION, (float)RESTITUTION);
            solve_velocity_joints<Traits>(e.b, e.jp, jpre, e.n_joints, dt);
        }
        integrate_positions(e.b, dt);
    #pragma unroll 1
    for (int it = 0; it < POSITION_ITERATIONS; ++it) {
            solve_position_contacts(e.b, c, (float)BAUMGARTE, (float)SLOP);
            solve_position_joints<Traits>(e.b, e.jp, e.n_joints, (float)BAUMGARTE, (float)SLOP);
        }
    }
    const float x_after = e.b.x[0], torso_z = e.b.y[0];
    float forward_velocity = (x_after - x_before) / (dt * (float)FRAME_SKIP);
    float forward_reward = (float)FORWARD_REWARD_WEIGHT * forward_velocity;
    float height_bonus = 0.0f;
    if (torso_z > (float)MIN_HEIGHT_FOR_BONUS) {
        float eff = torso_z;
        if (eff > (float)TARGET_HEIGHT) eff = (float)TARGET_HEIGHT;
        height_bonus = (float)HEIGHT_BONUS_WEIGHT * eff;
    }
    float ground_contact_penalty = 0.0f;  // contacts of the last sub-step, every body but the feet
#pragma unroll
    for (int k = 0; k < MAX_CONTACTS; ++k)
        if (k < c.n && c.body[k] != BODY_BFOOT && c.body[k] != BODY_FFOOT)
            ground_contact_penalty = ground_contact_penalty + (float)GROUND_CONTACT_PENALTY;
    reward_out = forward_reward - ctrl_cost + height_bonus - ground_contact_penalty;
    float step_count = s[METADATA_OFFSET + META_STEP_COUNT] + 1.0f;
    s[METADATA_OFFSET + META_STEP_COUNT] = step_count;
    done_out = step_count >= (float)MAX_STEPS ? 1.0f : 0.0f;  // TERMINATE_WHEN_UNHEALTHY is False
#pragma unroll
    for (int i = 0; i < NUM_BODIES; ++i) {
        float* body = s + BODIES_OFFSET + i * BODY_STATE_SIZE;
        body[IDX_X] = e.b.x[i]; body[IDX_Y] = e.b.y[i]; body[IDX_ANGLE] = e.b.a[i];
        body[IDX_VX] = e.b.vx[i]; body[IDX_VY] = e.b.vy[i]; body[IDX_OMEGA] = e.b.w[i];
        float* f = s + FORCES_OFFSET + i * 3;
        f[0] = 0.0f; f[1] = 0.0f; f[2] = 0.0f;
    }
    compute_obs(e.b, obs);
#pragma unroll
    for (int d = 0; d < OBS_DIM; ++d) s[d] = obs[d];
}

// _reset_env_gpu, cheetah_planar_v2.mojo:1175-1424, writing the reference row.
// Only the fields the reference writes are touched.
__device__ __forceinline__ void reset_row(float* s, int64_t seed) {
    Philox rng((uint64_t)seed, 0);
    float r[4];
    rng.step_uniform(r);
    const float init_x = 0.0f, init_y = (float)INIT_HEIGHT;
    const float init_vx = (r[0] * 2.0f - 1.0f) * 0.1f;
    const float init_vy = (r[1] * 2.0f - 1.0f) * 0.1f;
    const float back_hip_x = init_x - (float)(TORSO_LENGTH / 2), front_hip_x = init_x + (float)(TORSO_LENGTH / 2);
#pragma unroll
    for (int b = 0; b < NUM_BODIES; ++b) {
        float* p = s + BODIES_OFFSET + b * BODY_STATE_SIZE;
        float x = init_x, y = init_y, inv_m, inv_i;
        if (b == 0) {
            inv_m = (float)(1.0 / TORSO_MASS);
            inv_i = (float)(1.0 / (TORSO_MASS * TORSO_LENGTH * TORSO_LENGTH / 12.0));
        } else {
            const int k = b - 1;
            const double yoff = seg_center_drop(k);
            x = k < 3 ? back_hip_x : front_hip_x;
            y = init_y - (float)yoff;
            inv_m = (float)(1.0 / seg_mass(k));
            inv_i = (float)(12.0 / (seg_mass(k) * seg_length(k) * seg_length(k)));
        }
        p[IDX_X] = x; p[IDX_Y] = y; p[IDX_ANGLE] = 0.0f;
        p[IDX_VX] = init_vx; p[IDX_VY] = init_vy; p[IDX_OMEGA] = 0.0f;
        p[IDX_INV_MASS] = inv_m; p[IDX_INV_INERTIA] = inv_i;
        p[IDX_SHAPE] = (float)b;
    }
    s[JOINT_COUNT_OFFSET] = 6.0f;
#pragma unroll
    for (int j = 0; j < MAX_JOINTS; ++j) {
        float* jt = s + JOINTS_OFFSET + j * JOINT_DATA_SIZE;
        float ax, ay;
        if (j == 0) { ax = (float)(-TORSO_LENGTH / 2); ay = 0.0f; }
        else if (j == 3) { ax = (float)(TORSO_LENGTH / 2); ay = 0.0f; }
        else { ax = 0.0f; ay = (float)(-seg_length(j - 1) / 2); }
        jt[JOINT_TYPE] = 0.0f;
        jt[JOINT_BODY_A] = (float)Traits::ja(j);
        jt[JOINT_BODY_B] = (float)Traits::jb(j);
        jt[JOINT_ANCHOR_AX] = ax;
        jt[JOINT_ANCHOR_AY] = ay;
        jt[JOINT_ANCHOR_BX] = 0.0f;
        jt[JOINT_ANCHOR_BY] = (float)(seg_length(j) / 2);
        jt[JOINT_REF_ANGLE] = 0.0f;
        jt[JOINT_LOWER_LIMIT] = (float)limit_low(j);
        jt[JOINT_UPPER_LIMIT] = (float)limit_high(j);
        jt[JOINT_MAX_MOTOR_TORQUE] = (float)MAX_TORQUE;
        jt[JOINT_MOTOR_SPEED] = 0.0f;
        jt[JOINT_FLAGS] = (float)(JOINT_FLAG_LIMIT | JOINT_FLAG_MOTOR);
    }
#pragma unroll
    for (int i = 0; i < NUM_BODIES * 3; ++i) s[FORCES_OFFSET + i] = 0.0f;
    s[METADATA_OFFSET + META_STEP_COUNT] = 0.0f;
    s[METADATA_OFFSET + META_PREV_X] = init_x;
    s[METADATA_OFFSET + META_DONE] = 0.0f;
    s[METADATA_OFFSET + META_TOTAL_REWARD] = 0.0f;
    // observation of the fresh state: height, zero angles, the common velocity
#pragma unroll
    for (int d = 0; d < OBS_DIM; ++d) s[d] = 0.0f;
    s[0] = init_y;
    s[8] = init_vx;
    s[9] = init_vy;
}

// Int(seed_f32) * 2654435761 + (i + 1) * 12345 (cheetah_planar_v2.mojo:1109, :1151)
__host__ __device__ __forceinline__ int64_t combined_seed(float seed_f32, int env) {
    int64_t si = (int64_t)seed_f32;
    return (int64_t)((uint64_t)si * 2654435761ull + (uint64_t)(env + 1) * 12345ull);
}

}  // namespace cheetah
}  // namespace mrl
