// CPU ORACLE - test infrastructure, not product code.
//
// fp32 restatement of BipedalWalkerV2's GPU path:
// envs/bipedal_walker/bipedal_walker_v2.mojo:1372-2588, constants_v2.mojo.
// A hull and two two-segment legs on four motorised, limited revolute joints
// over a random-walk terrain of 128 edges, ten lidar rays from the hull.
// Reset draws come from Philox (see physics2d.hpp: parity unpinned at that
// boundary).
#pragma once
#include "physics2d.hpp"

namespace oracle {
namespace bipedal {

constexpr Layout L = BIPEDAL_LAYOUT;
constexpr int STATE_SIZE = L.state_size();  // 950
constexpr int OBS_DIM = 24, ACTION_DIM = 4, NUM_BODIES = 5, NUM_SHAPES = 5, MAX_CONTACTS = 20, MAX_JOINTS = 4,
              MAX_TERRAIN_EDGES = 128;
constexpr int OBS_OFFSET = 0, BODIES_OFFSET = L.bodies_offset(), FORCES_OFFSET = L.forces_offset(),
              JOINTS_OFFSET = L.joints_offset(), JOINT_COUNT_OFFSET = L.joint_count_offset(),
              EDGES_OFFSET = L.edges_offset(), EDGE_COUNT_OFFSET = L.edge_count_offset(),
              METADATA_OFFSET = L.metadata_offset();
constexpr int META_STEP_COUNT = 0, META_PREV_X = 1 /* the TOTAL_REWARD slot holds prev_x */, META_PREV_SHAPING = 2,
              META_DONE = 3, META_SCROLL = 4, META_LEFT_CONTACT = 5, META_RIGHT_CONTACT = 6, META_GAME_OVER = 7;

// envs/bipedal_walker/constants_v2.mojo
constexpr double FPS = 50.0, DT = 1.0 / FPS, SCALE = 30.0, GRAVITY_X = 0.0, GRAVITY_Y = -10.0, FRICTION = 2.5,
                 RESTITUTION = 0.0, BAUMGARTE = 0.2, SLOP = 0.005;
constexpr int VELOCITY_ITERATIONS = 6, POSITION_ITERATIONS = 2;
constexpr double MOTORS_TORQUE = 80.0, SPEED_HIP = 4.0, SPEED_KNEE = 6.0, LIDAR_RANGE = 160.0 / SCALE;
constexpr int NUM_LIDAR = 10, LIDAR_START_IDX = 14;
constexpr double LEG_DOWN = -8.0 / SCALE, LEG_H = 34.0 / SCALE, UPPER_LEG_W = 6.4 / SCALE, UPPER_LEG_H = 34.0 / SCALE,
                 LOWER_LEG_W = 5.12 / SCALE, LOWER_LEG_H = 34.0 / SCALE;
constexpr double HULL_MASS = 5.0, HULL_INERTIA = 2.0, LEG_MASS = 0.8, LEG_INERTIA = 0.1, LOWER_LEG_MASS = 0.5,
                 LOWER_LEG_INERTIA = 0.05;
constexpr double TERRAIN_STEP = 14.0 / SCALE, TERRAIN_HEIGHT = 400.0 / SCALE / 4.0;
constexpr int TERRAIN_LENGTH = 200, TERRAIN_GRASS = 10, TERRAIN_STARTPAD = 20;
constexpr double VIEWPORT_W = 600.0, VIEWPORT_H = 400.0;
constexpr double HIP_LIMIT_LOW = -0.8, HIP_LIMIT_HIGH = 1.1, KNEE_LIMIT_LOW = -1.6, KNEE_LIMIT_HIGH = -0.1;
constexpr double CRASH_PENALTY = -100.0;

// _init_shapes_gpu, bipedal_walker_v2.mojo:1899-1968
inline void init_shapes(float* shapes) {
    for (int i = 0; i < NUM_SHAPES * SHAPE_MAX_SIZE; ++i) shapes[i] = 0.0f;
    shapes[0] = (float)SHAPE_POLYGON; shapes[1] = 5.0f;
    shapes[2] = (float)(-30.0 / SCALE); shapes[3] = 0.0f;
    shapes[4] = (float)(-6.0 / SCALE);  shapes[5] = (float)(30.0 / SCALE);
    shapes[6] = (float)(6.0 / SCALE);   shapes[7] = (float)(30.0 / SCALE);
    shapes[8] = (float)(30.0 / SCALE);  shapes[9] = 0.0f;
    shapes[10] = 0.0f;                  shapes[11] = (float)(-12.0 / SCALE);
    for (int b = 1; b < 5; ++b) {
        float* sh = shapes + b * SHAPE_MAX_SIZE;
        const double w = (b == 1 || b == 3) ? UPPER_LEG_W : LOWER_LEG_W;
        const double h = (b == 1 || b == 3) ? UPPER_LEG_H : LOWER_LEG_H;
        sh[0] = (float)SHAPE_POLYGON; sh[1] = 4.0f;
        sh[2] = (float)(-w / 2); sh[3] = (float)(h / 2);
        sh[4] = (float)(-w / 2); sh[5] = (float)(-h / 2);
        sh[6] = (float)(w / 2);  sh[7] = (float)(-h / 2);
        sh[8] = (float)(w / 2);  sh[9] = (float)(h / 2);
    }
}

// Ten rays from the hull centre, 0 .. 1.5 rad below the hull's forward axis
// (bipedal_walker_v2.mojo:1843-1897 at reset, :2306-2388 per step); out[i] is the
// hit fraction of the range, 1.0 without a hit.
inline void lidar(const float* s, float* out) {
    const float* hull = s + BODIES_OFFSET;
    float hull_x = hull[IDX_X], hull_y = hull[IDX_Y], hull_angle = hull[IDX_ANGLE];
    int n_edges = (int)s[EDGE_COUNT_OFFSET];
    const float lidar_range = (float)LIDAR_RANGE;
    for (int i = 0; i < NUM_LIDAR; ++i) {
        float local_angle = (float)i * 1.5f / (float)(NUM_LIDAR - 1);
        float world_angle = hull_angle - local_angle - 1.5707963267948966f;
        float sn, cs;
        mrl_sincosf(world_angle, &sn, &cs);
        float ray_dx = cs * lidar_range, ray_dy = sn * lidar_range;
        float min_t = 1.0f;
        for (int e = 0; e < MAX_TERRAIN_EDGES; ++e) {
            if (e >= n_edges) break;
            const float* edge = s + EDGES_OFFSET + e * 6;
            float ex = edge[2] - edge[0], ey = edge[3] - edge[1];
            float denom = ray_dx * ey - ray_dy * ex;
            if (denom > -1e-10f && denom < 1e-10f) continue;
            float dx = hull_x - edge[0], dy = hull_y - edge[1];
            float t = (ex * dy - ey * dx) / denom;
            float u = (ray_dx * dy - ray_dy * dx) / denom;
            if (t >= 0.0f && t <= 1.0f && u >= 0.0f && u <= 1.0f) {
                if (t < min_t) min_t = t;
            }
        }
        out[i] = min_t;
    }
}

// Entries 0..13 of the observation; c1 / c2 are the leg contact flags
// (_extract_obs_gpu :2493-2588, _compute_initial_obs_reset_gpu :1755-1841).
inline void body_obs(const float* s, float c1, float c2, float* o) {
    auto body = [&](int b) { return s + BODIES_OFFSET + b * BODY_STATE_SIZE; };
    const float* hull = body(0);
    float hull_angle = hull[IDX_ANGLE], hull_omega = hull[IDX_OMEGA];
    o[0] = hull_angle;
    o[1] = hull_omega / 5.0f;
    o[2] = hull[IDX_VX] * (float)(VIEWPORT_W / SCALE / FPS);
    o[3] = hull[IDX_VY] * (float)(VIEWPORT_H / SCALE / FPS);
    for (int leg = 0; leg < 2; ++leg) {
        const float* up = body(leg * 2 + 1);
        const float* lo = body(leg * 2 + 2);
        float* q = o + 4 + leg * 5;
        q[0] = up[IDX_ANGLE] - hull_angle;
        q[1] = (up[IDX_OMEGA] - hull_omega) / 10.0f;
        q[2] = lo[IDX_ANGLE] - up[IDX_ANGLE];
        q[3] = (lo[IDX_OMEGA] - up[IDX_OMEGA]) / 10.0f;
        q[4] = leg == 0 ? c1 : c2;
    }
}

// _reset_env_gpu, bipedal_walker_v2.mojo:1513-1751
inline void reset_env(float* s, int64_t seed) {
    Philox rng((uint64_t)seed, 0);
    Philox terrain_rng((uint64_t)(seed + 1000), 0);
    const int n_edges = TERRAIN_LENGTH - 1 < MAX_TERRAIN_EDGES ? TERRAIN_LENGTH - 1 : MAX_TERRAIN_EDGES;
    s[EDGE_COUNT_OFFSET] = (float)n_edges;
    float y = (float)TERRAIN_HEIGHT, velocity = 0.0f, prev_y = y;
    for (int edge = 0; edge < n_edges; ++edge) {
        float x0 = (float)edge * (float)TERRAIN_STEP;
        float x1 = (float)(edge + 1) * (float)TERRAIN_STEP;
        prev_y = y;
        float terrain_height = (float)TERRAIN_HEIGHT;
        velocity = 0.8f * velocity + 0.01f * (terrain_height > y ? 1.0f : -1.0f);
        if (edge > TERRAIN_STARTPAD) {
            float r[4];
            terrain_rng.step_uniform(r);
            velocity = velocity + (r[0] * 2.0f - 1.0f) / (float)SCALE;
        }
        y = y + velocity;
        float dx = x1 - x0, dy = y - prev_y;
        float length = sqrtf(dx * dx + dy * dy);
        float nx = -dy / length, ny = dx / length;
        if (ny < 0.0f) { nx = -nx; ny = -ny; }
        float* e = s + EDGES_OFFSET + edge * 6;
        e[0] = x0; e[1] = prev_y; e[2] = x1; e[3] = y; e[4] = nx; e[5] = ny;
    }
    float r[4];
    rng.step_uniform(r);
    float init_x = (float)(TERRAIN_STARTPAD * TERRAIN_STEP);
    float init_y = (float)(TERRAIN_HEIGHT + 2.0 * LEG_H);
    float init_vx = (r[0] * 2.0f - 1.0f) * 0.1f;
    float init_vy = (r[1] * 2.0f - 1.0f) * 0.1f;
    auto set_body = [&](int b, float yy, double mass, double inertia) {
        float* p = s + BODIES_OFFSET + b * BODY_STATE_SIZE;
        p[IDX_X] = init_x; p[IDX_Y] = yy; p[IDX_ANGLE] = 0.0f;
        p[IDX_VX] = init_vx; p[IDX_VY] = init_vy; p[IDX_OMEGA] = 0.0f;
        p[IDX_INV_MASS] = (float)(1.0 / mass); p[IDX_INV_INERTIA] = (float)(1.0 / inertia);
        p[IDX_SHAPE] = (float)b;
    };
    set_body(0, init_y, HULL_MASS, HULL_INERTIA);
    for (int leg = 0; leg < 2; ++leg) {
        float upper_y = init_y + (float)LEG_DOWN - (float)(UPPER_LEG_H / 2);
        set_body(leg * 2 + 1, upper_y, LEG_MASS, LEG_INERTIA);
        float lower_y = upper_y - (float)(UPPER_LEG_H / 2) - (float)(LOWER_LEG_H / 2);
        set_body(leg * 2 + 2, lower_y, LOWER_LEG_MASS, LOWER_LEG_INERTIA);
    }
    s[JOINT_COUNT_OFFSET] = 4.0f;
    for (int leg = 0; leg < 2; ++leg) {
        for (int part = 0; part < 2; ++part) {  // 0 hip, 1 knee
            float* jt = s + JOINTS_OFFSET + (leg * 2 + part) * JOINT_DATA_SIZE;
            jt[JOINT_TYPE] = (float)JOINT_REVOLUTE;
            jt[JOINT_BODY_A] = part == 0 ? 0.0f : (float)(leg * 2 + 1);
            jt[JOINT_BODY_B] = (float)(leg * 2 + 1 + part);
            jt[JOINT_ANCHOR_AX] = 0.0f;
            jt[JOINT_ANCHOR_AY] = part == 0 ? (float)LEG_DOWN : (float)(-UPPER_LEG_H / 2);
            jt[JOINT_ANCHOR_BX] = 0.0f;
            jt[JOINT_ANCHOR_BY] = part == 0 ? (float)(UPPER_LEG_H / 2) : (float)(LOWER_LEG_H / 2);
            jt[JOINT_REF_ANGLE] = 0.0f;
            jt[JOINT_LOWER_LIMIT] = part == 0 ? (float)HIP_LIMIT_LOW : (float)KNEE_LIMIT_LOW;
            jt[JOINT_UPPER_LIMIT] = part == 0 ? (float)HIP_LIMIT_HIGH : (float)KNEE_LIMIT_HIGH;
            jt[JOINT_MAX_MOTOR_TORQUE] = (float)MOTORS_TORQUE;
            jt[JOINT_MOTOR_SPEED] = 0.0f;
            jt[JOINT_FLAGS] = (float)(JOINT_FLAG_LIMIT_ENABLED | JOINT_FLAG_MOTOR_ENABLED);
        }
    }
    for (int i = 0; i < NUM_BODIES * 3; ++i) s[FORCES_OFFSET + i] = 0.0f;
    body_obs(s, 0.0f, 0.0f, s + OBS_OFFSET);
    lidar(s, s + OBS_OFFSET + LIDAR_START_IDX);
    float* meta = s + METADATA_OFFSET;
    meta[META_STEP_COUNT] = 0.0f;
    meta[META_PREV_X] = init_x;
    meta[META_PREV_SHAPING] = 0.0f;
    meta[META_DONE] = 0.0f;
    meta[META_SCROLL] = 0.0f;
    meta[META_LEFT_CONTACT] = 0.0f;
    meta[META_RIGHT_CONTACT] = 0.0f;
    meta[META_GAME_OVER] = 0.0f;
}

// _apply_motor_actions_gpu, bipedal_walker_v2.mojo:2390-2490 (two sequential ifs for the clamp)
inline void apply_motor_actions(float* s, const float* action) {
    for (int j = 0; j < 4; ++j) {
        float* jt = s + JOINTS_OFFSET + j * JOINT_DATA_SIZE;
        float a = action[j];
        if (a > 1.0f) a = 1.0f;
        if (a < -1.0f) a = -1.0f;
        float sign = a >= 0.0f ? 1.0f : -1.0f;
        jt[JOINT_MOTOR_SPEED] = sign * (float)((j & 1) ? SPEED_KNEE : SPEED_HIP);
        float a_abs = a >= 0.0f ? a : -a;
        jt[JOINT_MAX_MOTOR_TORQUE] = (float)MOTORS_TORQUE * a_abs;
    }
}

// step_wrapper of _fused_step_gpu, bipedal_walker_v2.mojo:2040-2292
inline void step_env(float* s, const float* shapes, const float* action, float* reward_out, float* done_out) {
    apply_motor_actions(s, action);
    const float dt = (float)DT;
    int joint_count = (int)s[JOINT_COUNT_OFFSET], n_edges = (int)s[EDGE_COUNT_OFFSET];
    float contacts[MAX_CONTACTS * CONTACT_DATA_SIZE];
    integrate_velocities(s, NUM_BODIES, BODIES_OFFSET, FORCES_OFFSET, (float)GRAVITY_X, (float)GRAVITY_Y, dt);
    int contact_count = edge_terrain_detect(s, shapes, NUM_BODIES, BODIES_OFFSET, EDGES_OFFSET, MAX_TERRAIN_EDGES,
                                            n_edges, contacts, MAX_CONTACTS);
    for (int it = 0; it < VELOCITY_ITERATIONS; ++it) {
        solve_velocity_contacts(s, BODIES_OFFSET, contacts, contact_count, (float)FRICTION, (float)RESTITUTION);
        solve_velocity_joints(s, BODIES_OFFSET, JOINTS_OFFSET, MAX_JOINTS, joint_count, dt);
    }
    integrate_positions(s, NUM_BODIES, BODIES_OFFSET, dt);
    for (int it = 0; it < POSITION_ITERATIONS; ++it) {
        solve_position_contacts(s, BODIES_OFFSET, contacts, contact_count, (float)BAUMGARTE, (float)SLOP);
        solve_position_joints(s, BODIES_OFFSET, JOINTS_OFFSET, MAX_JOINTS, joint_count, (float)BAUMGARTE, (float)SLOP);
    }
    for (int i = 0; i < NUM_BODIES * 3; ++i) s[FORCES_OFFSET + i] = 0.0f;
    float hull_contact = 0.0f, left_leg_contact = 0.0f, right_leg_contact = 0.0f;
    for (int c = 0; c < contact_count; ++c) {
        int body_a = (int)contacts[c * CONTACT_DATA_SIZE + CONTACT_BODY_A];
        if (body_a == 0) hull_contact = 1.0f;
        else if (body_a == 2) left_leg_contact = 1.0f;
        else if (body_a == 4) right_leg_contact = 1.0f;
    }
    float* meta = s + METADATA_OFFSET;
    meta[META_LEFT_CONTACT] = left_leg_contact;
    meta[META_RIGHT_CONTACT] = right_leg_contact;
    meta[META_GAME_OVER] = hull_contact;
    lidar(s, s + OBS_OFFSET + LIDAR_START_IDX);
    body_obs(s, left_leg_contact, right_leg_contact, s + OBS_OFFSET);
    const float* hull = s + BODIES_OFFSET;
    float hull_x = hull[IDX_X], hull_y = hull[IDX_Y], hull_vx = hull[IDX_VX], hull_angle = hull[IDX_ANGLE];
    float step_count = meta[META_STEP_COUNT];
    meta[META_STEP_COUNT] = step_count + 1.0f;
    float prev_x = meta[META_PREV_X];
    float forward_progress = hull_x - prev_x;
    meta[META_PREV_X] = hull_x;
    float angle_abs = hull_angle >= 0.0f ? hull_angle : -hull_angle;
    float angle_penalty = 5.0f * angle_abs;
    float reward = (float)(130.0 / SCALE) * forward_progress - angle_penalty;
    float energy = 0.0f;  // |a0| + |a1| + |a2| + |a3| on the unclamped actions, left to right
    {
        float a0 = action[0] >= 0.0f ? action[0] : -action[0];
        float a1 = action[1] >= 0.0f ? action[1] : -action[1];
        float a2 = action[2] >= 0.0f ? action[2] : -action[2];
        float a3 = action[3] >= 0.0f ? action[3] : -action[3];
        energy = a0 + a1 + a2 + a3;
    }
    float energy_penalty = (float)(0.00035 * MOTORS_TORQUE) * energy;
    reward = reward - energy_penalty;
    const float min_height = (float)(TERRAIN_HEIGHT + LEG_H * 1.5);
    const float critical_height = (float)(TERRAIN_HEIGHT + LEG_H * 1.2);
    if (hull_y < min_height) reward = reward - 10.0f * (min_height - hull_y);
    float vel_x = hull_vx * (float)(VIEWPORT_W / SCALE / FPS);
    if (vel_x > 0.0f) reward = reward + 3.0f * vel_x;
    else { float vel_x_abs = -vel_x; reward = reward - 5.0f * vel_x_abs; }
    float done = 0.0f;
    float new_step_count = step_count + 1.0f;
    if (new_step_count >= 2000.0f) done = 1.0f;
    if (hull_contact > 0.5f) { done = 1.0f; reward = (float)CRASH_PENALTY; }
    if (hull_y < critical_height) { done = 1.0f; reward = -50.0f; }
    if (hull_x < 0.0f) { done = 1.0f; reward = (float)CRASH_PENALTY; }
    const float terrain_end = (float)(TERRAIN_LENGTH - TERRAIN_GRASS) * (float)TERRAIN_STEP;
    if (hull_x > terrain_end) done = 1.0f;
    *reward_out = reward;
    *done_out = done;
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

// bipedal_walker_v2.mojo:1442, :1488: Int(seed_f32) * 2654435761 + (i + 1) * 12345
inline int64_t combined_seed(uint64_t rng_seed, int env) {
    float seed_f = (float)rng_seed;
    int64_t si = (int64_t)seed_f;
    return (int64_t)((uint64_t)si * 2654435761ull + (uint64_t)(env + 1) * 12345ull);
}
inline void reset_all(float* states, int n, uint64_t rng_seed) {
    for (int i = 0; i < n; ++i) reset_env(states + (size_t)i * STATE_SIZE, combined_seed(rng_seed, i));
}
// bipedal_walker_v2.mojo:1456-1505: resets where done > 0.5 and clears the flag
inline void selective_reset(float* states, float* dones, int n, uint64_t rng_seed) {
    for (int i = 0; i < n; ++i)
        if (dones[i] > 0.5f) {
            reset_env(states + (size_t)i * STATE_SIZE, combined_seed(rng_seed, i));
            dones[i] = 0.0f;
        }
}

}  // namespace bipedal
}  // namespace oracle
