// BipedalWalkerV2 on the register-resident physics core.
// Reference: envs/bipedal_walker/bipedal_walker_v2.mojo:1372-2588 (GPU path),
// envs/bipedal_walker/constants_v2.mojo.  A hull and two two-segment legs on
// four motorised, limited revolute joints over a 128-edge terrain; ten lidar
// rays from the hull.
//
// The 3.8 kB row is mostly terrain (768 floats) that a step only reads.  Both
// consumers of the terrain - the vertex/edge collision test and the lidar -
// first pass once over the edges' x-ranges and keep a 128-bit candidate set;
// edges outside it fail the reference's own range test (collision) or cannot
// intersect any ray (lidar), so skipping them changes no result.
#pragma once
#include "physics2d.cuh"

namespace mrl {
namespace bipedal {

using namespace phys;

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

// physics2d/layout.mojo:268-277 (BipedalWalkerLayout)
constexpr int NUM_BODIES = 5, MAX_CONTACTS = 20, MAX_JOINTS = 4, MAX_TERRAIN_EDGES = 128, OBS_DIM = 24, ACTION_DIM = 4;
constexpr int BODIES_OFFSET = 24, FORCES_OFFSET = 89, JOINTS_OFFSET = 104, JOINT_COUNT_OFFSET = 172,
              EDGES_OFFSET = 173, EDGE_COUNT_OFFSET = 941, METADATA_OFFSET = 942, STATE_SIZE = 950;
constexpr int META_STEP_COUNT = 0, META_PREV_X = 1, META_PREV_SHAPING = 2, META_DONE = 3, META_SCROLL = 4,
              META_LEFT_CONTACT = 5, META_RIGHT_CONTACT = 6, META_GAME_OVER = 7;

struct Traits {  // hip, knee per leg
    __host__ __device__ static constexpr int ja(int j) { return (j & 1) ? j : 0; }
    __host__ __device__ static constexpr int jb(int j) { return j + 1; }
};

// Polygon vertices of _init_shapes_gpu (bipedal_walker_v2.mojo:1899-1968); the shape of body b is b.
__device__ __forceinline__ int shape_nverts(int body) { return body == 0 ? 5 : 4; }
__device__ __forceinline__ void shape_vertex(int body, int v, float& lx, float& ly) {
    if (body == 0) {
        const float hx[5] = {(float)(-30.0 / SCALE), (float)(-6.0 / SCALE), (float)(6.0 / SCALE),
                             (float)(30.0 / SCALE), 0.0f};
        const float hy[5] = {0.0f, (float)(30.0 / SCALE), (float)(30.0 / SCALE), 0.0f, (float)(-12.0 / SCALE)};
        lx = hx[v]; ly = hy[v];
    } else {
        const bool upper = (body == 1 || body == 3);
        const float w = upper ? (float)(UPPER_LEG_W / 2) : (float)(LOWER_LEG_W / 2);
        const float mw = upper ? (float)(-UPPER_LEG_W / 2) : (float)(-LOWER_LEG_W / 2);
        const float h = upper ? (float)(UPPER_LEG_H / 2) : (float)(LOWER_LEG_H / 2);
        const float mh = upper ? (float)(-UPPER_LEG_H / 2) : (float)(-LOWER_LEG_H / 2);
        lx = v < 2 ? mw : w;
        ly = (v == 0 || v == 3) ? h : mh;
    }
}

struct EdgeSet {  // 128 edges
    uint32_t w[4];
    __device__ __forceinline__ void clear() { w[0] = w[1] = w[2] = w[3] = 0u; }
    __device__ __forceinline__ void add(int e) { w[e >> 5] |= 1u << (e & 31); }
};

// Ten rays, hull-relative angles 0 .. 1.5 rad (bipedal_walker_v2.mojo:1843-1897, :2306-2388).
__device__ __forceinline__ void lidar(const float* __restrict__ s, float hull_x, float hull_y, float hull_angle,
                                      int n_edges, float (&out)[NUM_LIDAR]) {
    const float lidar_range = (float)LIDAR_RANGE;
    float rdx[NUM_LIDAR], rdy[NUM_LIDAR];
    float xlo = hull_x, xhi = hull_x;
#pragma unroll
    for (int i = 0; i < NUM_LIDAR; ++i) {
        float local_angle = (float)i * 1.5f / (float)(NUM_LIDAR - 1);
        float world_angle = hull_angle - local_angle - 1.5707963267948966f;
        const float2 sc = sincos_shared(world_angle);
        rdx[i] = sc.y * lidar_range;
        rdy[i] = sc.x * lidar_range;
        xlo = fminf(xlo, hull_x + rdx[i]);
        xhi = fmaxf(xhi, hull_x + rdx[i]);
        out[i] = 1.0f;
    }
    // A hit needs t and u in [0, 1]: the hit point lies on the ray and on the edge, so the edge's x-range
    // must reach the fan's x-range; the margin is orders of magnitude above the rounding of t and u.
    xlo -= 0.05f;
    xhi += 0.05f;
    for (int e = 0; e < MAX_TERRAIN_EDGES; ++e) {
        if (e >= n_edges) break;
        const float* edge = s + EDGES_OFFSET + e * 6;
        const float ex0 = edge[0], ex1 = edge[2];
        if (fmaxf(ex0, ex1) < xlo || fminf(ex0, ex1) > xhi) continue;
        const float ey0 = edge[1], ey1 = edge[3];
        const float ex = ex1 - ex0, ey = ey1 - ey0;
        const float dx = hull_x - ex0, dy = hull_y - ey0;
#pragma unroll
        for (int i = 0; i < NUM_LIDAR; ++i) {
            float denom = rdx[i] * ey - rdy[i] * ex;
            if (denom > -1e-10f && denom < 1e-10f) continue;
            float t = (ex * dy - ey * dx) / denom;
            float u = (rdx[i] * dy - rdy[i] * dx) / denom;
            if (t >= 0.0f && t <= 1.0f && u >= 0.0f && u <= 1.0f) {
                if (t < out[i]) out[i] = t;   // the minimum over edges does not depend on their order
            }
        }
    }
}

struct Env {
    Bodies<NUM_BODIES> b;
    JointParams jp[MAX_JOINTS];
    int n_joints, n_edges;
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
    e.n_edges = (int)s[EDGE_COUNT_OFFSET];
}

// Entries 0..13 of the observation (_extract_obs_gpu :2493-2588).
__device__ __forceinline__ void body_obs(const Bodies<NUM_BODIES>& b, float c1, float c2, float* o) {
    const float hull_angle = b.a[0], hull_omega = b.w[0];
    o[0] = hull_angle;
    o[1] = hull_omega / 5.0f;
    o[2] = b.vx[0] * (float)(VIEWPORT_W / SCALE / FPS);
    o[3] = b.vy[0] * (float)(VIEWPORT_H / SCALE / FPS);
#pragma unroll
    for (int leg = 0; leg < 2; ++leg) {
        const int up = leg * 2 + 1, lo = leg * 2 + 2;
        float* q = o + 4 + leg * 5;
        q[0] = b.a[up] - hull_angle;
        q[1] = (b.w[up] - hull_omega) / 10.0f;
        q[2] = b.a[lo] - b.a[up];
        q[3] = (b.w[lo] - b.w[up]) / 10.0f;
        q[4] = leg == 0 ? c1 : c2;
    }
}

// step_wrapper of _fused_step_gpu (bipedal_walker_v2.mojo:2040-2292) on the row at s (global memory).
__device__ __forceinline__ void step_row(float* s, const float* __restrict__ act, float (&obs)[OBS_DIM],
                                         float& reward_out, float& done_out) {
    Env e;
    load_row(s, e);
    const float dt = (float)DT;
    float action[ACTION_DIM];
#pragma unroll
    for (int j = 0; j < MAX_JOINTS; ++j) {  // _apply_motor_actions_gpu, :2390-2490
        action[j] = act[j];
        float a = action[j];
        if (a > 1.0f) a = 1.0f;
        if (a < -1.0f) a = -1.0f;
        const float sign = a >= 0.0f ? 1.0f : -1.0f;
        e.jp[j].motor_speed = sign * (float)((j & 1) ? SPEED_KNEE : SPEED_HIP);
        const float a_abs = a >= 0.0f ? a : -a;
        e.jp[j].max_torque = (float)MOTORS_TORQUE * a_abs;
        s[JOINTS_OFFSET + j * JOINT_DATA_SIZE + JOINT_MOTOR_SPEED] = e.jp[j].motor_speed;
        s[JOINTS_OFFSET + j * JOINT_DATA_SIZE + JOINT_MAX_MOTOR_TORQUE] = e.jp[j].max_torque;
    }
    float fx[NUM_BODIES], fy[NUM_BODIES], tau[NUM_BODIES];
#pragma unroll
    for (int i = 0; i < NUM_BODIES; ++i) {
        fx[i] = s[FORCES_OFFSET + i * 3 + 0];
        fy[i] = s[FORCES_OFFSET + i * 3 + 1];
        tau[i] = s[FORCES_OFFSET + i * 3 + 2];
    }
    integrate_velocities(e.b, fx, fy, tau, (float)GRAVITY_X, (float)GRAVITY_Y, dt);
    refresh_trig(e.b);
    // EdgeTerrainCollision.detect_single_env: body-major, vertex, edge order, capped at MAX_CONTACTS.
    constexpr int NV = 21;
    float wxs[NV], wys[NV];
    float vmin, vmax;
    {
        int idx = 0;
#pragma unroll
        for (int body = 0; body < NUM_BODIES; ++body) {
#pragma unroll
            for (int v = 0; v < 5; ++v) {
                if (v >= shape_nverts(body)) break;
                float lx, ly;
                shape_vertex(body, v, lx, ly);
                wxs[idx] = e.b.x[body] + lx * e.b.cs[body] - ly * e.b.sn[body];
                wys[idx] = e.b.y[body] + lx * e.b.sn[body] + ly * e.b.cs[body];
                ++idx;
            }
        }
        vmin = wxs[0]; vmax = wxs[0];
#pragma unroll
        for (int i = 1; i < NV; ++i) { vmin = fminf(vmin, wxs[i]); vmax = fmaxf(vmax, wxs[i]); }
    }
    EdgeSet cand;
    cand.clear();
    for (int ed = 0; ed < MAX_TERRAIN_EDGES; ++ed) {
        if (ed >= e.n_edges) break;
        const float x0 = s[EDGES_OFFSET + ed * 6], x1 = s[EDGES_OFFSET + ed * 6 + 2];
        float x_min = x0, x_max = x1;
        if (x0 > x1) { x_min = x1; x_max = x0; }
        if (!(vmax < x_min - 0.1f || vmin > x_max + 0.1f)) cand.add(ed);
    }
    Contacts<MAX_CONTACTS> c;
    c.n = 0;
    {
        int idx = 0;
#pragma unroll
        for (int body = 0; body < NUM_BODIES; ++body) {
#pragma unroll
            for (int v = 0; v < 5; ++v) {
                if (v >= shape_nverts(body)) break;
                const float wx = wxs[idx], wy = wys[idx];
                ++idx;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t m = cand.w[q];
                    while (m != 0) {
                        const int ed = q * 32 + __ffs(m) - 1;
                        m &= m - 1;
                        const float* p = s + EDGES_OFFSET + ed * 6;
                        vertex_edge_test(c, body, wx, wy, p[0], p[1], p[2], p[3], p[4], p[5]);
                    }
                }
            }
        }
    }
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
    float hull_contact = 0.0f, left_leg_contact = 0.0f, right_leg_contact = 0.0f;
#pragma unroll
    for (int k = 0; k < MAX_CONTACTS; ++k) {
        if (k < c.n) {
            if (c.body[k] == 0) hull_contact = 1.0f;
            else if (c.body[k] == 2) left_leg_contact = 1.0f;
            else if (c.body[k] == 4) right_leg_contact = 1.0f;
        }
    }
    float lid[NUM_LIDAR];
    lidar(s, e.b.x[0], e.b.y[0], e.b.a[0], e.n_edges, lid);
    body_obs(e.b, left_leg_contact, right_leg_contact, obs);
#pragma unroll
    for (int i = 0; i < NUM_LIDAR; ++i) obs[LIDAR_START_IDX + i] = lid[i];
    const float hull_x = e.b.x[0], hull_y = e.b.y[0], hull_vx = e.b.vx[0], hull_angle = e.b.a[0];
    float* meta = s + METADATA_OFFSET;
    const float step_count = meta[META_STEP_COUNT];
    const float prev_x = meta[META_PREV_X];
    float forward_progress = hull_x - prev_x;
    float angle_abs = hull_angle >= 0.0f ? hull_angle : -hull_angle;
    float angle_penalty = 5.0f * angle_abs;
    float reward = (float)(130.0 / SCALE) * forward_progress - angle_penalty;
    float a0 = action[0] >= 0.0f ? action[0] : -action[0];
    float a1 = action[1] >= 0.0f ? action[1] : -action[1];
    float a2 = action[2] >= 0.0f ? action[2] : -action[2];
    float a3 = action[3] >= 0.0f ? action[3] : -action[3];
    float energy = a0 + a1 + a2 + a3;
    float energy_penalty = (float)(0.00035 * MOTORS_TORQUE) * energy;
    reward = reward - energy_penalty;
    const float min_height = (float)(TERRAIN_HEIGHT + LEG_H * 1.5);
    const float critical_height = (float)(TERRAIN_HEIGHT + LEG_H * 1.2);
    if (hull_y < min_height) reward = reward - 10.0f * (min_height - hull_y);
    float vel_x = hull_vx * (float)(VIEWPORT_W / SCALE / FPS);
    if (vel_x > 0.0f) reward = reward + 3.0f * vel_x;
    else { float vel_x_abs = -vel_x; reward = reward - 5.0f * vel_x_abs; }
    float done = 0.0f;
    const float new_step_count = step_count + 1.0f;
    if (new_step_count >= 2000.0f) done = 1.0f;
    if (hull_contact > 0.5f) { done = 1.0f; reward = (float)CRASH_PENALTY; }
    if (hull_y < critical_height) { done = 1.0f; reward = -50.0f; }
    if (hull_x < 0.0f) { done = 1.0f; reward = (float)CRASH_PENALTY; }
    const float terrain_end = (float)(TERRAIN_LENGTH - TERRAIN_GRASS) * (float)TERRAIN_STEP;
    if (hull_x > terrain_end) done = 1.0f;
    reward_out = reward;
    done_out = done;
    // write back what the reference writes
#pragma unroll
    for (int i = 0; i < NUM_BODIES; ++i) {
        float* body = s + BODIES_OFFSET + i * BODY_STATE_SIZE;
        body[IDX_X] = e.b.x[i]; body[IDX_Y] = e.b.y[i]; body[IDX_ANGLE] = e.b.a[i];
        body[IDX_VX] = e.b.vx[i]; body[IDX_VY] = e.b.vy[i]; body[IDX_OMEGA] = e.b.w[i];
        float* f = s + FORCES_OFFSET + i * 3;
        f[0] = 0.0f; f[1] = 0.0f; f[2] = 0.0f;
    }
    meta[META_STEP_COUNT] = new_step_count;
    meta[META_PREV_X] = hull_x;
    meta[META_LEFT_CONTACT] = left_leg_contact;
    meta[META_RIGHT_CONTACT] = right_leg_contact;
    meta[META_GAME_OVER] = hull_contact;
#pragma unroll
    for (int d = 0; d < OBS_DIM; ++d) s[d] = obs[d];
}

// _reset_env_gpu, bipedal_walker_v2.mojo:1513-1751, writing the reference row in global memory.
// Only the fields the reference writes are touched.
__device__ __forceinline__ void reset_row(float* s, int64_t seed, float (&obs)[OBS_DIM]) {
    Philox rng((uint64_t)seed, 0);
    Philox terrain_rng((uint64_t)(seed + 1000), 0);
    constexpr int n_edges = TERRAIN_LENGTH - 1 < MAX_TERRAIN_EDGES ? TERRAIN_LENGTH - 1 : MAX_TERRAIN_EDGES;
    s[EDGE_COUNT_OFFSET] = (float)n_edges;
    float y = (float)TERRAIN_HEIGHT, velocity = 0.0f, prev_y = y;
    for (int edge = 0; edge < n_edges; ++edge) {
        float x0 = (float)edge * (float)TERRAIN_STEP;
        float x1 = (float)(edge + 1) * (float)TERRAIN_STEP;
        prev_y = y;
        const float terrain_height = (float)TERRAIN_HEIGHT;
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
        float* ep = s + EDGES_OFFSET + edge * 6;
        ep[0] = x0; ep[1] = prev_y; ep[2] = x1; ep[3] = y; ep[4] = nx; ep[5] = ny;
    }
    float r[4];
    rng.step_uniform(r);
    const float init_x = (float)(TERRAIN_STARTPAD * TERRAIN_STEP);
    const float init_y = (float)(TERRAIN_HEIGHT + 2.0 * LEG_H);
    const float init_vx = (r[0] * 2.0f - 1.0f) * 0.1f;
    const float init_vy = (r[1] * 2.0f - 1.0f) * 0.1f;
    const float upper_y = init_y + (float)LEG_DOWN - (float)(UPPER_LEG_H / 2);
    const float lower_y = upper_y - (float)(UPPER_LEG_H / 2) - (float)(LOWER_LEG_H / 2);
#pragma unroll
    for (int b = 0; b < NUM_BODIES; ++b) {
        float* p = s + BODIES_OFFSET + b * BODY_STATE_SIZE;
        const bool upper = (b == 1 || b == 3);
        p[IDX_X] = init_x;
        p[IDX_Y] = b == 0 ? init_y : (upper ? upper_y : lower_y);
        p[IDX_ANGLE] = 0.0f;
        p[IDX_VX] = init_vx; p[IDX_VY] = init_vy; p[IDX_OMEGA] = 0.0f;
        p[IDX_INV_MASS] = b == 0 ? (float)(1.0 / HULL_MASS) : (upper ? (float)(1.0 / LEG_MASS) : (float)(1.0 / LOWER_LEG_MASS));
        p[IDX_INV_INERTIA] = b == 0 ? (float)(1.0 / HULL_INERTIA)
                                    : (upper ? (float)(1.0 / LEG_INERTIA) : (float)(1.0 / LOWER_LEG_INERTIA));
        p[IDX_SHAPE] = (float)b;
    }
    s[JOINT_COUNT_OFFSET] = 4.0f;
#pragma unroll
    for (int j = 0; j < MAX_JOINTS; ++j) {
        float* jt = s + JOINTS_OFFSET + j * JOINT_DATA_SIZE;
        const bool knee = (j & 1) != 0;
        jt[JOINT_TYPE] = 0.0f;
        jt[JOINT_BODY_A] = (float)Traits::ja(j);
        jt[JOINT_BODY_B] = (float)Traits::jb(j);
        jt[JOINT_ANCHOR_AX] = 0.0f;
        jt[JOINT_ANCHOR_AY] = knee ? (float)(-UPPER_LEG_H / 2) : (float)LEG_DOWN;
        jt[JOINT_ANCHOR_BX] = 0.0f;
        jt[JOINT_ANCHOR_BY] = knee ? (float)(LOWER_LEG_H / 2) : (float)(UPPER_LEG_H / 2);
        jt[JOINT_REF_ANGLE] = 0.0f;
        jt[JOINT_LOWER_LIMIT] = knee ? (float)KNEE_LIMIT_LOW : (float)HIP_LIMIT_LOW;
        jt[JOINT_UPPER_LIMIT] = knee ? (float)KNEE_LIMIT_HIGH : (float)HIP_LIMIT_HIGH;
        jt[JOINT_MAX_MOTOR_TORQUE] = (float)MOTORS_TORQUE;
        jt[JOINT_MOTOR_SPEED] = 0.0f;
        jt[JOINT_FLAGS] = (float)(JOINT_FLAG_LIMIT | JOINT_FLAG_MOTOR);
    }
#pragma unroll
    for (int i = 0; i < NUM_BODIES * 3; ++i) s[FORCES_OFFSET + i] = 0.0f;
    // _compute_initial_obs_reset_gpu, :1755-1897: all bodies share the velocity, angles and omegas are zero
#pragma unroll
    for (int d = 0; d < OBS_DIM; ++d) obs[d] = 0.0f;
    obs[1] = 0.0f / 5.0f;
    obs[2] = init_vx * (float)(VIEWPORT_W / SCALE / FPS);
    obs[3] = init_vy * (float)(VIEWPORT_H / SCALE / FPS);
    float lid[NUM_LIDAR];
    lidar(s, init_x, init_y, 0.0f, n_edges, lid);
#pragma unroll
    for (int i = 0; i < NUM_LIDAR; ++i) obs[LIDAR_START_IDX + i] = lid[i];
#pragma unroll
    for (int d = 0; d < OBS_DIM; ++d) s[d] = obs[d];
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

// Int(seed_f32) * 2654435761 + (i + 1) * 12345 (bipedal_walker_v2.mojo:1442, :1488)
__host__ __device__ __forceinline__ int64_t combined_seed(float seed_f32, int env) {
    int64_t si = (int64_t)seed_f32;
    return (int64_t)((uint64_t)si * 2654435761ull + (uint64_t)(env + 1) * 12345ull);
}

}  // namespace bipedal
}  // namespace mrl
