// CPU ORACLE - test infrastructure, not product code.
//
// fp32 restatement of the reference's per-environment rigid-body routines, in
// the reference's own state layout (one row of floats per environment).  Each
// function cites the reference file:line it follows.  Compile with
// -ffp-contract=off so that every +,-,*,/ is one IEEE operation; sin/cos come
// from include/mrl_detmath.h (the reference's device libm is not available).
//
// Parity status: the reference cannot be executed in the build environment (no
// Mojo toolchain) and ships no recorded trajectory, so these routines are
// pinned only against the few known answers its tests state (free-fall
// velocity, layout sizes); everything else is "parity unpinned".
#pragma once
#include <cmath>
#include <cstdint>
#include "../include/mrl_detmath.h"

namespace oracle {

// physics2d/constants.mojo:20-48
constexpr int BODY_STATE_SIZE = 13;
constexpr int IDX_X = 0, IDX_Y = 1, IDX_ANGLE = 2, IDX_VX = 3, IDX_VY = 4, IDX_OMEGA = 5;
constexpr int IDX_FX = 6, IDX_FY = 7, IDX_TAU = 8, IDX_MASS = 9, IDX_INV_MASS = 10,
              IDX_INV_INERTIA = 11, IDX_SHAPE = 12;
// physics2d/constants.mojo:55-66
constexpr int SHAPE_MAX_SIZE = 20, SHAPE_POLYGON = 0, SHAPE_CIRCLE = 1, MAX_POLYGON_VERTS = 8;
// physics2d/constants.mojo:74-84
constexpr int CONTACT_DATA_SIZE = 9;
constexpr int CONTACT_BODY_A = 0, CONTACT_BODY_B = 1, CONTACT_POINT_X = 2, CONTACT_POINT_Y = 3,
              CONTACT_NORMAL_X = 4, CONTACT_NORMAL_Y = 5, CONTACT_DEPTH = 6,
              CONTACT_NORMAL_IMPULSE = 7, CONTACT_TANGENT_IMPULSE = 8;
// physics2d/constants.mojo:95-128
constexpr int JOINT_DATA_SIZE = 17, JOINT_REVOLUTE = 0;
constexpr int JOINT_TYPE = 0, JOINT_BODY_A = 1, JOINT_BODY_B = 2, JOINT_ANCHOR_AX = 3,
              JOINT_ANCHOR_AY = 4, JOINT_ANCHOR_BX = 5, JOINT_ANCHOR_BY = 6, JOINT_REF_ANGLE = 7,
              JOINT_LOWER_LIMIT = 8, JOINT_UPPER_LIMIT = 9, JOINT_MAX_MOTOR_TORQUE = 10,
              JOINT_MOTOR_SPEED = 11, JOINT_STIFFNESS = 12, JOINT_DAMPING = 13, JOINT_FLAGS = 14,
              JOINT_IMPULSE = 15, JOINT_MOTOR_IMPULSE = 16;
constexpr int JOINT_FLAG_LIMIT_ENABLED = 1, JOINT_FLAG_MOTOR_ENABLED = 2,
              JOINT_FLAG_SPRING_ENABLED = 4;

// physics2d/layout.mojo:41-239 - offsets of one environment row.
struct Layout {
    int num_bodies, max_contacts, max_joints, max_edges, obs_dim, metadata_size, num_shapes;
    constexpr int bodies_offset() const { return obs_dim; }
    constexpr int forces_offset() const { return bodies_offset() + num_bodies * BODY_STATE_SIZE; }
    constexpr int joints_offset() const { return forces_offset() + num_bodies * 3; }
    constexpr int joint_count_offset() const { return joints_offset() + max_joints * JOINT_DATA_SIZE; }
    constexpr int edges_offset() const { return joint_count_offset() + 1; }
    constexpr int edge_count_offset() const { return edges_offset() + max_edges * 6; }
    constexpr int metadata_offset() const { return edge_count_offset() + 1; }
    constexpr int state_size() const { return metadata_offset() + metadata_size; }
};
// physics2d/layout.mojo:247-299
constexpr Layout LUNAR_LAYOUT{3, 8, 2, 16, 8, 4, 3};
constexpr Layout BIPEDAL_LAYOUT{5, 20, 4, 128, 24, 8, 5};
constexpr Layout CHEETAH_LAYOUT{7, 14, 6, 2, 17, 8, 7};
static_assert(LUNAR_LAYOUT.state_size() == 192, "LunarLander row");
static_assert(BIPEDAL_LAYOUT.state_size() == 950, "BipedalWalker row");
static_assert(CHEETAH_LAYOUT.state_size() == 253, "HalfCheetah row");

// physics2d/integrators/euler.mojo:202-251
inline void integrate_velocities(float* s, int num_bodies, int bodies_off, int forces_off,
                                 float gx, float gy, float dt) {
    for (int b = 0; b < num_bodies; ++b) {
        float* body = s + bodies_off + b * BODY_STATE_SIZE;
        const float* f = s + forces_off + b * 3;
        float inv_mass = body[IDX_INV_MASS];
        float inv_inertia = body[IDX_INV_INERTIA];
        if (inv_mass == 0.0f) continue;
        float vx = body[IDX_VX], vy = body[IDX_VY], omega = body[IDX_OMEGA];
        vx = vx + (f[0] * inv_mass + gx) * dt;
        vy = vy + (f[1] * inv_mass + gy) * dt;
        omega = omega + f[2] * inv_inertia * dt;
        body[IDX_VX] = vx;
        body[IDX_VY] = vy;
        body[IDX_OMEGA] = omega;
    }
}

// physics2d/integrators/euler.mojo:255-311 (sequential ifs, not an elif chain)
inline void integrate_positions(float* s, int num_bodies, int bodies_off, float dt) {
    const float pi_val = (float)M_PI;
    const float two_pi_val = (float)(2.0 * M_PI);
    for (int b = 0; b < num_bodies; ++b) {
        float* body = s + bodies_off + b * BODY_STATE_SIZE;
        if (body[IDX_INV_MASS] == 0.0f) continue;
        float x = body[IDX_X] + body[IDX_VX] * dt;
        float y = body[IDX_Y] + body[IDX_VY] * dt;
        float angle = body[IDX_ANGLE] + body[IDX_OMEGA] * dt;
        if (angle > 100.0f || angle < -100.0f) angle = 0.0f;
        if (angle > pi_val) angle = angle - two_pi_val;
        if (angle > pi_val) angle = angle - two_pi_val;
        if (angle < -pi_val) angle = angle + two_pi_val;
        if (angle < -pi_val) angle = angle + two_pi_val;
        body[IDX_X] = x;
        body[IDX_Y] = y;
        body[IDX_ANGLE] = angle;
    }
}

inline void write_contact(float* c, int body, float px, float py, float nx, float ny, float depth) {
    c[CONTACT_BODY_A] = (float)body;
    c[CONTACT_BODY_B] = -1.0f;
    c[CONTACT_POINT_X] = px;
    c[CONTACT_POINT_Y] = py;
    c[CONTACT_NORMAL_X] = nx;
    c[CONTACT_NORMAL_Y] = ny;
    c[CONTACT_DEPTH] = depth;
    c[CONTACT_NORMAL_IMPULSE] = 0.0f;
    c[CONTACT_TANGENT_IMPULSE] = 0.0f;
}

// physics2d/collision/edge_terrain.mojo:784-1003.  Returns the contact count.
// Order of contacts: body-major, then vertex, then edge; stops at max_contacts.
inline int edge_terrain_detect(const float* s, const float* shapes, int num_bodies, int bodies_off,
                               int edges_off, int max_edges, int n_edges, float* contacts,
                               int max_contacts) {
    int count = 0;
    for (int b = 0; b < num_bodies; ++b) {
        const float* body = s + bodies_off + b * BODY_STATE_SIZE;
        float body_x = body[IDX_X], body_y = body[IDX_Y], body_angle = body[IDX_ANGLE];
        int shape_idx = (int)body[IDX_SHAPE];
        const float* shape = shapes + shape_idx * SHAPE_MAX_SIZE;
        int shape_type = (int)shape[0];
        float sin_a, cos_a;
        mrl_sincosf(body_angle, &sin_a, &cos_a);
        if (shape_type == SHAPE_POLYGON) {
            int n_verts = (int)shape[1];
            for (int v = 0; v < MAX_POLYGON_VERTS; ++v) {
                if (v >= n_verts) break;
                float local_x = shape[2 + v * 2], local_y = shape[3 + v * 2];
                float world_x = body_x + local_x * cos_a - local_y * sin_a;
                float world_y = body_y + local_x * sin_a + local_y * cos_a;
                for (int e = 0; e < max_edges; ++e) {
                    if (e >= n_edges) break;
                    const float* edge = s + edges_off + e * 6;
                    float e_x0 = edge[0], e_y0 = edge[1], e_x1 = edge[2], e_y1 = edge[3];
                    float e_nx = edge[4], e_ny = edge[5];
                    float x_min = e_x0, x_max = e_x1;
                    if (e_x0 > e_x1) { x_min = e_x1; x_max = e_x0; }
                    if (world_x < x_min - 0.1f || world_x > x_max + 0.1f) continue;
                    float edge_dx = e_x1 - e_x0, edge_dy = e_y1 - e_y0;
                    float edge_len_sq = edge_dx * edge_dx + edge_dy * edge_dy;
                    if (edge_len_sq < 1e-6f) continue;
                    float t = ((world_x - e_x0) * edge_dx + (world_y - e_y0) * edge_dy) / edge_len_sq;
                    if (t < 0.0f) t = 0.0f;
                    if (t > 1.0f) t = 1.0f;
                    float closest_x = e_x0 + t * edge_dx, closest_y = e_y0 + t * edge_dy;
                    float dist_x = world_x - closest_x, dist_y = world_y - closest_y;
                    float penetration = -(dist_x * e_nx + dist_y * e_ny);
                    if (penetration > 0.0f && count < max_contacts) {
                        write_contact(contacts + count * CONTACT_DATA_SIZE, b, world_x, world_y,
                                      e_nx, e_ny, penetration);
                        count += 1;
                    }
                }
            }
        } else if (shape_type == SHAPE_CIRCLE) {
            float radius = shape[1], off_x = shape[2], off_y = shape[3];
            float cx = body_x + off_x * cos_a - off_y * sin_a;
            float cy = body_y + off_x * sin_a + off_y * cos_a;
            for (int e = 0; e < max_edges; ++e) {
                if (e >= n_edges) break;
                const float* edge = s + edges_off + e * 6;
                float e_x0 = edge[0], e_y0 = edge[1], e_x1 = edge[2], e_y1 = edge[3];
                float e_nx = edge[4], e_ny = edge[5];
                float edge_dx = e_x1 - e_x0, edge_dy = e_y1 - e_y0;
                float edge_len_sq = edge_dx * edge_dx + edge_dy * edge_dy;
                if (edge_len_sq < 1e-6f) continue;
                float t = ((cx - e_x0) * edge_dx + (cy - e_y0) * edge_dy) / edge_len_sq;
                if (t < 0.0f) t = 0.0f;
                if (t > 1.0f) t = 1.0f;
                float closest_x = e_x0 + t * edge_dx, closest_y = e_y0 + t * edge_dy;
                float dist_x = cx - closest_x, dist_y = cy - closest_y;
                float dist = sqrtf(dist_x * dist_x + dist_y * dist_y);
                float penetration = radius - dist;
                if (penetration > 0.0f && count < max_contacts) {
                    float nx = e_nx, ny = e_ny;
                    if (dist > 1e-6f) { nx = dist_x / dist; ny = dist_y / dist; }
                    write_contact(contacts + count * CONTACT_DATA_SIZE, b, closest_x, closest_y, nx,
                                  ny, penetration);
                    count += 1;
                }
            }
        }
    }
    return count;
}

// physics2d/collision/flat_terrain.mojo:456-580 is restated next to its only
// caller (the planar cheetah) in half_cheetah.hpp.

// physics2d/solvers/impulse.mojo:419-628
inline void solve_velocity_contacts(float* s, int bodies_off, float* contacts, int contact_count,
                                    float friction, float restitution) {
    for (int c = 0; c < contact_count; ++c) {
        float* ct = contacts + c * CONTACT_DATA_SIZE;
        int body_a_idx = (int)ct[CONTACT_BODY_A];
        int body_b_idx = (int)ct[CONTACT_BODY_B];
        float* A = s + bodies_off + body_a_idx * BODY_STATE_SIZE;
        float point_x = ct[CONTACT_POINT_X], point_y = ct[CONTACT_POINT_Y];
        float normal_x = ct[CONTACT_NORMAL_X], normal_y = ct[CONTACT_NORMAL_Y];
        float pos_a_x = A[IDX_X], pos_a_y = A[IDX_Y];
        float vel_a_x = A[IDX_VX], vel_a_y = A[IDX_VY], omega_a = A[IDX_OMEGA];
        float inv_mass_a = A[IDX_INV_MASS], inv_inertia_a = A[IDX_INV_INERTIA];
        float inv_mass_b = 0.0f, inv_inertia_b = 0.0f, vel_b_x = 0.0f, vel_b_y = 0.0f, omega_b = 0.0f;
        float pos_b_x = point_x, pos_b_y = point_y;
        float* B = nullptr;
        if (body_b_idx >= 0) {
            B = s + bodies_off + body_b_idx * BODY_STATE_SIZE;
            pos_b_x = B[IDX_X]; pos_b_y = B[IDX_Y];
            vel_b_x = B[IDX_VX]; vel_b_y = B[IDX_VY]; omega_b = B[IDX_OMEGA];
            inv_mass_b = B[IDX_INV_MASS]; inv_inertia_b = B[IDX_INV_INERTIA];
        }
        float ra_x = point_x - pos_a_x, ra_y = point_y - pos_a_y;
        float rb_x = point_x - pos_b_x, rb_y = point_y - pos_b_y;
        float vel_at_a_x = vel_a_x - omega_a * ra_y, vel_at_a_y = vel_a_y + omega_a * ra_x;
        float vel_at_b_x = vel_b_x - omega_b * rb_y, vel_at_b_y = vel_b_y + omega_b * rb_x;
        float rel_vel_x = vel_at_a_x - vel_at_b_x, rel_vel_y = vel_at_a_y - vel_at_b_y;
        float vel_normal = rel_vel_x * normal_x + rel_vel_y * normal_y;
        if (vel_normal < 0.0f) {
            float ra_cross_n = ra_x * normal_y - ra_y * normal_x;
            float rb_cross_n = rb_x * normal_y - rb_y * normal_x;
            float k = inv_mass_a + inv_mass_b;
            k = k + inv_inertia_a * ra_cross_n * ra_cross_n;
            k = k + inv_inertia_b * rb_cross_n * rb_cross_n;
            float j_normal = -(1.0f + restitution) * vel_normal / k;
            float old_impulse = ct[CONTACT_NORMAL_IMPULSE];
            float new_impulse = old_impulse + j_normal;
            if (new_impulse < 0.0f) new_impulse = 0.0f;
            ct[CONTACT_NORMAL_IMPULSE] = new_impulse;
            j_normal = new_impulse - old_impulse;
            float impulse_x = j_normal * normal_x, impulse_y = j_normal * normal_y;
            A[IDX_VX] = vel_a_x + impulse_x * inv_mass_a;
            A[IDX_VY] = vel_a_y + impulse_y * inv_mass_a;
            A[IDX_OMEGA] = omega_a + (ra_x * impulse_y - ra_y * impulse_x) * inv_inertia_a;
            if (B) {
                B[IDX_VX] = vel_b_x - impulse_x * inv_mass_b;
                B[IDX_VY] = vel_b_y - impulse_y * inv_mass_b;
                B[IDX_OMEGA] = omega_b - (rb_x * impulse_y - rb_y * impulse_x) * inv_inertia_b;
            }
            vel_a_x = A[IDX_VX]; vel_a_y = A[IDX_VY]; omega_a = A[IDX_OMEGA];
            if (B) { vel_b_x = B[IDX_VX]; vel_b_y = B[IDX_VY]; omega_b = B[IDX_OMEGA]; }
            vel_at_a_x = vel_a_x - omega_a * ra_y; vel_at_a_y = vel_a_y + omega_a * ra_x;
            vel_at_b_x = vel_b_x - omega_b * rb_y; vel_at_b_y = vel_b_y + omega_b * rb_x;
            rel_vel_x = vel_at_a_x - vel_at_b_x; rel_vel_y = vel_at_a_y - vel_at_b_y;
            float tangent_x = -normal_y, tangent_y = normal_x;
            float vel_tangent = rel_vel_x * tangent_x + rel_vel_y * tangent_y;
            float ra_cross_t = ra_x * tangent_y - ra_y * tangent_x;
            float rb_cross_t = rb_x * tangent_y - rb_y * tangent_x;
            float k_t = inv_mass_a + inv_mass_b;
            k_t = k_t + inv_inertia_a * ra_cross_t * ra_cross_t;
            k_t = k_t + inv_inertia_b * rb_cross_t * rb_cross_t;
            float j_tangent = -vel_tangent / k_t;
            float max_friction = friction * ct[CONTACT_NORMAL_IMPULSE];
            float old_tangent = ct[CONTACT_TANGENT_IMPULSE];
            float new_tangent = old_tangent + j_tangent;
            if (new_tangent > max_friction) new_tangent = max_friction;
            else if (new_tangent < -max_friction) new_tangent = -max_friction;
            ct[CONTACT_TANGENT_IMPULSE] = new_tangent;
            j_tangent = new_tangent - old_tangent;
            float friction_x = j_tangent * tangent_x, friction_y = j_tangent * tangent_y;
            A[IDX_VX] = A[IDX_VX] + friction_x * inv_mass_a;
            A[IDX_VY] = A[IDX_VY] + friction_y * inv_mass_a;
            A[IDX_OMEGA] = A[IDX_OMEGA] + (ra_x * friction_y - ra_y * friction_x) * inv_inertia_a;
            if (B) {
                B[IDX_VX] = B[IDX_VX] - friction_x * inv_mass_b;
                B[IDX_VY] = B[IDX_VY] - friction_y * inv_mass_b;
                B[IDX_OMEGA] = B[IDX_OMEGA] - (rb_x * friction_y - rb_y * friction_x) * inv_inertia_b;
            }
        }
    }
}

// physics2d/solvers/impulse.mojo:905-980
inline void solve_position_contacts(float* s, int bodies_off, const float* contacts,
                                    int contact_count, float baumgarte, float slop) {
    for (int c = 0; c < contact_count; ++c) {
        const float* ct = contacts + c * CONTACT_DATA_SIZE;
        int body_a_idx = (int)ct[CONTACT_BODY_A];
        int body_b_idx = (int)ct[CONTACT_BODY_B];
        float* A = s + bodies_off + body_a_idx * BODY_STATE_SIZE;
        float normal_x = ct[CONTACT_NORMAL_X], normal_y = ct[CONTACT_NORMAL_Y];
        float correction = ct[CONTACT_DEPTH] - slop;
        if (correction <= 0.0f) continue;
        correction = baumgarte * correction;
        float inv_mass_a = A[IDX_INV_MASS], inv_mass_b = 0.0f;
        float* B = nullptr;
        if (body_b_idx >= 0) {
            B = s + bodies_off + body_b_idx * BODY_STATE_SIZE;
            inv_mass_b = B[IDX_INV_MASS];
        }
        float total_inv_mass = inv_mass_a + inv_mass_b;
        if (total_inv_mass == 0.0f) continue;
        float correction_a = correction * inv_mass_a / total_inv_mass;
        float correction_b = correction * inv_mass_b / total_inv_mass;
        A[IDX_X] = A[IDX_X] + normal_x * correction_a;
        A[IDX_Y] = A[IDX_Y] + normal_y * correction_a;
        if (B) {
            B[IDX_X] = B[IDX_X] - normal_x * correction_b;
            B[IDX_Y] = B[IDX_Y] - normal_y * correction_b;
        }
    }
}

// physics2d/joints/revolute.mojo:512-730.  Order inside one joint: point
// constraint, spring (pre-impulse omegas and angles), limit, motor.
inline void solve_velocity_joints(float* s, int bodies_off, int joints_off, int max_joints,
                                  int joint_count, float dt) {
    for (int j = 0; j < max_joints; ++j) {
        if (j >= joint_count) break;
        float* jt = s + joints_off + j * JOINT_DATA_SIZE;
        if ((int)jt[JOINT_TYPE] != JOINT_REVOLUTE) continue;
        float* A = s + bodies_off + (int)jt[JOINT_BODY_A] * BODY_STATE_SIZE;
        float* B = s + bodies_off + (int)jt[JOINT_BODY_B] * BODY_STATE_SIZE;
        float angle_a = A[IDX_ANGLE], vxa = A[IDX_VX], vya = A[IDX_VY], wa = A[IDX_OMEGA];
        float inv_ma = A[IDX_INV_MASS], inv_ia = A[IDX_INV_INERTIA];
        float angle_b = B[IDX_ANGLE], vxb = B[IDX_VX], vyb = B[IDX_VY], wb = B[IDX_OMEGA];
        float inv_mb = B[IDX_INV_MASS], inv_ib = B[IDX_INV_INERTIA];
        float local_ax = jt[JOINT_ANCHOR_AX], local_ay = jt[JOINT_ANCHOR_AY];
        float local_bx = jt[JOINT_ANCHOR_BX], local_by = jt[JOINT_ANCHOR_BY];
        float cos_a, sin_a, cos_b, sin_b;
        mrl_sincosf(angle_a, &sin_a, &cos_a);
        mrl_sincosf(angle_b, &sin_b, &cos_b);
        float rax = local_ax * cos_a - local_ay * sin_a, ray = local_ax * sin_a + local_ay * cos_a;
        float rbx = local_bx * cos_b - local_by * sin_b, rby = local_bx * sin_b + local_by * cos_b;
        float va_anchor_x = vxa - wa * ray, va_anchor_y = vya + wa * rax;
        float vb_anchor_x = vxb - wb * rby, vb_anchor_y = vyb + wb * rbx;
        float cdot_x = vb_anchor_x - va_anchor_x, cdot_y = vb_anchor_y - va_anchor_y;
        float k11 = inv_ma + inv_mb + inv_ia * ray * ray + inv_ib * rby * rby;
        float k12 = -inv_ia * rax * ray - inv_ib * rbx * rby;
        float k22 = inv_ma + inv_mb + inv_ia * rax * rax + inv_ib * rbx * rbx;
        float det = k11 * k22 - k12 * k12;
        if (det < 1e-10f) det = 1e-10f;
        float inv_det = 1.0f / det;
        float inv_k11 = k22 * inv_det, inv_k12 = -k12 * inv_det, inv_k22 = k11 * inv_det;
        float impulse_x = -(inv_k11 * cdot_x + inv_k12 * cdot_y);
        float impulse_y = -(inv_k12 * cdot_x + inv_k22 * cdot_y);
        A[IDX_VX] = vxa - inv_ma * impulse_x;
        A[IDX_VY] = vya - inv_ma * impulse_y;
        A[IDX_OMEGA] = wa - inv_ia * (rax * impulse_y - ray * impulse_x);
        B[IDX_VX] = vxb + inv_mb * impulse_x;
        B[IDX_VY] = vyb + inv_mb * impulse_y;
        B[IDX_OMEGA] = wb + inv_ib * (rbx * impulse_y - rby * impulse_x);

        int flags = (int)jt[JOINT_FLAGS];
        if (flags & JOINT_FLAG_SPRING_ENABLED) {
            float stiffness = jt[JOINT_STIFFNESS], damping = jt[JOINT_DAMPING];
            float ref_angle = jt[JOINT_REF_ANGLE];
            float current_angle = angle_b - angle_a;
            float angle_error = current_angle - ref_angle;
            float rel_omega = wb - wa;
            float spring_torque = -stiffness * angle_error - damping * rel_omega;
            float angular_impulse = spring_torque * dt;
            float eff_inertia = inv_ia + inv_ib;
            if (eff_inertia > 1e-10f) {
                A[IDX_OMEGA] = A[IDX_OMEGA] - inv_ia * angular_impulse / eff_inertia;
                B[IDX_OMEGA] = B[IDX_OMEGA] + inv_ib * angular_impulse / eff_inertia;
            }
        }
        if (flags & JOINT_FLAG_LIMIT_ENABLED) {
            float lower_limit = jt[JOINT_LOWER_LIMIT], upper_limit = jt[JOINT_UPPER_LIMIT];
            float lim_ref_angle = jt[JOINT_REF_ANGLE];
            float current_wa = A[IDX_OMEGA], current_wb = B[IDX_OMEGA];
            float relative_angle = B[IDX_ANGLE] - A[IDX_ANGLE] - lim_ref_angle;
            float rel_omega = current_wb - current_wa;
            float lim_eff_inertia = inv_ia + inv_ib;
            if (lim_eff_inertia > 1e-10f) {
                float limit_impulse = 0.0f;
                if (relative_angle <= lower_limit) {
                    if (rel_omega < 0.0f) limit_impulse = -rel_omega / lim_eff_inertia;
                } else if (relative_angle >= upper_limit) {
                    if (rel_omega > 0.0f) limit_impulse = -rel_omega / lim_eff_inertia;
                }
                if (limit_impulse != 0.0f) {
                    A[IDX_OMEGA] = current_wa - inv_ia * limit_impulse;
                    B[IDX_OMEGA] = current_wb + inv_ib * limit_impulse;
                }
            }
        }
        if (flags & JOINT_FLAG_MOTOR_ENABLED) {
            float motor_speed = jt[JOINT_MOTOR_SPEED], max_torque = jt[JOINT_MAX_MOTOR_TORQUE];
            float current_wa = A[IDX_OMEGA], current_wb = B[IDX_OMEGA];
            float rel_omega = current_wb - current_wa;
            float speed_error = motor_speed - rel_omega;
            float eff_inertia = inv_ia + inv_ib;
            if (eff_inertia > 1e-10f) {
                float motor_impulse = speed_error / eff_inertia;
                float max_impulse = max_torque * dt;
                if (motor_impulse > max_impulse) motor_impulse = max_impulse;
                if (motor_impulse < -max_impulse) motor_impulse = -max_impulse;
                A[IDX_OMEGA] = current_wa - inv_ia * motor_impulse;
                B[IDX_OMEGA] = current_wb + inv_ib * motor_impulse;
            }
        }
    }
}

// physics2d/joints/revolute.mojo:764-920.  A joint whose anchor error is below
// slop is skipped entirely, including its angle-limit correction.
inline void solve_position_joints(float* s, int bodies_off, int joints_off, int max_joints,
                                  int joint_count, float baumgarte, float slop) {
    for (int j = 0; j < max_joints; ++j) {
        if (j >= joint_count) break;
        float* jt = s + joints_off + j * JOINT_DATA_SIZE;
        if ((int)jt[JOINT_TYPE] != JOINT_REVOLUTE) continue;
        float* A = s + bodies_off + (int)jt[JOINT_BODY_A] * BODY_STATE_SIZE;
        float* B = s + bodies_off + (int)jt[JOINT_BODY_B] * BODY_STATE_SIZE;
        float xa = A[IDX_X], ya = A[IDX_Y], angle_a = A[IDX_ANGLE];
        float inv_ma = A[IDX_INV_MASS], inv_ia = A[IDX_INV_INERTIA];
        float xb = B[IDX_X], yb = B[IDX_Y], angle_b = B[IDX_ANGLE];
        float inv_mb = B[IDX_INV_MASS], inv_ib = B[IDX_INV_INERTIA];
        float local_ax = jt[JOINT_ANCHOR_AX], local_ay = jt[JOINT_ANCHOR_AY];
        float local_bx = jt[JOINT_ANCHOR_BX], local_by = jt[JOINT_ANCHOR_BY];
        float cos_a, sin_a, cos_b, sin_b;
        mrl_sincosf(angle_a, &sin_a, &cos_a);
        mrl_sincosf(angle_b, &sin_b, &cos_b);
        float rax = local_ax * cos_a - local_ay * sin_a, ray = local_ax * sin_a + local_ay * cos_a;
        float rbx = local_bx * cos_b - local_by * sin_b, rby = local_bx * sin_b + local_by * cos_b;
        float anchor_ax = xa + rax, anchor_ay = ya + ray;
        float anchor_bx = xb + rbx, anchor_by = yb + rby;
        float cx = anchor_bx - anchor_ax, cy = anchor_by - anchor_ay;
        float error = sqrtf(cx * cx + cy * cy);
        if (error < slop) continue;
        float k11 = inv_ma + inv_mb + inv_ia * ray * ray + inv_ib * rby * rby;
        float k12 = -inv_ia * rax * ray - inv_ib * rbx * rby;
        float k22 = inv_ma + inv_mb + inv_ia * rax * rax + inv_ib * rbx * rbx;
        float det = k11 * k22 - k12 * k12;
        if (det < 1e-10f) det = 1e-10f;
        float inv_det = 1.0f / det;
        float inv_k11 = k22 * inv_det, inv_k12 = -k12 * inv_det, inv_k22 = k11 * inv_det;
        float correction_x = -baumgarte * (inv_k11 * cx + inv_k12 * cy);
        float correction_y = -baumgarte * (inv_k12 * cx + inv_k22 * cy);
        A[IDX_X] = xa - inv_ma * correction_x;
        A[IDX_Y] = ya - inv_ma * correction_y;
        A[IDX_ANGLE] = angle_a - inv_ia * (rax * correction_y - ray * correction_x);
        B[IDX_X] = xb + inv_mb * correction_x;
        B[IDX_Y] = yb + inv_mb * correction_y;
        B[IDX_ANGLE] = angle_b + inv_ib * (rbx * correction_y - rby * correction_x);
        int flags = (int)jt[JOINT_FLAGS];
        if (flags & JOINT_FLAG_LIMIT_ENABLED) {
            float lower_limit = jt[JOINT_LOWER_LIMIT], upper_limit = jt[JOINT_UPPER_LIMIT];
            float pos_ref_angle = jt[JOINT_REF_ANGLE];
            float cur_angle_a = A[IDX_ANGLE], cur_angle_b = B[IDX_ANGLE];
            float relative_angle = cur_angle_b - cur_angle_a - pos_ref_angle;
            float pos_eff_inertia = inv_ia + inv_ib;
            if (pos_eff_inertia > 1e-10f) {
                float angle_correction = 0.0f;
                if (relative_angle < lower_limit)
                    angle_correction = baumgarte * (lower_limit - relative_angle);
                else if (relative_angle > upper_limit)
                    angle_correction = baumgarte * (upper_limit - relative_angle);
                if (angle_correction != 0.0f) {
                    A[IDX_ANGLE] = cur_angle_a - inv_ia * angle_correction / pos_eff_inertia;
                    B[IDX_ANGLE] = cur_angle_b + inv_ib * angle_correction / pos_eff_inertia;
                }
            }
        }
    }
}

// Counter-based Philox4x32-10 (Salmon, Moraes, Dror, Shaw, SC'11).  The
// reference draws from Mojo's stdlib `random.philox.Random(seed, offset)`,
// whose source is not in the reference tree (pinned by pixi.lock:117-119 to
// mojo 0.26.2.0.dev2026012305), so the (seed, offset) -> (key, counter) mapping
// and the uint32 -> float conversion below are this build's own, documented
// choice:  key = (seed lo32, seed hi32), counter = (offset lo32, offset hi32,
// 0, 0), each successive step_uniform() increments the counter by one, and a
// uniform is (x >> 8) * 2^-24 in [0, 1).  Parity unpinned at this boundary.
struct Philox {
    uint32_t key[2];
    uint32_t ctr[4];
    Philox(uint64_t seed, uint64_t offset) {
        key[0] = (uint32_t)seed; key[1] = (uint32_t)(seed >> 32);
        ctr[0] = (uint32_t)offset; ctr[1] = (uint32_t)(offset >> 32); ctr[2] = 0; ctr[3] = 0;
    }
    static void round(uint32_t c[4], const uint32_t k[2]) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0];
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1];
        uint32_t n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    }
    void step(uint32_t out[4]) {
        uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
        uint32_t k[2] = {key[0], key[1]};
        for (int i = 0; i < 10; ++i) {
            round(c, k);
            k[0] += 0x9E3779B9u;
            k[1] += 0xBB67AE85u;
        }
        for (int i = 0; i < 4; ++i) out[i] = c[i];
        if (++ctr[0] == 0) if (++ctr[1] == 0) if (++ctr[2] == 0) ++ctr[3];
    }
    void step_uniform(float out[4]) {
        uint32_t r[4];
        step(r);
        for (int i = 0; i < 4; ++i) out[i] = (float)(r[i] >> 8) * 5.9604644775390625e-8f;
    }
};

// deep_rl/gpu/random.mojo:11-41
inline uint32_t xorshift32(uint32_t x) {
    x ^= x << 13;
    x ^= x >> 17;
    x ^= x << 5;
    return x;
}
// value = float(new_state) / float(UINT32_MAX); both conversions round to
// nearest, so the divisor is 4294967296.0f and the value can equal 1.0.
inline float random_uniform(uint32_t& rng) {
    rng = xorshift32(rng);
    return (float)rng / (float)0xFFFFFFFFu;
}
inline float random_range(uint32_t& rng, float low, float high) {
    float u = random_uniform(rng);
    return low + u * (high - low);
}

}  // namespace oracle
