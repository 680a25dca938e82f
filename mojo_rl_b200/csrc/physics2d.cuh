// Register-resident rigid-body core shared by the physics2d environments
// (LunarLander, BipedalWalker, planar HalfCheetah).
//
// One thread owns one environment.  The dynamic state of its bodies lives in
// registers for the whole step; everything that the reference recomputes
// inside its solver iterations but that cannot change there (body sin/cos,
// joint lever arms and inverse constraint matrices, contact lever arms and
// effective masses - angles and positions are fixed during the velocity
// phase) is computed once per step.  The arithmetic per quantity is the same
// sequence of IEEE operations as in the reference routines:
//   physics2d/integrators/euler.mojo:202-311
//   physics2d/collision/edge_terrain.mojo:784-1003, flat_terrain.mojo:456-580
//   physics2d/solvers/impulse.mojo:419-628, :905-980
//   physics2d/joints/revolute.mojo:512-730, :764-920
// Terrain contacts always have the static ground as body B, so the B-side
// terms (all exactly zero there) are dropped.
//
// This translation unit must be compiled with -fmad=false: results are
// compared bit for bit with a CPU restatement.
#pragma once
#include "common.cuh"

namespace mrl {
namespace phys {

constexpr int BODY_STATE_SIZE = 13;
constexpr int IDX_X = 0, IDX_Y = 1, IDX_ANGLE = 2, IDX_VX = 3, IDX_VY = 4, IDX_OMEGA = 5,
              IDX_INV_MASS = 10, IDX_INV_INERTIA = 11, IDX_SHAPE = 12;
constexpr int JOINT_DATA_SIZE = 17;
constexpr int JOINT_TYPE = 0, JOINT_BODY_A = 1, JOINT_BODY_B = 2, JOINT_ANCHOR_AX = 3,
              JOINT_ANCHOR_AY = 4, JOINT_ANCHOR_BX = 5, JOINT_ANCHOR_BY = 6, JOINT_REF_ANGLE = 7,
              JOINT_LOWER_LIMIT = 8, JOINT_UPPER_LIMIT = 9, JOINT_MAX_MOTOR_TORQUE = 10,
              JOINT_MOTOR_SPEED = 11, JOINT_STIFFNESS = 12, JOINT_DAMPING = 13, JOINT_FLAGS = 14;
constexpr int JOINT_FLAG_LIMIT = 1, JOINT_FLAG_MOTOR = 2, JOINT_FLAG_SPRING = 4;
constexpr int CONTACT_DATA_SIZE = 9;

template <int NB>
struct Bodies {
    float x[NB], y[NB], a[NB], vx[NB], vy[NB], w[NB], inv_m[NB], inv_i[NB];
    float sn[NB], cs[NB];  // sin/cos of a[], refreshed by refresh_trig()
};

struct JointParams {
    float ax, ay, bx, by, ref, lo, hi, max_torque, motor_speed, stiffness, damping;
    int flags;
};

// Per-step constants of one joint during the velocity phase.
struct JointPre {
    float rax, ray, rbx, rby, ik11, ik12, ik22, angle_error, rel_angle;
};

template <int MAXC>
struct Contacts {
    int n;
    int body[MAXC];
    float px[MAXC], py[MAXC], nx[MAXC], ny[MAXC], depth[MAXC];
};

// Velocity-phase working set of the contacts (lever arm, effective masses,
// accumulated impulses).
template <int MAXC>
struct ContactPre {
    float rax[MAXC], ray[MAXC], k[MAXC], kt[MAXC], jn[MAXC], jt[MAXC];
};

// The step kernels are long straight-line programs run by one or two warps per SM, so their time goes
// into instruction fetch rather than arithmetic; the sine/cosine pair (~70 instructions, used a dozen
// times per step) is therefore one shared out-of-line routine instead of a dozen inlined copies.
static __device__ __noinline__ float2 sincos_shared(float a) {
    float s, c;
    mrl_sincosf(a, &s, &c);
    return make_float2(s, c);
}

template <int NB>
__device__ __forceinline__ void refresh_trig(Bodies<NB>& b) {
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const float2 sc = sincos_shared(b.a[i]);
        b.sn[i] = sc.x;
        b.cs[i] = sc.y;
    }
}

// euler.mojo:202-251 with the force slots passed in (fx, fy, tau per body).
template <int NB>
__device__ __forceinline__ void integrate_velocities(Bodies<NB>& b, const float (&fx)[NB],
                                                     const float (&fy)[NB], const float (&tau)[NB],
                                                     float gx, float gy, float dt) {
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        if (b.inv_m[i] == 0.0f) continue;
        b.vx[i] = b.vx[i] + (fx[i] * b.inv_m[i] + gx) * dt;
        b.vy[i] = b.vy[i] + (fy[i] * b.inv_m[i] + gy) * dt;
        b.w[i] = b.w[i] + tau[i] * b.inv_i[i] * dt;
    }
}

// euler.mojo:255-311
template <int NB>
__device__ __forceinline__ void integrate_positions(Bodies<NB>& b, float dt) {
    const float pi_val = 3.14159274101257324f;      // f32(pi)
    const float two_pi_val = 6.28318548202514648f;  // f32(2 pi)
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        if (b.inv_m[i] == 0.0f) continue;
        b.x[i] = b.x[i] + b.vx[i] * dt;
        b.y[i] = b.y[i] + b.vy[i] * dt;
        float angle = b.a[i] + b.w[i] * dt;
        if (angle > 100.0f || angle < -100.0f) angle = 0.0f;
        if (angle > pi_val) angle = angle - two_pi_val;
        if (angle > pi_val) angle = angle - two_pi_val;
        if (angle < -pi_val) angle = angle + two_pi_val;
        if (angle < -pi_val) angle = angle + two_pi_val;
        b.a[i] = angle;
    }
}

// One vertex against one terrain edge; edge_terrain.mojo:848-910.
template <int MAXC>
__device__ __forceinline__ void vertex_edge_test(Contacts<MAXC>& c, int body, float wx, float wy,
                                                 float e_x0, float e_y0, float e_x1, float e_y1,
                                                 float e_nx, float e_ny) {
    float x_min = e_x0, x_max = e_x1;
    if (e_x0 > e_x1) { x_min = e_x1; x_max = e_x0; }
    if (wx < x_min - 0.1f || wx > x_max + 0.1f) return;
    float edge_dx = e_x1 - e_x0, edge_dy = e_y1 - e_y0;
    float edge_len_sq = edge_dx * edge_dx + edge_dy * edge_dy;
    if (edge_len_sq < 1e-6f) return;
    float t = ((wx - e_x0) * edge_dx + (wy - e_y0) * edge_dy) / edge_len_sq;
    if (t < 0.0f) t = 0.0f;
    if (t > 1.0f) t = 1.0f;
    float closest_x = e_x0 + t * edge_dx, closest_y = e_y0 + t * edge_dy;
    float dist_x = wx - closest_x, dist_y = wy - closest_y;
    float penetration = -(dist_x * e_nx + dist_y * e_ny);
    if (penetration > 0.0f && c.n < MAXC) {
        int s = c.n;
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
            if (k == s) {
                c.body[k] = body; c.px[k] = wx; c.py[k] = wy;
                c.nx[k] = e_nx; c.ny[k] = e_ny; c.depth[k] = penetration;
            }
        c.n = s + 1;
    }
}

// Contact lever arms and effective masses (impulse.mojo:489-517, :573-583),
// positions being fixed during the velocity phase.
template <int NB, int MAXC>
__device__ __forceinline__ void prepare_contacts(const Bodies<NB>& b, const Contacts<MAXC>& c,
                                                 ContactPre<MAXC>& p) {
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
        if (k >= c.n) break;
        float bx = b.x[0], by = b.y[0], im = b.inv_m[0], ii = b.inv_i[0];
#pragma unroll
        for (int i = 1; i < NB; ++i)
            if (c.body[k] == i) { bx = b.x[i]; by = b.y[i]; im = b.inv_m[i]; ii = b.inv_i[i]; }
        float ra_x = c.px[k] - bx, ra_y = c.py[k] - by;
        float nx = c.nx[k], ny = c.ny[k];
        float ra_cross_n = ra_x * ny - ra_y * nx;
        float kn = im + 0.0f;
        kn = kn + ii * ra_cross_n * ra_cross_n;
        float tx = -ny, ty = nx;
        float ra_cross_t = ra_x * ty - ra_y * tx;
        float kt = im + 0.0f;
        kt = kt + ii * ra_cross_t * ra_cross_t;
        p.rax[k] = ra_x; p.ray[k] = ra_y; p.k[k] = kn; p.kt[k] = kt;
        p.jn[k] = 0.0f; p.jt[k] = 0.0f;
    }
}

// impulse.mojo:419-628 for ground contacts.
template <int NB, int MAXC>
__device__ __forceinline__ void solve_velocity_contacts(Bodies<NB>& b, const Contacts<MAXC>& c,
                                                        ContactPre<MAXC>& p, float friction,
                                                        float restitution) {
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
        if (k >= c.n) break;
        const int bi = c.body[k];
        float vx = b.vx[0], vy = b.vy[0], w = b.w[0], im = b.inv_m[0], ii = b.inv_i[0];
#pragma unroll
        for (int i = 1; i < NB; ++i)
            if (bi == i) { vx = b.vx[i]; vy = b.vy[i]; w = b.w[i]; im = b.inv_m[i]; ii = b.inv_i[i]; }
        const float ra_x = p.rax[k], ra_y = p.ray[k], nx = c.nx[k], ny = c.ny[k];
        float rel_x = vx - w * ra_y, rel_y = vy + w * ra_x;
        float vel_normal = rel_x * nx + rel_y * ny;
        if (vel_normal < 0.0f) {
            float j_normal = -(1.0f + restitution) * vel_normal / p.k[k];
            float old_impulse = p.jn[k];
            float new_impulse = old_impulse + j_normal;
            if (new_impulse < 0.0f) new_impulse = 0.0f;
            p.jn[k] = new_impulse;
            j_normal = new_impulse - old_impulse;
            float impulse_x = j_normal * nx, impulse_y = j_normal * ny;
            vx = vx + impulse_x * im;
            vy = vy + impulse_y * im;
            w = w + (ra_x * impulse_y - ra_y * impulse_x) * ii;
            rel_x = vx - w * ra_y;
            rel_y = vy + w * ra_x;
            float tx = -ny, ty = nx;
            float vel_tangent = rel_x * tx + rel_y * ty;
            float j_tangent = -vel_tangent / p.kt[k];
            float max_friction = friction * new_impulse;
            float old_tangent = p.jt[k];
            float new_tangent = old_tangent + j_tangent;
            if (new_tangent > max_friction) new_tangent = max_friction;
            else if (new_tangent < -max_friction) new_tangent = -max_friction;
            p.jt[k] = new_tangent;
            j_tangent = new_tangent - old_tangent;
            float friction_x = j_tangent * tx, friction_y = j_tangent * ty;
            vx = vx + friction_x * im;
            vy = vy + friction_y * im;
            w = w + (ra_x * friction_y - ra_y * friction_x) * ii;
#pragma unroll
            for (int i = 0; i < NB; ++i)
                if (bi == i) { b.vx[i] = vx; b.vy[i] = vy; b.w[i] = w; }
        }
    }
}

// impulse.mojo:905-980 for ground contacts (inv_mass_b = 0).
template <int NB, int MAXC>
__device__ __forceinline__ void solve_position_contacts(Bodies<NB>& b, const Contacts<MAXC>& c,
                                                        float baumgarte, float slop) {
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
        if (k >= c.n) break;
        float correction = c.depth[k] - slop;
        if (correction <= 0.0f) continue;
        correction = baumgarte * correction;
        const int bi = c.body[k];
        float im = b.inv_m[0];
#pragma unroll
        for (int i = 1; i < NB; ++i) if (bi == i) im = b.inv_m[i];
        float total_inv_mass = im + 0.0f;
        if (total_inv_mass == 0.0f) continue;
        float correction_a = correction * im / total_inv_mass;
        float dx = c.nx[k] * correction_a, dy = c.ny[k] * correction_a;
#pragma unroll
        for (int i = 0; i < NB; ++i)
            if (bi == i) { b.x[i] = b.x[i] + dx; b.y[i] = b.y[i] + dy; }
    }
}

// Lever arms and inverse point-constraint matrix of one joint
// (revolute.mojo:571-601); needs fresh b.sn / b.cs.
template <int NB>
__device__ __forceinline__ void joint_geometry(const Bodies<NB>& b, int A, int B,
                                               const JointParams& jp, float& rax, float& ray,
                                               float& rbx, float& rby, float& ik11, float& ik12,
                                               float& ik22) {
    const float cos_a = b.cs[A], sin_a = b.sn[A], cos_b = b.cs[B], sin_b = b.sn[B];
    rax = jp.ax * cos_a - jp.ay * sin_a;
    ray = jp.ax * sin_a + jp.ay * cos_a;
    rbx = jp.bx * cos_b - jp.by * sin_b;
    rby = jp.bx * sin_b + jp.by * cos_b;
    const float inv_ma = b.inv_m[A], inv_mb = b.inv_m[B], inv_ia = b.inv_i[A], inv_ib = b.inv_i[B];
    float k11 = inv_ma + inv_mb + inv_ia * ray * ray + inv_ib * rby * rby;
    float k12 = -inv_ia * rax * ray - inv_ib * rbx * rby;
    float k22 = inv_ma + inv_mb + inv_ia * rax * rax + inv_ib * rbx * rbx;
    float det = k11 * k22 - k12 * k12;
    if (det < 1e-10f) det = 1e-10f;
    float inv_det = 1.0f / det;
    ik11 = k22 * inv_det;
    ik12 = -k12 * inv_det;
    ik22 = k11 * inv_det;
}

// Traits::ja(j) / Traits::jb(j) give the compile-time topology.
template <class Traits, int NB, int NJ>
__device__ __forceinline__ void prepare_joints(const Bodies<NB>& b, const JointParams (&jp)[NJ],
                                               JointPre (&pre)[NJ]) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int A = Traits::ja(j), B = Traits::jb(j);
        joint_geometry(b, A, B, jp[j], pre[j].rax, pre[j].ray, pre[j].rbx, pre[j].rby, pre[j].ik11,
                       pre[j].ik12, pre[j].ik22);
        float current_angle = b.a[B] - b.a[A];
        pre[j].angle_error = current_angle - jp[j].ref;      // spring, revolute.mojo:627-628
        pre[j].rel_angle = b.a[B] - b.a[A] - jp[j].ref;      // limit,  revolute.mojo:672-674
    }
}

// revolute.mojo:512-730, one pass over the joints.
template <class Traits, int NB, int NJ>
__device__ __forceinline__ void solve_velocity_joints(Bodies<NB>& b, const JointParams (&jp)[NJ],
                                                      const JointPre (&pre)[NJ], int joint_count,
                                                      float dt) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        if (j >= joint_count) break;
        const int A = Traits::ja(j), B = Traits::jb(j);
        const JointPre& q = pre[j];
        const float inv_ma = b.inv_m[A], inv_mb = b.inv_m[B], inv_ia = b.inv_i[A], inv_ib = b.inv_i[B];
        const float vxa = b.vx[A], vya = b.vy[A], wa = b.w[A];
        const float vxb = b.vx[B], vyb = b.vy[B], wb = b.w[B];
        float va_anchor_x = vxa - wa * q.ray, va_anchor_y = vya + wa * q.rax;
        float vb_anchor_x = vxb - wb * q.rby, vb_anchor_y = vyb + wb * q.rbx;
        float cdot_x = vb_anchor_x - va_anchor_x, cdot_y = vb_anchor_y - va_anchor_y;
        float impulse_x = -(q.ik11 * cdot_x + q.ik12 * cdot_y);
        float impulse_y = -(q.ik12 * cdot_x + q.ik22 * cdot_y);
        b.vx[A] = vxa - inv_ma * impulse_x;
        b.vy[A] = vya - inv_ma * impulse_y;
        b.w[A] = wa - inv_ia * (q.rax * impulse_y - q.ray * impulse_x);
        b.vx[B] = vxb + inv_mb * impulse_x;
        b.vy[B] = vyb + inv_mb * impulse_y;
        b.w[B] = wb + inv_ib * (q.rbx * impulse_y - q.rby * impulse_x);
        const int flags = jp[j].flags;
        const float eff_inertia = inv_ia + inv_ib;
        if (flags & JOINT_FLAG_SPRING) {
            float rel_omega = wb - wa;  // pre-impulse values
            float spring_torque = -jp[j].stiffness * q.angle_error - jp[j].damping * rel_omega;
            float angular_impulse = spring_torque * dt;
            if (eff_inertia > 1e-10f) {
                b.w[A] = b.w[A] - inv_ia * angular_impulse / eff_inertia;
                b.w[B] = b.w[B] + inv_ib * angular_impulse / eff_inertia;
            }
        }
        if (flags & JOINT_FLAG_LIMIT) {
            float current_wa = b.w[A], current_wb = b.w[B];
            float rel_omega = current_wb - current_wa;
            if (eff_inertia > 1e-10f) {
                float limit_impulse = 0.0f;
                if (q.rel_angle <= jp[j].lo) {
                    if (rel_omega < 0.0f) limit_impulse = -rel_omega / eff_inertia;
                } else if (q.rel_angle >= jp[j].hi) {
                    if (rel_omega > 0.0f) limit_impulse = -rel_omega / eff_inertia;
                }
                if (limit_impulse != 0.0f) {
                    b.w[A] = current_wa - inv_ia * limit_impulse;
                    b.w[B] = current_wb + inv_ib * limit_impulse;
                }
            }
        }
        if (flags & JOINT_FLAG_MOTOR) {
            float current_wa = b.w[A], current_wb = b.w[B];
            float rel_omega = current_wb - current_wa;
            float speed_error = jp[j].motor_speed - rel_omega;
            if (eff_inertia > 1e-10f) {
                float motor_impulse = speed_error / eff_inertia;
                float max_impulse = jp[j].max_torque * dt;
                if (motor_impulse > max_impulse) motor_impulse = max_impulse;
                if (motor_impulse < -max_impulse) motor_impulse = -max_impulse;
                b.w[A] = current_wa - inv_ia * motor_impulse;
                b.w[B] = current_wb + inv_ib * motor_impulse;
            }
        }
    }
}

// revolute.mojo:764-920, one pass; angles move, so trig is recomputed per joint.
template <class Traits, int NB, int NJ>
__device__ __forceinline__ void solve_position_joints(Bodies<NB>& b, const JointParams (&jp)[NJ],
                                                      int joint_count, float baumgarte, float slop) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        if (j >= joint_count) break;
        const int A = Traits::ja(j), B = Traits::jb(j);
        {
            const float2 sa = sincos_shared(b.a[A]), sb = sincos_shared(b.a[B]);
            b.sn[A] = sa.x; b.cs[A] = sa.y;
            b.sn[B] = sb.x; b.cs[B] = sb.y;
        }
        float rax, ray, rbx, rby, ik11, ik12, ik22;
        joint_geometry(b, A, B, jp[j], rax, ray, rbx, rby, ik11, ik12, ik22);
        const float xa = b.x[A], ya = b.y[A], xb = b.x[B], yb = b.y[B];
        float anchor_ax = xa + rax, anchor_ay = ya + ray;
        float anchor_bx = xb + rbx, anchor_by = yb + rby;
        float cx = anchor_bx - anchor_ax, cy = anchor_by - anchor_ay;
        float error = sqrtf(cx * cx + cy * cy);
        if (error < slop) continue;
        const float inv_ma = b.inv_m[A], inv_mb = b.inv_m[B], inv_ia = b.inv_i[A], inv_ib = b.inv_i[B];
        float correction_x = -baumgarte * (ik11 * cx + ik12 * cy);
        float correction_y = -baumgarte * (ik12 * cx + ik22 * cy);
        b.x[A] = xa - inv_ma * correction_x;
        b.y[A] = ya - inv_ma * correction_y;
        b.a[A] = b.a[A] - inv_ia * (rax * correction_y - ray * correction_x);
        b.x[B] = xb + inv_mb * correction_x;
        b.y[B] = yb + inv_mb * correction_y;
        b.a[B] = b.a[B] + inv_ib * (rbx * correction_y - rby * correction_x);
        if (jp[j].flags & JOINT_FLAG_LIMIT) {
            float cur_angle_a = b.a[A], cur_angle_b = b.a[B];
            float relative_angle = cur_angle_b - cur_angle_a - jp[j].ref;
            float pos_eff_inertia = inv_ia + inv_ib;
            if (pos_eff_inertia > 1e-10f) {
                float angle_correction = 0.0f;
                if (relative_angle < jp[j].lo) angle_correction = baumgarte * (jp[j].lo - relative_angle);
                else if (relative_angle > jp[j].hi) angle_correction = baumgarte * (jp[j].hi - relative_angle);
                if (angle_correction != 0.0f) {
                    b.a[A] = cur_angle_a - inv_ia * angle_correction / pos_eff_inertia;
                    b.a[B] = cur_angle_b + inv_ib * angle_correction / pos_eff_inertia;
                }
            }
        }
    }
}

}  // namespace phys
}  // namespace mrl
