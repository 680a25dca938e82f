/*
 * mrl_detmath.h - deterministic single-precision elementary functions.
 *
 * The reference (denislabs/mojo-rl) calls Mojo's `math.sin/cos/exp/log/tanh`
 * inside its GPU kernels (e.g. physics2d/collision/edge_terrain.mojo:831-832,
 * deep_agents/ppo/ppo.mojo:4092-4121).  The bit patterns those produce depend
 * on the Mojo compiler's device libm, which is not part of the reference tree.
 * Contact detection and termination tests are threshold comparisons, so a
 * 1-ulp difference in sin/cos can flip a done flag.  To make "done flags and
 * action indices bit-exact" a checkable statement, the CUDA kernels and the
 * CPU checker evaluate the SAME sequence of IEEE-754 operations:
 *
 *   - every multiply-add that must be fused is written as fmaf() (one
 *     rounding on both x86 with FMA3 and sm_100a);
 *   - no expression here has the shape a*b+c outside fmaf(), so neither
 *     nvcc -fmad nor gcc -ffp-contract can change the result;
 *   - +, -, *, /, sqrtf are correctly rounded on both sides (nvcc default
 *     -prec-div=true -prec-sqrt=true, no -use_fast_math, no -ftz).
 *
 * Accuracy (checked on CPU against double-precision libm in
 * tests/test_detmath.py): <= 2 ulp for sin/cos on |x| <= 100, exp on
 * [-87, 88], log on positive normals; <= 4 ulp for tanh.
 *
 * Polynomials are plain Taylor / atanh series on the reduced argument; the
 * coefficients are 1/n! and 1/(2n+1).
 */
#ifndef MRL_DETMATH_H
#define MRL_DETMATH_H

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define MRL_HD __host__ __device__ __forceinline__
#else
#define MRL_HD static inline
#endif

MRL_HD float mrl_bits_to_float(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

MRL_HD uint32_t mrl_float_to_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

/* sin and cos of x together.  Cody-Waite reduction by pi/2 in three parts
 * (1.5703125 is exact in 8 bits, so kf*hi is exact for |kf| < 2^16). */
MRL_HD void mrl_sincosf(float x, float* s_out, float* c_out) {
    float kf = rintf(x * 0.636619772367581343f);
    float r = fmaf(kf, -1.5703125f, x);
    r = fmaf(kf, -4.837512969970703125e-4f, r);
    r = fmaf(kf, -7.54978995489188216e-8f, r);
    float r2 = r * r;
    /* sin(r) = r + r^3 * (-1/6 + r2/120 - r2^2/5040 + r2^3/362880) */
    float ps = fmaf(r2, 2.75573192239858907e-6f, -1.98412698412698413e-4f);
    ps = fmaf(ps, r2, 8.33333333333333333e-3f);
    ps = fmaf(ps, r2, -1.66666666666666667e-1f);
    float sr = fmaf(ps * r2, r, r);
    /* cos(r) = 1 - r2/2 + r2^2 * (1/24 - r2/720 + r2^2/40320 - r2^3/3628800) */
    float pc = fmaf(r2, -2.75573192239858907e-7f, 2.48015873015873016e-5f);
    pc = fmaf(pc, r2, -1.38888888888888889e-3f);
    pc = fmaf(pc, r2, 4.16666666666666667e-2f);
    float cr = fmaf(pc * r2, r2, fmaf(r2, -0.5f, 1.0f));
    int k = (int)kf;
    float s = (k & 1) ? cr : sr;
    float c = (k & 1) ? sr : cr;
    if (k & 2) s = -s;
    if ((k + 1) & 2) c = -c;
    *s_out = s;
    *c_out = c;
}

MRL_HD float mrl_sinf(float x) {
    float s, c;
    mrl_sincosf(x, &s, &c);
    return s;
}

MRL_HD float mrl_cosf(float x) {
    float s, c;
    mrl_sincosf(x, &s, &c);
    return c;
}

/* exp(x): x = k ln2 + r, |r| <= ln2/2, degree-7 Taylor, scale in two steps so
 * that results near the ends of the normal range round once. */
MRL_HD float mrl_expf(float x) {
    if (x != x) return x;
    if (x > 89.0f) x = 89.0f;    /* overflows to +inf below */
    if (x < -104.0f) x = -104.0f; /* underflows to 0 below   */
    float kf = rintf(x * 1.44269504088896341f);
    float r = fmaf(kf, -0.693359375f, x);
    r = fmaf(kf, 2.12194440054690583e-4f, r);
    float p = 1.98412698412698413e-4f;
    p = fmaf(p, r, 1.38888888888888889e-3f);
    p = fmaf(p, r, 8.33333333333333333e-3f);
    p = fmaf(p, r, 4.16666666666666667e-2f);
    p = fmaf(p, r, 1.66666666666666667e-1f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int k = (int)kf;
    int k1 = k / 2;
    int k2 = k - k1;
    float s1 = mrl_bits_to_float((uint32_t)(127 + k1) << 23);
    float s2 = mrl_bits_to_float((uint32_t)(127 + k2) << 23);
    return (p * s1) * s2;
}

/* log(x) for x > 0: x = 2^e * m, m in (sqrt(1/2), sqrt(2)], log m = 2 atanh(s),
 * s = (m-1)/(m+1), |s| <= 0.1716. */
MRL_HD float mrl_logf(float x) {
    if (x != x) return x;
    if (x < 0.0f) return mrl_bits_to_float(0x7fc00000u);
    if (x == 0.0f) return mrl_bits_to_float(0xff800000u);
    uint32_t u = mrl_float_to_bits(x);
    if (u == 0x7f800000u) return x;
    int e = 0;
    if (u < 0x00800000u) { /* subnormal: scale up by 2^23 (exact) */
        x = x * 8388608.0f;
        u = mrl_float_to_bits(x);
        e = -23;
    }
    e += (int)(u >> 23) - 127;
    float m = mrl_bits_to_float((u & 0x007fffffu) | 0x3f800000u);
    if (m > 1.41421356237309505f) {
        m = m * 0.5f;
        e += 1;
    }
    float s = (m - 1.0f) / (m + 1.0f);
    float s2 = s * s;
    float p = 9.09090909090909091e-2f;          /* 1/11 */
    p = fmaf(p, s2, 1.11111111111111111e-1f);   /* 1/9  */
    p = fmaf(p, s2, 1.42857142857142857e-1f);   /* 1/7  */
    p = fmaf(p, s2, 2.0e-1f);                   /* 1/5  */
    p = fmaf(p, s2, 3.33333333333333333e-1f);   /* 1/3  */
    float t = s + s;
    float lm = fmaf(p * s2, t, t);
    float ef = (float)e;
    return fmaf(ef, 0.693359375f, fmaf(ef, -2.12194440054690583e-4f, lm));
}

/* tanh(x): odd Taylor polynomial for |x| < 0.3, 1 - 2/(exp(2x)+1) otherwise. */
MRL_HD float mrl_tanhf(float x) {
    float ax = fabsf(x);
    if (ax < 0.3f) {
        float x2 = x * x;
        float p = -8.86323552990219657e-3f;          /* -1382/155925 */
        p = fmaf(p, x2, 2.18694885361552028e-2f);    /*  62/2835     */
        p = fmaf(p, x2, -5.39682539682539683e-2f);   /* -17/315      */
        p = fmaf(p, x2, 1.33333333333333333e-1f);    /*  2/15        */
        p = fmaf(p, x2, -3.33333333333333333e-1f);   /* -1/3         */
        return fmaf(p * x2, x, x);
    }
    if (ax > 10.0f) return x > 0.0f ? 1.0f : -1.0f;
    float e2 = mrl_expf(ax + ax);
    float t = 1.0f - 2.0f / (e2 + 1.0f);
    return x > 0.0f ? t : -t;
}

#endif /* MRL_DETMATH_H */
