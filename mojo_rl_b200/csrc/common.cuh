// Shared helpers of libmojorl_b200: status/error plumbing, launch counter,
// counter-based and xorshift RNGs, warp/block reductions.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/mojorl_b200.h"
#include "../../include/mrl_detmath.h"

namespace mrl {

// Last error text of the calling thread, returned by mrl_last_error_string().
void set_error(const char* fmt, ...);
// Every kernel launch of the library goes through MRL_LAUNCH so that
// mrl_kernel_launch_count() reports what actually ran on the device.
void count_launch(int n = 1);

#define MRL_CUDA_OK(expr)                                                              \
    do {                                                                               \
        cudaError_t _e = (expr);                                                       \
        if (_e != cudaSuccess) {                                                       \
            mrl::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #expr,                \
                           cudaGetErrorString(_e));                                    \
            return MRL_ERR_CUDA;                                                       \
        }                                                                              \
    } while (0)

#define MRL_CHECK_ARG(cond)                                                            \
    do {                                                                               \
        if (!(cond)) {                                                                 \
            mrl::set_error("%s:%d invalid argument: %s", __FILE__, __LINE__, #cond);   \
            return MRL_ERR_INVALID_ARG;                                                \
        }                                                                              \
    } while (0)

// Launch + count + check the launch status (not the execution status).
#define MRL_LAUNCH(kernel, grid, block, smem, stream, ...)                             \
    do {                                                                               \
        kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);                    \
        mrl::count_launch();                                                           \
        MRL_CUDA_OK(cudaGetLastError());                                               \
    } while (0)

// Optional per-kernel timing of the update path: when enabled, prof_mark(name)
// records a CUDA event after the launches it follows; mrl_profile_report sums
// the device time between consecutive marks by name.  Off by default.
void prof_mark(const char* name, cudaStream_t st);

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// ---------------------------------------------------------------------------
// RNGs.  xorshift32 is the reference's (deep_rl/gpu/random.mojo:11-41).
// Philox4x32-10 (Salmon et al., SC'11) stands in for Mojo's stdlib
// random.philox.Random, whose source is not part of the reference tree:
// key = (seed lo, seed hi), counter = (offset lo, offset hi, 0, 0), one
// counter increment per step, uniform = (x >> 8) * 2^-24.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t xorshift32(uint32_t x) {
    x ^= x << 13;
    x ^= x >> 17;
    x ^= x << 5;
    return x;
}
// float(state) / float(UINT32_MAX): both conversions round to nearest, the
// divisor is 2^32 and the result can be exactly 1.0.
__host__ __device__ __forceinline__ float xs_uniform(uint32_t& rng) {
    rng = xorshift32(rng);
    return (float)rng / 4294967296.0f;
}
__host__ __device__ __forceinline__ float xs_range(uint32_t& rng, float lo, float hi) {
    float u = xs_uniform(rng);
    return lo + u * (hi - lo);
}

struct Philox {
    uint32_t k0, k1, c0, c1, c2, c3;
    __host__ __device__ __forceinline__ Philox(uint64_t seed, uint64_t offset)
        : k0((uint32_t)seed), k1((uint32_t)(seed >> 32)), c0((uint32_t)offset),
          c1((uint32_t)(offset >> 32)), c2(0), c3(0) {}
    __host__ __device__ __forceinline__ void step(uint32_t out[4]) {
        uint32_t a0 = c0, a1 = c1, a2 = c2, a3 = c3, ka = k0, kb = k1;
#pragma unroll
        for (int i = 0; i < 10; ++i) {
#if defined(__CUDA_ARCH__)
            uint32_t hi0 = __umulhi(0xD2511F53u, a0), lo0 = 0xD2511F53u * a0;
            uint32_t hi1 = __umulhi(0xCD9E8D57u, a2), lo1 = 0xCD9E8D57u * a2;
#else
            uint64_t p0 = (uint64_t)0xD2511F53u * a0, p1 = (uint64_t)0xCD9E8D57u * a2;
            uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
            uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
#endif
            uint32_t n0 = hi1 ^ a1 ^ ka, n2 = hi0 ^ a3 ^ kb;
            a0 = n0; a1 = lo1; a2 = n2; a3 = lo0;
            ka += 0x9E3779B9u;
            kb += 0xBB67AE85u;
        }
        out[0] = a0; out[1] = a1; out[2] = a2; out[3] = a3;
        if (++c0 == 0) if (++c1 == 0) if (++c2 == 0) ++c3;
    }
    __host__ __device__ __forceinline__ void step_uniform(float out[4]) {
        uint32_t r[4];
        step(r);
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = (float)(r[i] >> 8) * 5.9604644775390625e-8f;
    }
};

// ---------------------------------------------------------------------------
// Reductions
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Sum over a block of up to 1024 threads; result valid in every thread.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T* smem32) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[w] = v;
    __syncthreads();
    int nw = (blockDim.x + 31) >> 5;
    T r = (threadIdx.x < nw) ? smem32[threadIdx.x] : (T)0;
    if (w == 0) r = warp_sum(r);
    if (threadIdx.x == 0) smem32[0] = r;
    __syncthreads();
    return smem32[0];
}

}  // namespace mrl
