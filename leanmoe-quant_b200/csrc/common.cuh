// Shared device helpers for the lemoq_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lemoq_b200.h"

namespace lemoq {

constexpr int kWarp = 32;

// ---- error plumbing (host) -------------------------------------------------
int set_error(int code, const char* fmt, ...);
int check_launch(const char* what);

#define LEMOQ_REQUIRE(cond, code, ...)                 \
    do {                                               \
        if (!(cond)) return ::lemoq::set_error(code, __VA_ARGS__); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- programmatic dependent launch ------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may
// start before its predecessor finishes; pdl_wait() blocks until the
// predecessor grid has completed and its writes are visible.  pdl_trigger()
// lets the successor start its own prologue.  Both are no-ops for a normal
// launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A token id read from device memory, clamped into [0, rows) (rows > 0); an id outside raises LEMOQ_FLAG_BAD_TOKEN.
__device__ __forceinline__ int64_t checked_token(const int64_t* token, int64_t rows, int* err_flag) {
    int64_t t = *token;
    if (rows > 0 && (t < 0 || t >= rows)) {
        if (err_flag && threadIdx.x == 0) atomicOr(err_flag, LEMOQ_FLAG_BAD_TOKEN);
        t = t < 0 ? 0 : rows - 1;
    }
    return t;
}

// ---- loads -------------------------------------------------------------------
// Streaming 128-bit load of read-once weight bytes: bypass L1 allocation.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Coherent 128-bit load of data another kernel (or another block) just wrote.
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ---- reductions -----------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the whole block; every thread gets the result.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    const float r = red[32];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    const float r = red[32];
    __syncthreads();
    return r;
}

// ---- int8 / fp16 unpacking -----------------------------------------------------
// Dot product of 16 int8 codes (one 128-bit word) with 16 fp32 activations.
__device__ __forceinline__ float dot16_s8(const uint4& w, const float* x) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        a = fmaf(static_cast<float>(static_cast<int8_t>(u[i] & 0xffu)), x[4 * i + 0], a);
        a = fmaf(static_cast<float>(static_cast<int8_t>((u[i] >> 8) & 0xffu)), x[4 * i + 1], a);
        a = fmaf(static_cast<float>(static_cast<int8_t>((u[i] >> 16) & 0xffu)), x[4 * i + 2], a);
        a = fmaf(static_cast<float>(static_cast<int8_t>(u[i] >> 24)), x[4 * i + 3], a);
    }
    return a;
}
// acc[j] += s * code[j] for 16 int8 codes.
__device__ __forceinline__ void axpy16_s8(const uint4& w, float s, float* acc) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc[4 * i + 0] = fmaf(s, static_cast<float>(static_cast<int8_t>(u[i] & 0xffu)), acc[4 * i + 0]);
        acc[4 * i + 1] = fmaf(s, static_cast<float>(static_cast<int8_t>((u[i] >> 8) & 0xffu)), acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(s, static_cast<float>(static_cast<int8_t>((u[i] >> 16) & 0xffu)), acc[4 * i + 2]);
        acc[4 * i + 3] = fmaf(s, static_cast<float>(static_cast<int8_t>(u[i] >> 24)), acc[4 * i + 3]);
    }
}
// 8 fp16 values (one 128-bit word) to fp32.
__device__ __forceinline__ void unpack8_h(const uint4& w, float* out) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&u[i]);
        const float2 f = __half22float2(h);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ float dot8_h(const uint4& w, const float* x) {
    float f[8];
    unpack8_h(w, f);
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) a = fmaf(f[i], x[i], a);
    return a;
}

// HF RMSNorm rounding chain for one element: fp16(x * rstd) then an fp16 multiply
// by the weight; returned widened to fp32.
__device__ __forceinline__ float norm_elem(__half x, float rstd, __half w) {
    const __half n = __float2half_rn(__half2float(x) * rstd);
    return __half2float(__hmul(n, w));
}

// Block-wide arg-max over `n` fp16 values in global memory, the FIRST maximal index wins (the rule of a host
// arg-max over the same row).  Every thread of the block calls it; thread 0 gets the result, others -1.
// `red_v` / `red_i` hold >= 32 entries each.
__device__ __forceinline__ int block_argmax_f16(const __half* __restrict__ v, int n, float* red_v, int* red_i) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    auto take = [&](float x, int i) {  // NaN counts as the largest value, the lowest index wins ties
        const bool xn = x != x, bn = best != best;
        if ((xn && (!bn || i < bi)) || (!xn && !bn && (x > best || (x == best && i < bi)))) {
            best = x;
            bi = i;
        }
    };
    const int chunks = (reinterpret_cast<uintptr_t>(v) & 15u) == 0 ? n / 8 : 0;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        float f[8];
        unpack8_h(ld_cg16(v + 8 * c), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) take(f[j], 8 * c + j);
    }
    for (int i = chunks * 8 + threadIdx.x; i < n; i += blockDim.x) take(__half2float(__ldcg(v + i)), i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        take(ob, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    if (lane == 0) {
        red_v[warp] = best;
        red_i[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < nwarp; ++w) take(red_v[w], red_i[w]);
        return (bi >= 0 && bi < n) ? bi : 0;
    }
    return -1;
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

}  // namespace lemoq
