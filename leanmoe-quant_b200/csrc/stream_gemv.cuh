// Device building blocks shared by the streaming GEMV kernels and the whole-step kernel.
#pragma once

#include "gemv_common.cuh"
#include "kernels.h"
#include "stream.cuh"

namespace lemoq {

// Activation slice of a lane in the form the chosen dot product wants.
template <int NCH, int MODE>
struct XSlice;
template <int NCH>
struct XSlice<NCH, DOT_F32_MAGIC> {
    float v[NCH][16];
    float neg[NCH];  // -32896 * sum of the 16 activations of the chunk
    __device__ __forceinline__ void set(int c, const float (&f)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[c][j] = f[j];
        neg[c] = -kMagicOffset * sum16(f);
    }
    __device__ __forceinline__ float dot(int c, const uint4& w) const { return magic_dot16(w, v[c]) + neg[c]; }
};
template <int NCH>
struct XSlice<NCH, DOT_F16_CVT> {
    float v[NCH][16];
    __device__ __forceinline__ void set(int c, const float (&f)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[c][j] = f[j];
    }
    __device__ __forceinline__ float dot(int c, const uint4& w) const { return exact_dot16_cvt(w, v[c]); }
};
template <int NCH>
struct XSlice<NCH, DOT_F16_FOLD> {
    float v[NCH][16];
    float neg[NCH];  // -1152 * sum of the 16 activations of the chunk
    __device__ __forceinline__ void set(int c, const float (&f)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[c][j] = f[j];
        neg[c] = -kFoldOffset * sum16(f);
    }
    __device__ __forceinline__ float dot(int c, const uint4& w) const { return fold_dot16(w, v[c]) + neg[c]; }
};
template <int NCH>
struct XSlice<NCH, DOT_F16_MIXED> {
    uint32_t h[NCH][8];
    __device__ __forceinline__ void set(int c, const float (&f)[16]) {  // f holds fp16-representable values
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __half2 p = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
            h[c][j] = *reinterpret_cast<const uint32_t*>(&p);
        }
    }
    __device__ __forceinline__ float dot(int c, const uint4& w) const { return exact_dot16_mixed(w, h[c]); }
};

// Fill the slice from a global fp16 vector, optionally through the fused RMSNorm.
template <int NCH, int MODE, bool NORM>
__device__ __forceinline__ void load_xslice(XSlice<NCH, MODE>& xs, const __half* __restrict__ x,
                                            const __half* __restrict__ nw, float eps, int K, int lane) {
    float tmp[NCH][16];
    if (NORM) {
        load_x_rmsnorm<NCH>(tmp, x, nw, eps, K, lane, nullptr);
    } else {
        load_x_plain<NCH>(tmp, x, K, lane);
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) xs.set(c, tmp[c]);
}

// Per-lane constants of the row layout: byte offset of the lane's chunk and the index of its scale.
template <int NCH>
struct LaneMap {
    int k0[NCH];
    int sidx[NCH];
    bool on[NCH];
    __device__ __forceinline__ void init(int K, int group_size, int lane) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            k0[c] = c * 512 + lane * 16;
            on[c] = k0[c] < K;
            sidx[c] = on[c] ? k0[c] / group_size : 0;
        }
    }
};

// sum over the lane's chunks of scale * (codes . x) for one row held in shared memory.
template <int NCH, int MODE>
__device__ __forceinline__ float row_partial(const unsigned char* __restrict__ row, const __half* __restrict__ scales,
                                             const LaneMap<NCH>& lm, const XSlice<NCH, MODE>& xs) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        if (lm.on[c]) {
            const uint4 w = *reinterpret_cast<const uint4*>(row + lm.k0[c]);
            acc = fmaf(xs.dot(c, w), __half2float(scales[lm.sidx[c]]), acc);
        }
    }
    return acc;
}

__device__ __forceinline__ void flag_timeout(int* err_flag) {
    if (err_flag && (threadIdx.x & 31) == 0) atomicOr(err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
}

}  // namespace lemoq
