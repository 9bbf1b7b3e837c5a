// Warp-per-row W8 GEMV building blocks.
//
// Layout of one weight row of K int8 codes across a warp: the row is cut into
// chunks of 512 bytes; in chunk c lane l owns the 16 codes [c*512 + l*16, +16),
// i.e. one coalesced 128-bit load per lane and chunk.  group_size is a multiple
// of 16, so a lane's 16 codes share one scale.  The activation slice a lane needs
// is the same for every row, so it lives in registers (NCH*16 fp32 values).
#pragma once

#include "common.cuh"

namespace lemoq {

template <int NCH>
struct RowW8 {
    uint4 w[NCH];
    __half s[NCH];
};

// Issue the loads of one row (codes + the scales this lane needs).  Lanes beyond K
// in the last chunk load nothing and contribute zero.
template <int NCH>
__device__ __forceinline__ void load_row_w8(RowW8<NCH>& r, const int8_t* __restrict__ codes_row,
                                            const __half* __restrict__ scale_row, int K, int group_size, int lane) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int k0 = c * 512 + lane * 16;
        if (k0 < K) {
            r.w[c] = ld_stream16(codes_row + k0);
            r.s[c] = scale_row[k0 / group_size];
        } else {
            r.w[c] = make_uint4(0, 0, 0, 0);
            r.s[c] = __float2half_rn(0.f);
        }
    }
}

// Per-lane partial of sum_k x[k]*code[k]*scale[k/g]; reduce with warp_sum().
template <int NCH>
__device__ __forceinline__ float dot_row_w8(const RowW8<NCH>& r, const float (&xr)[NCH][16]) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) acc = fmaf(dot16_s8(r.w[c], xr[c]), __half2float(r.s[c]), acc);
    return acc;
}

// fp16 weight row: 16 halves (two 128-bit words) per lane and chunk.
template <int NCH>
struct RowF16 {
    uint4 w[NCH][2];
};
template <int NCH>
__device__ __forceinline__ void load_row_f16(RowF16<NCH>& r, const __half* __restrict__ row, int K, int lane) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int k0 = c * 512 + lane * 16;
        if (k0 < K) {
            r.w[c][0] = ld_stream16(row + k0);
            r.w[c][1] = ld_stream16(row + k0 + 8);
        } else {
            r.w[c][0] = r.w[c][1] = make_uint4(0, 0, 0, 0);
        }
    }
}
template <int NCH>
__device__ __forceinline__ float dot_row_f16(const RowF16<NCH>& r, const float (&xr)[NCH][16]) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        acc += dot8_h(r.w[c][0], &xr[c][0]);
        acc += dot8_h(r.w[c][1], &xr[c][8]);
    }
    return acc;
}

// One interface over both weight formats (W8 = int8 codes + per-group fp16 scale).
template <int NCH, bool W8>
struct WRow;
template <int NCH>
struct WRow<NCH, true> {
    RowW8<NCH> r;
    __device__ __forceinline__ void load(const void* base, int64_t row, const __half* scale, int K, int group_size,
                                         int lane) {
        load_row_w8<NCH>(r, reinterpret_cast<const int8_t*>(base) + row * K, scale + row * (K / group_size), K,
                         group_size, lane);
    }
    __device__ __forceinline__ float dot(const float (&xr)[NCH][16]) const { return dot_row_w8<NCH>(r, xr); }
};
template <int NCH>
struct WRow<NCH, false> {
    RowF16<NCH> r;
    __device__ __forceinline__ void load(const void* base, int64_t row, const __half*, int K, int, int lane) {
        load_row_f16<NCH>(r, reinterpret_cast<const __half*>(base) + row * K, K, lane);
    }
    __device__ __forceinline__ float dot(const float (&xr)[NCH][16]) const { return dot_row_f16<NCH>(r, xr); }
};

// Activation slice of this lane, plain fp16 -> fp32.
template <int NCH>
__device__ __forceinline__ void load_x_plain(float (&xr)[NCH][16], const __half* __restrict__ x, int K, int lane) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int k0 = c * 512 + lane * 16;
        if (k0 < K) {
            const uint4 a = ld_cg16(x + k0);
            const uint4 b = ld_cg16(x + k0 + 8);
            unpack8_h(a, &xr[c][0]);
            unpack8_h(b, &xr[c][8]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) xr[c][j] = 0.f;
        }
    }
}

// Activation slice with the RMSNorm applied on the fly (HF rounding chain).  The
// block first reduces sum(x^2) over the K elements; `red` holds >= 33 floats.
// Must be called by every thread of the block.
template <int NCH>
__device__ __forceinline__ void load_x_rmsnorm(float (&xr)[NCH][16], const __half* __restrict__ x,
                                               const __half* __restrict__ nw, float eps, int K, int lane,
                                               float* red) {
    // Each warp reads the whole row; only warp 0's partial goes into the block sum
    // (the other warps need the raw values for their own slices anyway).
    uint4 raw[NCH][2];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int k0 = c * 512 + lane * 16;
        if (k0 < K) {
            raw[c][0] = ld_cg16(x + k0);
            raw[c][1] = ld_cg16(x + k0 + 8);
            float f[16];
            unpack8_h(raw[c][0], &f[0]);
            unpack8_h(raw[c][1], &f[8]);
#pragma unroll
            for (int j = 0; j < 16; ++j) ss = fmaf(f[j], f[j], ss);
        } else {
            raw[c][0] = raw[c][1] = make_uint4(0, 0, 0, 0);
        }
    }
    ss = warp_sum(ss);  // every warp holds the full sum of squares (same order in each warp)
    (void)red;
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(K) + eps);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int k0 = c * 512 + lane * 16;
        if (k0 < K) {
            const uint4 wa = *reinterpret_cast<const uint4*>(nw + k0);
            const uint4 wb = *reinterpret_cast<const uint4*>(nw + k0 + 8);
            const __half* xh0 = reinterpret_cast<const __half*>(&raw[c][0]);
            const __half* xh1 = reinterpret_cast<const __half*>(&raw[c][1]);
            const __half* wh0 = reinterpret_cast<const __half*>(&wa);
            const __half* wh1 = reinterpret_cast<const __half*>(&wb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xr[c][j] = norm_elem(xh0[j], rstd, wh0[j]);
                xr[c][8 + j] = norm_elem(xh1[j], rstd, wh1[j]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) xr[c][j] = 0.f;
        }
    }
}

}  // namespace lemoq
