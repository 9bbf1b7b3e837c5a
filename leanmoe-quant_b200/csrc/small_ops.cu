// Stand-alone element-wise / row ops of the decode step (each is also fused into a
// larger kernel on the whole-step path) and the offline weight quantiser.
#include "common.cuh"
#include "kernels.h"

namespace lemoq {

// ---------------------------------------------------------------------------
// RMSNorm, one block per row.  y = fp16(x * rstd) * w with an fp16 multiply.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rms_norm_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                       __half* __restrict__ y, int H, float eps) {
    __shared__ float red[40];
    pdl_wait();
    pdl_trigger();
    const __half* xr = x + static_cast<int64_t>(blockIdx.x) * H;
    __half* yr = y + static_cast<int64_t>(blockIdx.x) * H;
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
        float f[8];
        unpack8_h(ld_cg16(xr + i), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
        const uint4 xv = ld_cg16(xr + i);
        const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
        const __half* xh = reinterpret_cast<const __half*>(&xv);
        const __half* wh = reinterpret_cast<const __half*>(&wv);
        __align__(16) __half o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __hmul(__float2half_rn(__half2float(xh[j]) * rstd), wh[j]);
        *reinterpret_cast<uint4*>(yr + i) = *reinterpret_cast<const uint4*>(o);
    }
}

int launch_rms_norm(const __half* x, const __half* w, __half* y, int64_t rows, int H, float eps, const LaunchCfg& lc) {
    if (rows == 0) return LEMOQ_OK;
    return launch_kernel(rms_norm_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, lc, x, w, y, H, eps);
}

// ---------------------------------------------------------------------------
// Half-split RoPE on q and k, one block per head (q heads first, then k heads).
// ---------------------------------------------------------------------------
__global__ void rope_qk_kernel(const __half* __restrict__ q, int64_t q_hs, int heads_q, const __half* __restrict__ k,
                               int64_t k_hs, const __half* __restrict__ cos, const __half* __restrict__ sin, int D,
                               __half* __restrict__ q_out, __half* __restrict__ k_out) {
    pdl_wait();
    pdl_trigger();
    const int b = blockIdx.x;
    const bool is_q = b < heads_q;
    const int h = is_q ? b : b - heads_q;
    const __half* src = is_q ? q + h * q_hs : k + h * k_hs;
    __half* dst = (is_q ? q_out : k_out) + static_cast<int64_t>(h) * D;
    const int half_d = D / 2;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float x = __half2float(src[d]);
        const float rot = d < half_d ? -__half2float(src[d + half_d]) : __half2float(src[d - half_d]);
        const float a = __fmul_rn(x, __half2float(cos[d]));
        const float bb = __fmul_rn(rot, __half2float(sin[d]));
        dst[d] = __float2half_rn(__fadd_rn(a, bb));
    }
}

int launch_rope_qk(const __half* q, int64_t q_hs, int heads_q, const __half* k, int64_t k_hs, int heads_k,
                   const __half* cos, const __half* sin, int D, __half* q_out, __half* k_out, const LaunchCfg& lc) {
    const int threads = D >= 128 ? 128 : 64;
    return launch_kernel(rope_qk_kernel, dim3(heads_q + heads_k), dim3(threads), 0, lc, q, q_hs, heads_q, k, k_hs,
                         cos, sin, D, q_out, k_out);
}

// ---------------------------------------------------------------------------
// KV direct write: bit copy of the new K/V rows into slot *pos of the fp16 cache.
// grid = 2*heads (K heads then V heads).
// ---------------------------------------------------------------------------
__global__ void kv_direct_write_kernel(const __half* __restrict__ k_row, const __half* __restrict__ v_row,
                                       int64_t src_hs, __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                       const int64_t* __restrict__ pos_ptr, int heads, int max_len, int D,
                                       int* err_flag) {
    pdl_wait();
    pdl_trigger();
    const int64_t pos = *pos_ptr;
    if (pos < 0 || pos >= max_len) {
        if (err_flag && threadIdx.x == 0) atomicOr(err_flag, LEMOQ_FLAG_BAD_POSITION);
        return;
    }
    const bool is_k = blockIdx.x < heads;
    const int h = is_k ? blockIdx.x : blockIdx.x - heads;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(is_k ? k_row : v_row) + h * src_hs;
    uint16_t* dst = reinterpret_cast<uint16_t*>(is_k ? k_cache : v_cache) + (static_cast<int64_t>(h) * max_len + pos) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
}

int launch_kv_direct_write(const __half* k_row, const __half* v_row, int64_t src_hs, __half* k_cache, __half* v_cache,
                           const int64_t* pos, int heads, int max_len, int D, int* err_flag, const LaunchCfg& lc) {
    return launch_kernel(kv_direct_write_kernel, dim3(2 * heads), dim3(D >= 128 ? 128 : 64), 0, lc, k_row, v_row,
                         src_hs, k_cache, v_cache, pos, heads, max_len, D, err_flag);
}

// ---------------------------------------------------------------------------
// Per-token symmetric int8 quantisation (one warp per row):
//   amax (fp32) -> s = amax/127 (1.0 if amax == 0) -> rint(x / s) -> clamp +-127;
//   the scale is stored as fp16, the division uses the fp32 scale.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void quantize_row_warp(const __half* __restrict__ src, int8_t* __restrict__ codes,
                                                  __half* __restrict__ scale, int D) {
    const int lane = threadIdx.x & 31;
    float amax = 0.f;
    for (int d = lane; d < D; d += 32) amax = fmaxf(amax, fabsf(__half2float(src[d])));
    amax = warp_max(amax);
    const float s = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    for (int d = lane; d < D; d += 32) {
        float q = rintf(__fdiv_rn(__half2float(src[d]), s));
        q = fminf(fmaxf(q, -127.0f), 127.0f);
        codes[d] = static_cast<int8_t>(static_cast<int>(q));
    }
    if (lane == 0) *scale = __float2half_rn(s);
}

// grid = 2*heads, block = 32.
__global__ void __launch_bounds__(32) kv_int8_cache_write_kernel(const __half* __restrict__ k_row,
                                                                 const __half* __restrict__ v_row, int8_t* kc,
                                                                 __half* ks, int8_t* vc, __half* vs,
                                                                 const int64_t* __restrict__ pos_ptr, int heads, int S,
                                                                 int D, int* err_flag) {
    pdl_wait();
    pdl_trigger();
    const int64_t pos = pos_ptr ? *pos_ptr : 0;
    if (pos < 0 || pos >= S) {
        if (err_flag && threadIdx.x == 0) atomicOr(err_flag, LEMOQ_FLAG_BAD_POSITION);
        return;
    }
    const bool is_k = blockIdx.x < heads;
    const int h = is_k ? blockIdx.x : blockIdx.x - heads;
    const __half* src = (is_k ? k_row : v_row) + static_cast<int64_t>(h) * D;
    int8_t* codes = (is_k ? kc : vc) + (static_cast<int64_t>(h) * S + pos) * D;
    __half* scale = (is_k ? ks : vs) + static_cast<int64_t>(h) * S + pos;
    quantize_row_warp(src, codes, scale, D);
}

int launch_kv_int8_cache_write(const __half* k_row, const __half* v_row, int8_t* kc, __half* ks, int8_t* vc,
                               __half* vs, const int64_t* pos, int heads, int S, int D, int* err_flag,
                               const LaunchCfg& lc) {
    return launch_kernel(kv_int8_cache_write_kernel, dim3(2 * heads), dim3(32), 0, lc, k_row, v_row, kc, ks, vc, vs,
                         pos, heads, S, D, err_flag);
}

// Bulk: one warp per (tensor, head, slot); slots >= filled get code 0 / scale 1.
__global__ void __launch_bounds__(256) kv_int8_bulk_kernel(const __half* __restrict__ keys,
                                                           const __half* __restrict__ values, int8_t* kc, __half* ks,
                                                           int8_t* vc, __half* vs, int heads, int S, int D, int filled) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
    const int64_t rows = static_cast<int64_t>(heads) * S;
    if (row >= 2 * rows) return;
    const bool is_k = row < rows;
    const int64_t r = is_k ? row : row - rows;
    const int slot = static_cast<int>(r % S);
    const __half* src = (is_k ? keys : values) + r * D;
    int8_t* codes = (is_k ? kc : vc) + r * D;
    __half* scale = (is_k ? ks : vs) + r;
    if (filled >= 0 && slot >= filled) {
        for (int d = lane; d < D; d += 32) codes[d] = 0;
        if (lane == 0) *scale = __float2half_rn(1.0f);
        return;
    }
    quantize_row_warp(src, codes, scale, D);
}

int launch_kv_int8_bulk(const __half* keys, const __half* values, int8_t* kc, __half* ks, int8_t* vc, __half* vs,
                        int heads, int S, int D, int filled, const LaunchCfg& lc) {
    const int64_t rows = 2ll * heads * S;
    if (rows == 0) return LEMOQ_OK;
    const int wpb = 8;
    return launch_kernel(kv_int8_bulk_kernel, dim3(static_cast<unsigned>((rows + wpb - 1) / wpb)), dim3(wpb * 32), 0,
                         lc, keys, values, kc, ks, vc, vs, heads, S, D, filled);
}

// ---------------------------------------------------------------------------
// Weight RTN: one warp per (row, group).  scale = absmax/127 in fp32 (1.0 for a zero
// group); code = clamp(rint(w / scale), -128, 127); scale stored as fp16.
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void __launch_bounds__(256) rtn_quantize_kernel(const TW* __restrict__ w, int64_t n_groups_total,
                                                           int group_size, int8_t* __restrict__ codes,
                                                           __half* __restrict__ scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t g = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
    if (g >= n_groups_total) return;
    const TW* src = w + g * group_size;
    int8_t* dst = codes + g * group_size;
    float amax = 0.f;
    for (int i = lane; i < group_size; i += 32) amax = fmaxf(amax, fabsf(to_float(src[i])));
    amax = warp_max(amax);
    const float s = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    for (int i = lane; i < group_size; i += 32) {
        float q = rintf(__fdiv_rn(to_float(src[i]), s));
        q = fminf(fmaxf(q, -128.0f), 127.0f);
        dst[i] = static_cast<int8_t>(static_cast<int>(q));
    }
    if (lane == 0) scale[g] = __float2half_rn(s);
}

int launch_rtn_quantize(const void* w, int w_dtype, int64_t rows, int in_features, int group_size, int8_t* codes,
                        __half* scale, const LaunchCfg& lc) {
    const int64_t groups = rows * (in_features / group_size);
    if (groups == 0) return LEMOQ_OK;
    const int wpb = 8;
    const int64_t blocks = (groups + wpb - 1) / wpb;
    if (blocks > 0x7fffffffll) return set_error(LEMOQ_ERR_INVALID, "tensor too large for one quantisation launch");
    if (w_dtype == LEMOQ_DTYPE_F16)
        return launch_kernel(rtn_quantize_kernel<__half>, dim3(static_cast<unsigned>(blocks)), dim3(wpb * 32), 0, lc,
                             reinterpret_cast<const __half*>(w), groups, group_size, codes, scale);
    return launch_kernel(rtn_quantize_kernel<float>, dim3(static_cast<unsigned>(blocks)), dim3(wpb * 32), 0, lc,
                         reinterpret_cast<const float*>(w), groups, group_size, codes, scale);
}

}  // namespace lemoq
