// W8 rows against MANY activation vectors (batched decode and prefill: tens of tokens per call).
//
// The batch-1 kernels stream every weight row once per token.  With T tokens in flight that would read the
// weights T times; here a warp keeps a strip of 16 weight rows moving through its registers exactly once per
// block of up to 16 tokens and meets all of them on the way (weights-stationary).
//
//   1. quantise_tokens_kernel   x (T, K) fp16 -> three planes of 7-bit digits per token with one power-of-two
//      scale per group of 128: x = sx * (d2*2^14 + d1*2^7 + d0).  fp16 values within 2^9 of the group maximum
//      are exact, the rest good to 2^-20 of it.  Done once per call.
//   2. w8_tokens_mma_kernel     one warp per strip of 16 rows (gate/up mode: 8 gate rows + their 8 up rows).
//      The int8 weight codes are the A operand of mma.sync m16n8k32 s8 as they sit in memory; the B operand is
//      TWO tokens: columns (token, plane) = (0,0) (0,1) (0,2) - (1,0) (1,1) (1,2) -.  The int32 sums of a
//      128-group are exact; they are scaled by (row scale x token scale x plane weight) in fp32 and added up per
//      column, and the three columns of a token are added at the very end.  The bytes a lane loads for A and B
//      are the same permutation of k inside a 64-byte chunk, so 128-bit loads feed the fragments directly.
//      Weights come straight from global memory into registers, requested three groups ahead and bypassing L1.
//      All warps of a block work for the same expert, hence on the same tokens: the block stages the digit planes
//      of eight tokens in shared memory (the loads from L1/L2 were the kernel's limit: warps stalled on them
//      with the tensor pipe 5 % busy), every warp runs over its strip against them, then the next eight follow.
//      Segments: tokens [seg[e], seg[e+1]) use the weights of expert e (tokens sorted by expert).
//
// HBM-bound for a few tokens per expert.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace lemoq {

namespace {

constexpr int kStripWarps = 8;    // warps per block; a warp owns a strip of 16 rows
constexpr int kMaxPairs = 4;      // token pairs a warp carries through one pass over its strip
constexpr int kAhead = 3;         // groups of 128 codes a warp keeps requested ahead

// bytes of one quantised token: 3 planes x K digits, then K/128 group scales (fp32), rounded up to 16 so that every
// token starts on a 16-byte boundary (the planes are moved with 16-byte copies; K = 128 and 256 need the padding)
__host__ __device__ inline size_t token_plane_bytes(int K) {
    return (static_cast<size_t>(3) * K + static_cast<size_t>(K / 128) * 4 + 15) & ~static_cast<size_t>(15);
}

__device__ __forceinline__ void group_scale_pow2(float amax, float& sx, float& inv) {
    const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu);  // biased exponent
    if (amax > 0.f && e > 20) {
        sx = __uint_as_float(static_cast<uint32_t>(e - 19) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(254 - (e - 19)) << 23);
    } else {  // zero or denormal-range group: a fixed tiny scale keeps the arithmetic exact
        sx = __uint_as_float(static_cast<uint32_t>(2) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(252) << 23);
    }
}

// grid = T, block = K / 4 threads: a warp owns one group of 128 values, a thread four of them
__global__ void quantise_tokens_kernel(const __half* __restrict__ x, int K, uint8_t* __restrict__ planes) {
    const int t = blockIdx.x, item = threadIdx.x;
    const uint2 xv = *reinterpret_cast<const uint2*>(x + static_cast<int64_t>(t) * K + 4 * item);
    const __half* xh = reinterpret_cast<const __half*>(&xv);
    float f[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] = __half2float(xh[j]);
    float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sx, inv;
    group_scale_pow2(amax, sx, inv);
    uint32_t X[4], Y[4], Z[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        X[j] = __float_as_uint(fmaf(f[j], inv, 12582912.0f)) - 0x4B400000u;  // round to nearest even, |X| < 2^20
        Y[j] = X[j] >> 7;
        Z[j] = static_cast<uint32_t>(static_cast<int>(X[j]) >> 14);
    }
    uint8_t* tok = planes + static_cast<size_t>(t) * token_plane_bytes(K);
    uint32_t* d0 = reinterpret_cast<uint32_t*>(tok) + item;
    d0[0] = __byte_perm(__byte_perm(X[0], X[1], 0x0040), __byte_perm(X[2], X[3], 0x0040), 0x5410) & 0x7f7f7f7fu;
    d0[K / 4] = __byte_perm(__byte_perm(Y[0], Y[1], 0x0040), __byte_perm(Y[2], Y[3], 0x0040), 0x5410) & 0x7f7f7f7fu;
    d0[K / 2] = __byte_perm(__byte_perm(Z[0], Z[1], 0x0040), __byte_perm(Z[2], Z[3], 0x0040), 0x5410);
    if ((item & 31) == 0) reinterpret_cast<float*>(tok + static_cast<size_t>(3) * K)[item >> 5] = sx;
}

struct TokParams {
    const uint8_t* planes;    // (T, token_plane_bytes(K))
    const int8_t* codes;      // (E, N, K)
    const __half* scale;      // (E, N, K/group)
    const int32_t* seg;       // (E + 1) token offsets, or null: one segment [0, T)
    __half* y;                // (T, N) or, in gate/up mode, (T, N/2)
    int T, N, K, group, E, gate_up;
};

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The codes of one group of 128 of the warp's two rows per lane (rows g and g + 8 of the strip), and the rows'
// group scales.  A lane holds bytes [16q, 16q + 16) of each 64-byte chunk, q = lane & 3.
struct GroupRegs {
    uint4 lo[2], hi[2];  // [chunk of 64]: row g, row g + 8
    float ws_lo, ws_hi;
};

// What a lane knows about its strip and its columns.
struct Lane {
    const int8_t* w_lo;      // codes of row g of the strip, at byte 16q
    const int8_t* w_hi;      // codes of row g + 8
    const __half* s_lo;      // group scales of the two rows
    const __half* s_hi;
    uint32_t b_smem;         // shared address of this lane's plane row of token col_tok of pair 0, at byte 16q
    uint32_t b_zero;         // shared address of the row of zeros, at byte 16q
    uint32_t sx_smem;        // shared address of the group scales of token res_tok of pair 0
    uint32_t pair_stride;    // bytes between the plane rows of consecutive pairs (two tokens)
    uint32_t sx_pair_stride;
    int group;               // weight group size
    int col_tok;             // token of the pair whose (token, plane) column this lane feeds to B
    bool col_on;             // false: padding column
    float pw0, pw1;          // plane weights of the lane's two result columns
};

__device__ __forceinline__ void load_group(const Lane& L, GroupRegs& r, int grp) {
    const int k0 = grp << 7;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        r.lo[c] = ld_stream16(L.w_lo + k0 + 64 * c);
        r.hi[c] = ld_stream16(L.w_hi + k0 + 64 * c);
    }
    const int sg = k0 / L.group;
    r.ws_lo = __half2float(__ldg(L.s_lo + sg));
    r.ws_hi = __half2float(__ldg(L.s_hi + sg));
}

__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// One pass of a warp over the ngroups groups of its strip against the npairs token pairs staged in shared memory
// (ntok tokens; the second token of the last pair may be missing).  `ring` holds the first kAhead groups already.
// Pairs are taken two at a time: their loads, two independent chains of four MMAs, their fp32 updates.
__device__ __forceinline__ void strip_pass(const Lane& L, GroupRegs (&ring)[kAhead], int ngroups, int npairs, int ntok,
                                           float (&acc)[kMaxPairs][4]) {
    uint32_t b_addr[kMaxPairs], sx_addr[kMaxPairs];
#pragma unroll
    for (int pr = 0; pr < kMaxPairs; ++pr) {  // the padding column and a missing token read the row of zeros
        b_addr[pr] = L.col_on && 2 * pr + L.col_tok < ntok ? L.b_smem + pr * L.pair_stride : L.b_zero;
        sx_addr[pr] = L.sx_smem + pr * L.sx_pair_stride;
    }
    for (int grp0 = 0; grp0 < ngroups; grp0 += kAhead) {
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
            const int grp = grp0 + i;
            if (grp < ngroups) {
                const uint32_t koff = static_cast<uint32_t>(grp) << 7;
                const float f_lo0 = ring[i].ws_lo * L.pw0, f_lo1 = ring[i].ws_lo * L.pw1;
                const float f_hi0 = ring[i].ws_hi * L.pw0, f_hi1 = ring[i].ws_hi * L.pw1;
#pragma unroll
                for (int pb = 0; pb < kMaxPairs; pb += 2) {
                    if (pb < npairs) {  // warp-uniform
                        uint4 b[2][2];
                        float sx[2];
                        int c4[2][4];
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
#pragma unroll
                            for (int c = 0; c < 2; ++c) b[u][c] = lds_u128(b_addr[pb + u] + koff + 64 * c);
                            sx[u] = lds_f32(sx_addr[pb + u] + 4 * grp);
                            c4[u][0] = c4[u][1] = c4[u][2] = c4[u][3] = 0;
                        }
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
#pragma unroll
                            for (int u = 0; u < 2; ++u) mma_s8(c4[u], ring[i].lo[c].x, ring[i].hi[c].x, ring[i].lo[c].y, ring[i].hi[c].y, b[u][c].x, b[u][c].y);
#pragma unroll
                            for (int u = 0; u < 2; ++u) mma_s8(c4[u], ring[i].lo[c].z, ring[i].hi[c].z, ring[i].lo[c].w, ring[i].hi[c].w, b[u][c].z, b[u][c].w);
                        }
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            acc[pb + u][0] = fmaf(static_cast<float>(c4[u][0]), f_lo0 * sx[u], acc[pb + u][0]);
                            acc[pb + u][1] = fmaf(static_cast<float>(c4[u][1]), f_lo1 * sx[u], acc[pb + u][1]);
                            acc[pb + u][2] = fmaf(static_cast<float>(c4[u][2]), f_hi0 * sx[u], acc[pb + u][2]);
                            acc[pb + u][3] = fmaf(static_cast<float>(c4[u][3]), f_hi1 * sx[u], acc[pb + u][3]);
                        }
                    }
                }
                if (grp + kAhead < ngroups) load_group(L, ring[i], grp + kAhead);  // the slot is free again
            }
        }
    }
}

// Shared memory of a block: the digit planes of up to 2 * kMaxPairs tokens, rows [token][plane] of K + 64 bytes (the
// 64 bytes keep the 128-bit loads of a quarter warp on different banks), one row of zeros (what the padding column and a
// missing token read), then the tokens' group scales.
__host__ __device__ inline size_t stage_row_bytes(int K) { return static_cast<size_t>(K) + 64; }
__host__ __device__ inline size_t stage_bytes(int K) {
    return static_cast<size_t>(2 * kMaxPairs * 3 + 1) * stage_row_bytes(K) + static_cast<size_t>(2 * kMaxPairs) * (K / 128) * 4;
}

// grid = (token chunks, ceil(strips / kStripWarps), E), block = kStripWarps warps.  All warps of a block work for the
// same expert, hence on the same tokens: the block stages the planes of 2 * kMaxPairs tokens in shared memory, every
// warp runs over its strip against them, and the next tokens follow.  tok_chunk > 0 (dense linears with few rows)
// gives each block only tok_chunk of the tokens, so that more warps stream at the same time; the blocks that
// share rows are neighbours in the grid and meet in L2.
__global__ void __launch_bounds__(kStripWarps * 32, 2) w8_tokens_mma_kernel(const TokParams p, const int tok_chunk) {
    extern __shared__ __align__(16) uint8_t stage[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int e = blockIdx.z;
    int t0 = p.seg ? p.seg[e] : 0, t1 = p.seg ? p.seg[e + 1] : p.T;
    if (tok_chunk > 0) {
        t0 += static_cast<int>(blockIdx.x) * tok_chunk;
        t1 = min(t1, t0 + tok_chunk);
    }
    if (t1 <= t0) return;  // the whole block: every warp of a block has the same tokens
    const int half_rows = p.N / 2;
    const int strips = p.gate_up ? (half_rows + 7) / 8 : (p.N + 15) / 16;
    const int strip = blockIdx.y * kStripWarps + warp;
    const bool live = strip < strips;
    // the two rows of this lane; rows beyond the end are read as the last row and never stored
    const int out_lo = p.gate_up ? strip * 8 + g : strip * 16 + g;        // gate row n       | row
    const int out_hi = p.gate_up ? out_lo : out_lo + 8;                   // (same n)         | row + 8
    const int lim = p.gate_up ? half_rows : p.N;
    const int row_lo = max(0, min(out_lo, lim - 1)), row_hi = p.gate_up ? half_rows + row_lo : max(0, min(out_hi, lim - 1));
    const int ngroups = p.K >> 7, gK = p.K / p.group;
    const int64_t base = static_cast<int64_t>(e) * p.N;
    const uint32_t row_bytes = static_cast<uint32_t>(stage_row_bytes(p.K));
    const uint32_t stage_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(stage));
    const uint32_t zero_row = stage_u32 + static_cast<uint32_t>(2 * kMaxPairs * 3) * row_bytes;
    float* sx_stage = reinterpret_cast<float*>(stage + static_cast<size_t>(2 * kMaxPairs * 3 + 1) * row_bytes);
    for (uint32_t u = threadIdx.x * 16; u < row_bytes; u += blockDim.x * 16) *reinterpret_cast<uint4*>(stage + static_cast<size_t>(2 * kMaxPairs * 3) * row_bytes + u) = make_uint4(0, 0, 0, 0);
    Lane L;
    L.w_lo = p.codes + (base + row_lo) * p.K + 16 * q;
    L.w_hi = p.codes + (base + row_hi) * p.K + 16 * q;
    L.s_lo = p.scale + (base + row_lo) * gK;
    L.s_hi = p.scale + (base + row_hi) * gK;
    // B operand: column lane >> 2 = (token (lane >> 4) of the pair, plane (lane >> 2) & 3); plane 3 is padding
    L.col_tok = lane >> 4;
    L.col_on = (g & 3) < 3;
    L.b_smem = stage_u32 + (static_cast<uint32_t>(L.col_tok) * 3 + static_cast<uint32_t>(min(g & 3, 2))) * row_bytes + 16 * q;
    L.b_zero = zero_row + 64 + 16 * q;  // + 64: other banks than the plane row the neighbouring lanes read
    L.pair_stride = 6 * row_bytes;
    // result columns 2q and 2q + 1: token q >> 1 of the pair, planes 2 * (q & 1) and 2 * (q & 1) + 1
    L.sx_smem = static_cast<uint32_t>(__cvta_generic_to_shared(sx_stage)) + static_cast<uint32_t>(q >> 1) * ngroups * 4;
    L.sx_pair_stride = 2 * ngroups * 4;
    L.group = p.group;
    L.pw0 = (q & 1) ? 16384.f : 1.f;
    L.pw1 = (q & 1) ? 0.f : 128.f;
    const size_t tok_bytes = token_plane_bytes(p.K);
    const int units = p.K >> 4;  // 16-byte units of a plane row

    GroupRegs ring[kAhead];
    for (int tb = t0; tb < t1; tb += 2 * kMaxPairs) {
        const int ntok = min(2 * kMaxPairs, t1 - tb), npairs = (ntok + 1) >> 1;  // block-uniform
        // the first groups of the strip are requested before the tokens are staged: both latencies overlap
        if (live) {
#pragma unroll
            for (int i = 0; i < kAhead; ++i)
                if (i < ngroups) load_group(L, ring[i], i);
        }
        __syncthreads();  // the previous tokens have been consumed
        for (int u = threadIdx.x; u < ntok * 3 * units; u += blockDim.x) {
            const int r = u / units, c = u - r * units, t = r / 3;  // r = token * 3 + plane
            cp_async16(stage_u32 + static_cast<uint32_t>(r) * row_bytes + 16 * c,
                       p.planes + static_cast<size_t>(tb + t) * tok_bytes + static_cast<size_t>(r - 3 * t) * p.K + 16 * c);
        }
        for (int u = threadIdx.x; u < ntok * ngroups; u += blockDim.x) {
            const int t = u / ngroups;
            sx_stage[u] = __ldg(reinterpret_cast<const float*>(p.planes + static_cast<size_t>(tb + t) * tok_bytes + static_cast<size_t>(3) * p.K) + (u - t * ngroups));
        }
        // a missing second token of the last pair: its scales are read (and multiplied by zero sums)
        if ((ntok & 1) && threadIdx.x < ngroups) sx_stage[ntok * ngroups + threadIdx.x] = 0.f;
        cp_async_wait_all();
        __syncthreads();
        if (!live) continue;  // took part in the staging only
        float acc[kMaxPairs][4];
#pragma unroll
        for (int i = 0; i < kMaxPairs; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        strip_pass(L, ring, ngroups, npairs, ntok, acc);
        // planes of a token: two columns in this lane, the third (and the padding) in the lane next to it
#pragma unroll
        for (int pr = 0; pr < kMaxPairs; ++pr) {
            if (pr < npairs) {  // warp-uniform
                float v_lo = acc[pr][0] + acc[pr][1], v_hi = acc[pr][2] + acc[pr][3];
                v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 1);
                v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 1);
                const int tok = tb + 2 * pr + (q >> 1);
                if ((q & 1) == 0 && tok < t1) {
                    if (p.gate_up) {
                        if (out_lo < half_rows)
                            p.y[static_cast<int64_t>(tok) * half_rows + out_lo] = __float2half_rn(v_lo * (1.0f / (1.0f + expf(-v_lo))) * v_hi);
                    } else {
                        if (out_lo < p.N) p.y[static_cast<int64_t>(tok) * p.N + out_lo] = __float2half_rn(v_lo);
                        if (out_hi < p.N) p.y[static_cast<int64_t>(tok) * p.N + out_hi] = __float2half_rn(v_hi);
                    }
                }
            }
        }
    }
}

}  // namespace
}  // namespace lemoq

using namespace lemoq;

extern "C" size_t lemoq_w8_token_planes_bytes(int T, int K) {
    if (T <= 0 || K <= 0 || K % 128 != 0) return 0;
    return static_cast<size_t>(T) * token_plane_bytes(K);
}

extern "C" int lemoq_w8_quantise_tokens(const void* x, int T, int K, void* planes, void* stream) {
    LEMOQ_REQUIRE(T >= 0 && K > 0, LEMOQ_ERR_INVALID, "w8_quantise_tokens: bad shape");
    LEMOQ_REQUIRE(K % 128 == 0 && K <= 4096, LEMOQ_ERR_UNSUPPORTED, "w8_quantise_tokens: K=%d must be a multiple of 128, <= 4096", K);
    if (T == 0) return LEMOQ_OK;
    LEMOQ_REQUIRE(x && planes && aligned16(x) && aligned16(planes), LEMOQ_ERR_INVALID, "w8_quantise_tokens: null or unaligned pointer");
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    return launch_kernel(quantise_tokens_kernel, dim3(T), dim3(K / 4), 0, lc, reinterpret_cast<const __half*>(x), K,
                         reinterpret_cast<uint8_t*>(planes));
}

extern "C" int lemoq_w8_rows_tokens(const void* planes, int T, const int8_t* codes, const void* scale, int N, int K, int group_size,
                                    const int32_t* seg_offsets, int E, int gate_up, void* y, void* stream) {
    LEMOQ_REQUIRE(T >= 0 && N > 0 && K > 0 && E >= 1, LEMOQ_ERR_INVALID, "w8_rows_tokens: bad shape");
    LEMOQ_REQUIRE(N % 2 == 0, LEMOQ_ERR_UNSUPPORTED, "w8_rows_tokens: N=%d must be even", N);
    LEMOQ_REQUIRE(K % 128 == 0 && K <= 4096, LEMOQ_ERR_UNSUPPORTED, "w8_rows_tokens: K=%d must be a multiple of 128, <= 4096", K);
    LEMOQ_REQUIRE(group_size > 0 && K % group_size == 0, LEMOQ_ERR_INVALID, "w8_rows_tokens: bad group_size %d", group_size);
    LEMOQ_REQUIRE(group_size % 128 == 0, LEMOQ_ERR_UNSUPPORTED, "w8_rows_tokens: group_size=%d must be a multiple of 128", group_size);
    LEMOQ_REQUIRE(E == 1 || seg_offsets, LEMOQ_ERR_INVALID, "w8_rows_tokens: several experts need segment offsets");
    if (T == 0) return LEMOQ_OK;
    LEMOQ_REQUIRE(planes && codes && scale && y && aligned16(planes) && aligned16(codes), LEMOQ_ERR_INVALID,
                  "w8_rows_tokens: null or unaligned pointer");
    TokParams p;
    p.planes = reinterpret_cast<const uint8_t*>(planes);
    p.codes = codes;
    p.scale = reinterpret_cast<const __half*>(scale);
    p.seg = seg_offsets;
    p.y = reinterpret_cast<__half*>(y);
    p.T = T; p.N = N; p.K = K; p.group = group_size; p.E = E; p.gate_up = gate_up ? 1 : 0;
    const int strips = gate_up ? (N / 2 + 7) / 8 : (N + 15) / 16;
    // a dense linear with few strips: give every block only a part of the tokens, so that the machine has enough
    // warps streaming (148 SMs x 8 and more); with experts the tokens of a block are its expert's segment
    int tok_chunk = 0, chunks = 1;
    if (E == 1) {
        const int want = (148 * 8 + strips - 1) / strips;                   // blocks wanted per strip
        chunks = std::min(std::max(want, (T + 2 * kMaxPairs - 1) / (2 * kMaxPairs)), (T + 1) / 2);  // and one pass per block
        tok_chunk = ((T + chunks - 1) / chunks + 1) & ~1;                 // even: tokens travel in pairs
        chunks = (T + tok_chunk - 1) / tok_chunk;
    }
    dim3 grid(chunks, (strips + kStripWarps - 1) / kStripWarps, E), block(kStripWarps * 32);
    const size_t smem = stage_bytes(K);
    {  // per device and idempotent; not a stream operation, so legal under capture
        const cudaError_t err = cudaFuncSetAttribute(w8_tokens_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(stage_bytes(4096)));
        if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(err));
    }
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    return launch_kernel(w8_tokens_mma_kernel, grid, block, smem, lc, p, tok_chunk);
}
