// W8 rows against MANY activation vectors (batched decode: tens of tokens per step).
//
// The batch-1 kernels stream every weight row once per token.  With T tokens in flight that would read
// the weights T times; here a warp keeps its two weight rows in registers and walks all the tokens of its
// segment, so every weight byte is read from memory once per call whatever T is (weights-stationary).
//
//   1. quantise_tokens_kernel   x (T, K) fp16 -> digit planes: per 16-element chunk a power-of-two scale sx
//      and three planes of 7-bit digits, x = sx * (d2*2^14 + d1*2^7 + d0) (fp16 values within 2^9 of the
//      chunk maximum are exact, the rest good to 2^-20 of it).  Done once per call, not once per block.
//   2. w8_tokens_kernel         block = 8 warps x 2 rows; token tiles of 8 are staged in shared memory and
//      shared by the block's warps; int8 codes meet the planes in dp4a (exact int32 partial sums), fp32
//      combine and scale, fp16 result.  Segments: tokens [seg[e], seg[e+1]) use the weights of expert e
//      (tokens sorted by expert), so a resident expert's rows are read once for all its tokens.
//      Modes: plain rows (dense linears, expert down) and gate/up with the SwiGLU epilogue.
//
// HBM/L2-bound integer work on CUDA cores; no tensor cores.
#include "common.cuh"
#include "kernels.h"

namespace lemoq {

namespace {

constexpr int kTokTile = 8;     // tokens staged per tile
constexpr int kRowWarps = 8;    // warps per block, two rows each
constexpr int kMaxChunks = 4;   // K <= 2048

// words of one quantised token: 3 planes x (K/16) lane chunks x 4 words, then K/16 chunk scales
__host__ __device__ inline int plane_words(int K) { return 3 * (K / 16) * 4 + K / 16; }

__device__ __forceinline__ void chunk_scale_pow2(float amax, float& sx, float& inv) {
    const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu);
    if (amax > 0.f && e > 20) {
        sx = __uint_as_float(static_cast<uint32_t>(e - 19) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(254 - (e - 19)) << 23);
    } else {
        sx = __uint_as_float(static_cast<uint32_t>(2) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(252) << 23);
    }
}

// grid = T, block = K / 4 threads (four consecutive threads share a 16-element chunk)
__global__ void quantise_tokens_kernel(const __half* __restrict__ x, int K, uint32_t* __restrict__ planes) {
    const int t = blockIdx.x, item = threadIdx.x;
    const int nlc = K / 16;
    const uint2 xv = *reinterpret_cast<const uint2*>(x + static_cast<int64_t>(t) * K + 4 * item);
    const __half* xh = reinterpret_cast<const __half*>(&xv);
    float f[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] = __half2float(xh[j]);
    float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float sx, inv;
    chunk_scale_pow2(amax, sx, inv);
    uint32_t X[4], Y[4], Z[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        X[j] = __float_as_uint(fmaf(f[j], inv, 12582912.0f)) - 0x4B400000u;  // round to nearest even, |X| < 2^20
        Y[j] = X[j] >> 7;
        Z[j] = static_cast<uint32_t>(static_cast<int>(X[j]) >> 14);
    }
    uint32_t* dst = planes + static_cast<int64_t>(t) * plane_words(K);
    const int lc = item >> 2, w = item & 3;
    dst[(0 * nlc + lc) * 4 + w] = __byte_perm(__byte_perm(X[0], X[1], 0x0040), __byte_perm(X[2], X[3], 0x0040), 0x5410) & 0x7f7f7f7fu;
    dst[(1 * nlc + lc) * 4 + w] = __byte_perm(__byte_perm(Y[0], Y[1], 0x0040), __byte_perm(Y[2], Y[3], 0x0040), 0x5410) & 0x7f7f7f7fu;
    dst[(2 * nlc + lc) * 4 + w] = __byte_perm(__byte_perm(Z[0], Z[1], 0x0040), __byte_perm(Z[2], Z[3], 0x0040), 0x5410);
    if (w == 0) reinterpret_cast<float*>(dst + 3 * nlc * 4)[lc] = sx;
}

struct TokParams {
    const uint32_t* planes;   // (T, plane_words(K))
    const int8_t* codes;      // (E, N, K)
    const __half* scale;      // (E, N, K/group)
    const int32_t* seg;       // (E + 1) token offsets, or null: one segment [0, T)
    __half* y;                // (T, N) or, in gate/up mode, (T, N/2)
    int T, N, K, group, E, gate_up;
};

// Sixteen per-lane partial sums -> sixteen warp totals with 16 shuffles: every round halves the values a
// lane carries and doubles the lanes that agree.  Afterwards lane L holds the total of value
// ((L>>4)&1)*8 + ((L>>3)&1)*4 + ((L>>2)&1)*2 + ((L>>1)&1) (both lanes of an even/odd pair hold the same).
__device__ __forceinline__ float warp_reduce16(float (&v)[16], int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const bool up = (lane & 16) != 0;
        const float keep = up ? v[i + 8] : v[i], give = up ? v[i] : v[i + 8];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const bool up = (lane & 8) != 0;
        const float keep = up ? v[i + 4] : v[i], give = up ? v[i] : v[i + 4];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const bool up = (lane & 4) != 0;
        const float keep = up ? v[i + 2] : v[i], give = up ? v[i] : v[i + 2];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, give, 4);
    }
    {
        const bool up = (lane & 2) != 0;
        const float keep = up ? v[1] : v[0], give = up ? v[0] : v[1];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, give, 2);
    }
    return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}

// grid = (ceil(row pairs / kRowWarps), E); dynamic smem = kTokTile * plane_words(K) * 4 bytes.
// One row pair per warp: its weights stay in registers while the warp walks all token tiles of the segment.
// (A variant that kept the token tile and walked eight row pairs per warp was slower for the experts: the
// serial weight loads of a warp are not hidden, thousands of small blocks hide them better.)
template <int NCH>
__global__ void __launch_bounds__(kRowWarps * 32) w8_tokens_kernel(const TokParams p) {
    extern __shared__ __align__(16) uint32_t tile[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.y;
    const int t0 = p.seg ? p.seg[e] : 0, t1 = p.seg ? p.seg[e + 1] : p.T;
    if (t1 <= t0) return;
    const int pairs = p.N / 2;
    const int nlc = p.K / 16, gK = p.K / p.group, pw = plane_words(p.K);
    const int64_t base = static_cast<int64_t>(e) * p.N;
    uint4 w[2][NCH];
    float sc[2][NCH];
    auto load_rows = [&](int pair) {
        // rows of the pair: (2i, 2i+1), or (n, N/2 + n) when the gate and the up row meet in the SwiGLU epilogue
        const int r0 = p.gate_up ? pair : 2 * pair, r1 = p.gate_up ? pairs + pair : 2 * pair + 1;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int lc = c * 32 + lane;
            const bool on = pair < pairs && lc < nlc;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int64_t row = base + (r == 0 ? r0 : r1);
                w[r][c] = on ? ld_stream16(p.codes + row * p.K + lc * 16) : make_uint4(0, 0, 0, 0);
                sc[r][c] = on ? __half2float(p.scale[row * gK + (lc * 16) / p.group]) : 0.f;
            }
        }
    };
    auto stage_tile = [&](int tb, int nt) {
        __syncthreads();  // the previous tile has been consumed
        const uint4* src = reinterpret_cast<const uint4*>(p.planes + static_cast<int64_t>(tb) * pw);
        uint4* dst = reinterpret_cast<uint4*>(tile);
        for (int i = threadIdx.x; i < nt * pw / 4; i += blockDim.x) dst[i] = __ldg(src + i);
        __syncthreads();
    };
    auto compute_tile = [&](int pair, int tb, int nt) {
        float acc[16];  // [token][row]
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll
        for (int tt = 0; tt < kTokTile; ++tt) {
            if (tt < nt) {
                const uint32_t* xq = tile + tt * pw;
                const float* sxs = reinterpret_cast<const float*>(xq + 3 * nlc * 4);
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const int lc = c * 32 + lane;
                    if (lc < nlc) {
                        const uint4 x0 = *reinterpret_cast<const uint4*>(xq + (0 * nlc + lc) * 4);
                        const uint4 x1 = *reinterpret_cast<const uint4*>(xq + (1 * nlc + lc) * 4);
                        const uint4 x2 = *reinterpret_cast<const uint4*>(xq + (2 * nlc + lc) * 4);
                        const float sx = sxs[lc];
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const uint4 ww = w[r][c];
                            int s0 = __dp4a(static_cast<int>(ww.x), static_cast<int>(x0.x), 0);
                            int s1 = __dp4a(static_cast<int>(ww.x), static_cast<int>(x1.x), 0);
                            int s2 = __dp4a(static_cast<int>(ww.x), static_cast<int>(x2.x), 0);
                            s0 = __dp4a(static_cast<int>(ww.y), static_cast<int>(x0.y), s0);
                            s1 = __dp4a(static_cast<int>(ww.y), static_cast<int>(x1.y), s1);
                            s2 = __dp4a(static_cast<int>(ww.y), static_cast<int>(x2.y), s2);
                            s0 = __dp4a(static_cast<int>(ww.z), static_cast<int>(x0.z), s0);
                            s1 = __dp4a(static_cast<int>(ww.z), static_cast<int>(x1.z), s1);
                            s2 = __dp4a(static_cast<int>(ww.z), static_cast<int>(x2.z), s2);
                            s0 = __dp4a(static_cast<int>(ww.w), static_cast<int>(x0.w), s0);
                            s1 = __dp4a(static_cast<int>(ww.w), static_cast<int>(x1.w), s1);
                            s2 = __dp4a(static_cast<int>(ww.w), static_cast<int>(x2.w), s2);
                            const float tsum = fmaf(static_cast<float>(s2), 16384.f, fmaf(static_cast<float>(s1), 128.f, static_cast<float>(s0)));
                            acc[2 * tt + r] = fmaf(tsum, sx * sc[r][c], acc[2 * tt + r]);
                        }
                    }
                }
            }
        }
        const float total = warp_reduce16(acc, lane);
        // this lane's value: token tt, row r
        const int idx = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
        const int tt = idx >> 1, r = idx & 1;
        // gate (r = 0) and up (r = 1) of one token sit in lanes that differ in bit 1 (every lane takes part)
        const float other = __shfl_xor_sync(0xffffffffu, total, 2);
        if (pair < pairs && tt < nt && (lane & 1) == 0) {
            const int64_t tok = tb + tt;
            if (p.gate_up) {
                if (r == 0) p.y[tok * pairs + pair] = __float2half_rn(total * (1.0f / (1.0f + expf(-total))) * other);
            } else {
                p.y[tok * p.N + (r == 0 ? 2 * pair : 2 * pair + 1)] = __float2half_rn(total);
            }
        }
    };
    const int pair = blockIdx.x * kRowWarps + warp;
    load_rows(pair);
    for (int tb = t0; tb < t1; tb += kTokTile) {
        const int nt = min(kTokTile, t1 - tb);
        stage_tile(tb, nt);
        compute_tile(pair, tb, nt);
    }
}

}  // namespace
}  // namespace lemoq

using namespace lemoq;

extern "C" size_t lemoq_w8_token_planes_bytes(int T, int K) {
    if (T <= 0 || K <= 0 || K % 16 != 0) return 0;
    return static_cast<size_t>(T) * plane_words(K) * sizeof(uint32_t);
}

extern "C" int lemoq_w8_quantise_tokens(const void* x, int T, int K, void* planes, void* stream) {
    LEMOQ_REQUIRE(T >= 0 && K > 0, LEMOQ_ERR_INVALID, "w8_quantise_tokens: bad shape");
    LEMOQ_REQUIRE(K % 128 == 0 && K <= 2048 * 2, LEMOQ_ERR_UNSUPPORTED, "w8_quantise_tokens: K=%d must be a multiple of 128, <= 4096", K);
    if (T == 0) return LEMOQ_OK;
    LEMOQ_REQUIRE(x && planes && aligned16(x) && aligned16(planes), LEMOQ_ERR_INVALID, "w8_quantise_tokens: null or unaligned pointer");
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    return launch_kernel(quantise_tokens_kernel, dim3(T), dim3(K / 4), 0, lc, reinterpret_cast<const __half*>(x), K,
                         reinterpret_cast<uint32_t*>(planes));
}

extern "C" int lemoq_w8_rows_tokens(const void* planes, int T, const int8_t* codes, const void* scale, int N, int K, int group_size,
                                    const int32_t* seg_offsets, int E, int gate_up, void* y, void* stream) {
    LEMOQ_REQUIRE(T >= 0 && N > 0 && K > 0 && E >= 1, LEMOQ_ERR_INVALID, "w8_rows_tokens: bad shape");
    LEMOQ_REQUIRE(N % 2 == 0, LEMOQ_ERR_UNSUPPORTED, "w8_rows_tokens: N=%d must be even", N);
    LEMOQ_REQUIRE(K % 512 == 0 && K <= 512 * kMaxChunks, LEMOQ_ERR_UNSUPPORTED, "w8_rows_tokens: K=%d must be a multiple of 512, <= 2048", K);
    LEMOQ_REQUIRE(group_size > 0 && group_size % 16 == 0 && K % group_size == 0, LEMOQ_ERR_INVALID, "w8_rows_tokens: bad group_size %d", group_size);
    LEMOQ_REQUIRE(E == 1 || seg_offsets, LEMOQ_ERR_INVALID, "w8_rows_tokens: several experts need segment offsets");
    if (T == 0) return LEMOQ_OK;
    LEMOQ_REQUIRE(planes && codes && scale && y && aligned16(planes) && aligned16(codes), LEMOQ_ERR_INVALID,
                  "w8_rows_tokens: null or unaligned pointer");
    TokParams p;
    p.planes = reinterpret_cast<const uint32_t*>(planes);
    p.codes = codes;
    p.scale = reinterpret_cast<const __half*>(scale);
    p.seg = seg_offsets;
    p.y = reinterpret_cast<__half*>(y);
    p.T = T; p.N = N; p.K = K; p.group = group_size; p.E = E; p.gate_up = gate_up ? 1 : 0;
    const int pairs = N / 2;
    dim3 grid((pairs + kRowWarps - 1) / kRowWarps, E), block(kRowWarps * 32);
    const size_t smem = static_cast<size_t>(kTokTile) * plane_words(K) * sizeof(uint32_t);
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    const int nch = K / 512;
#define LEMOQ_TOK_CASE(NCHV)                                                                                          \
    case NCHV: {                                                                                                      \
        if (smem > 48 * 1024) {                                                                                       \
            const cudaError_t err = cudaFuncSetAttribute(w8_tokens_kernel<NCHV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(err)); \
        }                                                                                                             \
        return launch_kernel(w8_tokens_kernel<NCHV>, grid, block, smem, lc, p);                                       \
    }
    switch (nch) {
        LEMOQ_TOK_CASE(1)
        LEMOQ_TOK_CASE(2)
        LEMOQ_TOK_CASE(3)
        LEMOQ_TOK_CASE(4)
        default: break;
    }
#undef LEMOQ_TOK_CASE
    return set_error(LEMOQ_ERR_UNSUPPORTED, "w8_rows_tokens: K=%d", K);
}
