// The whole decode step as ONE persistent cooperative kernel, built on 8-row weight tiles and the
// int8 tensor-core dot product.
//
// One block per SM stays resident for the whole step.  All weights move as TILES: 8 whole rows and the rows'
// group scales, brought into a 16.9 KB shared-memory stage by three to six bulk asynchronous copies, each issued by
// a lane of its own: the codes in runs of four rows (adjacent in memory; every run lands 64 bytes further than its
// natural place, so that the 16-byte reads of rows r and r + 4, which one request of a quarter warp combines, hit
// different banks), the scales in one or two runs.  The block has ten stages.  Ten CONSUMER warps own one stage
// each and do all the arithmetic; five PRODUCER warps do nothing but issue copies: each keeps two stages filled,
// walking the block's tile sequence of the WHOLE STEP in order (a copy instruction occupies the issuing warp for
// well over a thousand cycles, which is why the consumers do not issue their own).  A stage is handed back and
// forth through a full/empty pair of shared-memory barriers.  The producers run ahead across phases and layers:
// q.k.v, KV-cache, o_proj, router and lm_head tiles do not depend on activations, so they land while the
// consumers still work on the phase before; only the expert tiles wait, on the block's own top-k.
//
// Between phases the blocks exchange small vectors (the residual stream, q.k.v, router logits, the SwiGLU
// activations) through global memory as flagged 8-byte words that the readers poll, see "flagged words" below.
// The one place where every block needs everything every other block wrote in bulk - the attention partials
// before o_proj - is a grid barrier: one per layer, plus one at the end of the step.
//
// Arithmetic: the activation vector of a phase is turned once per block into three planes of signed
// 7-bit digits with one power-of-two scale per group of 128 (x = sx * (d2*2^14 + d1*2^7 + d0)).  The
// planes are the B operand of mma.sync m16n8k32 s8, the int8 weight codes are the A operand as they
// sit in memory.  The 16 rows of the instruction are the 8 rows of the tile, twice (instruction row g is tile row
// g/2 + 4 (g mod 2)): rows 0-7 take the first half of k, rows 8-15 the second half, and B carries the planes of
// the first half in columns 0-2 and those of the second half in columns 3-5.  One instruction thus multiplies 8 rows x 64 codes;
// the int32 sums of a 128-group are exact and are scaled by (row scale x sx) in fp32.  The bytes a
// lane loads for A and B are a permutation of k inside a 64-byte chunk, the same on both sides, so
// 128-bit shared loads feed the fragments directly.  The router rows (fp16) go through mma.sync
// m16n8k16 f16 the same way: 4 rows x 4 quarters of k, the fp16 activations of the quarters in
// columns 0-3.
//
// A warp finishes the rows of its tile by itself (fp16 rounding, residual add, SwiGLU of a tile of
// 4 gate + 4 up rows); only the expert down rows, whose eight routed experts are eight tiles, leave
// partial sums in shared memory that the block adds in slot order.  No atomics on data: results are
// bit-identical run to run.
//
// Phases per layer (what a block waits for -> what it publishes):
//   A  q.k.v tiles          flagged x of the layer before; planes of RMSNorm(x)   -> flagged qkv + sum-of-squares partials
//   B  attention            flagged qkv; one (head, split) per block, KV tiles of 16, 32 or 64 positions through the
//                           same stages; q/k norm + RoPE + KV row write fused     -> (m, l, acc) partial per unit
//      grid barrier
//   C  o_proj tiles         splits of each head merged while the planes are built; + residual -> flagged x1
//   D  router tiles (fp16)  flagged x1; planes of h2 = RMSNorm(x1) stay in shared memory for E -> flagged logits
//   E  expert gate/up       flagged logits; one warp per block derives the top-k; SwiGLU -> flagged act
//   F  expert down          flagged act; routing-weighted sum + residual          -> flagged x2
// then the lm_head tiles on RMSNorm(x2) as the q.k.v tiles of a pseudo layer, with the greedy pick.
#include <algorithm>
#include <cstddef>
#include <cstdio>
#include <cstdlib>

#include "step_kernel.h"
#include "stream.cuh"

namespace lemoq {
namespace tile {

constexpr int kStreamWarps = 10;        // consumer warps: one stage each, they do all the arithmetic
constexpr int kProducerWarps = 5;       // producer warps: each keeps two stages filled, nothing else
constexpr int kWarps = kStreamWarps;    // warps that take part in the block-wide work of a phase
constexpr int kConsumerThreads = kStreamWarps * 32;
constexpr int kThreads = (kStreamWarps + kProducerWarps) * 32;
constexpr int kPad = 64;                // plane segments and vector quarters sit 64 bytes off their natural stride
constexpr int kRunPad = 64;             // every run of four code rows of a tile sits this much further than the one before
constexpr int kScaleOff = 8 * 2048 + 256;  // the group scales of a tile sit behind its rows (at most four runs)
constexpr int kStageBytes = kScaleOff + 256;
constexpr int kKvTile = 64;             // cached positions per attention tile
constexpr int kMaxLayers = 33;
constexpr int kMaxSplits = 9;
constexpr int kHeadDim = 128;
constexpr int kQPlaneStride = kHeadDim + kPad;
constexpr int kPartFloats = 1024;       // partial sums of the down phase (8 per tile)
constexpr uint32_t kBarrierSpinLimit = 1u << 24;

enum Kind : int { KA = 0, KB = 1, KC = 2, KD = 3, KE = 4, KF = 5, KEND = 6 };

// ---------------------------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint2 ld_cg8(const void* p) {
    uint2 v;
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
// ---- flagged words: how the blocks hand small vectors to each other without a grid barrier --------------------
// A value travels as one 8-byte word {32 bits of data, 32-bit tag}; the tag is the sequence number of the layer
// (unique over launches).  8-byte accesses are single-copy atomic, so a reader that sees the tag it waits for (or
// a later one) holds the data that was stored with it: it polls the very words it needs and starts as soon as
// they are there - one memory round trip behind the producer's store, where a barrier costs an arrival, a poll
// and then the load.  Buffers alternate with the layer's parity; the one grid barrier per layer that remains
// (attention -> o_proj) keeps every block within one layer of every other, so no word is overwritten while
// somebody still waits for its previous content.
constexpr uint32_t kFlagSpinLimit = 1u << 21;  // default of the limit below
// Polls of a flagged word before a wait gives up (raising LEMOQ_FLAG_WAIT_TIMEOUT; the step then goes on with what the
// word held).  lemoq_set_tuning key 5 changes it on the current device: the time-out path can be tested by making it 1.
__constant__ uint32_t c_flag_spin_limit = kFlagSpinLimit;
__device__ __forceinline__ void flag_store(unsigned long long* p, uint32_t data, uint32_t tag) {
    const unsigned long long w = (static_cast<unsigned long long>(tag) << 32) | data;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long flag_load(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
// Four neighbouring words in one request: a whole 32-byte sector instead of four requests for a quarter of it each
// (every word is still its own single-copy atomic access).  32-byte aligned.
__device__ __forceinline__ void flag_load4(const unsigned long long* p, unsigned long long (&w)[4]) {
    asm volatile("ld.relaxed.gpu.global.v4.u64 {%0, %1, %2, %3}, [%4];" : "=l"(w[0]), "=l"(w[1]), "=l"(w[2]), "=l"(w[3]) : "l"(p) : "memory");
}
__device__ __forceinline__ bool tag_reached(unsigned long long w, uint32_t tag) {
    return static_cast<int>(static_cast<uint32_t>(w >> 32) - tag) >= 0;
}
// A wait that ran out anywhere in the grid shortens every later one: every 1024 failed polls a waiting thread looks at
// the step's flag word, where time-outs are reported, and gives up too.  (After a lost store the step thus ends within
// milliseconds of the first time-out instead of running every wait to its limit.  The word is sticky: the host clears it.)
__device__ __forceinline__ bool others_gave_up(const int* err_flag, uint32_t it) {
    if ((it & 1023u) != 1023u || err_flag == nullptr) return false;
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(err_flag) : "memory");
    return (v & LEMOQ_FLAG_WAIT_TIMEOUT) != 0;
}
// N words of this thread (src[0..N), used where on[i]) until all carry the tag: data[i] = their data.  Bounded.
template <int N>
__device__ __forceinline__ bool flag_wait(const unsigned long long* src, const bool (&on)[N], uint32_t tag, uint32_t (&data)[N],
                                          const int* err_flag) {
    const uint32_t limit = c_flag_spin_limit;
    bool have[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        have[i] = !on[i];
        data[i] = 0;
    }
#pragma unroll 1  // one look per trip: an unrolled poll loop multiplies the traffic of everybody who waits
    for (uint32_t it = 0; it < limit; ++it) {
        bool ok = true;
        static_assert(N % 4 == 0, "words are looked at four at a time");
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            if (!(have[i] && have[i + 1] && have[i + 2] && have[i + 3])) {  // only sectors with a word still missing
                unsigned long long w[4];
                flag_load4(src + i, w);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (!have[i + j]) {
                        have[i + j] = tag_reached(w[j], tag);
                        data[i + j] = static_cast<uint32_t>(w[j]);
                    }
                    ok = ok && have[i + j];
                }
            }
        }
        if (ok) return true;
        if (others_gave_up(err_flag, it)) return false;
    }
    return false;
}

// Block barrier of the consumer warps (the producer warps never take part in it).
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }
// D = A (16x32 s8, rows) x B (32x8 s8, columns) + D, int32 accumulate.
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D = A (16x16 f16) x B (16x8 f16) + D, fp32 accumulate.
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void stamp(const StepParams& p, int slot) {
    if (p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.stamps[slot] = t;
    }
}

// ---------------------------------------------------------------------------------------------
// activations as digit planes
// ---------------------------------------------------------------------------------------------
// Four activations (fp32 holding fp16-representable values) -> one packed word per plane.  `inv` is the
// exact power-of-two reciprocal of the group scale.  X = round(f * inv) (|X| < 2^20) is split in two's
// complement: X = d2 * 2^14 + d1 * 2^7 + d0 with d0, d1 in [0, 127] and d2 in [-64, 63].
__device__ __forceinline__ void quantise4(const float (&f)[4], float inv, uint32_t& w0, uint32_t& w1, uint32_t& w2) {
    uint32_t X[4], Y[4], Z[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // round to nearest even through the 1.5 * 2^23 offset: the integer sits in the low mantissa bits
        X[j] = __float_as_uint(fmaf(f[j], inv, 12582912.0f)) - 0x4B400000u;
        Y[j] = X[j] >> 7;
        Z[j] = static_cast<uint32_t>(static_cast<int>(X[j]) >> 14);
    }
    w0 = __byte_perm(__byte_perm(X[0], X[1], 0x0040), __byte_perm(X[2], X[3], 0x0040), 0x5410) & 0x7f7f7f7fu;
    w1 = __byte_perm(__byte_perm(Y[0], Y[1], 0x0040), __byte_perm(Y[2], Y[3], 0x0040), 0x5410) & 0x7f7f7f7fu;
    w2 = __byte_perm(__byte_perm(Z[0], Z[1], 0x0040), __byte_perm(Z[2], Z[3], 0x0040), 0x5410);
}
// Group scale sx = 2^(floor(log2(amax)) - 19) (a fixed tiny scale for a zero group) and its reciprocal.
__device__ __forceinline__ void group_scale(float amax, float& sx, float& inv) {
    const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu);  // biased exponent
    if (amax > 0.f && e > 20) {
        sx = __uint_as_float(static_cast<uint32_t>(e - 19) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(254 - (e - 19)) << 23);
    } else {  // zero or denormal-range group: fixed tiny scale keeps the arithmetic exact
        sx = __uint_as_float(static_cast<uint32_t>(2) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(252) << 23);
    }
}
// Maximum over the 16 lanes of a half warp (both halves at once).
__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// One group of 128 values, eight per lane of a half warp (fp32 holding fp16-representable values), of vector
// element range [k0, k0 + 128) into the plane segments at `planes`: segment (half * 3 + plane) of K/2 + 64 bytes
// each.  `on` = this half warp has a group at all (the shuffles are executed by everyone).  Returns the group scale.
__device__ __forceinline__ float store_group_planes(const float (&f)[8], unsigned char* planes, int K, int k0, int lane16, bool on) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    amax = half_warp_max(amax);
    float s, inv;
    group_scale(amax, s, inv);
    const float lo[4] = {f[0], f[1], f[2], f[3]}, hi[4] = {f[4], f[5], f[6], f[7]};
    uint2 w0, w1, w2;
    quantise4(lo, inv, w0.x, w1.x, w2.x);
    quantise4(hi, inv, w0.y, w1.y, w2.y);
    if (on) {
        const int half_k = K >> 1, seg = half_k + kPad;
        const int hf = k0 >= half_k ? 1 : 0;
        unsigned char* base = planes + hf * 3 * seg + (k0 - hf * half_k) + lane16 * 8;
        *reinterpret_cast<uint2*>(base) = w0;
        *reinterpret_cast<uint2*>(base + seg) = w1;
        *reinterpret_cast<uint2*>(base + 2 * seg) = w2;
    }
    return s;
}

// Plane weights of the four accumulator registers of a lane (t = lane & 3; c0/c2 are column 2t, c1/c3 column
// 2t+1).  one_vector: columns 0-2 for all 16 rows.  Otherwise rows 0-7 use columns 0-2, rows 8-15 columns 3-5.
__device__ __forceinline__ void plane_weights(int t, bool one_vector, float (&pw)[4]) {
    pw[0] = t == 0 ? 1.f : (t == 1 ? 16384.f : 0.f);
    pw[1] = t == 0 ? 128.f : 0.f;
    if (one_vector) {
        pw[2] = pw[0];
        pw[3] = pw[1];
    } else {
        pw[2] = t == 2 ? 128.f : 0.f;
        pw[3] = t == 1 ? 1.f : (t == 2 ? 16384.f : 0.f);
    }
}

// NB group steps (128 codes of both half rows each) of an int8 tile with NB independent accumulator sets: the
// tensor-core instruction has a long latency, so consecutive instructions must not depend on each other.
template <int NB>
__device__ __forceinline__ float tile_s8_steps(const unsigned char* alo, const unsigned char* ahi, const unsigned char* bp, const float* sx,
                                               const __half* sc, int gh, int gs0, const float (&pw)[4], float acc) {
    int c[NB][4];
#pragma unroll
    for (int u = 0; u < NB; ++u) c[u][0] = c[u][1] = c[u][2] = c[u][3] = 0;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
        uint4 a[NB], b[NB], x[NB];
#pragma unroll
        for (int u = 0; u < NB; ++u) {
            const int off = (gs0 + u) * 128 + jj * 64;
            a[u] = *reinterpret_cast<const uint4*>(alo + off);
            b[u] = *reinterpret_cast<const uint4*>(ahi + off);
            x[u] = *reinterpret_cast<const uint4*>(bp + off);
        }
#pragma unroll
        for (int u = 0; u < NB; ++u) mma_s8(c[u], a[u].x, b[u].x, a[u].y, b[u].y, x[u].x, x[u].y);
#pragma unroll
        for (int u = 0; u < NB; ++u) mma_s8(c[u], a[u].z, b[u].z, a[u].w, b[u].w, x[u].z, x[u].w);
    }
#pragma unroll
    for (int u = 0; u < NB; ++u) {
        const int gs = gs0 + u;
        const float s_lo = __half2float(sc[gs]) * sx[gs];
        const float s_hi = __half2float(sc[gh + gs]) * sx[gh + gs];
        acc = fmaf(fmaf(static_cast<float>(c[u][1]), pw[1], static_cast<float>(c[u][0]) * pw[0]), s_lo, acc);
        acc = fmaf(fmaf(static_cast<float>(c[u][3]), pw[3], static_cast<float>(c[u][2]) * pw[2]), s_hi, acc);
    }
    return acc;
}

// One int8 tile: 8 rows of K codes in a stage (tile row r at r * K + (r >> 2) * kRunPad) against the plane segments
// of a vector.  r: the tile row of this lane's instruction row (tile_row()).  bp: this lane's segment pointer (+ t*16
// applied here).  sx: the K/128 group scales of the vector.  sc: the K/128 fp16 group scales of row r.  Returns the
// lane's share of row r (to be added over the 4 lanes of a group).
__device__ __forceinline__ float tile_s8(const unsigned char* st, int K, int r, int t, const unsigned char* bp, const float* sx,
                                         const __half* sc, const float (&pw)[4]) {
    const int half_k = K >> 1, gh = K >> 8;  // bytes per half row, groups per half
    const unsigned char* alo = st + r * K + (r >> 2) * kRunPad + t * 16;
    const unsigned char* ahi = alo + half_k;
    bp += t * 16;
    float acc = 0.f;
    if (gh >= 4) {
#pragma unroll 1
        for (int gs0 = 0; gs0 < gh; gs0 += 4) acc = tile_s8_steps<4>(alo, ahi, bp, sx, sc, gh, gs0, pw, acc);
    } else {
        acc = tile_s8_steps<2>(alo, ahi, bp, sx, sc, gh, 0, pw, acc);
    }
    return acc;
}

// One fp16 tile: 4 rows of H values (row stride 2H bytes) against the fp16 vector xh, whose quarters sit
// H/2 + 64 bytes apart.  Instruction row v = quarter (v >> 2), tile row (v & 3); B column n = quarter n.
// Four independent accumulator sets (see above).  Returns this lane's share of tile row (g & 3) (to be added over
// the lanes g, g ^ 4 with t = 0, 1).
__device__ __forceinline__ float tile_f16(const unsigned char* st, int H, int g, int t, const unsigned char* xh) {
    const int qb = H >> 1;  // bytes of a quarter row
    const unsigned char* alo = st + (g & 3) * (2 * H) + (g >> 2) * qb + t * 16;
    const unsigned char* ahi = alo + 2 * qb;
    const unsigned char* bp = xh + (g & 3) * (qb + kPad) + t * 16;
    float c[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) c[u][0] = c[u][1] = c[u][2] = c[u][3] = 0.f;
#pragma unroll 1
    for (int off = 0; off < qb; off += 256) {
        uint4 a[4], b[4], x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            a[u] = *reinterpret_cast<const uint4*>(alo + off + u * 64);
            b[u] = *reinterpret_cast<const uint4*>(ahi + off + u * 64);
            x[u] = *reinterpret_cast<const uint4*>(bp + off + u * 64);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) mma_f16(c[u], a[u].x, b[u].x, a[u].y, b[u].y, x[u].x, x[u].y);
#pragma unroll
        for (int u = 0; u < 4; ++u) mma_f16(c[u], a[u].z, b[u].z, a[u].w, b[u].w, x[u].z, x[u].w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) c[0][i] = (c[0][i] + c[1][i]) + (c[2][i] + c[3][i]);
    // instruction row g holds quarter g >> 2 (column g >> 2), row g + 8 quarter 2 + (g >> 2)
    const float lo = g < 4 ? c[0][0] : c[0][1], hi = g < 4 ? c[0][2] : c[0][3];
    return t == 0 ? lo : (t == 1 ? hi : 0.f);
}

// ---------------------------------------------------------------------------------------------
// shared-memory layout
// ---------------------------------------------------------------------------------------------
struct AttnSm {
    float wm[kStreamWarps];
    float wl[kStreamWarps];
    float wacc[kStreamWarps][kHeadDim];
    __align__(4) short pq[kStreamWarps][kKvTile];  // 15-bit softmax weights of a warp's tile
    __align__(16) unsigned char qplanes[3 * kQPlaneStride];
    __align__(16) uint32_t newk[32];
    __align__(16) uint32_t newv[32];
    float qsx;
    unsigned short newks, newvs;  // fp16 bit patterns of the new row's scales
    // fp16-KV arm: the query as it is (fp16 after RoPE), the new token's K and V rows, the softmax weights of a tile
    __align__(16) __half q16[kHeadDim];
    __align__(16) uint2 newk16[32];
    __align__(16) uint2 newv16[32];
    float p32[kStreamWarps][32];
};

// Sizes, shifts and this block's place in the grid (all row widths are powers of two between 512 and 2048).
struct Geo {
    int H, A, F, E, K, S, V, G, b, layers;
    int shF4;       // log2(F / 4): gate/up tiles per routed expert
    int fpair;      // down phase: a tile holds the rows of two routed experts (ffn <= 1024)
    int ftiles;     // down phase: tiles per block of 8 output rows
    int f_magic;    // ceil(65536 / ftiles)
    int f_blocks;   // down phase: blocks of 8 output rows this block owns
    // attention: the same in every layer of the step
    int pos;        // position of the new token (clamped into the cache)
    int nf;         // filled length (clamped)
    int h, split;   // this block's (head, split) unit
    int tile0;      // first KV tile of this block's slice
    int owner;      // the slice contains the new token: this block writes its K/V row
    int kvt;        // cached positions per KV tile: 16, 32 or 64 (int8 codes, chosen per step) or 32 (fp16 values)
    int kv16;       // the cache is read as fp16 (no int8 mirror)
    int has_unit;   // this block has a unit at all
    int nt[8];      // tiles of this block per kind (index 6: the lm_head tiles)
};

constexpr int kXPlaneBytes = 6 * (1024 + kPad);                    // plane segments of one vector of up to 2048 values
constexpr int kBigPlaneBytes = 6 * 4096 + 16 * 6 * kPad;            // plane segments of the routed experts' activations (<= 8192 values in <= 16 vectors)
constexpr int kBigBytes = kBigPlaneBytes + 64 * 4;                  // + their group scales
struct Smem {
    __align__(128) unsigned char ring[kStreamWarps * kStageBytes];
    __align__(8) unsigned long long full_bars[kStreamWarps];   // a tile has landed in the stage
    __align__(8) unsigned long long empty_bars[kStreamWarps];  // the consumer is done with the stage
    volatile int ready_layer;                                  // the routing of layers <= this is in route_id
    __align__(128) unsigned char xplanes[kXPlaneBytes];
    float xsx[16];
    __align__(128) unsigned char xh[4 * (1024 + kPad)];  // fp16 copy of the normalised vector, in quarters (router rows)
    __align__(128) unsigned char big[kBigBytes > static_cast<int>(sizeof(AttnSm)) ? kBigBytes : static_cast<int>(sizeof(AttnSm))];
    float part[kPartFloats];
    float red[64];
    float cs[2 * kHeadDim];
    int route_id[32];
    float route_w[32];
    Geo geo;
    StepLayer layers[kMaxLayers];
};

__device__ __forceinline__ int udiv_small(int q, int magic) { return (q * magic) >> 16; }  // q / d for q < 65536 / d, magic = ceil(65536 / d)

// ---------------------------------------------------------------------------------------------
// per-warp tile stream
// ---------------------------------------------------------------------------------------------
// The bulk copies of tile (layer, kind, lt) of this block into a stage (a few large copies: starting a copy costs
// a warp some hundred cycles).  Global tile index of local tile lt: b + lt * G (down phase: row block b + j * G with
// the top_k routed experts as consecutive tiles).
__device__ __noinline__ void issue_tile(const Smem& S, int layer, int kind, int lt, uint32_t stage, uint32_t bar) {
    const Geo& geo = S.geo;
    const StepLayer& L = S.layers[layer];
    const int lane = threadIdx.x & 31;
    const char* src = nullptr;
    uint32_t bytes = 0, dst = 0, tx = 0;
    if (kind == KB) {  // cached positions of this block's head: keys and values (int8: the consumer reads the scales itself)
        const int first = (geo.tile0 + lt) * geo.kvt;
        const uint32_t npos = static_cast<uint32_t>(min(geo.kvt, geo.S - first));  // the last tile of a head may be short
        const uint32_t p0 = static_cast<uint32_t>(geo.h * geo.S + first);
        const uint32_t row = geo.kv16 ? 2 * kHeadDim : kHeadDim;  // bytes of a position
        tx = 2 * npos * row;
        if (lane < 2) {
            const void* base = geo.kv16 ? static_cast<const void*>(lane == 0 ? L.keys : L.values) : static_cast<const void*>(lane == 0 ? L.kc : L.vc);
            src = reinterpret_cast<const char*>(base) + static_cast<size_t>(p0) * row;
            bytes = npos * row;
            dst = lane * kKvTile * kHeadDim;
        }
    } else if (kind == KD) {  // 4 router rows (fp16) in one copy; fewer than 4 experts left: only those
        const int row0 = (geo.b + lt * geo.G) * 4;
        const uint32_t nrows = static_cast<uint32_t>(min(4, geo.E - row0));
        tx = nrows * 2 * geo.H;
        if (lane == 0) {
            src = reinterpret_cast<const char*>(L.router) + static_cast<size_t>(row0) * 2 * geo.H;
            bytes = tx;
        }
    } else {
        // The code rows of a tile land in runs of four, each run 64 bytes further than its natural place (tile row r at
        // r * K + (r >> 2) * 64): the eight lanes that read 16 bytes each of tile rows r and r + 4 in one request then
        // hit different banks.  Lanes 0-3 copy one run of codes each, lanes 4-5 the group scales (rows of a run are
        // consecutive in memory; gate/up: the gate run and the up run; down: the runs of one routed expert or of two).
        const int tg = geo.b + lt * geo.G;
        const uint32_t run = lane & 3, half = lane & 1;  // code lanes: run of four rows; scale lanes 4, 5: first / second part
        uint32_t K = geo.H;          // row width
        uint32_t crow = 0, srow = 0; // first row of this lane's run of codes / part of the scales
        uint32_t nruns = 2;          // runs of four code rows in the tile
        uint32_t sparts = 1, srows = 8;  // parts of the scales and rows per part
        const char* cbase;
        const char* sbase;
        if (kind == KE) {  // 4 gate rows + 4 up rows of one routed expert
            const int slot = tg >> geo.shF4, n0 = (tg - (slot << geo.shF4)) * 4;
            crow = srow = static_cast<uint32_t>(S.route_id[slot]) * 2 * geo.F + n0 + (half ? geo.F : 0);
            sparts = 2;
            srows = 4;
            cbase = reinterpret_cast<const char*>(L.gu_codes);
            sbase = reinterpret_cast<const char*>(L.gu_scale);
        } else if (kind == KF) {  // 8 down rows of one routed expert, or of two (runs 2-3 and scale part 1: the second one)
            const int j = udiv_small(lt, geo.f_magic), pp = lt - j * geo.ftiles;
            const bool two = geo.fpair && 2 * pp + 1 < geo.K;
            const uint32_t first = (geo.b + j * geo.G) * 8;
            const int cslot = geo.fpair ? 2 * pp + static_cast<int>(run >> 1) : pp, sslot = geo.fpair ? 2 * pp + static_cast<int>(half) : pp;
            crow = static_cast<uint32_t>(S.route_id[min(cslot, geo.K - 1)]) * geo.H + first + (run & 1) * 4;
            srow = static_cast<uint32_t>(S.route_id[min(sslot, geo.K - 1)]) * geo.H + first;
            nruns = two ? 4 : 2;
            sparts = two ? 2 : 1;
            K = geo.F;
            cbase = reinterpret_cast<const char*>(L.dn_codes);
            sbase = reinterpret_cast<const char*>(L.dn_scale);
        } else {  // 8 consecutive rows of q.k.v / lm_head (KA) or o_proj (KC)
            crow = tg * 8 + run * 4;
            srow = tg * 8;
            K = kind == KA ? geo.H : geo.A;
            cbase = reinterpret_cast<const char*>(kind == KA ? L.qkv_codes : L.o_codes);
            sbase = reinterpret_cast<const char*>(kind == KA ? L.qkv_scale : L.o_scale);
        }
        const uint32_t sb = (K >> 7) * 2;  // bytes of one row of group scales
        tx = nruns * 4u * (K + sb);
        if (lane < 4) {
            if (run < nruns) {
                src = cbase + static_cast<size_t>(crow) * K;
                bytes = 4 * K;
                dst = run * (4 * K + kRunPad);
            }
        } else if (lane < 6 && half < sparts) {
            src = sbase + static_cast<size_t>(srow) * sb;
            bytes = srows * sb;
            dst = kScaleOff + half * srows * sb;
        }
    }
    if (lane == 0) mbar_expect_tx(bar, tx);
    __syncwarp();
    if (bytes != 0) bulk_g2s(stage + dst, src, bytes, bar);
}

// Place in the block's tile sequence of the tiles that go through one stage.  The tiles of a block form one
// sequence over all phases of the step; tile q of the sequence goes through stage q mod 10 and is consumed by warp
// q mod 10, so the stages that free up first in a phase take the tiles that are needed first in the next one.
struct Cursor {
    int layer, kind, lt;  // next tile of the stage
    int base;             // place of the first tile of (layer, kind) in the sequence, modulo the stages
    __device__ __forceinline__ void start(const Geo& geo, int stage) {
        layer = 0;
        kind = KA;
        base = 0;
        lt = stage;
        normalise(geo, stage);
    }
    __device__ __forceinline__ void normalise(const Geo& geo, int stage) {
        while (kind != KEND) {
            const int n = layer == geo.layers ? (kind == KA ? geo.nt[6] : 0) : geo.nt[kind];
            if (lt < n) return;
            base = (base + n) % kStreamWarps;
            lt = stage - base + (stage < base ? kStreamWarps : 0);
            if (layer == geo.layers) {
                kind = KEND;
                return;
            }
            if (kind == KF) {
                kind = KA;
                ++layer;
            } else {
                ++kind;
            }
        }
    }
};

// A producer warp: fills its two stages in sequence order for the whole step.  A stage is refilled as soon as its
// consumer gives it back, whatever phase the consumers are in; only the expert tiles wait for the routing of
// their layer.  Every wait is bounded: a producer that gives up raises the flag word and stops, and the consumers
// then run into their own bounded waits.
__device__ __noinline__ void producer_loop(Smem& S, int* err_flag, int first_stage) {
    const Geo& geo = S.geo;
    const int lane = threadIdx.x & 31;
    Cursor c0, c1;
    c0.start(geo, first_stage);
    c1.start(geo, first_stage + 1);
    uint32_t used0 = 0, used1 = 0;  // fills of each stage so far
    bool ok = true;
#pragma unroll 1
    while (ok && (c0.kind != KEND || c1.kind != KEND)) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            Cursor& c = i == 0 ? c0 : c1;
            uint32_t& used = i == 0 ? used0 : used1;
            if (!ok || c.kind == KEND) continue;
            const int stage = first_stage + i;
            if (c.kind >= KE) {  // expert tiles: the routing of the layer must be known
                uint32_t n = 0;
                while (S.ready_layer < c.layer) {
                    __nanosleep(64);
                    if (++n > (1u << 22)) {
                        ok = false;
                        break;
                    }
                }
                __threadfence_block();
            }
            if (ok && used > 0) ok = mbar_wait(smem_u32(&S.empty_bars[stage]), (used - 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            issue_tile(S, c.layer, c.kind, c.lt, smem_u32(S.ring) + static_cast<uint32_t>(stage) * kStageBytes, smem_u32(&S.full_bars[stage]));
            ++used;
            c.lt += kStreamWarps;
            c.normalise(geo, stage);
        }
    }
    if (!ok && err_flag && lane == 0) atomicOr(err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
}

// Consumer side of a stage: wait for the tile (warp-uniform result; false on time-out), give the stage back.
__device__ __forceinline__ bool stage_acquire(uint32_t full_bar, uint32_t parity, int* err_flag) {
    bool ok = mbar_wait(full_bar, parity);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && err_flag && (threadIdx.x & 31) == 0) atomicOr(err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
    return ok;
}
__device__ __forceinline__ void stage_release(uint32_t empty_bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar) : "memory");
}

// ---------------------------------------------------------------------------------------------
// routing: softmax + top-k of the E fp16 logits (E <= 128, flagged words) by one warp.  Probabilities are positive
// floats, so their bit patterns order like unsigned integers: a warp-wide integer maximum plus a ballot
// gives the largest probability and its lowest index per round.
// ---------------------------------------------------------------------------------------------
template <int PER>  // experts per lane: 2 for E <= 64, 4 for E <= 128
__device__ __forceinline__ void warp_topk_per(const unsigned long long* logits, uint32_t tag, int* err_flag, int E, int K, bool norm,
                                              int lane, int& id_reg, float& w_reg) {
    float v[PER];
    float mx = -INFINITY;
    {
        uint32_t d[PER];
        bool on[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) on[j] = lane + 32 * j < E;
        // lane-strided words: word j of this lane sits 32 words further
        bool good = true;
        const uint32_t limit = c_flag_spin_limit;
#pragma unroll 1
        for (uint32_t it = 0; it < limit; ++it) {
            good = true;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const unsigned long long w = on[j] ? flag_load(logits + lane + 32 * j) : (static_cast<unsigned long long>(tag) << 32);
                good = good && tag_reached(w, tag);
                d[j] = static_cast<uint32_t>(w);
            }
            if (good || others_gave_up(err_flag, it)) break;
        }
        if (!good && err_flag) atomicOr(err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            v[j] = on[j] ? __half2float(__ushort_as_half(static_cast<unsigned short>(d[j] & 0xffffu))) : -INFINITY;
            mx = fmaxf(mx, v[j]);
        }
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? expf(v[j] - mx) : 0.f;
        sum += v[j];
    }
    sum = warp_sum(sum);
    unsigned int key[PER];  // bits of the probability + 1; 0 = absent or already taken
#pragma unroll
    for (int j = 0; j < PER; ++j) key[j] = (lane + 32 * j) < E ? __float_as_uint(v[j] / sum) + 1u : 0u;
    float wsum = 0.f;
    id_reg = 0;
    w_reg = 0.f;
#pragma unroll 1
    for (int k = 0; k < K; ++k) {
        unsigned int own = key[0];
#pragma unroll
        for (int j = 1; j < PER; ++j) own = max(own, key[j]);
        const unsigned int top = __reduce_max_sync(0xffffffffu, own);
        int bi = -1;
#pragma unroll
        for (int j = PER - 1; j >= 0; --j) {
            const unsigned int b = __ballot_sync(0xffffffffu, key[j] == top);
            if (b) bi = 32 * j + __ffs(b) - 1;
        }
        const float best = __uint_as_float(top - 1u);
        wsum += best;
        if (lane == k) {
            id_reg = bi;
            w_reg = best;
        }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int j = 0; j < PER; ++j)
                if (j == (bi >> 5)) key[j] = 0u;
        }
    }
    if (norm) w_reg = w_reg / wsum;
    w_reg = __half2float(__float2half_rn(w_reg));  // the routing weights are used in fp16
}
__device__ __noinline__ void warp_topk(const unsigned long long* logits, uint32_t tag, int* err_flag, int E, int K, bool norm, int lane,
                                       int& id_reg, float& w_reg) {
    if (E <= 64) warp_topk_per<2>(logits, tag, err_flag, E, K, norm, lane, id_reg, w_reg);
    else warp_topk_per<4>(logits, tag, err_flag, E, K, norm, lane, id_reg, w_reg);
}

// ---------------------------------------------------------------------------------------------
// block-wide preparation of a phase's activation vectors
// ---------------------------------------------------------------------------------------------
// ngroups groups of 128 fp16 values (contiguous at src; vectors of K values each) -> plane segments (vector v at
// planes + v * 6 * (K/2 + 64)) and group scales sx[group].  With nw (one vector of at most 2048 values) the values
// are RMS-normalised first; xh, when given, receives them as fp16 in quarters.  A half warp handles a group (eight
// values per lane), the block twenty groups per pass (at most four passes, all requested before any is worked on).
// The values come from a plain fp16 vector (src) or from flagged words (fsrc: `pack` values per word, waited for
// until they carry `tag`).
__device__ __noinline__ void prepare(float eps, const __half* __restrict__ src, const unsigned long long* fsrc, uint32_t tag, int pack,
                                     const __half* __restrict__ nw, int K, int ngroups, unsigned char* planes, float* sx,
                                     unsigned char* xh, float* red, int* err_flag) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, lane16 = lane & 15;
    constexpr int kPerPass = 2 * kStreamWarps, kMaxPass = 4;
    const int gi0 = warp * 2 + (lane >> 4);
    // the raw fp16 values of this half warp's groups (pass q: group gi0 + 20 q), eight per lane
    uint4 raw[kMaxPass];
    bool good = true;
    if (fsrc == nullptr) {  // plain fp16 vector (the embedding row)
#pragma unroll
        for (int q = 0; q < kMaxPass; ++q) {
            const int gi = gi0 + q * kPerPass;
            raw[q] = gi < ngroups ? *reinterpret_cast<const uint4*>(src + gi * 128 + lane16 * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
    } else if (pack == 1) {  // one value per flagged word
#pragma unroll
        for (int q = 0; q < kMaxPass; ++q) {
            const int gi = gi0 + q * kPerPass;
            uint32_t d[8];
            const bool act = gi < ngroups;
            const bool on[8] = {act, act, act, act, act, act, act, act};
            good = flag_wait<8>(fsrc + (act ? gi : 0) * 128 + lane16 * 8, on, tag, d, err_flag) && good;
            raw[q] = make_uint4((d[0] & 0xffffu) | (d[1] << 16), (d[2] & 0xffffu) | (d[3] << 16), (d[4] & 0xffffu) | (d[5] << 16),
                                (d[6] & 0xffffu) | (d[7] << 16));
            if (q == 0 && ngroups <= kPerPass) break;
        }
    } else {  // two values per flagged word
#pragma unroll
        for (int q = 0; q < kMaxPass; ++q) {
            const int gi = gi0 + q * kPerPass;
            uint32_t d[4];
            const bool act = gi < ngroups;
            const bool on[4] = {act, act, act, act};
            good = flag_wait<4>(fsrc + (act ? gi : 0) * 64 + lane16 * 4, on, tag, d, err_flag) && good;
            raw[q] = make_uint4(d[0], d[1], d[2], d[3]);
        }
    }
    if (!good && err_flag) atomicOr(err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
    __syncwarp();
    uint4 wv = make_uint4(0u, 0u, 0u, 0u);
    float rstd = 0.f;
    if (nw != nullptr) {  // one pass: at most 16 groups
        if (gi0 < ngroups) wv = *reinterpret_cast<const uint4*>(nw + gi0 * 128 + lane16 * 8);
        float xf[8];
        unpack8_h(gi0 < ngroups ? raw[0] : make_uint4(0u, 0u, 0u, 0u), xf);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(xf[j], xf[j], ss);
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        consumer_sync();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kStreamWarps; ++w) tot += red[w];
        rstd = 1.0f / sqrtf(tot / static_cast<float>(K) + eps);
    }
    const int kshift = 31 - __clz(K);
#pragma unroll
    for (int q = 0; q < kMaxPass; ++q) {
        const int gi = gi0 + q * kPerPass;
        if (q * kPerPass >= ngroups) break;
        const __half* xv = reinterpret_cast<const __half*>(&raw[q]);
        const __half* wh = reinterpret_cast<const __half*>(&wv);
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = nw != nullptr ? norm_elem(xv[j], rstd, wh[j]) : __half2float(xv[j]);
        const bool on = gi < ngroups;
        const int v = (gi * 128) >> kshift, k0 = gi * 128 - (v << kshift);
        const float s = store_group_planes(f, planes + v * 6 * ((K >> 1) + kPad), K, k0, lane16, on);
        if (on && lane16 == 0) sx[gi] = s;
        if (xh != nullptr && on) {
            uint4 o;
            __half2 h;
            h = __floats2half2_rn(f[0], f[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[2], f[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[4], f[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[6], f[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
            const int qv = K >> 2, qq = k0 >> (kshift - 2);  // values per quarter, quarter of this group
            *reinterpret_cast<uint4*>(xh + qq * (2 * qv + kPad) + (k0 - qq * qv) * 2 + lane16 * 16) = o;
        }
    }
    consumer_sync();
}

// The attention output as the o_proj input: a half warp merges the splits of one head (partials (m, l, acc[128]) of
// the (head, split) units, taken four splits at a time in split order), rounds to fp16 and builds the planes of the
// head's group.  Lane i of the half warp holds dimensions 8i .. 8i+7.
__device__ __noinline__ void prepare_attention_output(const StepParams& p, Smem& S) {
    constexpr int D = kHeadDim;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, lane16 = lane & 15;
    const int head = warp * 2 + (lane >> 4);
    const bool on = head < p.heads;
    const int hd = on ? head : 0;
    const float* hacc = p.attn_part + static_cast<int64_t>(hd) * p.splits * D + lane16 * 8;
    const float* hml = p.attn_part + static_cast<int64_t>(p.heads) * p.splits * D + static_cast<int64_t>(hd) * p.splits * 2;
    float big = -INFINITY, den = 0.f;
    float num[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int j0 = 0; j0 < p.splits; j0 += 4) {
        float4 a0[4], a1[4];
        float2 mv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j0 + j < p.splits) {
                a0[j] = __ldcg(reinterpret_cast<const float4*>(hacc + (j0 + j) * D));
                a1[j] = __ldcg(reinterpret_cast<const float4*>(hacc + (j0 + j) * D + 4));
                mv[j] = __ldcg(reinterpret_cast<const float2*>(hml + 2 * (j0 + j)));
            } else {
                a0[j] = a1[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                mv[j] = make_float2(-INFINITY, 0.f);
            }
        }
        float nb = big;
#pragma unroll
        for (int j = 0; j < 4; ++j) nb = fmaxf(nb, mv[j].x);
        const float ref = nb > -INFINITY ? nb : 0.f;
        const float keep = exp2f(big - ref);  // 0 for the first batch (big = -inf)
        den *= keep;
#pragma unroll
        for (int i = 0; i < 8; ++i) num[i] *= keep;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float w = exp2f(mv[j].x - ref);
            den = fmaf(mv[j].y, w, den);
            num[0] = fmaf(a0[j].x, w, num[0]);
            num[1] = fmaf(a0[j].y, w, num[1]);
            num[2] = fmaf(a0[j].z, w, num[2]);
            num[3] = fmaf(a0[j].w, w, num[3]);
            num[4] = fmaf(a1[j].x, w, num[4]);
            num[5] = fmaf(a1[j].y, w, num[5]);
            num[6] = fmaf(a1[j].z, w, num[6]);
            num[7] = fmaf(a1[j].w, w, num[7]);
        }
        big = nb;
    }
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __half2float(__float2half_rn(den > 0.f ? num[j] / den : num[j]));
    const float s = store_group_planes(f, S.xplanes, p.heads * D, hd * D, lane16, on);
    if (on && lane16 == 0) S.xsx[hd] = s;
    consumer_sync();
}

// ---------------------------------------------------------------------------------------------
// attention phase (one (head, split) unit per block; head_dim 128, int8 KV with per-token scales)
// ---------------------------------------------------------------------------------------------
// Warp 0: q (RMSNorm over all heads, RoPE, softmax scale, digit planes).  Warp 1 / warp 2 of the block that owns
// the new position: the new K row (norm, RoPE) / V row into the fp16 cache and, quantised, into the int8 mirror
// and shared memory.  Lane i holds dimensions 4i .. 4i+3; the RoPE partner (d +- 64) lives 16 lanes away.
__device__ __noinline__ void attention_prologue(const StepParams& p, const StepLayer& L, Smem& S, const unsigned long long* fqkv,
                                                const unsigned long long* fstats, uint32_t tag) {
    constexpr int D = kHeadDim;
    AttnSm& sm = *reinterpret_cast<AttnSm*>(S.big);
    const Geo& geo = S.geo;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp == 0 || (geo.owner && warp < 3)) {
        const int A = geo.A, h = geo.h;
        // this lane's four values of the head's q (k, v) row: flagged words written by the q.k.v phase
        uint32_t d4[4];
        const bool on4[4] = {true, true, true, true};
        bool good = flag_wait<4>(fqkv + warp * A + h * D + lane * 4, on4, tag, d4, p.err_flag);
        const uint2 raw = make_uint2((d4[0] & 0xffffu) | (d4[1] << 16), (d4[2] & 0xffffu) | (d4[3] << 16));
        const __half* rh = reinterpret_cast<const __half*>(&raw);
        float f[4];
        if (warp < 2) {
            const uint2 wv = *reinterpret_cast<const uint2*>((warp == 0 ? L.q_norm : L.k_norm) + h * D + lane * 4);
            const __half* wh = reinterpret_cast<const __half*>(&wv);
            // sum of squares of the whole q (k) row: one partial per block of the grid, added in a fixed order
            float s = 0.f;
#pragma unroll 1
            for (int b0 = 0; b0 < geo.G; b0 += 128) {
                uint32_t d[4];
                bool on[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) on[i] = b0 + lane + 32 * i < geo.G;
                const uint32_t limit = c_flag_spin_limit;
#pragma unroll 1
                for (uint32_t it = 0; it < limit; ++it) {
                    bool ok = true;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const unsigned long long w = on[i] ? flag_load(fstats + warp * 1024 + b0 + lane + 32 * i) : (static_cast<unsigned long long>(tag) << 32);
                        ok = ok && tag_reached(w, tag);
                        d[i] = static_cast<uint32_t>(w);
                    }
                    if (ok) break;
                    if (it + 1 == limit || others_gave_up(p.err_flag, it)) {
                        good = false;
                        break;
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) s += on[i] ? __uint_as_float(d[i]) : 0.f;
            }
            __syncwarp();
            s = warp_sum(s);
            const float rstd = 1.0f / sqrtf(s / static_cast<float>(A) + p.eps);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float x = norm_elem(rh[j], rstd, wh[j]);
                const float o = __shfl_xor_sync(0xffffffffu, x, 16);
                const float rot = lane < 16 ? -o : o;
                f[j] = __half2float(__float2half_rn(__fadd_rn(__fmul_rn(x, S.cs[4 * lane + j]), __fmul_rn(rot, S.cs[D + 4 * lane + j]))));
            }
        } else {
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] = __half2float(rh[j]);
        }
        if (!good && p.err_flag) atomicOr(p.err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
        if (warp == 0 && geo.kv16) {  // the query as fp16 (exact: it was rounded after the rotation); scores are scaled in fp32
            __half2 h01 = __floats2half2_rn(f[0], f[1]), h23 = __floats2half2_rn(f[2], f[3]);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&h01);
            o.y = *reinterpret_cast<uint32_t*>(&h23);
            *reinterpret_cast<uint2*>(sm.q16 + lane * 4) = o;
        } else if (warp == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] *= p.qk_scale_log2;
            const float amax = warp_max(fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3]))));
            float s, inv;
            group_scale(amax, s, inv);
            uint32_t w0, w1, w2;
            quantise4(f, inv, w0, w1, w2);
            *reinterpret_cast<uint32_t*>(sm.qplanes + 4 * lane) = w0;
            *reinterpret_cast<uint32_t*>(sm.qplanes + kQPlaneStride + 4 * lane) = w1;
            *reinterpret_cast<uint32_t*>(sm.qplanes + 2 * kQPlaneStride + 4 * lane) = w2;
            if (lane == 0) sm.qsx = s;
        } else {
            const int64_t at = (static_cast<int64_t>(h) * geo.S + geo.pos) * D + lane * 4;
            __half2 h01 = __floats2half2_rn(f[0], f[1]), h23 = __floats2half2_rn(f[2], f[3]);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&h01);
            o.y = *reinterpret_cast<uint32_t*>(&h23);
            *reinterpret_cast<uint2*>((warp == 1 ? L.keys : L.values) + at) = o;
            if (geo.kv16) {  // the fp16 cache is what attention reads: keep the row for the tile that holds the new slot
                (warp == 1 ? sm.newk16 : sm.newv16)[lane] = o;
            } else {  // the int8 mirror: quantise the row, write codes and scale, keep both
                const float amax = warp_max(fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3]))));
                const float sc = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
                uint32_t packed = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = static_cast<int>(fminf(fmaxf(rintf(__fdiv_rn(f[j], sc)), -127.0f), 127.0f));
                    packed |= (static_cast<uint32_t>(c) & 0xffu) << (8 * j);
                }
                *reinterpret_cast<uint32_t*>((warp == 1 ? L.kc : L.vc) + at) = packed;
                (warp == 1 ? sm.newk : sm.newv)[lane] = packed;
                if (lane == 0) {
                    const __half hs = __float2half_rn(sc);
                    (warp == 1 ? L.ks : L.vs)[static_cast<int64_t>(h) * geo.S + geo.pos] = hs;
                    (warp == 1 ? sm.newks : sm.newvs) = __half_as_ushort(hs);
                }
            }
        }
    }
    consumer_sync();
}

// One KV tile (T = 16, 32 or 64 positions in a stage: keys at its start, values 8 KB further) of the warp: scores
// through the int8 dot product against the planes of q (instruction rows = positions), online softmax (base 2),
// values with each lane owning four output dimensions.
template <int T>
__device__ __forceinline__ void attention_tile(unsigned char* st, AttnSm& sm, const Geo& geo, int lt, int lane, int warp, const float (&pw)[4],
                                               const float (&kscale)[2], const float (&vscale)[2], float& m_i, float& l_i, float (&acc)[4]) {
    constexpr int D = kHeadDim, VO = kKvTile * kHeadDim;  // VO: where the values start
    const int g = lane >> 2, t = lane & 3;
    const int base = (geo.tile0 + lt) * T;
    const int nvalid = min(T, geo.nf - base);
    if (geo.owner && geo.pos >= base && geo.pos < base + T) {
        // the row of the new token: the codes this block has just derived (the copy may have read the slot before the write)
        const int row = geo.pos - base;
        reinterpret_cast<uint32_t*>(st + row * D)[lane] = sm.newk[lane];
        reinterpret_cast<uint32_t*>(st + VO + row * D)[lane] = sm.newv[lane];
        __syncwarp();
    }
    // kscale[r] / vscale[r] of this lane belong to position 32 r + lane of the tile
    auto scale_of = [&](const float (&sc)[2], int pi) { return __shfl_sync(0xffffffffu, (T <= 32 || pi < 32) ? sc[0] : sc[1], pi & 31); };
    const unsigned char* qp = sm.qplanes + (g < 3 ? g : (g & 1)) * kQPlaneStride + t * 16;
    const float qsx = sm.qsx;
    float s[T / 8];
#pragma unroll
    for (int blk = 0; blk < T / 16; ++blk) {
        int c[4] = {0, 0, 0, 0};
        const unsigned char* alo = st + (blk * 16 + g) * D + t * 16;
        const unsigned char* ahi = alo + 8 * D;
#pragma unroll
        for (int jd = 0; jd < 2; ++jd) {
            const uint4 a = *reinterpret_cast<const uint4*>(alo + jd * 64);
            const uint4 b = *reinterpret_cast<const uint4*>(ahi + jd * 64);
            const uint4 x = *reinterpret_cast<const uint4*>(qp + jd * 64);
            mma_s8(c, a.x, b.x, a.y, b.y, x.x, x.y);
            mma_s8(c, a.z, b.z, a.w, b.w, x.z, x.w);
        }
        float vlo = fmaf(static_cast<float>(c[1]), pw[1], static_cast<float>(c[0]) * pw[0]);
        float vhi = fmaf(static_cast<float>(c[3]), pw[3], static_cast<float>(c[2]) * pw[2]);
        vlo += __shfl_xor_sync(0xffffffffu, vlo, 1);
        vhi += __shfl_xor_sync(0xffffffffu, vhi, 1);
        vlo += __shfl_xor_sync(0xffffffffu, vlo, 2);
        vhi += __shfl_xor_sync(0xffffffffu, vhi, 2);
        const int plo = blk * 16 + g, phi = plo + 8;
        const float klo = scale_of(kscale, plo), khi = scale_of(kscale, phi);
        s[2 * blk] = plo < nvalid ? vlo * qsx * klo : -INFINITY;
        s[2 * blk + 1] = phi < nvalid ? vhi * qsx * khi : -INFINITY;
    }
    float mx = s[0];
#pragma unroll
    for (int i = 1; i < T / 8; ++i) mx = fmaxf(mx, s[i]);
    const float m_new = fmaxf(m_i, warp_max(mx));  // finite: position 0 of the tile is valid
    const float alpha = exp2f(m_i - m_new);
    float lsum = 0.f;
#pragma unroll
    for (int i = 0; i < T / 8; ++i) {
        s[i] = s[i] > -INFINITY ? exp2f(s[i] - m_new) : 0.f;
        lsum += s[i];
    }
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 4);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 8);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 16);
    l_i = fmaf(l_i, alpha, lsum);
    m_i = m_new;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] *= alpha;
    // values: the weights w_j = p_j * vscale_j of the tile as 15-bit integers (relative to the tile's largest), two
    // positions per word; a lane owns four output dimensions and takes the positions in pairs: two byte permutes put
    // the codes of a pair next to each other, four 2-way integer dot products add both positions to the four sums
    float wj[T / 8], wmax = 0.f;
#pragma unroll
    for (int i = 0; i < T / 8; ++i) {
        const int pi = (i >> 1) * 16 + g + (i & 1) * 8;
        const float vsc = scale_of(vscale, pi);
        wj[i] = pi < nvalid ? s[i] * vsc : 0.f;
        wmax = fmaxf(wmax, wj[i]);
    }
    wmax = warp_max(wmax);
    const float qs = wmax > 0.f ? 32767.0f / wmax : 0.f;
    __syncwarp();
    if (t == 0) {
#pragma unroll
        for (int i = 0; i < T / 8; ++i) {
            const int pi = (i >> 1) * 16 + g + (i & 1) * 8;
            sm.pq[warp][pi] = static_cast<short>(__float2int_rn(wj[i] * qs));
        }
    }
    __syncwarp();
    const unsigned char* vrow = st + VO + lane * 4;
    const uint32_t* pq = reinterpret_cast<const uint32_t*>(sm.pq[warp]);
    int ai[4] = {0, 0, 0, 0};
#pragma unroll 4
    for (int j2 = 0; j2 < T / 2; ++j2) {
        const int pp = static_cast<int>(pq[j2]);
        const uint32_t v0 = *reinterpret_cast<const uint32_t*>(vrow + (2 * j2) * D);
        const uint32_t v1 = *reinterpret_cast<const uint32_t*>(vrow + (2 * j2 + 1) * D);
        const int w01 = static_cast<int>(__byte_perm(v0, v1, 0x5140));  // dimension 0 of both positions, then dimension 1
        const int w23 = static_cast<int>(__byte_perm(v0, v1, 0x7362));  // dimension 2 of both positions, then dimension 3
        ai[0] = __dp2a_lo(pp, w01, ai[0]);
        ai[1] = __dp2a_hi(pp, w01, ai[1]);
        ai[2] = __dp2a_lo(pp, w23, ai[2]);
        ai[3] = __dp2a_hi(pp, w23, ai[3]);
    }
    const float back = wmax * (1.0f / 32767.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = fmaf(static_cast<float>(ai[j]), back, acc[j]);
}

// One KV tile of the fp16-KV arm (32 positions in a stage: 8 KB of keys, 8 KB of values): a lane owns one position
// for the scores (its key row against the query, 16-byte chunks taken in a rotated order so that the eight lanes of a
// quarter warp hit different banks), online softmax (base 2), then four output dimensions for the values.
__device__ __forceinline__ void attention_tile16(unsigned char* st, AttnSm& sm, const Geo& geo, int lt, int lane, int warp, float qk_scale_log2,
                                                 float& m_i, float& l_i, float (&acc)[4]) {
    constexpr int D = kHeadDim, T = 32;
    const int base = (geo.tile0 + lt) * T;
    const int nvalid = min(T, geo.nf - base);
    if (geo.owner && geo.pos >= base && geo.pos < base + T) {
        // the row of the new token: what this block has just written (the copy may have read the slot before the write)
        const int row = geo.pos - base;
        reinterpret_cast<uint2*>(st + row * 2 * D)[lane] = sm.newk16[lane];
        reinterpret_cast<uint2*>(st + kKvTile * D + row * 2 * D)[lane] = sm.newv16[lane];
        __syncwarp();
    }
    float dot = 0.f;
    const unsigned char* krow = st + lane * 2 * D;
#pragma unroll 4
    for (int c = 0; c < 16; ++c) {
        const int cc = (c + lane) & 15;
        const uint4 kv = *reinterpret_cast<const uint4*>(krow + cc * 16);
        const uint4 qv = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sm.q16) + cc * 16);
        const __half2* kh = reinterpret_cast<const __half2*>(&kv);
        const __half2* qh = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 kf = __half22float2(kh[j]), qf = __half22float2(qh[j]);
            dot = fmaf(kf.x, qf.x, dot);
            dot = fmaf(kf.y, qf.y, dot);
        }
    }
    const float s = lane < nvalid ? dot * qk_scale_log2 : -INFINITY;
    const float m_new = fmaxf(m_i, warp_max(s));  // finite: position 0 of the tile is valid
    const float alpha = exp2f(m_i - m_new);
    const float pj = s > -INFINITY ? exp2f(s - m_new) : 0.f;
    l_i = fmaf(l_i, alpha, warp_sum(pj));
    m_i = m_new;
    sm.p32[warp][lane] = pj;
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] *= alpha;
    const unsigned char* vcol = st + kKvTile * D + lane * 8;
#pragma unroll 8
    for (int j = 0; j < nvalid; ++j) {  // rows behind the filled length are not numbers that may be multiplied by zero
        const float w = sm.p32[warp][j];
        const uint2 vv = *reinterpret_cast<const uint2*>(vcol + j * 2 * D);
        const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&vv.x)), v23 = __half22float2(*reinterpret_cast<const __half2*>(&vv.y));
        acc[0] = fmaf(w, v01.x, acc[0]);
        acc[1] = fmaf(w, v01.y, acc[1]);
        acc[2] = fmaf(w, v23.x, acc[2]);
        acc[3] = fmaf(w, v23.y, acc[3]);
    }
    __syncwarp();
}

// Merge of the block's warps into the unit's partial (m, l, acc[128]).
__device__ __noinline__ void attention_partial(const StepParams& p, Smem& S) {
    constexpr int D = kHeadDim;
    AttnSm& sm = *reinterpret_cast<AttnSm*>(S.big);
    const Geo& geo = S.geo;
    const int tid = threadIdx.x;
    // partial layout: acc[(h*splits + split)*D + d], then the (m, l) pairs
    if (tid < D) {
        constexpr int nactive = kStreamWarps;  // warps without a tile hold (-inf, 0, 0)
        float big = -INFINITY;
#pragma unroll 1
        for (int w = 0; w < nactive; ++w) big = fmaxf(big, sm.wm[w]);
        const float bs = big > -INFINITY ? big : 0.f;
        float a = 0.f, l = 0.f;
#pragma unroll 1
        for (int w = 0; w < nactive; ++w) {
            const float wt = exp2f(sm.wm[w] - bs);
            a = fmaf(sm.wacc[w][tid], wt, a);
            l = fmaf(sm.wl[w], wt, l);
        }
        p.attn_part[(static_cast<int64_t>(geo.h) * p.splits + geo.split) * D + tid] = a;
        if (tid == 0) {
            float* ml = p.attn_part + static_cast<int64_t>(p.heads) * p.splits * D + (static_cast<int64_t>(geo.h) * p.splits + geo.split) * 2;
            ml[0] = big;
            ml[1] = l;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int count_of(int n, int b, int G) { return n > b ? (n - b + G - 1) / G : 0; }
__device__ __forceinline__ int log2i(int v) { return 31 - __clz(v); }

// greedy pick: is candidate (v, i) better than (best, bi)?  NaN counts as the largest value (the rule of a
// host arg-max), the lowest index wins ties.
__device__ __noinline__ bool better(float v, int i, float best, int bi) {
    const bool vn = v != v, bn = best != best;
    if (vn != bn) return vn;
    if (vn) return i < bi;
    return v > best || (v == best && i < bi);
}

__global__ void __launch_bounds__(kThreads, 1) step_tile_kernel(const __grid_constant__ StepParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int gr = (g >> 1) + 4 * (g & 1);  // int8 weight tiles: the tile row of instruction row g (rows r and r + 4 are neighbours)
    const int G = gridDim.x, b = blockIdx.x;
    const int A = p.heads * p.D;
    {
        const uint64_t* src = reinterpret_cast<const uint64_t*>(p.L);
        uint64_t* dst = reinterpret_cast<uint64_t*>(S.layers);
        const int words = (p.layers + 1) * static_cast<int>(sizeof(StepLayer) / 8);
        for (int i = tid; i < words; i += kThreads) dst[i] = src[i];
    }

    // Position, cache slice, RoPE row and the tile counts are the same in every layer of the step.
    int64_t tok = *p.token;
    {
        int nf = *p.filled;
        int64_t pos = *p.cache_position;
        if (nf < 0 || nf > p.S) {
            if (p.err_flag && tid == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_LENGTH);
            nf = nf < 0 ? 0 : p.S;
        }
        const bool pos_ok = pos >= 0 && pos < p.S;
        if (!pos_ok) {
            if (p.err_flag && tid == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_POSITION);
            pos = pos < 0 ? 0 : p.S - 1;
        }
        if (tok < 0 || tok >= p.V) {
            if (p.err_flag && tid == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_TOKEN);
            tok = tok < 0 ? 0 : p.V - 1;
        }
        if (tid == 0) {
            Geo& geo = S.geo;
            geo.H = p.H; geo.A = A; geo.F = p.F; geo.E = p.E; geo.K = p.K; geo.S = p.S; geo.V = p.V; geo.G = G; geo.b = b;
            geo.layers = p.layers;
            geo.shF4 = log2i(p.F >> 2);
            geo.fpair = p.F <= 1024 && p.K >= 2;
            geo.ftiles = geo.fpair ? (p.K + 1) / 2 : p.K;
            geo.f_magic = (65536 + geo.ftiles - 1) / geo.ftiles;
            geo.f_blocks = count_of(p.H / 8, b, G);
            const bool has_unit = b < p.heads * p.splits;
            const int unit = has_unit ? b : 0;
            geo.kv16 = p.kv_int8 ? 0 : 1;
            // int8 codes: the smallest tile of 16, 32 or 64 positions with which no warp of a unit gets a second tile (a tile
            // is one warp's serial work, so short contexts are cut finer); fp16 values: 32 positions (8 KB of keys)
            geo.kvt = kKvTile / 2;
            if (p.kv_int8) {
                geo.kvt = 16;
                while (geo.kvt < kKvTile && ((nf + geo.kvt - 1) / geo.kvt + p.splits - 1) / p.splits > kStreamWarps) geo.kvt *= 2;
            }
            const int ntile_total = (nf + geo.kvt - 1) / geo.kvt;
            const int tps = (ntile_total + p.splits - 1) / p.splits;
            geo.h = unit / p.splits;
            geo.split = unit - geo.h * p.splits;
            geo.pos = static_cast<int>(pos);
            geo.nf = nf;
            geo.has_unit = has_unit ? 1 : 0;
            geo.tile0 = geo.split * tps;
            const int tile1 = min(geo.tile0 + tps, ntile_total);
            const int ptile = static_cast<int>(pos) / geo.kvt;
            geo.owner = has_unit && pos_ok && pos < nf && ptile >= geo.tile0 && ptile < tile1;
            geo.nt[KA] = count_of(3 * A / 8, b, G);
            geo.nt[KB] = has_unit && tile1 > geo.tile0 ? tile1 - geo.tile0 : 0;
            geo.nt[KC] = count_of(p.H / 8, b, G);
            geo.nt[KD] = count_of((p.E + 3) / 4, b, G);
            geo.nt[KE] = count_of(p.K * p.F / 4, b, G);
            geo.nt[KF] = geo.f_blocks * geo.ftiles;
            geo.nt[6] = count_of(p.V / 8, b, G);
            geo.nt[7] = 0;
        }
        if (tid < kHeadDim) {
            S.cs[tid] = __half2float(p.rope_cos[pos * kHeadDim + tid]);
            S.cs[kHeadDim + tid] = __half2float(p.rope_sin[pos * kHeadDim + tid]);
        }
    }
    if (tid == 0) {
        for (int st = 0; st < kStreamWarps; ++st) {
            mbar_init(smem_u32(&S.full_bars[st]), 1u);
            mbar_init(smem_u32(&S.empty_bars[st]), 1u);
        }
        mbar_fence_init();
        S.ready_layer = -1;
    }
    __syncthreads();  // the one barrier of all warps: from here on producers and consumers only meet at the stages
    if (warp >= kStreamWarps) {
        producer_loop(S, p.err_flag, 2 * (warp - kStreamWarps));
        return;
    }
    const Geo& geo = S.geo;
    const uint32_t full_bar = smem_u32(&S.full_bars[warp]), empty_bar = smem_u32(&S.empty_bars[warp]);
    uint32_t c_par = 0;  // parity of the next tile's arrival in this warp's stage
    int cbase = 0;  // the same place for the phase being worked on
    unsigned char* const my_stage = S.ring + static_cast<size_t>(warp) * kStageBytes;

    const uint32_t epoch = ld_acquire_u32(p.bar_epoch);
    unsigned int bar_target = epoch * static_cast<unsigned int>(p.barriers_per_launch) * gridDim.x;
    const uint32_t tag0 = epoch * 64u;  // tag of layer l's exchanges: tag0 + l + 1 (at most 33 layers per launch)
    const __half* const embed_row = p.embed + tok * static_cast<int64_t>(p.H);
    float pw1v[4], pw2v[4];
    plane_weights(t, true, pw1v);
    plane_weights(t, false, pw2v);
    const int bseg = g < 6 ? g : (g & 1);  // plane segment this lane feeds to B: first half planes 0-2, second half planes 0-2
    float* const fsx = reinterpret_cast<float*>(S.big + kBigPlaneBytes);  // group scales of the routed experts' activations
    float pick_v = -INFINITY;
    int pick_i = 0x7fffffff;
    int l = 0, ph = 0;  // phase: 0 q.k.v / lm_head, 1 attention, 2 o_proj, 3 router, 4 gate/up, 5 down
    const int nphases = 6 * p.layers + 1;

    auto grid_arrive = [&]() {  // after a block barrier: the writes of the whole block are ordered before the arrival
        bar_target += gridDim.x;
        if (tid == 0) red_release_add(p.bar_counter, 1u);
    };
    auto grid_wait = [&]() {
        if (tid == 0) {
            unsigned int n = 0;
            while (static_cast<int>(ld_acquire_u32(p.bar_counter) - bar_target) < 0) {
                if (++n > kBarrierSpinLimit || others_gave_up(p.err_flag, n)) {
                    if (p.err_flag) atomicOr(p.err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
                    break;
                }
            }
        }
        consumer_sync();
    };

#pragma unroll 1
    for (int step = 0; step < nphases; ++step) {
        stamp(p, step);
        const StepLayer& L = S.layers[l];
        const bool last = l == p.layers;
        const int ntiles = last ? geo.nt[6] : geo.nt[ph];
        const int lt0 = warp - cbase + (warp < cbase ? kStreamWarps : 0);  // this warp's first tile of the phase
        cbase = (cbase + ntiles) % kStreamWarps;
        // flagged-word buffers of this layer (parity l & 1) and of the previous layer's output
        const int par = l & 1, ppar = par ^ 1;
        const uint32_t tag = tag0 + l + 1;
        unsigned long long* const f_x2 = p.fl_x + par * 2048;            // this layer's output (down phase)
        const unsigned long long* const f_xin = p.fl_x + ppar * 2048;    // the previous layer's output
        unsigned long long* const f_xa = p.fl_x + (2 + par) * 2048;      // residual stream after attention
        unsigned long long* const f_qkv = p.fl_qkv + par * 3 * 2048;
        unsigned long long* const f_stats = p.fl_stats + par * 2048;
        unsigned long long* const f_logits = p.fl_logits + par * 128;
        unsigned long long* const f_act = p.fl_act + par * 4096;
        float sq = 0.f, sk = 0.f;  // phase A: sums of squares of the q / k values this lane stored

        if (ph == 1) {
            if (geo.has_unit) {
                AttnSm& sm = *reinterpret_cast<AttnSm*>(S.big);
                attention_prologue(p, L, S, f_qkv, f_stats, tag);
                {
                    float m_i = -INFINITY, l_i = 0.f;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                    for (int lt = lt0; lt < ntiles; lt += kStreamWarps) {
                        if (geo.kv16) {
                            if (!stage_acquire(full_bar, c_par, p.err_flag)) break;
                            c_par ^= 1u;
                            attention_tile16(my_stage, sm, geo, lt, lane, warp, p.qk_scale_log2, m_i, l_i, acc);
                            stage_release(empty_bar);
                            continue;
                        }
                        // the scales of the tile's positions (two per lane), requested before the wait for the codes
                        float kscale[2], vscale[2];
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const int pos = (geo.tile0 + lt) * geo.kvt + 32 * r + lane;
                            const bool in = 32 * r + lane < geo.kvt && pos < geo.nf;
                            const int64_t at = static_cast<int64_t>(geo.h) * geo.S + (in ? pos : 0);
                            const bool fresh = geo.owner && pos == geo.pos;  // the new token: the scales this block has just derived
                            kscale[r] = fresh ? __half2float(__ushort_as_half(sm.newks)) : (in ? __half2float(__ldcg(L.ks + at)) : 0.f);
                            vscale[r] = fresh ? __half2float(__ushort_as_half(sm.newvs)) : (in ? __half2float(__ldcg(L.vs + at)) : 0.f);
                        }
                        if (!stage_acquire(full_bar, c_par, p.err_flag)) break;
                        c_par ^= 1u;
                        if (geo.kvt == 16) attention_tile<16>(my_stage, sm, geo, lt, lane, warp, pw1v, kscale, vscale, m_i, l_i, acc);
                        else if (geo.kvt == 32) attention_tile<32>(my_stage, sm, geo, lt, lane, warp, pw1v, kscale, vscale, m_i, l_i, acc);
                        else attention_tile<kKvTile>(my_stage, sm, geo, lt, lane, warp, pw1v, kscale, vscale, m_i, l_i, acc);
                        stage_release(empty_bar);
                    }
                    *reinterpret_cast<float4*>(&sm.wacc[warp][lane * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    if (lane == 0) {
                        sm.wm[warp] = m_i;
                        sm.wl[warp] = l_i;
                    }
                }
                consumer_sync();
                attention_partial(p, S);
            }
            // the one grid barrier of the layer: the o_proj phase of every block merges the partials of all units
            consumer_sync();
            grid_arrive();
        } else {
            // ---- block-wide preparation of the phase -----------------------------------------------------
            if (ph == 4) {
                if (warp == 0) {  // one warp routes, the others pick the result up from shared memory
                    int id;
                    float w;
                    warp_topk(f_logits, tag, p.err_flag, p.E, p.K, p.norm_topk != 0, lane, id, w);
                    S.route_id[lane] = id;
                    S.route_w[lane] = lane < p.K ? w : 0.f;
                    if (b == 0 && lane < p.K) {
                        p.top_i[static_cast<int64_t>(l) * p.K + lane] = id;
                        p.top_w[lane] = __float2half_rn(w);
                    }
                    __threadfence_block();
                    if (lane == 0) S.ready_layer = l;  // the producers may start the expert tiles of this layer
                }
                consumer_sync();
            } else if (ph == 2) {
                grid_wait();
                prepare_attention_output(p, S);
            } else if (ph == 0) {
                if (!last && geo.has_unit && !geo.kv16) {
                    // the scales of this warp's first KV tile of the coming attention phase, towards the L2 cache
                    const int ltb = warp - cbase + (warp < cbase ? kStreamWarps : 0);
                    const int pos = (geo.tile0 + ltb) * geo.kvt + lane;
                    if (ltb < geo.nt[KB] && lane < geo.kvt && pos < geo.nf) {
                        const int64_t at = static_cast<int64_t>(geo.h) * geo.S + pos;
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(L.ks + at));
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(L.vs + at));
                        if (geo.kvt > 32 && pos + 32 < geo.nf) {
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(L.ks + at + 32));
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(L.vs + at + 32));
                        }
                    }
                }
                prepare(p.eps, embed_row, l == 0 ? nullptr : f_xin, tag - 1, 2, L.ln1, p.H, p.H >> 7, S.xplanes, S.xsx, nullptr, S.red, p.err_flag);
            } else if (ph == 3) {
                prepare(p.eps, nullptr, f_xa, tag, 2, L.ln2, p.H, p.H >> 7, S.xplanes, S.xsx, S.xh, S.red, p.err_flag);
            } else {
                prepare(p.eps, nullptr, f_act, tag, 2, nullptr, p.F, (p.K * p.F) >> 7, S.big, fsx, nullptr, S.red, p.err_flag);
            }
            // ---- this warp's tiles of the phase: a warp finishes the rows of its tile by itself ------------------
            {
                const int K = ph == 2 ? A : (ph == 5 ? p.F : p.H);
#pragma unroll 1
                for (int lt = lt0; lt < ntiles; lt += kStreamWarps) {
                    const int tg = b + lt * G;  // global tile index (not in the down phase)
                    __half resid = __float2half_rn(0.f);
                    if (ph == 2) {  // the residual of this lane's row (this block has seen the tag of every word in phase A)
                        const int n = tg * 8 + gr;
                        resid = l == 0 ? embed_row[n] : __ushort_as_half(static_cast<unsigned short>((flag_load(f_xin + (n >> 1)) >> (16 * (n & 1))) & 0xffffu));
                    }
                    if (!stage_acquire(full_bar, c_par, p.err_flag)) break;
                    c_par ^= 1u;
                    float val;
                    if (ph == 3) {
                        val = tile_f16(my_stage, p.H, g, t, S.xh);
                        val += __shfl_xor_sync(0xffffffffu, val, 1);
                        val += __shfl_xor_sync(0xffffffffu, val, 16);
                    } else if (ph == 5) {
                        // one or two routed experts' rows of the same 8 outputs: each against its own activation planes
                        const int j = udiv_small(lt, geo.f_magic), pp = lt - j * geo.ftiles;
                        const int seg = (K >> 1) + kPad, slot = geo.fpair ? 2 * pp : pp;
                        const __half* sc = reinterpret_cast<const __half*>(my_stage + kScaleOff) + gr * (K >> 7);
                        val = tile_s8(my_stage, K, gr, t, S.big + slot * 6 * seg + bseg * seg, fsx + slot * (K >> 7), sc, pw2v);
                        val += __shfl_xor_sync(0xffffffffu, val, 1);
                        val += __shfl_xor_sync(0xffffffffu, val, 2);
                        if (t == 0) S.part[(j * p.K + slot) * 8 + gr] = val;
                        if (geo.fpair && slot + 1 < p.K) {  // tile rows 8-15: two runs further
                            val = tile_s8(my_stage + 8 * K + 2 * kRunPad, K, gr, t, S.big + (slot + 1) * 6 * seg + bseg * seg, fsx + (slot + 1) * (K >> 7),
                                          sc + 8 * (K >> 7), pw2v);
                            val += __shfl_xor_sync(0xffffffffu, val, 1);
                            val += __shfl_xor_sync(0xffffffffu, val, 2);
                            if (t == 0) S.part[(j * p.K + slot + 1) * 8 + gr] = val;
                        }
                    } else {
                        val = tile_s8(my_stage, K, gr, t, S.xplanes + bseg * ((K >> 1) + kPad), S.xsx,
                                      reinterpret_cast<const __half*>(my_stage + kScaleOff) + gr * (K >> 7), pw2v);
                        val += __shfl_xor_sync(0xffffffffu, val, 1);
                        val += __shfl_xor_sync(0xffffffffu, val, 2);
                    }
                    stage_release(empty_bar);
                    if (ph == 0) {
                        const int n = tg * 8 + gr;
                        const __half hv = __float2half_rn(val);
                        const float f = __half2float(hv);
                        if (t == 0) {
                            if (!last) {
                                flag_store(f_qkv + n, __half_as_ushort(hv), tag);
                                if (n < A) sq = fmaf(f, f, sq);
                                else if (n < 2 * A) sk = fmaf(f, f, sk);
                            } else {
                                p.logits[n] = hv;
                                if (better(f, n, pick_v, pick_i)) {
                                    pick_v = f;
                                    pick_i = n;
                                }
                            }
                        }
                    } else if (ph == 2) {
                        // the residual stream travels two values per word: tile rows r and r + 1 meet in the even row's lane
                        // (the lanes of tile row r + 1 are those of instruction row g + 2)
                        const uint32_t mine = __half_as_ushort(__hadd(__float2half_rn(val), resid));
                        const uint32_t next = __shfl_down_sync(0xffffffffu, mine, 8);
                        if (t == 0 && (gr & 1) == 0) flag_store(f_xa + ((tg * 8 + gr) >> 1), mine | (next << 16), tag);
                    } else if (ph == 3) {
                        const int e = tg * 4 + g;
                        if (t == 0 && g < 4 && e < p.E) {
                            const __half hv = __float2half_rn(val);
                            flag_store(f_logits + e, __half_as_ushort(hv), tag);
                            p.router_logits[static_cast<int64_t>(l) * p.E + e] = hv;  // kept for inspection
                        }
                    } else if (ph == 4) {
                        const float up = __shfl_down_sync(0xffffffffu, val, 4);  // tile rows 4-7 are the up rows: the next instruction row
                        const uint32_t mine = __half_as_ushort(__float2half_rn(val * (1.0f / (1.0f + expf(-val))) * up));
                        const uint32_t next = __shfl_down_sync(0xffffffffu, mine, 8);  // the activation of the next tile row
                        const int slot = tg >> geo.shF4, n = ((tg - (slot << geo.shF4)) << 2) + gr;
                        if (t == 0 && (gr == 0 || gr == 2)) flag_store(f_act + ((slot * p.F + n) >> 1), mine | (next << 16), tag);  // two per word
                    }
                }
            }
            if (ph == 5) {
                // the routed experts of a down row are consecutive tiles: routing-weighted sum in slot order
                const int nrows = geo.f_blocks * 8;
                consumer_sync();
#pragma unroll 1
                for (int i0 = 0; i0 < nrows; i0 += kConsumerThreads) {  // every thread makes every trip: the rows meet in pairs
                    const int i = i0 + tid;
                    const bool on = i < nrows;
                    const int j = i >> 3, r = i & 7;
                    const int n = (b + j * G) * 8 + r;
                    uint32_t mine = 0;
                    if (on) {
                        float out = 0.f;
#pragma unroll 1
                        for (int slot = 0; slot < p.K; ++slot) out = fmaf(S.route_w[slot], S.part[(j * p.K + slot) * 8 + r], out);
                        // the residual: this block has seen the tag of every word of the stream in the router phase
                        const __half resid = __ushort_as_half(static_cast<unsigned short>((flag_load(f_xa + (n >> 1)) >> (16 * (n & 1))) & 0xffffu));
                        mine = __half_as_ushort(__hadd(__float2half_rn(out), resid));
                    }
                    const uint32_t next = __shfl_down_sync(0xffffffffu, mine, 1);  // row n + 1: the neighbouring thread
                    if (on && (r & 1) == 0) flag_store(f_x2 + (n >> 1), mine | (next << 16), tag);
                }
            } else if (ph == 0) {
                if (!last) {
                    sq = warp_sum(sq);
                    sk = warp_sum(sk);
                    if (lane == 0) {
                        S.red[warp] = sq;
                        S.red[kWarps + warp] = sk;
                    }
                } else {
#pragma unroll 1
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, pick_v, o);
                        const int oi = __shfl_xor_sync(0xffffffffu, pick_i, o);
                        if (better(ov, oi, pick_v, pick_i)) {
                            pick_v = ov;
                            pick_i = oi;
                        }
                    }
                    if (lane == 0) {
                        S.red[warp] = pick_v;
                        reinterpret_cast<int*>(S.red)[kWarps + warp] = pick_i;
                    }
                }
            }
            // ---- end of the phase: the block's shared buffers are free again ----------------------------------------
            consumer_sync();
            if (ph == 0 && tid == 0) {
                if (!last) {
                    // this block's share of the sums of squares of the q and k rows (its rows as stored, in fp16)
                    float a = 0.f, c = 0.f;
                    for (int w = 0; w < kStreamWarps; ++w) {
                        a += S.red[w];
                        c += S.red[kWarps + w];
                    }
                    flag_store(f_stats + b, __float_as_uint(a), tag);
                    flag_store(f_stats + 1024 + b, __float_as_uint(c), tag);
                } else if (p.next_token != nullptr) {
                    // this block's candidate for the greedy pick
                    float best = S.red[0];
                    int bi = reinterpret_cast<int*>(S.red)[kWarps];
                    for (int w = 1; w < kStreamWarps; ++w) {
                        const float v = S.red[w];
                        const int i = reinterpret_cast<int*>(S.red)[kWarps + w];
                        if (better(v, i, best, bi)) {
                            best = v;
                            bi = i;
                        }
                    }
                    p.attn_part[2 * b] = best;
                    p.attn_part[2 * b + 1] = __int_as_float(bi);
                }
            }
            if (last) grid_arrive();  // the logits and this block's candidate are out
        }
        if (++ph == 6) {
            ph = 0;
            ++l;
        }
    }
    stamp(p, nphases);
    if (b != 0) return;
    grid_wait();  // block 0 ends the step: every block has delivered its logits and its candidate
    if (p.next_token != nullptr && b == 0 && warp == 0) {
        // greedy pick on the device: one candidate per block (written before the last barrier), merged here
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int bb = lane; bb < G; bb += 32) {
            const float v = __ldcg(p.attn_part + 2 * bb);
            const int i = __float_as_int(__ldcg(p.attn_part + 2 * bb + 1));
            if (better(v, i, best, bi)) {
                best = v;
                bi = i;
            }
        }
#pragma unroll 1
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ob, oi, best, bi)) {
                best = ob;
                bi = oi;
            }
        }
        if (lane == 0) {
            const int64_t pick = (bi >= 0 && bi < p.V) ? bi : 0;
            *p.next_token = pick;
            if (p.token_log != nullptr) p.token_log[geo.pos] = pick;
            if (p.self_feed) {
                // every block read the three step scalars before its first grid barrier, long ago: the next launch
                // finds the picked token, the next slot and the next length
                *const_cast<int64_t*>(p.token) = pick;
                *const_cast<int64_t*>(p.cache_position) += 1;
                *const_cast<int32_t*>(p.filled) += 1;
            }
        }
    }
    if (b == 0 && tid == 0) atomicAdd(p.bar_epoch, 1u);
}

}  // namespace tile

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static_assert(sizeof(tile::Smem) + 128 <= 227 * 1024, "the block's shared memory must fit one SM");
size_t tile_smem_bytes() { return sizeof(tile::Smem) + 128; }

int set_flag_spin_limit(int polls) {
    if (polls < 1 || polls > (1 << 24)) return set_error(LEMOQ_ERR_INVALID, "set_tuning: flag poll limit %d outside [1, 2^24]", polls);
    const uint32_t v = static_cast<uint32_t>(polls);
    const cudaError_t err = cudaMemcpyToSymbol(tile::c_flag_spin_limit, &v, sizeof(v));
    if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "set_tuning: %s", cudaGetErrorString(err));
    return LEMOQ_OK;
}
bool tile_eligible(const lemoq_step_desc& d) {
    const int A = d.heads * d.head_dim;
    if (d.group_size != 128) return false;
    auto ok_dim = [](int n) { return n == 512 || n == 1024 || n == 2048; };  // row widths: powers of two, halves of whole 128-groups
    if (!ok_dim(d.hidden) || !ok_dim(A) || !ok_dim(d.ffn)) return false;
    if (d.head_dim != tile::kHeadDim) return false;
    if (d.experts > 128 || d.top_k > 32 || d.top_k > d.experts) return false;
    if (d.top_k * d.ffn > 8192) return false;                      // planes of the routed experts' activations
    if (d.vocab % 8 != 0 || d.layers + 1 > tile::kMaxLayers) return false;
    return true;
}

// Attention splits per head for the tile form: every (head, split) unit should have at most one KV tile per
// streaming warp.  A tile is one warp's serial work and every further split makes the merge of the partials longer
// (it takes the splits four at a time), so a short int8 cache is cut into tiles of 32 positions, about 8 per unit and
// at most 6 splits, and a long one into tiles of 64, 10 per unit (measured at 1024 and 4096 cached positions).
int tile_attention_splits(const lemoq_step_desc& d, int grid) {
    const int tiles64 = (d.max_len + tile::kKvTile - 1) / tile::kKvTile, tiles32 = (d.max_len + 31) / 32;
    int s;
    if (d.kv_int8 && tiles64 <= 30) s = std::min(6, (tiles32 + 7) / 8);
    else s = ((d.kv_int8 ? tiles64 : tiles32) + tile::kStreamWarps - 1) / tile::kStreamWarps;
    s = std::max(1, std::min(s, tile::kMaxSplits));
    return std::max(1, std::min(s, grid / d.heads));
}

int tile_grid(const lemoq_step_desc& d) {
    const bool verbose = getenv("LEMOQ_VERBOSE") != nullptr;
    int dev = 0, sms = 0, per_sm = 0, coop = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(tile::step_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tile_smem_bytes()));
    if (err == cudaSuccess)
        err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tile::step_tile_kernel, tile::kThreads, tile_smem_bytes());
    if (verbose)
        fprintf(stderr, "lemoq: tile step kernel: %s, sms %d, cooperative %d, blocks/SM %d, smem %zu\n", cudaGetErrorString(err), sms,
                coop, per_sm, tile_smem_bytes());
    if (err != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (!(coop && per_sm >= 1) || sms < d.heads) return 0;
    // the partial sums of the down phase of the fullest block must fit their array
    const int down_tiles = (d.hidden / 8 + sms - 1) / sms * d.top_k;
    return down_tiles * 8 <= tile::kPartFloats ? sms : 0;
}

int launch_step_tile(const StepParams& p, int grid, cudaStream_t stream) {
    StepParams local = p;
    void* args[] = {&local};
    const cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(tile::step_tile_kernel), dim3(grid), dim3(tile::kThreads),
                                                        args, tile_smem_bytes(), stream);
    if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "cooperative launch of the step kernel failed: %s", cudaGetErrorString(err));
    return LEMOQ_OK;
}

}  // namespace lemoq
