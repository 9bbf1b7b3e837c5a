// The whole decode step as ONE persistent cooperative kernel.
//
// Why: on B200 a dependent global-memory round trip costs ~0.7 us and a kernel boundary inside a
// graph 3-5 us, while a whole layer of the step only streams ~11 us worth of bytes.  With six
// all-to-all dependencies per layer, separate kernels spend most of the step waiting.  Here one
// block per SM stays resident for the whole step; the phases of a layer are separated by a grid
// barrier (~1.2 us), and every warp keeps a private ring of shared-memory stages that it fills
// with bulk asynchronous copies IN PROGRAM ORDER ACROSS PHASES: while a warp waits at a barrier the
// weights of its next tasks (q.k.v, o_proj, router and lm_head rows do not depend on activations)
// are already streaming in.  Only the expert rows have to wait for the routing.
//
// Arithmetic of the W8 rows: the activation vector of a phase is converted once per block into
// three planes of signed 7-bit digits (x = sx * (d2*2^14 + d1*2^7 + d0), sx a power of two chosen
// per 16-element lane chunk, so fp16 activations within 2^9 of the chunk maximum are represented
// exactly and the rest to 2^-20 of it); the int8 weight codes are then consumed as they are by the
// integer dot-product instruction (dp4a), 12 per 16 codes, with exact int32 partial sums that are
// combined and scaled in fp32.  No int8->float conversion of the weights takes place.
//
// Phases per layer (all blocks take part in each):
//   A  q.k.v rows          x = RMSNorm(x_prev)                                   -> qkv
//   B  attention           one (head, split) per block; fused q/k norm + RoPE + KV write; the block that
//                          arrives last at a head's counter merges the head's splits   -> attn
//   C  o_proj rows         + residual                                             -> x1
//   D  router rows (fp16)  h2 = RMSNorm(x1) (its planes stay in shared memory for E) -> router logits
//   E  expert gate/up      one warp per block derives the top-k from the logits; SwiGLU -> act
//   F  expert down         routing-weighted sum + residual                        -> x2
// then the lm_head rows on RMSNorm(x2), streamed as the q.k.v rows of a pseudo layer.
//
// The per-layer code runs once per layer, so it is cold in the first-level instruction cache every time:
// cold loops are rolled and the phases share one task loop, one activation-prep routine and one refill
// site on purpose (code size showed up directly in the step time).
#include <cstddef>
#include <cstdio>
#include <cstdlib>

#include "step_mega.h"
#include "stream.cuh"

namespace lemoq {

constexpr int kMegaWarps = 16;
constexpr int kMegaThreads = kMegaWarps * 32;
constexpr int kMegaStages = 2;
constexpr int kMegaStageBytes = 4224;  // 2 rows x 2048 codes + 2 x 32 bytes of scales, padded to 128
constexpr int kMegaScratchBytes = 28672 + 16384 + 4096 + 128;  // planes, raw staging, norm weights, reductions
constexpr int NCH = 4;  // activations up to 2048 wide
constexpr int kMegaMaxLayers = 33;  // layer descriptors kept in shared memory (layers + 1)
constexpr int kMaxSplits = 9;   // attention splits per head the merge is unrolled for
constexpr uint32_t kBarrierSpinLimit = 1u << 24;


// ---------------------------------------------------------------------------------------------
// grid barrier: monotonically increasing arrival counter, wrap-safe comparison, bounded spin
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct GridBarrier {
    unsigned int* counter;
    unsigned int target;  // value the counter reaches when everyone has arrived at the next barrier
    int* err_flag;
    __device__ __forceinline__ void sync() {
        __syncthreads();
        target += gridDim.x;
        if (threadIdx.x == 0) {
            // release at gpu scope is cumulative: it orders the writes of the whole block, which the block
            // barrier above made visible to this thread, before the arrival
            red_release_add(counter, 1u);
            unsigned int n = 0;
            while (static_cast<int>(ld_acquire_u32(counter) - target) < 0) {
                if (++n > kBarrierSpinLimit) {
                    if (err_flag) atomicOr(err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
                    break;
                }
            }
        }
        __syncthreads();
    }
};

// Phase time stamps (block 0, thread 0; nanoseconds of the global timer) for profiling the step.
__device__ __forceinline__ void stamp(const MegaParams& p, int slot) {
    if (p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.stamps[slot] = t;
    }
}

// Finer stamps of layer 1 only (64 extra slots after the phase stamps), for profiling.
__device__ __forceinline__ void substamp(const MegaParams& p, int l, int idx) {
    if (p.stamps != nullptr && l == 1 && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.stamps[6 * p.layers + 2 + idx] = t;
    }
}

// SM cycle counter of block 0 / thread 0 into the extra stamp slots 32.. (profiling; last writer wins).
__device__ __forceinline__ void dbg_clock(const MegaParams& p, int idx) {
#ifndef LEMOQ_MEGA_PROFILE
    (void)p;
    (void)idx;
    return;
#endif
    if (p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.stamps[6 * p.layers + 2 + 32 + idx] = clock64();
}

// ---------------------------------------------------------------------------------------------
// activation vectors as digit planes in shared memory
// ---------------------------------------------------------------------------------------------
// Layout of one quantised vector of up to NV lane chunks (a lane chunk = 16 consecutive elements;
// chunk index lc = k / 16): plane p word w of lane chunk lc at ((p * nlc + lc) * 4 + w) words; the
// chunk scales follow as floats.  A lane reads its chunk of a plane with one 128-bit load.

// Four activations (fp32 holding fp16-representable values) -> one packed word per plane.  `inv` is
// the exact power-of-two reciprocal of the chunk scale.  X = round(f * inv) (|X| < 2^20) is split in
// two's complement: X = d2 * 2^14 + d1 * 2^7 + d0 with d0, d1 in [0, 127] and d2 in [-64, 63].
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
// Chunk scale sx = 2^(floor(log2(amax)) - 19) (1 for an all-zero chunk) and its reciprocal.
__device__ __forceinline__ void chunk_scale(float amax, float& sx, float& inv) {
    const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu);  // biased exponent
    if (amax > 0.f && e > 20) {
        sx = __uint_as_float(static_cast<uint32_t>(e - 19) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(254 - (e - 19)) << 23);
    } else {  // zero or denormal-range chunk: fixed tiny scale keeps the arithmetic exact
        sx = __uint_as_float(static_cast<uint32_t>(2) << 23);
        inv = __uint_as_float(static_cast<uint32_t>(252) << 23);
    }
}

// One 4-element item of a vector of nlc lane chunks: four consecutive threads share a lane chunk, whole
// warps call this together (threads whose item lies past the end pass on = false and zeros).
__device__ __forceinline__ void quantise_item(uint32_t* dst, int nlc, int item, bool on, const float (&f)[4]) {
    float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float sx, inv;
    chunk_scale(amax, sx, inv);
    uint32_t w0, w1, w2;
    quantise4(f, inv, w0, w1, w2);
    if (on) {
        const int lc = item >> 2, w = item & 3;
        dst[(0 * nlc + lc) * 4 + w] = w0;
        dst[(1 * nlc + lc) * 4 + w] = w1;
        dst[(2 * nlc + lc) * 4 + w] = w2;
        if (w == 0) reinterpret_cast<float*>(dst + 3 * nlc * 4)[lc] = sx;
    }
}

// R W8 rows (codes and per-group scales in shared memory) against a quantised vector in shared memory:
// per-lane partial sums.  Lane `lane` owns the lane chunks c*32 + lane, i.e. codes c*512 + lane*16 .. +15.
template <int R>
__device__ __forceinline__ void dp_rows(float (&acc)[R], const unsigned char* const (&row)[R], const __half* const (&sc)[R],
                                        const uint32_t* __restrict__ xq, int K, int lane, int sbase, int sstride) {
    const int nlc = K >> 4;
    const float* sxs = reinterpret_cast<const float*>(xq + 3 * nlc * 4);
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int lc = c * 32 + lane;
        if (lc < nlc) {
            const uint4 x0 = *reinterpret_cast<const uint4*>(xq + (0 * nlc + lc) * 4);
            const uint4 x1 = *reinterpret_cast<const uint4*>(xq + (1 * nlc + lc) * 4);
            const uint4 x2 = *reinterpret_cast<const uint4*>(xq + (2 * nlc + lc) * 4);
            const float sx = sxs[lc];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint4 w = *reinterpret_cast<const uint4*>(row[r] + lc * 16);
                int s0 = __dp4a(static_cast<int>(w.x), static_cast<int>(x0.x), 0);
                int s1 = __dp4a(static_cast<int>(w.x), static_cast<int>(x1.x), 0);
                int s2 = __dp4a(static_cast<int>(w.x), static_cast<int>(x2.x), 0);
                s0 = __dp4a(static_cast<int>(w.y), static_cast<int>(x0.y), s0);
                s1 = __dp4a(static_cast<int>(w.y), static_cast<int>(x1.y), s1);
                s2 = __dp4a(static_cast<int>(w.y), static_cast<int>(x2.y), s2);
                s0 = __dp4a(static_cast<int>(w.z), static_cast<int>(x0.z), s0);
                s1 = __dp4a(static_cast<int>(w.z), static_cast<int>(x1.z), s1);
                s2 = __dp4a(static_cast<int>(w.z), static_cast<int>(x2.z), s2);
                s0 = __dp4a(static_cast<int>(w.w), static_cast<int>(x0.w), s0);
                s1 = __dp4a(static_cast<int>(w.w), static_cast<int>(x1.w), s1);
                s2 = __dp4a(static_cast<int>(w.w), static_cast<int>(x2.w), s2);
                const float t = fmaf(static_cast<float>(s2), 16384.f, fmaf(static_cast<float>(s1), 128.f, static_cast<float>(s0)));
                acc[r] = fmaf(t, sx * __half2float(sc[r][c * sstride + sbase]), acc[r]);
            }
        }
    }
}

// The same for R rows that each have their OWN quantised vector (the routed experts of one down row).
template <int R>
__device__ __forceinline__ void dp_rows_each(float (&acc)[R], const unsigned char* const (&row)[R], const __half* const (&sc)[R],
                                             const uint32_t* const (&xq)[R], int K, int lane, int sbase, int sstride) {
    const int nlc = K >> 4;
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
#pragma unroll 1
    for (int c = 0; c < NCH; ++c) {
        const int lc = c * 32 + lane;
        if (lc < nlc) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint4 x0 = *reinterpret_cast<const uint4*>(xq[r] + (0 * nlc + lc) * 4);
                const uint4 x1 = *reinterpret_cast<const uint4*>(xq[r] + (1 * nlc + lc) * 4);
                const uint4 x2 = *reinterpret_cast<const uint4*>(xq[r] + (2 * nlc + lc) * 4);
                const float sx = reinterpret_cast<const float*>(xq[r] + 3 * nlc * 4)[lc];
                const uint4 w = *reinterpret_cast<const uint4*>(row[r] + lc * 16);
                int s0 = __dp4a(static_cast<int>(w.x), static_cast<int>(x0.x), 0);
                int s1 = __dp4a(static_cast<int>(w.x), static_cast<int>(x1.x), 0);
                int s2 = __dp4a(static_cast<int>(w.x), static_cast<int>(x2.x), 0);
                s0 = __dp4a(static_cast<int>(w.y), static_cast<int>(x0.y), s0);
                s1 = __dp4a(static_cast<int>(w.y), static_cast<int>(x1.y), s1);
                s2 = __dp4a(static_cast<int>(w.y), static_cast<int>(x2.y), s2);
                s0 = __dp4a(static_cast<int>(w.z), static_cast<int>(x0.z), s0);
                s1 = __dp4a(static_cast<int>(w.z), static_cast<int>(x1.z), s1);
                s2 = __dp4a(static_cast<int>(w.z), static_cast<int>(x2.z), s2);
                s0 = __dp4a(static_cast<int>(w.w), static_cast<int>(x0.w), s0);
                s1 = __dp4a(static_cast<int>(w.w), static_cast<int>(x1.w), s1);
                s2 = __dp4a(static_cast<int>(w.w), static_cast<int>(x2.w), s2);
                const float t = fmaf(static_cast<float>(s2), 16384.f, fmaf(static_cast<float>(s1), 128.f, static_cast<float>(s0)));
                acc[r] = fmaf(t, sx * __half2float(sc[r][c * sstride + sbase]), acc[r]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// per-warp task stream: the order in which a warp will consume weight tasks over the whole step
// ---------------------------------------------------------------------------------------------
// Task kinds and what one stage holds (K = input width of the rows):
//   KIND_A  q.k.v rows (and the lm_head rows, as the q.k.v of a pseudo layer): two consecutive rows
//           [codes 2*K][scales 2*(K/group) halves]
//   KIND_C  o_proj rows, same layout
//   KIND_D  one fp16 router row [2*K]
//   KIND_E  gate row n and up row n of one routed expert [gate K][up K][gate scales][up scales]
//   KIND_F  down row n of `sps` consecutive routed experts [codes sps*F][scales sps*(F/group) halves]
// Every bulk copy of a kind is described by one CopyDesc in shared memory; lane c of the warp issues
// copy c, so the issue path is a handful of instructions whatever the kind.
enum Kind : int { KIND_A = 0, KIND_C = 1, KIND_D = 2, KIND_E = 3, KIND_F = 4, KIND_END = 5 };

struct CopyDesc {
    uint32_t field;     // byte offset of the source base pointer inside MegaLayer
    uint32_t bytes;     // size of the copy
    uint32_t dst;       // byte offset inside the stage
    uint32_t t_stride;  // source bytes per task index (row index n for E and F)
    uint32_t e_stride;  // source bytes per expert
    uint32_t cst;       // constant source offset
    uint32_t pad0, pad1;
};
struct StreamTable {
    CopyDesc copy[5][4];
    uint32_t ncopies[5];
    uint32_t tx[5];
};

#define LEMOQ_FIELD(name) static_cast<uint32_t>(offsetof(MegaLayer, name))

__device__ __forceinline__ void build_stream_table(StreamTable& t, const MegaParams& p, int sps) {
    const uint32_t H = p.H, A = p.heads * p.D, F = p.F, g = p.group;
    auto set = [&](int kind, int c, uint32_t field, uint32_t bytes, uint32_t dst, uint32_t ts, uint32_t es, uint32_t cst) {
        t.copy[kind][c] = CopyDesc{field, bytes, dst, ts, es, cst, 0u, 0u};
    };
    set(KIND_A, 0, LEMOQ_FIELD(qkv_codes), 2 * H, 0, 2 * H, 0, 0);
    set(KIND_A, 1, LEMOQ_FIELD(qkv_scale), 4 * (H / g), 2 * H, 4 * (H / g), 0, 0);
    t.ncopies[KIND_A] = 2;
    t.tx[KIND_A] = 2 * H + 4 * (H / g);
    set(KIND_C, 0, LEMOQ_FIELD(o_codes), 2 * A, 0, 2 * A, 0, 0);
    set(KIND_C, 1, LEMOQ_FIELD(o_scale), 4 * (A / g), 2 * A, 4 * (A / g), 0, 0);
    t.ncopies[KIND_C] = 2;
    t.tx[KIND_C] = 2 * A + 4 * (A / g);
    set(KIND_D, 0, LEMOQ_FIELD(router), 2 * H, 0, 2 * H, 0, 0);
    t.ncopies[KIND_D] = 1;
    t.tx[KIND_D] = 2 * H;
    const uint32_t sb = 2 * (H / g);
    set(KIND_E, 0, LEMOQ_FIELD(gu_codes), H, 0, H, 2 * F * H, 0);
    set(KIND_E, 1, LEMOQ_FIELD(gu_codes), H, H, H, 2 * F * H, F * H);
    set(KIND_E, 2, LEMOQ_FIELD(gu_scale), sb, 2 * H, sb, 2 * F * sb, 0);
    set(KIND_E, 3, LEMOQ_FIELD(gu_scale), sb, 2 * H + sb, sb, 2 * F * sb, F * sb);
    t.ncopies[KIND_E] = 4;
    t.tx[KIND_E] = 2 * H + 2 * sb;
    const uint32_t gb = 2 * (F / g);
    set(KIND_F, 0, LEMOQ_FIELD(dn_codes), F, 0, F, H * F, 0);
    set(KIND_F, 1, LEMOQ_FIELD(dn_scale), gb, sps * F, gb, H * gb, 0);
    t.ncopies[KIND_F] = 2;  // per routed expert of the stage
    t.tx[KIND_F] = F + gb;  // per routed expert of the stage
    if (p.debug & 1) {  // timing experiment (wrong results): no separate copies of the scales
        t.ncopies[KIND_A] = 1; t.tx[KIND_A] = 2 * H;
        t.ncopies[KIND_C] = 1; t.tx[KIND_C] = 2 * A;
        t.ncopies[KIND_E] = 2; t.tx[KIND_E] = 2 * H;
    }
}

struct WarpStream {
    const MegaParams* P;
    const StreamTable* T;
    const MegaLayer* LS;      // layer descriptors in shared memory
    WarpRing<kMegaStages> ring;
    const unsigned char* my;  // generic pointer to this warp's stage 0
    int wg, G, lane;
    int cnt[5];               // tasks of this warp per kind in a layer
    int cnt_lm;               // lm_head tasks of this warp
    int sps;                  // routed experts per stage in kind F
    int inflight;             // stages issued and not yet released
    int depth;                // upper bound of inflight
    int i_stage;              // next stage to fill
    int c_stage, c_par;       // next stage to consume and its barrier parity
    int ids_ready_layer;      // expert tasks of layers <= this may be issued
    int ids_reg;              // lane k holds the k-th expert id of ids_ready_layer
    // issue cursor: layer, kind, tasks left in the kind, task index, routed-expert slot, row inside the expert (E)
    int c_layer, c_kind, c_left, c_task, c_slot, c_n;
    // this lane's bulk copy of the current kind (lane c issues copy c; in kind F lane 2j + c copies for routed expert j)
    const char* lc_base;
    uint32_t lc_ts, lc_es, lc_bytes, lc_dst;
    uint32_t k_tx, k_ncop;    // bytes and copies per task (per routed expert in kind F) of the current kind

    __device__ __noinline__ static int count_of(int n, int wg, int G) { return n > wg ? (n - wg + G - 1) / G : 0; }
    __device__ __forceinline__ int count(int n) const { return count_of(n, wg, G); }
    __device__ __forceinline__ int kind_cnt(int k) const {
        int v = cnt[0];
#pragma unroll
        for (int i = 1; i < 5; ++i) v = k == i ? cnt[i] : v;
        return v;
    }
    __device__ __forceinline__ void enter_kind() {  // position the cursor on the first task of c_kind
        c_task = wg;
        c_slot = 0;
        c_n = wg;
        if (c_kind == KIND_E) {
            while (c_n >= P->F) {
                c_n -= P->F;
                ++c_slot;
            }
        }
        const bool isF = c_kind == KIND_F;
        const int ci = isF ? lane & 1 : lane;
        k_tx = T->tx[c_kind];
        k_ncop = T->ncopies[c_kind];
        lc_bytes = 0;
        lc_base = nullptr;
        lc_ts = lc_es = lc_dst = 0;
        if (ci < static_cast<int>(k_ncop)) {  // the table only describes the copies the kind has
            const CopyDesc d = T->copy[c_kind][ci];
            lc_base = *reinterpret_cast<const char* const*>(reinterpret_cast<const char*>(LS + c_layer) + d.field) + d.cst;
            lc_ts = d.t_stride;
            lc_es = d.e_stride;
            lc_bytes = d.bytes;
            lc_dst = d.dst + (isF ? (lane >> 1) * d.bytes : 0u);
        }
    }
    __device__ __forceinline__ void next_kind() {
        do {
            if (c_layer == P->layers) {  // the pseudo layer only has the lm_head rows
                c_kind = KIND_END;
                return;
            }
            if (c_kind == KIND_F) {
                c_kind = KIND_A;
                ++c_layer;
            } else {
                ++c_kind;
            }
            c_left = c_layer == P->layers ? cnt_lm : kind_cnt(c_kind);
        } while (c_left == 0);
        enter_kind();
    }
    __device__ __forceinline__ void start() {
        c_layer = 0;
        c_kind = KIND_A;
        c_left = cnt[KIND_A];
        if (c_left == 0) next_kind();
        else enter_kind();
    }
    __device__ __forceinline__ void advance() {
        if (c_kind == KIND_F) {
            c_slot += sps;
            if (c_slot < P->K) return;
            c_slot = 0;
        } else if (c_kind == KIND_E) {
            c_n += G;
            while (c_n >= P->F) {
                c_n -= P->F;
                ++c_slot;
            }
        }
        c_task += G;
        if (--c_left == 0) next_kind();
    }
    __device__ __forceinline__ bool allowed() const {
        if (c_kind == KIND_END) return false;
        return c_kind < KIND_E || c_layer <= ids_ready_layer;
    }
    // keep the ring full (called by the whole warp)
    __device__ __forceinline__ void pump() {
        while (inflight < depth && allowed()) {
            const uint32_t dst = ring.stage(i_stage), bar = ring.bar(i_stage);
            const bool isF = c_kind == KIND_F;
            const int nsl = isF ? min(sps, P->K - c_slot) : 1;
            // expert of this lane's copy (ignored by the kinds whose expert stride is zero)
            const int expert = __shfl_sync(0xffffffffu, ids_reg, (c_slot + (isF ? lane >> 1 : 0)) & 31);
            if (lane == 0) mbar_expect_tx(bar, k_tx * nsl);
            __syncwarp();
            if (lane < static_cast<int>(k_ncop) * nsl) {
                const uint32_t t = c_kind == KIND_E ? c_n : c_task;
                const uint64_t off = static_cast<uint64_t>(expert) * lc_es + static_cast<uint64_t>(t) * lc_ts;
                bulk_g2s(dst + lc_dst, lc_base + off, lc_bytes, bar);
            }
            i_stage = i_stage + 1 == kMegaStages ? 0 : i_stage + 1;
            ++inflight;
            advance();
        }
    }
    // wait for the oldest stage; returns its generic address (nullptr on timeout)
    __device__ __forceinline__ const unsigned char* acquire() {
        if (!mbar_wait(ring.bar(c_stage), c_par)) {
            if (P->err_flag && lane == 0) atomicOr(P->err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
            return nullptr;
        }
        return my + static_cast<size_t>(c_stage) * kMegaStageBytes;
    }
    // the stage after the oldest one (both are then released in order)
    __device__ __forceinline__ const unsigned char* acquire_next() {
        const int s = c_stage + 1 == kMegaStages ? 0 : c_stage + 1;
        const int par = c_stage + 1 == kMegaStages ? c_par ^ 1 : c_par;
        if (!mbar_wait(ring.bar(s), par)) {
            if (P->err_flag && lane == 0) atomicOr(P->err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
            return nullptr;
        }
        return my + static_cast<size_t>(s) * kMegaStageBytes;
    }
    __device__ __forceinline__ void release(int n) {  // the n oldest stages
        __syncwarp();
        c_stage += n;
        if (c_stage >= kMegaStages) {
            c_stage -= kMegaStages;
            c_par ^= 1;
        }
        inflight -= n;
        pump();
    }
};

// ---------------------------------------------------------------------------------------------
// routing: every warp derives softmax + top-k from the E fp16 logits (E <= 128), identically.
// Probabilities are positive floats, so their bit patterns order like unsigned integers: a warp-wide
// integer maximum plus a ballot gives the largest probability and its lowest index per round.
// ---------------------------------------------------------------------------------------------
struct TopK {
    int id;   // lane k: k-th expert id
    float w;  // lane k: its routing weight (fp16-rounded)
};
template <int PER>  // experts per lane: 2 for E <= 64, 4 for E <= 128
__device__ __noinline__ TopK warp_topk(const __half* __restrict__ logits, int E, int K, bool norm, int lane) {
    int id_reg;
    float w_reg;
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? __half2float(__ldcg(logits + e)) : -INFINITY;
        mx = fmaxf(mx, v[j]);
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
    return TopK{id_reg, w_reg};
}

// ---------------------------------------------------------------------------------------------
// attention phase (one (head, split) unit per block; head_dim 128, int8 KV with per-token scales)
// ---------------------------------------------------------------------------------------------
// Scores: one LANE per cached position.  The lane reads its position's 128 codes as eight 128-bit words
// and multiplies them with the digit planes of the roped query through dp4a (the planes sit in shared
// memory and are read as broadcasts), so a warp scores 32 positions with no shuffle at all.
// Values: the 32 probabilities of the warp go through shared memory; each lane then owns four output
// dimensions and walks the 32 positions, reading 4 codes (a coalesced 128-byte row per position).
// The block's warps are merged in shared memory, the block writes the (m, l, acc[128]) partial of its
// unit, and the block that arrives last at the head's counter merges the splits of the head.
constexpr int kHeadDim = 128;

struct AttnScratch {
    float q[kHeadDim];
    float kx[kHeadDim];
    float red[2 * kMegaWarps];
    float amax[8];
    float wm[kMegaWarps];
    float wl[kMegaWarps];
    float wacc[kMegaWarps][kHeadDim];
    float pbuf[kMegaWarps][32];
    __align__(16) uint32_t qplanes[3 * 8 * 4 + 8];
    int last_flag;
};

// What every layer's attention phase shares (computed once per step).
struct AttnConst {
    int pos;      // position of the new token (clamped into the cache)
    int n_start;  // this block's slice of the cached positions
    int n_end;
    int owner;    // the slice contains the new token: this block writes its K/V row
};

__device__ __forceinline__ float rope_elem(const float* __restrict__ xs, int d, float c, float s) {
    const float rot = d < kHeadDim / 2 ? -xs[d + kHeadDim / 2] : xs[d - kHeadDim / 2];
    return __half2float(__float2half_rn(__fadd_rn(__fmul_rn(xs[d], c), __fmul_rn(rot, s))));
}

__device__ __noinline__ void attention_phase(const MegaParams& p, const MegaLayer& L, AttnScratch& sm, const AttnConst ac,
                                             const float* __restrict__ cs /* cos[128], sin[128] of the position */) {
    constexpr int D = kHeadDim;
    const int unit = blockIdx.x;
    if (unit >= p.heads * p.splits) return;
    const int h = unit / p.splits, split = unit - h * p.splits;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int A = p.heads * D;
    const int64_t hs = static_cast<int64_t>(p.S) * D;
    int8_t* kc = L.kc + h * hs;
    int8_t* vc = L.vc + h * hs;
    __half* ks = L.ks + static_cast<int64_t>(h) * p.S;
    __half* vs = L.vs + static_cast<int64_t>(h) * p.S;

    // ---- q (and, for the owner, the new K/V row): RMSNorm over all heads, RoPE, int8 row -------------
    float ssq = 0.f, ssk = 0.f;
#pragma unroll 1
    for (int i = tid * 8; i < A; i += kMegaThreads * 8) {
        const uint4 qv = ld_cg16(p.qkv + i);
        const uint4 kv = ld_cg16(p.qkv + A + i);
        float f[8];
        unpack8_h(qv, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ssq = fmaf(f[j], f[j], ssq);
        unpack8_h(kv, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ssk = fmaf(f[j], f[j], ssk);
    }
    __half qraw = __float2half_rn(0.f), kraw = qraw, vraw = qraw, qw = qraw, kw = qraw;
    if (tid < D) {
        qraw = __ldcg(p.qkv + h * D + tid);
        kraw = __ldcg(p.qkv + A + h * D + tid);
        vraw = __ldcg(p.qkv + 2 * A + h * D + tid);
        qw = L.q_norm[h * D + tid];
        kw = L.k_norm[h * D + tid];
    }
    ssq = warp_sum(ssq);
    ssk = warp_sum(ssk);
    if (lane == 0) {
        sm.red[warp] = ssq;
        sm.red[kMegaWarps + warp] = ssk;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
#pragma unroll 1
    for (int w = 0; w < kMegaWarps; ++w) {
        tq += sm.red[w];
        tk += sm.red[kMegaWarps + w];
    }
    if (tid < D) {
        sm.q[tid] = norm_elem(qraw, 1.0f / sqrtf(tq / static_cast<float>(A) + p.eps), qw);
        sm.kx[tid] = norm_elem(kraw, 1.0f / sqrtf(tk / static_cast<float>(A) + p.eps), kw);
    }
    __syncthreads();
    float qd = 0.f, kn = 0.f;
    if (tid < D) {
        qd = rope_elem(sm.q, tid, cs[tid], cs[D + tid]);
        kn = rope_elem(sm.kx, tid, cs[tid], cs[D + tid]);
        if (ac.owner) {
            L.keys[h * hs + static_cast<int64_t>(ac.pos) * D + tid] = __float2half_rn(kn);
            L.values[h * hs + static_cast<int64_t>(ac.pos) * D + tid] = vraw;
            const float ak = warp_max(fabsf(kn)), av = warp_max(fabsf(__half2float(vraw)));
            if (lane == 0) {
                sm.amax[warp] = ak;
                sm.amax[4 + warp] = av;
            }
        }
    }
    __syncthreads();  // the un-rotated q has been read by everyone; the owner's maxima are in place
    if (tid < D) {
        sm.q[tid] = qd * p.qk_scale_log2;
        if (ac.owner) {
            const float amk = fmaxf(fmaxf(sm.amax[0], sm.amax[1]), fmaxf(sm.amax[2], sm.amax[3]));
            const float amv = fmaxf(fmaxf(sm.amax[4], sm.amax[5]), fmaxf(sm.amax[6], sm.amax[7]));
            const float sk = amk > 0.f ? __fdiv_rn(amk, 127.0f) : 1.0f;
            const float sv = amv > 0.f ? __fdiv_rn(amv, 127.0f) : 1.0f;
            const float qk = fminf(fmaxf(rintf(__fdiv_rn(kn, sk)), -127.0f), 127.0f);
            const float qv = fminf(fmaxf(rintf(__fdiv_rn(__half2float(vraw), sv)), -127.0f), 127.0f);
            kc[static_cast<int64_t>(ac.pos) * D + tid] = static_cast<int8_t>(static_cast<int>(qk));
            vc[static_cast<int64_t>(ac.pos) * D + tid] = static_cast<int8_t>(static_cast<int>(qv));
            if (tid == 0) {
                ks[ac.pos] = __float2half_rn(sk);
                vs[ac.pos] = __float2half_rn(sv);
            }
        }
    }
    __threadfence_block();
    __syncthreads();
    if (warp == 0) {  // the scaled, roped q as digit planes: 8 lane chunks of 16 dims
        const float f[4] = {sm.q[4 * lane], sm.q[4 * lane + 1], sm.q[4 * lane + 2], sm.q[4 * lane + 3]};
        quantise_item(sm.qplanes, 8, lane, true, f);
    }
    __syncthreads();

    // ---- scores and values: each warp takes blocks of 32 positions --------------------------------------
    float m_i = -INFINITY, l_i = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const float* qsx = reinterpret_cast<const float*>(sm.qplanes + 3 * 8 * 4);
#pragma unroll 1
    for (int base = ac.n_start + warp * 32; base < ac.n_end; base += kMegaWarps * 32) {
        const int n = min(base + lane, ac.n_end - 1);
        const bool has = base + lane < ac.n_end;
        uint4 kw8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) kw8[c] = ld_cg16(kc + static_cast<int64_t>(n) * D + c * 16);
        const float kscale = __half2float(__ldcg(ks + n));
        const float vscale = __half2float(__ldcg(vs + n));
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint4 x0 = *reinterpret_cast<const uint4*>(sm.qplanes + (0 * 8 + c) * 4);
            const uint4 x1 = *reinterpret_cast<const uint4*>(sm.qplanes + (1 * 8 + c) * 4);
            const uint4 x2 = *reinterpret_cast<const uint4*>(sm.qplanes + (2 * 8 + c) * 4);
            const uint4 w = kw8[c];
            int s0 = __dp4a(static_cast<int>(w.x), static_cast<int>(x0.x), 0);
            int s1 = __dp4a(static_cast<int>(w.x), static_cast<int>(x1.x), 0);
            int s2 = __dp4a(static_cast<int>(w.x), static_cast<int>(x2.x), 0);
            s0 = __dp4a(static_cast<int>(w.y), static_cast<int>(x0.y), s0);
            s1 = __dp4a(static_cast<int>(w.y), static_cast<int>(x1.y), s1);
            s2 = __dp4a(static_cast<int>(w.y), static_cast<int>(x2.y), s2);
            s0 = __dp4a(static_cast<int>(w.z), static_cast<int>(x0.z), s0);
            s1 = __dp4a(static_cast<int>(w.z), static_cast<int>(x1.z), s1);
            s2 = __dp4a(static_cast<int>(w.z), static_cast<int>(x2.z), s2);
            s0 = __dp4a(static_cast<int>(w.w), static_cast<int>(x0.w), s0);
            s1 = __dp4a(static_cast<int>(w.w), static_cast<int>(x1.w), s1);
            s2 = __dp4a(static_cast<int>(w.w), static_cast<int>(x2.w), s2);
            const float t = fmaf(static_cast<float>(s2), 16384.f, fmaf(static_cast<float>(s1), 128.f, static_cast<float>(s0)));
            s = fmaf(t, qsx[c], s);
        }
        // the value codes of the block (the key registers are free now): in flight during the softmax reductions
        uint32_t vw[32];
        {
            const int lastj = min(32, ac.n_end - base) - 1;
            const int8_t* vrow = vc + static_cast<int64_t>(base) * D + lane * 4;
#pragma unroll
            for (int j = 0; j < 32; ++j) vw[j] = __ldcg(reinterpret_cast<const uint32_t*>(vrow + static_cast<int64_t>(min(j, lastj)) * D));
        }
        s = has ? s * kscale : -INFINITY;
        const float m_new = fmaxf(m_i, warp_max(s));  // finite: lane 0 always has a position
        const float alpha = exp2f(m_i - m_new);
        const float pw = has ? exp2f(s - m_new) : 0.f;
        l_i = fmaf(l_i, alpha, warp_sum(pw));
        m_i = m_new;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] *= alpha;
        __syncwarp();
        sm.pbuf[warp][lane] = pw * vscale;
        __syncwarp();
        const int cnt = min(32, ac.n_end - base);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float pj = j < cnt ? sm.pbuf[warp][j] : 0.f;
            acc[0] = fmaf(pj, static_cast<float>(static_cast<int8_t>(vw[j] & 0xffu)), acc[0]);
            acc[1] = fmaf(pj, static_cast<float>(static_cast<int8_t>((vw[j] >> 8) & 0xffu)), acc[1]);
            acc[2] = fmaf(pj, static_cast<float>(static_cast<int8_t>((vw[j] >> 16) & 0xffu)), acc[2]);
            acc[3] = fmaf(pj, static_cast<float>(static_cast<int8_t>(vw[j] >> 24)), acc[3]);
        }
    }
    // ---- merge the warps of the block ----------------------------------------------------------------------
    *reinterpret_cast<float4*>(&sm.wacc[warp][lane * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if (lane == 0) {
        sm.wm[warp] = m_i;
        sm.wl[warp] = l_i;
    }
    __syncthreads();
    // partial layout: acc[(h*S + split)*D + d], then the (m, l) pairs
    if (tid < D) {
        // only the warps that had a block of positions hold anything
        const int nactive = min(kMegaWarps, (max(ac.n_end - ac.n_start, 0) + 31) >> 5);
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
        p.attn_part[(static_cast<int64_t>(h) * p.splits + split) * D + tid] = a;
        if (tid == 0) {
            float* ml = p.attn_part + static_cast<int64_t>(p.heads) * p.splits * D + (static_cast<int64_t>(h) * p.splits + split) * 2;
            ml[0] = big;
            ml[1] = l;
        }
    }
    // ---- the block that arrives last at its head's counter merges the splits of the head -------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int prev = atomicAdd(p.attn_counters + h, 1u);
        const bool is_last = prev + 1u == static_cast<unsigned int>(p.splits);
        if (is_last) p.attn_counters[h] = 0u;  // everyone of this layer has arrived: ready for the next one
        sm.last_flag = is_last ? 1 : 0;
    }
    __syncthreads();
    if (sm.last_flag != 0 && tid < D) {
        __threadfence();
        const float* hacc = p.attn_part + static_cast<int64_t>(h) * p.splits * D + tid;
        const float* hml = p.attn_part + static_cast<int64_t>(p.heads) * p.splits * D + static_cast<int64_t>(h) * p.splits * 2;
        float av[kMaxSplits];
        float2 mv[kMaxSplits];
#pragma unroll
        for (int j = 0; j < kMaxSplits; ++j) {
            if (j < p.splits) {
                av[j] = __ldcg(hacc + j * D);
                mv[j] = __ldcg(reinterpret_cast<const float2*>(hml + 2 * j));
            }
        }
        float big = -INFINITY;
#pragma unroll
        for (int j = 0; j < kMaxSplits; ++j)
            if (j < p.splits) big = fmaxf(big, mv[j].x);
        big = big > -INFINITY ? big : 0.f;
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxSplits; ++j) {
            if (j < p.splits) {
                const float w = exp2f(mv[j].x - big);
                den = fmaf(mv[j].y, w, den);
                num = fmaf(av[j], w, num);
            }
        }
        p.attn[h * D + tid] = __float2half_rn(den > 0.f ? num / den : num);
    }
}

// ---------------------------------------------------------------------------------------------
// block-wide preparation of a phase's activation vector
// ---------------------------------------------------------------------------------------------
// Sum over the block with ONE barrier: every thread adds the per-warp partials in warp order.
// `red` (>= kMegaWarps floats) must not be reused before the next block barrier.
__device__ __forceinline__ float block_sum_once(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kMegaWarps; ++w) t += red[w];
    return t;
}

// Scratch layout (bytes): [0, kRawOff) digit planes / attention scratch / reductions, then the raw fp16
// staging of the phase's activation vectors (16 KB) and of the norm weights (4 KB).
constexpr int kRawOff = 28672;
constexpr int kRawBytes = 16384;
constexpr int kNormWOff = kRawOff + kRawBytes;
constexpr int kNormWBytes = 4096;

// One routine prepares the activations of every weight phase.  Thread 0 brings `total` fp16 values
// (and the RMSNorm weights, when given) into shared memory with bulk copies; everyone waits on the
// copy's mbarrier; then the values are normalised (nw != null), quantised into digit planes
// (vectors of 2^vshift values each, vector v at dst + v * vec_words) and, when f32out is given,
// also stored as fp32 in the lane-major layout ((c*4 + q)*32 + ln)*4 + r for k = c*512 + ln*16 + q*4 + r.
__device__ __noinline__ void prepare_vectors(unsigned char* scratch, uint32_t bar, int parity, const MegaParams& p,
                                             const __half* __restrict__ src, const __half* __restrict__ nw, int total, int vshift,
                                             uint32_t* dst, int vec_words, float* f32out) {
    const __half* raw = reinterpret_cast<const __half*>(scratch + kRawOff);
    const __half* nws = reinterpret_cast<const __half*>(scratch + kNormWOff);
    float* red = reinterpret_cast<float*>(scratch + kNormWOff + kNormWBytes);
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, static_cast<uint32_t>(2 * total * (nw != nullptr ? 2 : 1)));
        bulk_g2s(smem_u32(raw), src, static_cast<uint32_t>(2 * total), bar);
        if (nw != nullptr) bulk_g2s(smem_u32(nws), nw, static_cast<uint32_t>(2 * total), bar);
    }
    if (!mbar_wait(bar, parity)) {
        if (p.err_flag && threadIdx.x == 0) atomicOr(p.err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
    }
    const int items = total >> 2;
    float rstd = 0.f;
    if (nw != nullptr) {
        float ss = 0.f;
#pragma unroll 1
        for (int item = threadIdx.x; item < items; item += kMegaThreads) {
            const uint2 xv = *reinterpret_cast<const uint2*>(raw + 4 * item);
            const __half* xh = reinterpret_cast<const __half*>(&xv);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss = fmaf(__half2float(xh[j]), __half2float(xh[j]), ss);
        }
        rstd = 1.0f / sqrtf(block_sum_once(ss, red) / static_cast<float>(total) + p.eps);
    }
    const int vmask = (1 << (vshift - 2)) - 1;  // items per vector - 1
#pragma unroll 1
    for (int item = threadIdx.x; item - static_cast<int>(threadIdx.x & 31) < items; item += kMegaThreads) {
        const bool on = item < items;
        float f[4] = {0.f, 0.f, 0.f, 0.f};
        if (on) {
            const uint2 xv = *reinterpret_cast<const uint2*>(raw + 4 * item);
            const __half* xh = reinterpret_cast<const __half*>(&xv);
            if (nw != nullptr) {
                const uint2 wv = *reinterpret_cast<const uint2*>(nws + 4 * item);
                const __half* wh = reinterpret_cast<const __half*>(&wv);
#pragma unroll
                for (int j = 0; j < 4; ++j) f[j] = norm_elem(xh[j], rstd, wh[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) f[j] = __half2float(xh[j]);
            }
        }
        const int vec = item >> (vshift - 2), within = item & vmask;
        quantise_item(dst + vec * vec_words, 1 << (vshift - 4), within, on, f);
        if (f32out != nullptr && on) {
            const int k = 4 * item;
            const int c = k >> 9, ln = (k & 511) >> 4, q = (k & 15) >> 2;
            *reinterpret_cast<float4*>(f32out + (((c * 4 + q) * 32 + ln) << 2)) = make_float4(f[0], f[1], f[2], f[3]);
        }
    }
    __syncthreads();
}

// L2 prefetch of a byte range by the whole block (128-byte lines).
__device__ __noinline__ void prefetch_l2(const void* ptr, int64_t bytes) {
    const char* c = reinterpret_cast<const char*>(ptr);
    for (int64_t off = static_cast<int64_t>(threadIdx.x) * 128; off < bytes; off += static_cast<int64_t>(kMegaThreads) * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
// One loop over the 6*layers + 1 phases with one task loop inside: the instruction footprint of a
// layer stays small enough to live in the instruction cache (every phase runs once per layer, so
// straight-line per-phase code would be fetched from L2 again in every layer).
__global__ void __launch_bounds__(kMegaThreads, 1) step_mega_kernel(const __grid_constant__ MegaParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* scratch = smem + kMegaWarps * kMegaStages * kMegaStageBytes + kMegaWarps * kMegaStages * 8 + 128;
    scratch = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(scratch) + 127) & ~uintptr_t(127));
    uint32_t* xq_s = reinterpret_cast<uint32_t*>(scratch);  // quantised activation vector (<= 6.7 KB)
    float* h2f = reinterpret_cast<float*>(scratch + 7680);   // fp32 h2, lane-major, for the fp16 router rows (8 KB)
    StreamTable& table = *reinterpret_cast<StreamTable*>(scratch + kMegaScratchBytes);
    float* cs_s = reinterpret_cast<float*>(scratch + kMegaScratchBytes + ((sizeof(StreamTable) + 127) & ~size_t(127)));  // cos, sin
    int* route_s = reinterpret_cast<int*>(cs_s + 2 * kHeadDim);  // routed expert ids and weights of the layer
    MegaLayer* layers_s = reinterpret_cast<MegaLayer*>(route_s + 64);  // the layer descriptors (layers + 1 of them)
    {
        const uint64_t* src = reinterpret_cast<const uint64_t*>(p.L);
        uint64_t* dst = reinterpret_cast<uint64_t*>(layers_s);
        const int words = (p.layers + 1) * static_cast<int>(sizeof(MegaLayer) / 8);
        for (int i = threadIdx.x; i < words; i += kMegaThreads) dst[i] = src[i];
    }

    WarpStream ws;
    ws.P = &p;
    ws.T = &table;
    ws.LS = layers_s;
    ws.G = gridDim.x * kMegaWarps;
    ws.wg = warp * gridDim.x + blockIdx.x;
    ws.lane = lane;
    ws.cnt[KIND_A] = ws.count(3 * p.heads * p.D / 2);
    ws.cnt[KIND_C] = ws.count(p.H / 2);
    ws.cnt[KIND_D] = ws.count(p.E);
    ws.cnt[KIND_E] = ws.count(p.K * p.F);
    ws.cnt[KIND_F] = ws.count(p.H);
    ws.cnt_lm = ws.count(p.V / 2);
    ws.sps = min(min(4, p.K), kMegaStageBytes / (p.F + 2 * (p.F / p.group)));
    if (threadIdx.x == 0) build_stream_table(table, p, ws.sps);
    ws.ring.init(smem, warp, kMegaWarps, kMegaStageBytes, lane);
    const uint32_t prep_bar = smem_u32(smem) + kMegaWarps * kMegaStages * kMegaStageBytes + kMegaWarps * kMegaStages * 8 + 64;
    if (threadIdx.x == 0) {
        mbar_init(prep_bar, 1u);
        mbar_fence_init();
    }
    ws.my = smem + static_cast<size_t>(warp) * kMegaStages * kMegaStageBytes;
    ws.inflight = 0;
    ws.depth = min(max(p.depth, 1), kMegaStages);
    ws.i_stage = ws.c_stage = ws.c_par = 0;
    ws.ids_ready_layer = -1;
    ws.ids_reg = 0;
    __syncthreads();
    ws.start();

    GridBarrier bar;
    bar.counter = p.bar_counter;
    bar.err_flag = p.err_flag;
    bar.target = ld_acquire_u32(p.bar_epoch) * static_cast<unsigned int>(p.barriers_per_launch) * gridDim.x;

    stamp(p, 0);
    const int A = p.heads * p.D;
    const int lane16 = lane * 16;
    const int sbase = lane16 / p.group, sstride = 512 / p.group;
    const int vec_words = 3 * (p.F / 16) * 4 + p.F / 16;  // one quantised expert activation vector

    // Position, cache slice and RoPE row are the same in every layer of the step.
    AttnConst ac;
    int kv_first = 0, kv_count = 0;
    {
        int nf = *p.filled;
        int64_t pos = *p.cache_position;
        if (nf < 0 || nf > p.S) {
            if (p.err_flag && threadIdx.x == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_LENGTH);
            nf = nf < 0 ? 0 : p.S;
        }
        const bool pos_ok = pos >= 0 && pos < p.S;
        if (!pos_ok) {
            if (p.err_flag && threadIdx.x == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_POSITION);
            pos = pos < 0 ? 0 : p.S - 1;
        }
        const int unit = blockIdx.x < static_cast<unsigned int>(p.heads * p.splits) ? blockIdx.x : 0;
        const int h = unit / p.splits, split = unit - h * p.splits;
        const int chunk = (nf + p.splits - 1) / p.splits;
        ac.pos = static_cast<int>(pos);
        ac.n_start = split * chunk;
        ac.n_end = min(ac.n_start + chunk, nf);
        ac.owner = pos_ok && pos >= ac.n_start && pos < ac.n_end;
        if (static_cast<int>(blockIdx.x) < p.heads * p.splits) {
            kv_first = h * p.S + ac.n_start;
            kv_count = ac.n_end > ac.n_start ? ac.n_end - ac.n_start : 0;
        }
        if (threadIdx.x < kHeadDim) {
            cs_s[threadIdx.x] = __half2float(p.rope_cos[pos * kHeadDim + threadIdx.x]);
            cs_s[kHeadDim + threadIdx.x] = __half2float(p.rope_sin[pos * kHeadDim + threadIdx.x]);
        }
    }

    const __half* x_prev = p.embed + (*p.token) * static_cast<int64_t>(p.H);
    float tw_reg = 0.f;
    float pick_v = -INFINITY;  // greedy pick over the logits this warp produced
    int pick_i = 0x7fffffff;
    int prep_par = 0;
    int l = 0, ph = 0;  // phase: 0 q.k.v / lm_head, 1 attention, 2 o_proj, 3 router, 4 gate/up, 5 down
    const int nphases = 6 * p.layers + 1;

#pragma unroll 1
    for (int step = 0; step < nphases; ++step) {
        const MegaLayer& L = layers_s[l];
        const bool last = l == p.layers;
        int ntasks = 0, K = p.H, nst = 1;
        if (ph == 0) dbg_clock(p, 24);
        if (ph == 2) dbg_clock(p, 25);
        // ---- block-wide preparation of the phase -----------------------------------------------------
        if (ph == 0 || ph == 2 || ph == 3) {
            if (ph == 0 && !last && kv_count > 0) {
                prefetch_l2(L.kc + static_cast<int64_t>(kv_first) * p.D, static_cast<int64_t>(kv_count) * p.D);
                prefetch_l2(L.vc + static_cast<int64_t>(kv_first) * p.D, static_cast<int64_t>(kv_count) * p.D);
                prefetch_l2(L.ks + kv_first, static_cast<int64_t>(kv_count) * 2);
                prefetch_l2(L.vs + kv_first, static_cast<int64_t>(kv_count) * 2);
            }
            if (ph == 2) K = A;
            prepare_vectors(scratch, prep_bar, prep_par, p, ph == 0 ? x_prev : (ph == 2 ? p.attn : p.xa),
                            ph == 0 ? L.ln1 : (ph == 2 ? nullptr : L.ln2), K, 31 - __clz(K), xq_s, 0, ph == 3 ? h2f : nullptr);
            prep_par ^= 1;
            ntasks = ph == 0 ? (last ? ws.cnt_lm : ws.cnt[KIND_A]) : (ph == 2 ? ws.cnt[KIND_C] : ws.cnt[KIND_D]);
        } else if (ph == 1) {
            AttnScratch& sm = *reinterpret_cast<AttnScratch*>(scratch);
            attention_phase(p, L, sm, ac, cs_s);
        } else if (ph == 4) {
            dbg_clock(p, 30);
            // one warp routes, the others pick the result up from shared memory
            if (warp == 0) {
                const __half* lg = p.router_logits + static_cast<int64_t>(l) * p.E;
                const TopK tk = p.E <= 64 ? warp_topk<2>(lg, p.E, p.K, p.norm_topk != 0, lane) : warp_topk<4>(lg, p.E, p.K, p.norm_topk != 0, lane);
                route_s[lane] = tk.id;
                route_s[32 + lane] = __float_as_int(tk.w);
            }
            dbg_clock(p, 31);
            __syncthreads();
            dbg_clock(p, 32);
            ws.ids_reg = route_s[lane];
            tw_reg = __int_as_float(route_s[32 + lane]);
            ws.ids_ready_layer = l;
            if (blockIdx.x == 0 && warp == 0 && lane < p.K) {
                p.top_i[static_cast<int64_t>(l) * p.K + lane] = ws.ids_reg;
                p.top_w[lane] = __float2half_rn(tw_reg);
            }
            ntasks = ws.cnt[KIND_E];
        } else {
            prepare_vectors(scratch, prep_bar, prep_par, p, p.act, nullptr, p.K * p.F, 31 - __clz(p.F),
                            reinterpret_cast<uint32_t*>(scratch), vec_words, nullptr);
            prep_par ^= 1;
            K = p.F;
            ntasks = ws.cnt[KIND_F];
            nst = (p.K + ws.sps - 1) / ws.sps;
        }
        ws.pump();  // the one place besides release(): start of the step, and the expert rows once the routing is known
        substamp(p, l, 2 * ph);
        const int gK = K / p.group;

        // ---- this warp's tasks of the phase ---------------------------------------------------------------
        // Every iteration takes one or two stages off the ring: two two-row W8 tasks at once (four rows against
        // one read of the activation planes), one router row, or the two stages of one down row.
        const bool rows2 = ph == 0 || ph == 2 || ph == 4;
#pragma unroll 1
        for (int i = 0; i < ntasks; i += rows2 ? 2 : 1) {
            const bool two = rows2 ? i + 1 < ntasks : nst > 1;
            const bool prof = ph == 5 && i == 0;
            if (prof) dbg_clock(p, 50);
            const unsigned char* st0 = ws.acquire();
            const unsigned char* st1 = two ? ws.acquire_next() : st0;
            if (!st0 || !st1) break;
            if (prof) dbg_clock(p, 51);
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            if (rows2) {
                const __half* sc0 = reinterpret_cast<const __half*>(st0 + 2 * K);
                const __half* sc1 = reinterpret_cast<const __half*>(st1 + 2 * K);
                const unsigned char* const rows[4] = {st0, st0 + K, st1, st1 + K};
                const __half* const scs[4] = {sc0, sc0 + gK, sc1, sc1 + gK};
                dp_rows<4>(part, rows, scs, xq_s, K, lane, sbase, sstride);
            } else if (ph == 3) {  // one fp16 router row against the fp32 h2
#pragma unroll 1
                for (int c = 0; c < NCH; ++c) {
                    const int k0 = c * 512 + lane16;
                    if (k0 < p.H) {
                        float hf[16];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 v = *reinterpret_cast<const float4*>(h2f + (((c * 4 + q) * 32 + lane) << 2));
                            hf[4 * q] = v.x;
                            hf[4 * q + 1] = v.y;
                            hf[4 * q + 2] = v.z;
                            hf[4 * q + 3] = v.w;
                        }
                        part[0] += dot8_h(*reinterpret_cast<const uint4*>(st0 + 2 * k0), &hf[0]);
                        part[0] += dot8_h(*reinterpret_cast<const uint4*>(st0 + 2 * k0 + 16), &hf[8]);
                    }
                }
            } else {  // down row n of the routed experts: sps (4) of them per stage, each against its own activations
                const uint32_t* planes = reinterpret_cast<const uint32_t*>(scratch);
#pragma unroll 1
                for (int s = 0; s < nst; ++s) {
                    const unsigned char* st = s == 0 ? st0 : st1;
                    const int slot0 = s * ws.sps;
                    const __half* sc = reinterpret_cast<const __half*>(st + ws.sps * p.F);
                    // slots past top_k (a last, partly filled stage) repeat the last valid one with weight zero
                    const int j1 = min(1, p.K - 1 - slot0), j2 = min(2, p.K - 1 - slot0), j3 = min(3, p.K - 1 - slot0);
                    const unsigned char* const rows[4] = {st, st + j1 * p.F, st + j2 * p.F, st + j3 * p.F};
                    const __half* const scs[4] = {sc, sc + j1 * gK, sc + j2 * gK, sc + j3 * gK};
                    const uint32_t* const xqs[4] = {planes + slot0 * vec_words, planes + (slot0 + j1) * vec_words,
                                                    planes + (slot0 + j2) * vec_words, planes + (slot0 + j3) * vec_words};
                    float one[4];
                    dp_rows_each<4>(one, rows, scs, xqs, p.F, lane, sbase, sstride);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool valid = j < ws.sps && slot0 + j < p.K;
                        const float tw = __shfl_sync(0xffffffffu, tw_reg, min(slot0 + j, 31));
                        part[0] = fmaf(valid ? tw : 0.f, one[j], part[0]);
                    }
                }
            }
            if (prof) dbg_clock(p, 52);
            ws.release(two ? 2 : 1);
            if (prof) dbg_clock(p, 53);
#pragma unroll
            for (int r = 0; r < 4; ++r) part[r] = warp_sum(part[r]);
            if (prof) dbg_clock(p, 54);
#pragma unroll 1
            for (int t = 0; t < (rows2 && two ? 2 : 1); ++t) {
                const int task = ws.wg + (i + t) * ws.G;
                const float a0 = t ? part[2] : part[0], a1 = t ? part[3] : part[1];
                if (ph == 0) {
                    if (lane < 2) (last ? p.logits : p.qkv)[task * 2 + lane] = __float2half_rn(lane == 0 ? a0 : a1);
                    if (last) {  // running greedy pick over this warp's logits (as stored: rounded to fp16), lowest index on ties
                        const float v0 = __half2float(__float2half_rn(a0)), v1 = __half2float(__float2half_rn(a1));
                        if (v0 > pick_v || (v0 == pick_v && task * 2 < pick_i)) {
                            pick_v = v0;
                            pick_i = task * 2;
                        }
                        if (v1 > pick_v || (v1 == pick_v && task * 2 + 1 < pick_i)) {
                            pick_v = v1;
                            pick_i = task * 2 + 1;
                        }
                    }
                } else if (ph == 2) {
                    if (lane < 2) {
                        const int n = task * 2 + lane;
                        p.xa[n] = __hadd(__float2half_rn(lane == 0 ? a0 : a1), __ldcg(x_prev + n));
                    }
                } else if (ph == 3) {
                    if (lane == 0) p.router_logits[static_cast<int64_t>(l) * p.E + task] = __float2half_rn(a0);
                } else if (ph == 4) {
                    if (lane == 0) p.act[task] = __float2half_rn(a0 * (1.0f / (1.0f + expf(-a0))) * a1);
                } else {
                    if (lane == 0) p.xb[task] = __hadd(__float2half_rn(a0), __ldcg(p.xa + task));
                }
            }
        }
        if (ph == 5) dbg_clock(p, 55);
        substamp(p, l, 2 * ph + 1);
        if (last && p.next_token != nullptr) {
            // this block's candidate for the greedy pick (the attention partials buffer is free by now)
            float* cv = reinterpret_cast<float*>(scratch);
            int* ci = reinterpret_cast<int*>(scratch + 256);
            if (lane == 0) {
                cv[warp] = pick_v;
                ci[warp] = pick_i;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                float best = cv[0];
                int bi = ci[0];
                for (int w = 1; w < kMegaWarps; ++w) {
                    if (cv[w] > best || (cv[w] == best && ci[w] < bi)) {
                        best = cv[w];
                        bi = ci[w];
                    }
                }
                p.attn_part[2 * blockIdx.x] = best;
                p.attn_part[2 * blockIdx.x + 1] = __int_as_float(bi);
            }
        }
        bar.sync();
        stamp(p, step + 1);
        if (++ph == 6) {
            ph = 0;
            ++l;
            x_prev = p.xb;
        }
    }
    if (p.next_token != nullptr && blockIdx.x == 0) {
        // greedy pick on the device: one candidate per block (written before the last barrier), merged here
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int b = lane; b < static_cast<int>(gridDim.x); b += 32) {
            const float v = __ldcg(p.attn_part + 2 * b);
            const int i = __float_as_int(__ldcg(p.attn_part + 2 * b + 1));
            if (v > best || (v == best && i < bi)) {
                best = v;
                bi = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) {
                best = ob;
                bi = oi;
            }
        }
        if (threadIdx.x == 0) *p.next_token = bi;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(p.bar_epoch, 1u);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
size_t mega_smem_bytes() {
    return static_cast<size_t>(kMegaWarps) * kMegaStages * kMegaStageBytes + kMegaWarps * kMegaStages * 8 + 512 +
           kMegaScratchBytes + sizeof(StreamTable) + 128 + 2 * kHeadDim * sizeof(float) + 64 * sizeof(int) + kMegaMaxLayers * sizeof(MegaLayer);
}

bool mega_eligible(const lemoq_step_desc& d) {
    const int A = d.heads * d.head_dim;
    const int g = d.group_size;
    if (g <= 0 || g % 16 != 0 || 512 % g != 0) return false;
    auto ok_dim = [&](int n) { return n % 512 == 0 && n <= 2048 && n % g == 0 && ((n / g) * 2 * 2) % 16 == 0; };
    if (!ok_dim(d.hidden) || !ok_dim(A) || !ok_dim(d.ffn)) return false;
    // one expert row of scales (gate/up rows and down rows are copied singly) must be a 16-byte multiple
    if (((d.hidden / g) * 2) % 16 != 0 || ((d.ffn / g) * 2) % 16 != 0) return false;
    if (d.ffn + 2 * (d.ffn / g) > kMegaStageBytes) return false;
    {  // the routed experts of one down row must fit the ring: at most kMegaStages stages per task
        int sps = kMegaStageBytes / (d.ffn + 2 * (d.ffn / g));
        sps = sps > 4 ? 4 : sps;
        if ((d.top_k + sps - 1) / sps > kMegaStages) return false;
        if (sps != 4 && sps < d.top_k) return false;  // the down rows are taken four routed experts at a time
    }
    if (d.head_dim != kHeadDim || !d.kv_int8) return false;  // the fp16-KV arm runs as chained kernels
    if (d.experts > 128 || d.top_k > 32 || d.top_k > d.experts) return false;
    if (d.vocab % 2 != 0 || d.layers + 1 > kMegaMaxLayers) return false;
    const size_t vec_words = 3 * (d.ffn / 16) * 4 + d.ffn / 16;
    if (static_cast<size_t>(d.top_k) * vec_words * 4 > kRawOff) return false;
    auto pow2 = [](int n) { return n > 0 && (n & (n - 1)) == 0; };
    if (!pow2(d.hidden) || !pow2(A) || !pow2(d.ffn)) return false;  // vectors are addressed by shifts
    if (static_cast<size_t>(d.top_k) * d.ffn * 2 > kRawBytes || d.hidden * 2 > kNormWBytes || A * 2 > kNormWBytes) return false;
    if (sizeof(AttnScratch) > kRawOff) return false;
    return true;
}

int mega_grid(const lemoq_step_desc& d, int splits) {
    (void)d;
    (void)splits;
    const bool verbose = getenv("LEMOQ_VERBOSE") != nullptr;
    int dev = 0, sms = 0, per_sm = 0, coop = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (err == cudaSuccess)
        err = cudaFuncSetAttribute(step_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(mega_smem_bytes()));
    if (err == cudaSuccess)
        err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, step_mega_kernel, kMegaThreads, mega_smem_bytes());
    if (verbose)
        fprintf(stderr, "lemoq: whole-step kernel: %s, sms %d, cooperative %d, blocks/SM %d, smem %zu\n",
                cudaGetErrorString(err), sms, coop, per_sm, mega_smem_bytes());
    if (err != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return (coop && per_sm >= 1) ? sms : 0;
}

int launch_step_mega(const MegaParams& p, int grid, cudaStream_t stream) {
    MegaParams local = p;
    void* args[] = {&local};
    const cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(step_mega_kernel), dim3(grid),
                                                        dim3(kMegaThreads), args, mega_smem_bytes(), stream);
    if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "cooperative launch of the step kernel failed: %s", cudaGetErrorString(err));
    return LEMOQ_OK;
}

}  // namespace lemoq
