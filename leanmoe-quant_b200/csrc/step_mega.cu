// The whole decode step as ONE persistent cooperative kernel.
//
// Why: on B200 a dependent global-memory round trip costs ~0.7 us and a kernel boundary inside a
// graph 3-5 us, while a whole layer of the step only streams ~11 us worth of bytes.  With six
// all-to-all dependencies per layer, separate kernels spend most of the step waiting.  Here one
// block per SM stays resident for the whole step; the six phases of a layer are separated by a
// grid barrier (~1.2 us), and every warp keeps a private ring of shared-memory stages that it
// fills with bulk asynchronous copies IN PROGRAM ORDER ACROSS PHASES: while a warp waits at a
// barrier the weights of its next tasks (q.k.v, o_proj, router and lm_head rows do not depend
// on activations) are already streaming in.  Only the expert rows have to wait for the routing.
//
// Phases per layer (all blocks take part in each):
//   A  q.k.v rows          x = RMSNorm(x_prev)                         -> qkv
//   B  attention           one (head, split) per block, fused q/k norm + RoPE + KV write; the last
//                          block of a head merges the splits              -> attn
//   C  o_proj rows         + residual                                     -> x1
//   D  router rows (fp16)  h2 = RMSNorm(x1)                               -> router logits
//   E  expert gate/up      every warp derives the top-k itself from the logits; SwiGLU -> act
//   F  expert down         routing-weighted sum + residual                -> x2
// then the lm_head rows on RMSNorm(x2).
//
// Numerics are those of the separate kernels (same rounding points, same reduction orders).
#include "step_mega.h"
#include "stream_gemv.cuh"

namespace lemoq {

constexpr int kMegaWarps = 12;
constexpr int kMegaThreads = kMegaWarps * 32;
constexpr int kMegaStages = 4;
constexpr int kMegaStageBytes = 4224;  // 2 rows x 2048 codes + 2 x 32 bytes of scales, padded to 128
constexpr int kMegaScratchBytes = 16384;
constexpr int kMegaMode = DOT_F16_FOLD;
constexpr int NCH = 4;  // activations up to 2048 wide
constexpr uint32_t kBarrierSpinLimit = 1u << 24;

enum Phase : int { PH_A = 0, PH_C = 1, PH_D = 2, PH_E = 3, PH_F = 4, PH_LM = 5, PH_END = 6 };

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
            __threadfence();
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

// ---------------------------------------------------------------------------------------------
// per-warp task stream: the order in which a warp will consume weight tasks over the whole step
// ---------------------------------------------------------------------------------------------
struct Cursor {
    int layer, phase, i, slot;
};

struct WarpStream {
    const MegaParams* P;
    WarpRing<kMegaStages> ring;
    const unsigned char* my;  // generic pointer to this warp's stage 0
    int wg, G, lane;
    int n_issued, n_consumed;
    int ids_ready_layer;  // expert tasks of layers <= this may be issued
    long long ids_reg;    // lane k holds the k-th expert id of ids_ready_layer
    Cursor cur;

    __device__ __forceinline__ int count(int n) const { return n > wg ? (n - wg + G - 1) / G : 0; }
    __device__ __forceinline__ int phase_count(int phase) const {
        const MegaParams& p = *P;
        switch (phase) {
            case PH_A: return count(3 * p.heads * p.D / 2);
            case PH_C: return count(p.H / 2);
            case PH_D: return count(p.E);
            case PH_E: return count(p.K * p.F);
            case PH_F: return count(p.H / 2);
            default: return count(p.V / 2);
        }
    }
    // move the cursor to the next valid task (or PH_END)
    __device__ __forceinline__ void normalise() {
        const MegaParams& p = *P;
        while (cur.phase != PH_END) {
            if (cur.i < phase_count(cur.phase)) return;
            cur.i = 0;
            cur.slot = 0;
            if (cur.phase == PH_LM) {
                cur.phase = PH_END;
            } else if (cur.phase == PH_F) {
                ++cur.layer;
                cur.phase = cur.layer < p.layers ? PH_A : PH_LM;
            } else {
                ++cur.phase;
            }
        }
    }
    __device__ __forceinline__ void advance() {
        if (cur.phase == PH_F) {
            if (++cur.slot < P->K) return;
            cur.slot = 0;
        }
        ++cur.i;
        normalise();
    }
    __device__ __forceinline__ bool allowed() const {
        if (cur.phase == PH_END) return false;
        if (cur.phase == PH_E || cur.phase == PH_F) return cur.layer <= ids_ready_layer;
        return true;
    }
    // lane 0: enqueue the copies of the cursor's task into stage s
    __device__ __forceinline__ void issue(int s, int expert) {
        const MegaParams& p = *P;
        const MegaLayer& L = p.L[cur.layer < p.layers ? cur.layer : 0];
        const int task = wg + cur.i * G;
        const uint32_t dst = ring.stage(s), bar = ring.bar(s);
        const int A = p.heads * p.D;
        switch (cur.phase) {
            case PH_A: {
                const int g = p.H / p.group;
                const uint32_t cb = 2 * p.H, sb = 2 * g * 2;
                mbar_expect_tx(bar, cb + sb);
                bulk_g2s(dst, L.qkv_codes + static_cast<int64_t>(task) * 2 * p.H, cb, bar);
                bulk_g2s(dst + cb, L.qkv_scale + static_cast<int64_t>(task) * 2 * g, sb, bar);
                break;
            }
            case PH_C: {
                const int g = A / p.group;
                const uint32_t cb = 2 * A, sb = 2 * g * 2;
                mbar_expect_tx(bar, cb + sb);
                bulk_g2s(dst, L.o_codes + static_cast<int64_t>(task) * 2 * A, cb, bar);
                bulk_g2s(dst + cb, L.o_scale + static_cast<int64_t>(task) * 2 * g, sb, bar);
                break;
            }
            case PH_D: {
                const uint32_t cb = 2 * p.H;
                mbar_expect_tx(bar, cb);
                bulk_g2s(dst, L.router + static_cast<int64_t>(task) * p.H, cb, bar);
                break;
            }
            case PH_E: {
                const int g = p.H / p.group;
                const int slot = task / p.F, n = task - slot * p.F;
                (void)slot;
                const int64_t rg = static_cast<int64_t>(expert) * 2 * p.F + n, ru = rg + p.F;
                const uint32_t rb = p.H, sb = g * 2;
                mbar_expect_tx(bar, 2 * rb + 2 * sb);
                bulk_g2s(dst, L.gu_codes + rg * p.H, rb, bar);
                bulk_g2s(dst + rb, L.gu_codes + ru * p.H, rb, bar);
                bulk_g2s(dst + 2 * rb, L.gu_scale + rg * g, sb, bar);
                bulk_g2s(dst + 2 * rb + sb, L.gu_scale + ru * g, sb, bar);
                break;
            }
            case PH_F: {
                const int g = p.F / p.group;
                const int64_t row = static_cast<int64_t>(expert) * p.H + 2 * task;
                const uint32_t cb = 2 * p.F, sb = 2 * g * 2;
                mbar_expect_tx(bar, cb + sb);
                bulk_g2s(dst, L.dn_codes + row * p.F, cb, bar);
                bulk_g2s(dst + cb, L.dn_scale + row * g, sb, bar);
                break;
            }
            default: {
                const int g = p.H / p.group;
                const uint32_t cb = 2 * p.H, sb = 2 * g * 2;
                mbar_expect_tx(bar, cb + sb);
                bulk_g2s(dst, p.lm_codes + static_cast<int64_t>(task) * 2 * p.H, cb, bar);
                bulk_g2s(dst + cb, p.lm_scale + static_cast<int64_t>(task) * 2 * g, sb, bar);
                break;
            }
        }
    }
    // keep the ring full (called by the whole warp)
    __device__ __forceinline__ void pump() {
        while (n_issued - n_consumed < kMegaStages && allowed()) {
            int expert = 0;
            if (cur.phase == PH_E) {
                expert = static_cast<int>(__shfl_sync(0xffffffffu, ids_reg, (wg + cur.i * G) / P->F));
            } else if (cur.phase == PH_F) {
                expert = static_cast<int>(__shfl_sync(0xffffffffu, ids_reg, cur.slot));
            }
            if (lane == 0) issue(n_issued % kMegaStages, expert);
            ++n_issued;
            advance();
        }
    }
    // wait for the oldest stage; returns its generic address (nullptr on timeout)
    __device__ __forceinline__ const unsigned char* acquire() {
        const int s = n_consumed % kMegaStages;
        if (!mbar_wait(ring.bar(s), (n_consumed / kMegaStages) & 1)) {
            if (P->err_flag && lane == 0) atomicOr(P->err_flag, LEMOQ_FLAG_WAIT_TIMEOUT);
            return nullptr;
        }
        return my + static_cast<size_t>(s) * kMegaStageBytes;
    }
    __device__ __forceinline__ void release() {
        __syncwarp();
        ++n_consumed;
        pump();
    }
};

// ---------------------------------------------------------------------------------------------
// row dot product with the lane layout derived on the fly (group_size divides 512)
// ---------------------------------------------------------------------------------------------
struct LaneLite {
    int lane16;   // lane * 16: byte offset of the lane inside a 512-byte chunk
    int sbase;    // scale index of the lane inside a chunk
    int sstride;  // scales per chunk
};
__device__ __forceinline__ float row_dot(const unsigned char* __restrict__ row, const __half* __restrict__ scales, int K,
                                         const LaneLite& ll, const XSlice<NCH, kMegaMode>& xs) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int k0 = c * 512 + ll.lane16;
        if (k0 < K) {
            const uint4 w = *reinterpret_cast<const uint4*>(row + k0);
            acc = fmaf(xs.dot(c, w), __half2float(scales[c * ll.sstride + ll.sbase]), acc);
        }
    }
    return acc;
}

// Activation slice loaders that convert chunk by chunk (low register peak).
__device__ __forceinline__ void slice_plain(XSlice<NCH, kMegaMode>& xs, const __half* __restrict__ x, int K, int lane16) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int k0 = c * 512 + lane16;
        float f[16];
        if (k0 < K) {
            unpack8_h(ld_cg16(x + k0), &f[0]);
            unpack8_h(ld_cg16(x + k0 + 8), &f[8]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] = 0.f;
        }
        xs.set(c, f);
    }
}
// Raw row words of the lane plus the RMSNorm statistic (every warp covers the row exactly once).
struct RawRow {
    uint4 w[NCH][2];
    float rstd;
    __device__ __forceinline__ void load(const __half* __restrict__ x, int K, int lane16, float eps) {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int k0 = c * 512 + lane16;
            if (k0 < K) {
                w[c][0] = ld_cg16(x + k0);
                w[c][1] = ld_cg16(x + k0 + 8);
                float f[16];
                unpack8_h(w[c][0], &f[0]);
                unpack8_h(w[c][1], &f[8]);
#pragma unroll
                for (int j = 0; j < 16; ++j) ss = fmaf(f[j], f[j], ss);
            } else {
                w[c][0] = w[c][1] = make_uint4(0, 0, 0, 0);
            }
        }
        ss = warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / static_cast<float>(K) + eps);
    }
    // normalised values of chunk c (HF rounding chain), as fp32
    __device__ __forceinline__ void chunk(int c, const __half* __restrict__ nw, int K, int lane16, float (&f)[16]) const {
        const int k0 = c * 512 + lane16;
        if (k0 < K) {
            const uint4 wa = *reinterpret_cast<const uint4*>(nw + k0);
            const uint4 wb = *reinterpret_cast<const uint4*>(nw + k0 + 8);
            const __half* xh0 = reinterpret_cast<const __half*>(&w[c][0]);
            const __half* xh1 = reinterpret_cast<const __half*>(&w[c][1]);
            const __half* wh0 = reinterpret_cast<const __half*>(&wa);
            const __half* wh1 = reinterpret_cast<const __half*>(&wb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                f[j] = norm_elem(xh0[j], rstd, wh0[j]);
                f[8 + j] = norm_elem(xh1[j], rstd, wh1[j]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] = 0.f;
        }
    }
};
__device__ __forceinline__ void slice_norm(XSlice<NCH, kMegaMode>& xs, const __half* __restrict__ x,
                                           const __half* __restrict__ nw, float eps, int K, int lane16) {
    RawRow r;
    r.load(x, K, lane16, eps);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        float f[16];
        r.chunk(c, nw, K, lane16, f);
        xs.set(c, f);
    }
}

// ---------------------------------------------------------------------------------------------
// routing: every warp derives softmax + top-k from the E fp16 logits (E <= 128), identically
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void warp_topk(const __half* __restrict__ logits, int E, int K, bool norm, int lane,
                                          long long& id_reg, float& w_reg) {
    float v[4];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? __half2float(__ldcg(logits + e)) : -INFINITY;
        mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? expf(v[j] - mx) : 0.f;
        sum += v[j];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (lane + 32 * j) < E ? v[j] / sum : -1.0e30f;
    float wsum = 0.f;
    id_reg = 0;
    w_reg = 0.f;
    for (int k = 0; k < K; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (v[j] > best) {
                best = v[j];
                bi = lane + 32 * j;
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
        wsum += best;
        if (lane == k) {
            id_reg = bi;
            w_reg = best;
        }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j == (bi >> 5)) v[j] = -1.0e30f;
        }
    }
    if (norm) w_reg = w_reg / wsum;
    w_reg = __half2float(__float2half_rn(w_reg));  // the routing weights are used in fp16
}

// ---------------------------------------------------------------------------------------------
// attention phase (one (head, split) unit per block)
// ---------------------------------------------------------------------------------------------
struct AttnScratch {
    float q[128];
    float tmp[128];
    float red[40];
    float wm[kMegaWarps];
    float wl[kMegaWarps];
    float wacc[kMegaWarps][132];
    int last;
};

__device__ __forceinline__ float block_rstd(const __half* __restrict__ row, int A, float eps, float* red) {
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < A; i += blockDim.x * 8) {
        float f[8];
        unpack8_h(ld_cg16(row + i), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = block_sum(ss, red);
    return 1.0f / sqrtf(ss / static_cast<float>(A) + eps);
}

template <int D>
__device__ __forceinline__ __half rope_one(const float* __restrict__ xs, int d, const __half* __restrict__ cos,
                                           const __half* __restrict__ sin) {
    const float x = xs[d];
    const float rot = d < D / 2 ? -xs[d + D / 2] : xs[d - D / 2];
    return __float2half_rn(__fadd_rn(__fmul_rn(x, __half2float(cos[d])), __fmul_rn(rot, __half2float(sin[d]))));
}

template <int D, bool INT8>
__device__ __noinline__ void attention_phase(const MegaParams& p, const MegaLayer& L, AttnScratch& sm) {
    constexpr int LPP = D / 16;  // lanes per position
    constexpr int GW = 32 / LPP;  // position groups per warp
    const int unit = blockIdx.x;
    if (unit >= p.heads * p.splits) return;
    const int h = unit / p.splits, split = unit - h * p.splits;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane % LPP, grp = lane / LPP;
    const int A = p.heads * D;

    int n_filled = *p.filled;
    if (n_filled < 0 || n_filled > p.S) {
        if (p.err_flag && tid == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_LENGTH);
        n_filled = n_filled < 0 ? 0 : p.S;
    }
    const int chunk = (n_filled + p.splits - 1) / p.splits;
    const int n_start = split * chunk;
    const int n_end = min(n_start + chunk, n_filled);
    int64_t pos = *p.cache_position;
    const bool pos_ok = pos >= 0 && pos < p.S;
    if (!pos_ok) {
        if (p.err_flag && tid == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_POSITION);
        pos = pos < 0 ? 0 : p.S - 1;
    }
    const __half* cos = p.rope_cos + pos * D;
    const __half* sin = p.rope_sin + pos * D;
    const int64_t hs = static_cast<int64_t>(p.S) * D;
    int8_t* kc = L.kc + h * hs;
    int8_t* vc = L.vc + h * hs;
    __half* ks = L.ks + static_cast<int64_t>(h) * p.S;
    __half* vs = L.vs + static_cast<int64_t>(h) * p.S;
    __half* kh = L.keys + h * hs;
    __half* vh = L.values + h * hs;

    const float rstd_q = block_rstd(p.qkv, A, p.eps, sm.red);
    if (tid < D) sm.tmp[tid] = norm_elem(__ldcg(p.qkv + h * D + tid), rstd_q, L.q_norm[h * D + tid]);
    __syncthreads();
    if (tid < D) sm.q[tid] = __half2float(rope_one<D>(sm.tmp, tid, cos, sin));
    __syncthreads();
    const bool owner = pos_ok && pos >= n_start && pos < n_end;
    if (owner) {
        const float rstd_k = block_rstd(p.qkv + A, A, p.eps, sm.red);
        if (tid < D) sm.tmp[tid] = norm_elem(__ldcg(p.qkv + A + h * D + tid), rstd_k, L.k_norm[h * D + tid]);
        __syncthreads();
        __half kn = __float2half_rn(0.f), vn = __float2half_rn(0.f);
        if (tid < D) {
            kn = rope_one<D>(sm.tmp, tid, cos, sin);
            vn = __ldcg(p.qkv + 2 * A + h * D + tid);
            kh[pos * D + tid] = kn;
            vh[pos * D + tid] = vn;
        }
        if (INT8) {
            const float kf = __half2float(kn), vf = __half2float(vn);
            const float amk = block_max(tid < D ? fabsf(kf) : 0.f, sm.red);
            const float amv = block_max(tid < D ? fabsf(vf) : 0.f, sm.red);
            const float sk = amk > 0.f ? __fdiv_rn(amk, 127.0f) : 1.0f;
            const float sv = amv > 0.f ? __fdiv_rn(amv, 127.0f) : 1.0f;
            if (tid < D) {
                float qk = fminf(fmaxf(rintf(__fdiv_rn(kf, sk)), -127.0f), 127.0f);
                float qv = fminf(fmaxf(rintf(__fdiv_rn(vf, sv)), -127.0f), 127.0f);
                kc[pos * D + tid] = static_cast<int8_t>(static_cast<int>(qk));
                vc[pos * D + tid] = static_cast<int8_t>(static_cast<int>(qv));
            }
            if (tid == 0) {
                ks[pos] = __float2half_rn(sk);
                vs[pos] = __float2half_rn(sv);
            }
        }
        __threadfence_block();
        __syncthreads();
    }

    float q[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) q[j] = sm.q[sub * 16 + j];
    float m_i = -INFINITY, l_i = 0.f;
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;

    constexpr int GROUPS = kMegaWarps * GW;
    const int group = warp * GW + grp;
    for (int base = n_start; base < n_end; base += 2 * GROUPS) {
        const int n0 = base + group, n1 = n0 + GROUPS;
        const bool has0 = n0 < n_end, has1 = n1 < n_end;
        const uint4 z = make_uint4(0, 0, 0, 0);
        uint4 k0a = z, k0b = z, v0a = z, v0b = z, k1a = z, k1b = z, v1a = z, v1b = z;
        float ks0 = 1.f, vs0 = 1.f, ks1 = 1.f, vs1 = 1.f;
        if (INT8) {
            if (has0) {
                k0a = ld_cg16(kc + static_cast<int64_t>(n0) * D + sub * 16);
                v0a = ld_cg16(vc + static_cast<int64_t>(n0) * D + sub * 16);
                ks0 = __half2float(__ldcg(ks + n0));
                vs0 = __half2float(__ldcg(vs + n0));
            }
            if (has1) {
                k1a = ld_cg16(kc + static_cast<int64_t>(n1) * D + sub * 16);
                v1a = ld_cg16(vc + static_cast<int64_t>(n1) * D + sub * 16);
                ks1 = __half2float(__ldcg(ks + n1));
                vs1 = __half2float(__ldcg(vs + n1));
            }
        } else {
            if (has0) {
                k0a = ld_cg16(kh + static_cast<int64_t>(n0) * D + sub * 16);
                k0b = ld_cg16(kh + static_cast<int64_t>(n0) * D + sub * 16 + 8);
                v0a = ld_cg16(vh + static_cast<int64_t>(n0) * D + sub * 16);
                v0b = ld_cg16(vh + static_cast<int64_t>(n0) * D + sub * 16 + 8);
            }
            if (has1) {
                k1a = ld_cg16(kh + static_cast<int64_t>(n1) * D + sub * 16);
                k1b = ld_cg16(kh + static_cast<int64_t>(n1) * D + sub * 16 + 8);
                v1a = ld_cg16(vh + static_cast<int64_t>(n1) * D + sub * 16);
                v1b = ld_cg16(vh + static_cast<int64_t>(n1) * D + sub * 16 + 8);
            }
        }
        float d0, d1;
        if (INT8) {
            d0 = dot16_s8(k0a, q);
            d1 = dot16_s8(k1a, q);
        } else {
            d0 = dot8_h(k0a, &q[0]) + dot8_h(k0b, &q[8]);
            d1 = dot8_h(k1a, &q[0]) + dot8_h(k1b, &q[8]);
        }
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) {
            d0 += __shfl_xor_sync(0xffffffffu, d0, o);
            d1 += __shfl_xor_sync(0xffffffffu, d1, o);
        }
        auto step = [&](float s, float v_scale, const uint4& va, const uint4& vb) {
            const float m_new = fmaxf(m_i, s);
            const float alpha = exp2f(m_i - m_new);
            const float pw = exp2f(s - m_new);
            l_i = fmaf(l_i, alpha, pw);
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] *= alpha;
            if (INT8) {
                axpy16_s8(va, pw * v_scale, acc);
            } else {
                float f[16];
                unpack8_h(va, &f[0]);
                unpack8_h(vb, &f[8]);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] = fmaf(pw, f[j], acc[j]);
            }
            m_i = m_new;
        };
        if (has0) step(INT8 ? d0 * p.qk_scale_log2 * ks0 : d0 * p.qk_scale_log2, vs0, v0a, v0b);
        if (has1) step(INT8 ? d1 * p.qk_scale_log2 * ks1 : d1 * p.qk_scale_log2, vs1, v1a, v1b);
    }

    // merge the position groups of the warp (fixed xor order), then the warps of the block
#pragma unroll
    for (int o = LPP; o < 32; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m_i, o);
        const float lo = __shfl_xor_sync(0xffffffffu, l_i, o);
        const float mn = fmaxf(m_i, mo);
        const float base = mn > -INFINITY ? mn : 0.f;
        const float wa = exp2f(m_i - base), wb = exp2f(mo - base);
        l_i = l_i * wa + lo * wb;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float ao = __shfl_xor_sync(0xffffffffu, acc[j], o);
            acc[j] = acc[j] * wa + ao * wb;
        }
        m_i = mn;
    }
    if (lane < LPP) {
#pragma unroll
        for (int j = 0; j < 16; ++j) sm.wacc[warp][lane * 16 + j] = acc[j];
        if (lane == 0) {
            sm.wm[warp] = m_i;
            sm.wl[warp] = l_i;
        }
    }
    __syncthreads();
    float* part = p.attn_part + (static_cast<int64_t>(h) * p.splits + split) * (D + 2);
    if (tid < D) {
        float big = -INFINITY;
        for (int w = 0; w < kMegaWarps; ++w) big = fmaxf(big, sm.wm[w]);
        const float base = big > -INFINITY ? big : 0.f;
        float a = 0.f, l = 0.f;
        for (int w = 0; w < kMegaWarps; ++w) {
            const float wt = exp2f(sm.wm[w] - base);
            a = fmaf(sm.wacc[w][tid], wt, a);
            l = fmaf(sm.wl[w], wt, l);
        }
        part[2 + tid] = a;
        if (tid == 0) {
            part[0] = big;
            part[1] = l;
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(p.attn_counters + h, 1u);
        sm.last = (ticket == static_cast<unsigned int>(p.splits) - 1u);
    }
    __syncthreads();
    if (!sm.last) return;
    __threadfence();
    if (tid < D) {
        const float* hp = p.attn_part + static_cast<int64_t>(h) * p.splits * (D + 2);
        float big = -INFINITY;
        for (int j = 0; j < p.splits; ++j) big = fmaxf(big, __ldcg(hp + j * (D + 2)));
        big = big > -INFINITY ? big : 0.f;
        float num = 0.f, den = 0.f;
        for (int j = 0; j < p.splits; ++j) {
            const float w = exp2f(__ldcg(hp + j * (D + 2)) - big);
            num = fmaf(__ldcg(hp + j * (D + 2) + 2 + tid), w, num);
            den = fmaf(__ldcg(hp + j * (D + 2) + 1), w, den);
        }
        p.attn[h * D + tid] = __float2half_rn(den > 0.f ? num / den : num);
    }
    if (tid == 0) p.attn_counters[h] = 0u;
}

// Phase time stamps (block 0, thread 0; nanoseconds of the global timer) for profiling the step.
__device__ __forceinline__ void stamp(const MegaParams& p, int slot) {
    if (p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.stamps[slot] = t;
    }
}

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMegaThreads, 1) step_mega_kernel(const __grid_constant__ MegaParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* scratch = smem + kMegaWarps * kMegaStages * kMegaStageBytes + kMegaWarps * kMegaStages * 8 + 128;
    scratch = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(scratch) + 127) & ~uintptr_t(127));

    WarpStream ws;
    ws.P = &p;
    ws.ring.init(smem, warp, kMegaWarps, kMegaStageBytes, lane);
    ws.my = smem + static_cast<size_t>(warp) * kMegaStages * kMegaStageBytes;
    ws.G = gridDim.x * kMegaWarps;
    ws.wg = warp * gridDim.x + blockIdx.x;
    ws.lane = lane;
    ws.n_issued = ws.n_consumed = 0;
    ws.ids_ready_layer = -1;
    ws.ids_reg = 0;
    ws.cur = Cursor{0, PH_A, 0, 0};
    ws.normalise();
    ws.pump();

    GridBarrier bar;
    bar.counter = p.bar_counter;
    bar.err_flag = p.err_flag;
    bar.target = ld_acquire_u32(p.bar_epoch) * static_cast<unsigned int>(p.barriers_per_launch) * gridDim.x;

    stamp(p, 0);
    const int A = p.heads * p.D;
    LaneLite ll;
    ll.lane16 = lane * 16;
    ll.sbase = (lane * 16) / p.group;
    ll.sstride = 512 / p.group;
    const int gH = p.H / p.group, gA = A / p.group, gF = p.F / p.group;

    const __half* x_prev = p.embed + (*p.token) * static_cast<int64_t>(p.H);
    XSlice<NCH, kMegaMode> xs;

    for (int l = 0; l < p.layers; ++l) {
        const MegaLayer& L = p.L[l];
        // ---- A: q.k.v -------------------------------------------------------------------------------
        {
            const int cnt = ws.phase_count(PH_A);
            if (cnt > 0) slice_norm(xs, x_prev, L.ln1, p.eps, p.H, ll.lane16);
            for (int i = 0; i < cnt; ++i) {
                const unsigned char* st = ws.acquire();
                if (!st) break;
                const __half* sc = reinterpret_cast<const __half*>(st + 2 * p.H);
                float a0 = row_dot(st, sc, p.H, ll, xs);
                float a1 = row_dot(st + p.H, sc + gH, p.H, ll, xs);
                ws.release();
                a0 = warp_sum(a0);
                a1 = warp_sum(a1);
                if (lane < 2) p.qkv[(ws.wg + i * ws.G) * 2 + lane] = __float2half_rn(lane == 0 ? a0 : a1);
            }
        }
        bar.sync();
        stamp(p, 6 * l + 1);
        // ---- B: attention ---------------------------------------------------------------------------
        {
            AttnScratch& sm = *reinterpret_cast<AttnScratch*>(scratch);
            if (p.D == 128) {
                if (p.kv_int8) attention_phase<128, true>(p, L, sm);
                else attention_phase<128, false>(p, L, sm);
            } else {
                if (p.kv_int8) attention_phase<64, true>(p, L, sm);
                else attention_phase<64, false>(p, L, sm);
            }
        }
        bar.sync();
        stamp(p, 6 * l + 2);
        // ---- C: o_proj + residual -------------------------------------------------------------------
        {
            const int cnt = ws.phase_count(PH_C);
            if (cnt > 0) slice_plain(xs, p.attn, A, ll.lane16);
            for (int i = 0; i < cnt; ++i) {
                const unsigned char* st = ws.acquire();
                if (!st) break;
                const __half* sc = reinterpret_cast<const __half*>(st + 2 * A);
                float a0 = row_dot(st, sc, A, ll, xs);
                float a1 = row_dot(st + A, sc + gA, A, ll, xs);
                ws.release();
                a0 = warp_sum(a0);
                a1 = warp_sum(a1);
                if (lane < 2) {
                    const int n = (ws.wg + i * ws.G) * 2 + lane;
                    p.xa[n] = __hadd(__float2half_rn(lane == 0 ? a0 : a1), __ldcg(x_prev + n));
                }
            }
        }
        bar.sync();
        stamp(p, 6 * l + 3);
        // ---- D: router logits -----------------------------------------------------------------------
        {
            const int cnt = ws.phase_count(PH_D);
            RawRow rr;
            if (cnt > 0) rr.load(p.xa, p.H, ll.lane16, p.eps);
            for (int i = 0; i < cnt; ++i) {
                const unsigned char* st = ws.acquire();
                if (!st) break;
                float a = 0.f;
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const int k0 = c * 512 + ll.lane16;
                    if (k0 < p.H) {
                        float hf[16];
                        rr.chunk(c, L.ln2, p.H, ll.lane16, hf);
                        const uint4 w0 = *reinterpret_cast<const uint4*>(st + 2 * k0);
                        const uint4 w1 = *reinterpret_cast<const uint4*>(st + 2 * k0 + 16);
                        a += dot8_h(w0, &hf[0]);
                        a += dot8_h(w1, &hf[8]);
                    }
                }
                ws.release();
                a = warp_sum(a);
                if (lane == 0) p.router_logits[static_cast<int64_t>(l) * p.E + ws.wg + i * ws.G] = __float2half_rn(a);
            }
        }
        bar.sync();
        stamp(p, 6 * l + 4);
        // ---- E: routing (per warp) + expert gate/up ----------------------------------------------------
        float tw_reg;
        {
            warp_topk(p.router_logits + static_cast<int64_t>(l) * p.E, p.E, p.K, p.norm_topk != 0, lane, ws.ids_reg, tw_reg);
            ws.ids_ready_layer = l;
            ws.pump();
            if (blockIdx.x == 0 && warp == 0 && lane < p.K) {
                p.top_i[static_cast<int64_t>(l) * p.K + lane] = ws.ids_reg;
                p.top_w[lane] = __float2half_rn(tw_reg);
            }
            const int cnt = ws.phase_count(PH_E);
            if (cnt > 0) slice_norm(xs, p.xa, L.ln2, p.eps, p.H, ll.lane16);
            for (int i = 0; i < cnt; ++i) {
                const unsigned char* st = ws.acquire();
                if (!st) break;
                const __half* sc = reinterpret_cast<const __half*>(st + 2 * p.H);
                float g = row_dot(st, sc, p.H, ll, xs);
                float u = row_dot(st + p.H, sc + gH, p.H, ll, xs);
                ws.release();
                g = warp_sum(g);
                u = warp_sum(u);
                if (lane == 0) p.act[ws.wg + i * ws.G] = __float2half_rn(g * (1.0f / (1.0f + expf(-g))) * u);
            }
        }
        bar.sync();
        stamp(p, 6 * l + 5);
        // ---- F: expert down + residual ----------------------------------------------------------------
        {
            // stage the K activation vectors as packed fp16, lane-major
            const int per_slot = p.F / 8;
            const int nchF = (p.F + 511) / 512;
            for (int idx = threadIdx.x; idx < p.K * per_slot; idx += blockDim.x) {
                const int slot = idx / per_slot;
                const int k = (idx - slot * per_slot) * 8;
                const uint4 raw = ld_cg16(p.act + static_cast<int64_t>(slot) * p.F + k);
                const int c = k >> 9, ln = (k & 511) >> 4, hi = (k >> 3) & 1;
                *reinterpret_cast<uint4*>(scratch + (static_cast<size_t>((slot * nchF + c) * 32 + ln) * 16 + hi * 8) * 2) = raw;
            }
            __syncthreads();
            const int cnt = ws.phase_count(PH_F);
            for (int i = 0; i < cnt; ++i) {
                float acc0 = 0.f, acc1 = 0.f;
                bool dead = false;
                for (int slot = 0; slot < p.K; ++slot) {
                    const unsigned char* st = ws.acquire();
                    if (!st) {
                        dead = true;
                        break;
                    }
                    const __half* sc = reinterpret_cast<const __half*>(st + 2 * p.F);
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        if (c * 512 + ll.lane16 < p.F) {
                            const unsigned char* src = scratch + static_cast<size_t>((slot * nchF + c) * 32 + lane) * 32;
                            float f[16];
                            unpack8_h(*reinterpret_cast<const uint4*>(src), &f[0]);
                            unpack8_h(*reinterpret_cast<const uint4*>(src + 16), &f[8]);
                            xs.set(c, f);
                        }
                    }
                    const float p0 = row_dot(st, sc, p.F, ll, xs);
                    const float p1 = row_dot(st + p.F, sc + gF, p.F, ll, xs);
                    ws.release();
                    const float tw = __shfl_sync(0xffffffffu, tw_reg, slot);
                    acc0 = fmaf(tw, p0, acc0);
                    acc1 = fmaf(tw, p1, acc1);
                }
                if (dead) break;
                acc0 = warp_sum(acc0);
                acc1 = warp_sum(acc1);
                if (lane < 2) {
                    const int n = (ws.wg + i * ws.G) * 2 + lane;
                    p.xb[n] = __hadd(__float2half_rn(lane == 0 ? acc0 : acc1), __ldcg(p.xa + n));
                }
            }
        }
        bar.sync();
        stamp(p, 6 * l + 6);
        x_prev = p.xb;
    }
    // ---- lm_head ------------------------------------------------------------------------------------------
    {
        const int cnt = ws.phase_count(PH_LM);
        if (cnt > 0) slice_norm(xs, x_prev, p.final_norm, p.eps, p.H, ll.lane16);
        for (int i = 0; i < cnt; ++i) {
            const unsigned char* st = ws.acquire();
            if (!st) break;
            const __half* sc = reinterpret_cast<const __half*>(st + 2 * p.H);
            float a0 = row_dot(st, sc, p.H, ll, xs);
            float a1 = row_dot(st + p.H, sc + gH, p.H, ll, xs);
            ws.release();
            a0 = warp_sum(a0);
            a1 = warp_sum(a1);
            if (lane < 2) p.logits[(ws.wg + i * ws.G) * 2 + lane] = __float2half_rn(lane == 0 ? a0 : a1);
        }
    }
    bar.sync();
    stamp(p, 6 * p.layers + 1);
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(p.bar_epoch, 1u);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
size_t mega_smem_bytes() {
    return static_cast<size_t>(kMegaWarps) * kMegaStages * kMegaStageBytes + kMegaWarps * kMegaStages * 8 + 256 +
           kMegaScratchBytes;
}

bool mega_eligible(const lemoq_step_desc& d) {
    const int A = d.heads * d.head_dim;
    const int g = d.group_size;
    if (g <= 0 || g % 16 != 0 || 512 % g != 0) return false;
    auto ok_dim = [&](int n) { return n % 512 == 0 && n <= 2048 && n % g == 0 && ((n / g) * 2 * 2) % 16 == 0; };
    if (!ok_dim(d.hidden) || !ok_dim(A) || !ok_dim(d.ffn)) return false;
    if (((d.hidden / g) * 2) % 16 != 0) return false;  // one expert row of scales must be a 16-byte multiple
    if (d.head_dim != 64 && d.head_dim != 128) return false;
    if (d.experts > 128 || d.top_k > 32 || d.top_k > d.experts) return false;
    if (d.vocab % 2 != 0) return false;
    if (static_cast<size_t>(d.top_k) * ((d.ffn + 511) / 512) * 512 * 2 > kMegaScratchBytes) return false;
    if (sizeof(AttnScratch) > kMegaScratchBytes) return false;
    return true;
}

int mega_grid(const lemoq_step_desc& d, int splits) {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaFuncSetAttribute(step_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(mega_smem_bytes())) != cudaSuccess)
        return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, step_mega_kernel, kMegaThreads, mega_smem_bytes()) !=
            cudaSuccess ||
        per_sm < 1)
        return 0;
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop) return 0;
    (void)d;
    (void)splits;
    return sms;
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
