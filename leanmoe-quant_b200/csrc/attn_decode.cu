// Split-KV decode attention (batch 1, one query row per head) over a static cache,
// reading either fp16 K/V or the per-token symmetric int8 mirror with the scales
// folded into the scores (K) and the softmax weights (V).
//
// grid = (num_splits, heads), block = 128.  A "lane group" of D/16 lanes owns one cache
// position at a time (16 head-dim elements per lane: one 128-bit word of int8 codes
// or two of fp16) and keeps its own online-softmax state (m, l, acc[16]) in base 2.
// The groups of a block are merged in shared memory in a fixed order, the block
// writes its (m, l, acc[D]) partial, and the last block of a head to arrive merges
// the head's splits in split order.  No atomics on data: results are bit-identical
// from run to run.
//
// FUSED variant: the block derives q (and the split that owns the new position
// derives k, v) from the raw packed q.k.v projection row: RMSNorm over the full
// projection width, head split, half-split RoPE, then writes the new K/V row into
// the fp16 cache and the int8 mirror before attending to it.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace lemoq {

constexpr int kAttnThreads = 128;

template <int D>
struct AttnSmem {
    float q[D];
    float tmp[D];
    float red[40];
    float m[kAttnThreads / (D / 16)];
    float l[kAttnThreads / (D / 16)];
    float acc[kAttnThreads / (D / 16)][D + 4];
    int last;
};

// RMSNorm statistics of one projection row of width A, reduced by the whole block.
__device__ __forceinline__ float row_rstd(const __half* __restrict__ row, int A, float eps, float* red) {
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

// Half-split RoPE of element d given the normalised row in shared memory:
// fp32 products and sum, each rounded (no contraction), one rounding to fp16.
template <int D>
__device__ __forceinline__ __half rope_elem(const float* __restrict__ xs, int d, const __half* __restrict__ cos,
                                            const __half* __restrict__ sin) {
    const float x = xs[d];
    const float rot = d < D / 2 ? -xs[d + D / 2] : xs[d - D / 2];
    const float a = __fmul_rn(x, __half2float(cos[d]));
    const float b = __fmul_rn(rot, __half2float(sin[d]));
    return __float2half_rn(__fadd_rn(a, b));
}

// Per-token symmetric int8 of one value given the row's amax (fp32 rules of the cache).
__device__ __forceinline__ float kv_scale_of(float amax) { return amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f; }
__device__ __forceinline__ int8_t kv_code_of(float x, float s) {
    float q = rintf(__fdiv_rn(x, s));
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return static_cast<int8_t>(static_cast<int>(q));
}

template <int D, bool INT8, bool FUSED>
__global__ void __launch_bounds__(kAttnThreads) attn_split_kernel(AttnParams p) {
    constexpr int LPP = D / 16;                 // lanes per position
    constexpr int G = kAttnThreads / LPP;       // lane groups per block
    __shared__ AttnSmem<D> sm;
    const int tid = threadIdx.x;
    const int split = blockIdx.x;
    const int h = blockIdx.y;
    const int group = tid / LPP;
    const int sub = tid % LPP;                  // which 16 dims of the head this lane owns

    pdl_wait();
    pdl_trigger();

    int n_filled = *p.filled;
    if (n_filled < 0 || n_filled > p.S) {
        if (p.err_flag && tid == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_LENGTH);
        n_filled = n_filled < 0 ? 0 : p.S;
    }
    const int chunk = (n_filled + p.num_splits - 1) / p.num_splits;
    const int n_start = split * chunk;
    const int n_end = min(n_start + chunk, n_filled);

    const int8_t* kc = reinterpret_cast<const int8_t*>(p.k) + h * p.kv_head_stride;
    const int8_t* vc = reinterpret_cast<const int8_t*>(p.v) + h * p.kv_head_stride;
    const __half* kh = reinterpret_cast<const __half*>(p.k) + h * p.kv_head_stride;
    const __half* vh = reinterpret_cast<const __half*>(p.v) + h * p.kv_head_stride;
    const __half* ks = INT8 ? p.ks + static_cast<int64_t>(h) * p.S : nullptr;
    const __half* vs = INT8 ? p.vs + static_cast<int64_t>(h) * p.S : nullptr;

    // ---- q (and, for the owning split, the new K/V row) --------------------------------
    if (FUSED) {
        const int A = p.heads * D;
        int64_t pos = *p.cache_position;
        bool pos_ok = pos >= 0 && pos < p.S;
        if (!pos_ok) {
            if (p.err_flag && tid == 0) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_POSITION);
            pos = pos < 0 ? 0 : p.S - 1;
        }
        const __half* cos = p.rope_cos + pos * D;
        const __half* sin = p.rope_sin + pos * D;
        const float rstd_q = row_rstd(p.qkv, A, p.eps, sm.red);
        if (tid < D) sm.tmp[tid] = norm_elem(p.qkv[h * D + tid], rstd_q, p.q_norm_w[h * D + tid]);
        __syncthreads();
        if (tid < D) sm.q[tid] = __half2float(rope_elem<D>(sm.tmp, tid, cos, sin));
        __syncthreads();
        const bool owner = pos_ok && pos >= n_start && pos < n_end;
        if (owner) {
            const float rstd_k = row_rstd(p.qkv + A, A, p.eps, sm.red);
            if (tid < D) sm.tmp[tid] = norm_elem(p.qkv[A + h * D + tid], rstd_k, p.k_norm_w[h * D + tid]);
            __syncthreads();
            __half kn = __float2half_rn(0.f), vn = __float2half_rn(0.f);
            if (tid < D) {
                kn = rope_elem<D>(sm.tmp, tid, cos, sin);
                vn = p.qkv[2 * A + h * D + tid];
                const int64_t o = static_cast<int64_t>(h) * p.S * D + pos * D + tid;
                p.keys_fp16[o] = kn;
                p.values_fp16[o] = vn;
            }
            if (INT8) {
                const float kf = __half2float(kn), vf = __half2float(vn);
                const float sk = kv_scale_of(block_max(tid < D ? fabsf(kf) : 0.f, sm.red));
                const float sv = kv_scale_of(block_max(tid < D ? fabsf(vf) : 0.f, sm.red));
                if (tid < D) {
                    const int64_t o = pos * D + tid;
                    const_cast<int8_t*>(kc)[o] = kv_code_of(kf, sk);
                    const_cast<int8_t*>(vc)[o] = kv_code_of(vf, sv);
                }
                if (tid == 0) {
                    const_cast<__half*>(ks)[pos] = __float2half_rn(sk);
                    const_cast<__half*>(vs)[pos] = __float2half_rn(sv);
                }
            }
            // the block's own loads below go to L2 (ld.cg), where these stores are visible
            __threadfence_block();
            __syncthreads();
        }
    } else {
        if (tid < D) sm.q[tid] = __half2float(p.q[h * D + tid]);
        __syncthreads();
    }

    float q[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) q[j] = sm.q[sub * 16 + j];

    // ---- this block's slice of the cache ---------------------------------------------------
    float m_i = -INFINITY, l_i = 0.f;
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;

    auto step = [&](float s, float v_scale, const uint4& v0, const uint4& v1) {
        const float m_new = fmaxf(m_i, s);
        const float alpha = exp2f(m_i - m_new);
        const float pw = exp2f(s - m_new);
        l_i = fmaf(l_i, alpha, pw);
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] *= alpha;
        if (INT8) {
            axpy16_s8(v0, pw * v_scale, acc);
        } else {
            float f[16];
            unpack8_h(v0, &f[0]);
            unpack8_h(v1, &f[8]);
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = fmaf(pw, f[j], acc[j]);
        }
        m_i = m_new;
    };
    auto group_sum = [&](float v) {
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    };

    // Two positions per group and iteration so that four 128-bit loads per lane are in
    // flight.  The trip count is uniform over the block (the group reductions shuffle
    // across the whole warp); positions past the end are predicated off.
    for (int base = n_start; base < n_end; base += 2 * G) {
        const int n0 = base + group;
        const int n1 = n0 + G;
        const bool has0 = n0 < n_end;
        const bool has1 = n1 < n_end;
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
        d0 = group_sum(d0);
        d1 = group_sum(d1);
        if (has0) {
            const float s0 = INT8 ? d0 * p.qk_scale_log2 * ks0 : d0 * p.qk_scale_log2;
            step(s0, vs0, v0a, v0b);
        }
        if (has1) {
            const float s1 = INT8 ? d1 * p.qk_scale_log2 * ks1 : d1 * p.qk_scale_log2;
            step(s1, vs1, v1a, v1b);
        }
    }

    // ---- merge the block's lane groups (fixed order) ----------------------------------------
    if (sub == 0) {
        sm.m[group] = m_i;
        sm.l[group] = l_i;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) sm.acc[group][sub * 16 + j] = acc[j];
    __syncthreads();
    float* part = p.part + (static_cast<int64_t>(h) * p.num_splits + split) * (D + 2);
    if (tid < D) {
        float big = -INFINITY;
        for (int g = 0; g < G; ++g) big = fmaxf(big, sm.m[g]);
        const float base = big > -INFINITY ? big : 0.f;
        float a = 0.f, l = 0.f;
        for (int g = 0; g < G; ++g) {
            const float w = exp2f(sm.m[g] - base);
            a = fmaf(sm.acc[g][tid], w, a);
            l = fmaf(sm.l[g], w, l);
        }
        part[2 + tid] = a;
        if (tid == 0) {
            part[0] = big;
            part[1] = l;
        }
    }

    // ---- last block of the head merges the splits in split order ----------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(p.counters + h, 1u);
        sm.last = (ticket == static_cast<unsigned int>(p.num_splits) - 1u);
    }
    __syncthreads();
    if (!sm.last) return;
    __threadfence();
    if (tid < D) {
        const float* hp = p.part + static_cast<int64_t>(h) * p.num_splits * (D + 2);
        float big = -INFINITY;
        for (int j = 0; j < p.num_splits; ++j) big = fmaxf(big, __ldcg(hp + j * (D + 2)));
        big = big > -INFINITY ? big : 0.f;
        float num = 0.f, den = 0.f;
        for (int j = 0; j < p.num_splits; ++j) {
            const float w = exp2f(__ldcg(hp + j * (D + 2)) - big);
            num = fmaf(__ldcg(hp + j * (D + 2) + 2 + tid), w, num);
            den = fmaf(__ldcg(hp + j * (D + 2) + 1), w, den);
        }
        const float o = den > 0.f ? num / den : num;
        p.out[h * D + tid] = __float2half_rn(o);
    }
    if (tid == 0) p.counters[h] = 0u;
}

template <int D>
static int launch_attn_d(const AttnParams& p, bool int8_kv, bool fused, const LaunchCfg& lc) {
    dim3 grid(p.num_splits, p.heads), block(kAttnThreads);
    if (int8_kv) {
        return fused ? launch_kernel(attn_split_kernel<D, true, true>, grid, block, 0, lc, p)
                     : launch_kernel(attn_split_kernel<D, true, false>, grid, block, 0, lc, p);
    }
    return fused ? launch_kernel(attn_split_kernel<D, false, true>, grid, block, 0, lc, p)
                 : launch_kernel(attn_split_kernel<D, false, false>, grid, block, 0, lc, p);
}

int launch_attn_decode(const AttnParams& p, bool int8_kv, bool fused, const LaunchCfg& lc) {
    if (p.D == 128) return launch_attn_d<128>(p, int8_kv, fused, lc);
    if (p.D == 64) return launch_attn_d<64>(p, int8_kv, fused, lc);
    return set_error(LEMOQ_ERR_UNSUPPORTED, "head_dim %d: the attention kernel is built for 64 and 128", p.D);
}

}  // namespace lemoq

// ---------------------------------------------------------------------------------------------------
// Int8 decode attention for callers that cannot hand over a workspace.
//
// Some hosts of this library may not allocate device memory where they call it: a serving loop that
// has already given every byte of the device to its own pools, a plugin that runs inside another
// framework's stream callback or graph construction where allocation calls are forbidden, a process
// whose memory budget was fixed at start-up.  For them the split partials and the per-head arrival
// counters of the attention kernel live in the fixed array below, which is part of the library image:
// nothing is allocated or freed, here or in any routine this entry point calls.
//
// The array holds kStaticAttnScratchBytes (1 MiB).  Its first kStaticAttnCounterBytes (16 KiB) are the
// arrival counters of up to 4096 heads, at the same place for every shape; the split partials of the
// call start right behind them.  A call with more heads, or whose heads x splits x (D + 2) partials do
// not fit behind the counters, is refused with LEMOQ_ERR_INVALID.  The counters must be zero when a
// launch starts: the array is zeroed when the module is loaded, every launch leaves its counters at
// zero again, and each call also enqueues a clear of its own counters ahead of its kernel, so a launch
// that was aborted earlier cannot poison later calls.  The partials keep the last call's contents; they
// are always written before they are read.  ALL calls on a device share the one array: two calls whose
// kernels may run at the same time on that device (other streams, other threads) race on it and give
// wrong results - order them on one stream.
// ---------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticAttnScratchBytes = size_t(1) << 20;
constexpr size_t kStaticAttnCounterBytes = size_t(16) << 10;  // fixed counter region: 4096 heads
constexpr int kStaticMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticAttnScratchBytes];

// Address of the array on each device, looked up once per device with that device current.
void* g_static_attn_ptr[kStaticMaxDevices] = {};
std::mutex g_static_attn_mutex;

int static_attn_scratch(void** out) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return lemoq::set_error(LEMOQ_ERR_CUDA, "attn_decode_int8_static: cudaGetDevice: %s", cudaGetErrorString(err));
    if (dev < 0 || dev >= kStaticMaxDevices)
        return lemoq::set_error(LEMOQ_ERR_UNSUPPORTED, "attn_decode_int8_static: device ordinal %d above %d", dev, kStaticMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_static_attn_mutex);
    if (g_static_attn_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_static_attn_scratch);
        if (err != cudaSuccess || ptr == nullptr)
            return lemoq::set_error(LEMOQ_ERR_CUDA, "attn_decode_int8_static: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
        g_static_attn_ptr[dev] = ptr;
    }
    *out = g_static_attn_ptr[dev];
    return LEMOQ_OK;
}

}  // namespace

extern "C" size_t lemoq_attn_static_scratch_bytes(void) { return kStaticAttnScratchBytes; }

extern "C" int lemoq_attn_decode_int8_static(const void* q, const int8_t* kc, const void* ks, const int8_t* vc, const void* vs,
                                             int64_t kv_head_stride, const int32_t* filled, void* out, int heads, int S, int D,
                                             int num_splits, float scale, int* err_flag, void* stream) {
    using namespace lemoq;
    LEMOQ_REQUIRE(q && filled && out && kc && ks && vc && vs, LEMOQ_ERR_INVALID, "attn_decode_int8_static: null pointer");
    LEMOQ_REQUIRE(heads > 0 && S > 0, LEMOQ_ERR_INVALID, "attn_decode_int8_static: heads and cache capacity must be positive");
    LEMOQ_REQUIRE(D == 64 || D == 128, LEMOQ_ERR_UNSUPPORTED, "attn_decode_int8_static: head_dim=%d, built for 64 and 128", D);
    LEMOQ_REQUIRE(num_splits >= 1 && num_splits <= 4096, LEMOQ_ERR_INVALID, "attn_decode_int8_static: num_splits must be in [1, 4096]");
    LEMOQ_REQUIRE(aligned16(kc) && aligned16(vc) && kv_head_stride % 16 == 0, LEMOQ_ERR_INVALID,
                  "attn_decode_int8_static: codes must be 16-byte aligned with a head stride that is a multiple of 16");
    LEMOQ_REQUIRE(kv_head_stride >= static_cast<int64_t>(S) * D, LEMOQ_ERR_INVALID,
                  "attn_decode_int8_static: heads overlap (head stride < S*D)");
    // counters in a region of fixed size (so that calls of different shapes never lay partials over
    // another shape's counters), then the partials
    LEMOQ_REQUIRE(sizeof(unsigned int) * static_cast<size_t>(heads) <= kStaticAttnCounterBytes, LEMOQ_ERR_INVALID,
                  "attn_decode_int8_static: heads=%d, the fixed array holds counters for %zu heads", heads,
                  kStaticAttnCounterBytes / sizeof(unsigned int));
    const size_t counters = kStaticAttnCounterBytes;
    const size_t need = counters + sizeof(float) * static_cast<size_t>(heads) * num_splits * (D + 2);
    LEMOQ_REQUIRE(need <= kStaticAttnScratchBytes, LEMOQ_ERR_INVALID,
                  "attn_decode_int8_static: heads=%d x num_splits=%d x head_dim=%d needs %zu bytes of scratch, the fixed array holds %zu",
                  heads, num_splits, D, need, kStaticAttnScratchBytes);
    void* scratch = nullptr;
    if (int rc = static_attn_scratch(&scratch)) return rc;
    AttnParams p;
    p.q = reinterpret_cast<const __half*>(q);
    p.filled = filled;
    p.out = reinterpret_cast<__half*>(out);
    p.heads = heads;
    p.S = S;
    p.D = D;
    p.num_splits = num_splits;
    p.qk_scale_log2 = scale * 1.4426950408889634f;
    p.counters = reinterpret_cast<unsigned int*>(scratch);
    p.part = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + counters);
    p.err_flag = err_flag;
    p.k = kc;
    p.v = vc;
    p.ks = reinterpret_cast<const __half*>(ks);
    p.vs = reinterpret_cast<const __half*>(vs);
    p.kv_head_stride = kv_head_stride;
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    // the counters of this call start at zero whatever an earlier (possibly aborted) launch left behind
    const cudaError_t cerr = cudaMemsetAsync(scratch, 0, sizeof(unsigned int) * static_cast<size_t>(heads), lc.stream);
    if (cerr != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "attn_decode_int8_static: clearing the counters: %s", cudaGetErrorString(cerr));
    return launch_attn_decode(p, true, false, lc);
}

