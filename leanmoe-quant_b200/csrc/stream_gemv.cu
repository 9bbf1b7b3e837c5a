// Persistent weight-streaming W8 GEMV kernels (the decode step's hot kernels).
//
// One block per SM, 8 warps.  Each warp walks its share of the row tasks and streams them
// through a private ring of shared-memory stages filled by cp.async.bulk (see stream.cuh):
// the bytes in flight per SM are set by the ring depth, not by registers or occupancy, and a
// warp never waits for another warp.  Weights that do not depend on the previous kernel are
// requested before griddepcontrol.wait, so under programmatic dependent launch the HBM
// stream of a kernel starts while its predecessor is still finishing.
//
// Dequantisation runs on the ALU/FMA pipes (PRMT + FFMA per code, see magic_dot16), fp32
// accumulation, one fp16 scale per 16-code lane chunk, warp-shuffle reduction, no atomics.
#include "stream_gemv.cuh"
#include "step_kernel.h"

namespace lemoq {

constexpr int kMaxStreamWarps = 16;
constexpr int kStreamStages = 3;
constexpr int kDownStages = 4;

// Tunables (set through lemoq_set_tuning; defaults are the measured best).
int g_stream_warps = 16;
int g_dot_mode = DOT_F16_FOLD;
extern int g_step_use_whole;

// ---------------------------------------------------------------------------
// Dense GEMV: a task is ROWS=2 consecutive weight rows (codes and scales contiguous).
// ---------------------------------------------------------------------------
template <int NCH, int MODE, bool NORM, bool RESID>
__global__ void __launch_bounds__(kMaxStreamWarps * 32, 1) stream_gemv_w8_kernel(GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int ROWS = 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int groups = p.K / p.group_size;
    const uint32_t code_bytes = ROWS * p.K, scale_bytes = ROWS * groups * 2;
    const uint32_t stage_bytes = (code_bytes + scale_bytes + 127u) & ~127u;
    WarpRing<kStreamStages> ring;
    ring.init(smem, warp, warps, stage_bytes, lane);
    const unsigned char* my = smem + static_cast<size_t>(warp) * kStreamStages * stage_bytes;

    const int n_tasks = p.N / ROWS;
    const int stride = gridDim.x * warps;
    const int first = warp * gridDim.x + blockIdx.x;

    auto issue = [&](int s, int task) {
        const int n = task * ROWS;
        mbar_expect_tx(ring.bar(s), code_bytes + scale_bytes);
        bulk_g2s(ring.stage(s), p.codes + static_cast<int64_t>(n) * p.K, code_bytes, ring.bar(s));
        bulk_g2s(ring.stage(s) + code_bytes, p.scale + static_cast<int64_t>(n) * groups, scale_bytes, ring.bar(s));
    };
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStreamStages; ++s) {
            const int t = first + s * stride;
            if (t < n_tasks) issue(s, t);
        }
    }
    LaneMap<NCH> lm;
    lm.init(p.K, p.group_size, lane);

    pdl_wait();
    pdl_trigger();

    int64_t x_off = 0;
    if (p.x_token != nullptr) x_off = checked_token(p.x_token, p.token_rows, p.err_flag) * static_cast<int64_t>(p.K);
    XSlice<NCH, MODE> xs;
    load_xslice<NCH, MODE, NORM>(xs, p.x + x_off, p.norm_w, p.eps, p.K, lane);

    int it = 0;
    for (int task = first; task < n_tasks; task += stride, ++it) {
        const int s = it % kStreamStages;
        if (!mbar_wait(ring.bar(s), (it / kStreamStages) & 1)) {
            flag_timeout(p.err_flag);
            return;
        }
        const unsigned char* st = my + static_cast<size_t>(s) * stage_bytes;
        const __half* sc = reinterpret_cast<const __half*>(st + code_bytes);
        float acc0 = row_partial<NCH, MODE>(st, sc, lm, xs);
        float acc1 = row_partial<NCH, MODE>(st + p.K, sc + groups, lm, xs);
        __syncwarp();  // every lane has read the stage: it may be refilled
        if (lane == 0) {
            const int nt = task + kStreamStages * stride;
            if (nt < n_tasks) issue(s, nt);
        }
        acc0 = warp_sum(acc0);
        acc1 = warp_sum(acc1);
        if (lane < ROWS) {
            const int n = task * ROWS + lane;
            __half h = __float2half_rn(lane == 0 ? acc0 : acc1);
            if (RESID) {
                int64_t ro = n;
                if (p.resid_token != nullptr) ro = checked_token(p.resid_token, p.token_rows, nullptr) * static_cast<int64_t>(p.N) + n;
                h = __hadd(h, p.resid[ro]);
            }
            reinterpret_cast<__half*>(p.y)[n] = h;
        }
    }
}

// ---------------------------------------------------------------------------
// Expert gate/up: a task is (slot, n): the gate row n and the up row n of expert ids[slot].
// ---------------------------------------------------------------------------
template <int NCH, int MODE>
__global__ void __launch_bounds__(kMaxStreamWarps * 32, 1) stream_gate_up_kernel(MoeParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int groups = p.H / p.group_size;
    const uint32_t row_bytes = p.H, srow_bytes = groups * 2;
    const uint32_t code_bytes = 2 * row_bytes;
    const uint32_t stage_bytes = (code_bytes + 2 * srow_bytes + 127u) & ~127u;
    WarpRing<kStreamStages> ring;
    ring.init(smem, warp, warps, stage_bytes, lane);
    const unsigned char* my = smem + static_cast<size_t>(warp) * kStreamStages * stage_bytes;

    const int n_tasks = p.K * p.F;
    const int stride = gridDim.x * warps;
    const int first = warp * gridDim.x + blockIdx.x;
    LaneMap<NCH> lm;
    lm.init(p.H, p.group_size, lane);

    // the expert ids are produced by the previous kernel
    pdl_wait();
    pdl_trigger();

    const int8_t* codes = reinterpret_cast<const int8_t*>(p.gate_up);
    auto issue = [&](int s, int task) {
        const int slot = task / p.F, n = task - slot * p.F;
        int64_t e = p.ids[slot];
        if (e < 0 || e >= p.E) {
            if (p.err_flag) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_EXPERT);
            e = e < 0 ? 0 : p.E - 1;
        }
        const int64_t rg = e * 2 * p.F + n, ru = rg + p.F;
        mbar_expect_tx(ring.bar(s), code_bytes + 2 * srow_bytes);
        bulk_g2s(ring.stage(s), codes + rg * p.H, row_bytes, ring.bar(s));
        bulk_g2s(ring.stage(s) + row_bytes, codes + ru * p.H, row_bytes, ring.bar(s));
        bulk_g2s(ring.stage(s) + code_bytes, p.gu_scale + rg * groups, srow_bytes, ring.bar(s));
        bulk_g2s(ring.stage(s) + code_bytes + srow_bytes, p.gu_scale + ru * groups, srow_bytes, ring.bar(s));
    };
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStreamStages; ++s) {
            const int t = first + s * stride;
            if (t < n_tasks) issue(s, t);
        }
    }

    XSlice<NCH, MODE> xs;
    load_xslice<NCH, MODE, false>(xs, p.x, nullptr, 0.f, p.H, lane);

    int it = 0;
    for (int task = first; task < n_tasks; task += stride, ++it) {
        const int s = it % kStreamStages;
        if (!mbar_wait(ring.bar(s), (it / kStreamStages) & 1)) {
            flag_timeout(p.err_flag);
            return;
        }
        const unsigned char* st = my + static_cast<size_t>(s) * stage_bytes;
        const __half* sc = reinterpret_cast<const __half*>(st + code_bytes);
        float g = row_partial<NCH, MODE>(st, sc, lm, xs);
        float u = row_partial<NCH, MODE>(st + row_bytes, sc + groups, lm, xs);
        __syncwarp();
        if (lane == 0) {
            const int nt = task + kStreamStages * stride;
            if (nt < n_tasks) issue(s, nt);
        }
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) p.act[task] = __float2half_rn(g * (1.0f / (1.0f + expf(-g))) * u);  // act is (K, F): index = task
    }
}

// ---------------------------------------------------------------------------
// Expert down: a task is ROWS=2 output rows; it streams K slot stages (2 rows of expert
// ids[slot] each).  The K activation vectors sit in shared memory in a lane-major layout:
// fp32 for the fp32 dot modes, packed fp16 for the mixed-precision mode.
// ---------------------------------------------------------------------------
template <int NCHF, int MODE, bool RESID>
__global__ void __launch_bounds__(kMaxStreamWarps * 32, 1) stream_down_kernel(MoeParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int ROWS = 2;
    constexpr int STAGES = kDownStages;
    constexpr bool HALF_ACT = MODE == DOT_F16_MIXED;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int groups = p.F / p.group_size;
    const uint32_t code_bytes = ROWS * p.F, scale_bytes = ROWS * groups * 2;
    const uint32_t stage_bytes = (code_bytes + scale_bytes + 127u) & ~127u;
    WarpRing<STAGES> ring;
    ring.init(smem, warp, warps, stage_bytes, lane);
    const unsigned char* my = smem + static_cast<size_t>(warp) * STAGES * stage_bytes;
    unsigned char* s_act = smem + ((WarpRing<STAGES>::smem_bytes(warps, stage_bytes) + 127) & ~size_t(127));
    // element e = (slot, c, lane, j): word index ((slot*NCHF + c)*32 + lane)*16 + j  (j-th of the lane's 16)

    const int n_tasks = p.H / ROWS;
    const int stride = gridDim.x * warps;
    const int first = warp * gridDim.x + blockIdx.x;
    const int my_tasks = first < n_tasks ? (n_tasks - first + stride - 1) / stride : 0;
    const int my_sub = my_tasks * p.K;  // sub-task = (task, slot)

    const int8_t* codes = reinterpret_cast<const int8_t*>(p.down);
    // ids were written two kernels upstream: legal to read before the dependency wait
    auto issue = [&](int s, int sub) {
        const int j = sub / p.K, slot = sub - j * p.K;
        const int n = (first + j * stride) * ROWS;
        int64_t e = p.ids[slot];
        if (e < 0 || e >= p.E) {
            if (p.err_flag) atomicOr(p.err_flag, LEMOQ_FLAG_BAD_EXPERT);
            e = e < 0 ? 0 : p.E - 1;
        }
        const int64_t row = e * p.H + n;
        mbar_expect_tx(ring.bar(s), code_bytes + scale_bytes);
        bulk_g2s(ring.stage(s), codes + row * p.F, code_bytes, ring.bar(s));
        bulk_g2s(ring.stage(s) + code_bytes, p.dn_scale + row * groups, scale_bytes, ring.bar(s));
    };
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
            if (s < my_sub) issue(s, s);
    }
    LaneMap<NCHF> lm;
    lm.init(p.F, p.group_size, lane);

    pdl_wait();
    pdl_trigger();

    // stage the K activation vectors, lane-major: each 16-byte piece of 8 halves goes to its lane's slot
    {
        const int per_slot = p.F / 8;
        for (int idx = threadIdx.x; idx < p.K * per_slot; idx += blockDim.x) {
            const int slot = idx / per_slot;
            const int k = (idx - slot * per_slot) * 8;
            const uint4 raw = ld_cg16(p.act + static_cast<int64_t>(slot) * p.F + k);
            const int c = k >> 9, l = (k & 511) >> 4, hi = (k >> 3) & 1;
            const int base = ((slot * NCHF + c) * 32 + l) * 16 + hi * 8;  // element index
            if (HALF_ACT) {
                *reinterpret_cast<uint4*>(s_act + static_cast<size_t>(base) * 2) = raw;
            } else {
                float f[8];
                unpack8_h(raw, f);
                float* dst = reinterpret_cast<float*>(s_act) + base;
                *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
        __syncthreads();
    }

    float acc0 = 0.f, acc1 = 0.f;
    for (int sub = 0; sub < my_sub; ++sub) {
        const int s = sub % STAGES;
        if (!mbar_wait(ring.bar(s), (sub / STAGES) & 1)) {
            flag_timeout(p.err_flag);
            return;
        }
        const int j = sub / p.K, slot = sub - j * p.K;
        const unsigned char* st = my + static_cast<size_t>(s) * stage_bytes;
        const __half* sc = reinterpret_cast<const __half*>(st + code_bytes);
        XSlice<NCHF, MODE> xs;
#pragma unroll
        for (int c = 0; c < NCHF; ++c) {
            const int base = ((slot * NCHF + c) * 32 + lane) * 16;
            if (HALF_ACT) {
                const uint4 a = *reinterpret_cast<const uint4*>(s_act + static_cast<size_t>(base) * 2);
                const uint4 b = *reinterpret_cast<const uint4*>(s_act + static_cast<size_t>(base) * 2 + 16);
                float f[16];
                unpack8_h(a, &f[0]);  // dead code for the packed mode once set() is inlined on raw words
                unpack8_h(b, &f[8]);
                xs.set(c, f);
            } else {
                const float* src = reinterpret_cast<const float*>(s_act) + base;
                float f[16];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 v = *reinterpret_cast<const float4*>(src + 4 * q);
                    f[4 * q + 0] = v.x;
                    f[4 * q + 1] = v.y;
                    f[4 * q + 2] = v.z;
                    f[4 * q + 3] = v.w;
                }
                xs.set(c, f);
            }
        }
        const float p0 = row_partial<NCHF, MODE>(st, sc, lm, xs);
        const float p1 = row_partial<NCHF, MODE>(st + p.F, sc + groups, lm, xs);
        __syncwarp();
        if (lane == 0) {
            const int ns = sub + STAGES;
            if (ns < my_sub) issue(s, ns);
        }
        const float tw = __half2float(p.top_w[slot]);
        acc0 = fmaf(tw, p0, acc0);
        acc1 = fmaf(tw, p1, acc1);
        if (slot == p.K - 1) {
            acc0 = warp_sum(acc0);
            acc1 = warp_sum(acc1);
            if (lane < ROWS) {
                const int n = (first + j * stride) * ROWS + lane;
                __half h = __float2half_rn(lane == 0 ? acc0 : acc1);
                if (RESID) h = __hadd(h, p.resid[n]);
                p.out[n] = h;
            }
            acc0 = acc1 = 0.f;
        }
    }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
static int sm_count() {
    static int cached = 0;
    if (cached) return cached;
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
        cached = v;
    else
        cached = 148;
    return cached;
}

template <typename Kern>
static int set_smem(Kern kern, size_t smem) {
    if (smem > 227 * 1024) return set_error(LEMOQ_ERR_UNSUPPORTED, "streaming kernel needs %zu bytes of shared memory", smem);
    if (smem > 48 * 1024) {
        const cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(err));
    }
    return LEMOQ_OK;
}

// Warps per block: the tuned count, reduced until the rings (plus `extra` bytes) fit in shared memory.
static int pick_warps(size_t per_warp_bytes, size_t extra) {
    int w = g_stream_warps < 1 ? 1 : (g_stream_warps > kMaxStreamWarps ? kMaxStreamWarps : g_stream_warps);
    while (w > 1 && w * per_warp_bytes + extra + 256 > 220 * 1024) --w;
    return w;
}

static int grid_for(int tasks, int warps) {
    const int need = (tasks + warps - 1) / warps;
    const int sms = sm_count();
    return need < sms ? need : sms;
}

int set_stream_tuning(int key, int value) {
    if (key == 0 && value >= 0 && value <= 3) {
        g_dot_mode = value;
        return LEMOQ_OK;
    }
    if (key == 1 && value >= 1 && value <= kMaxStreamWarps) {
        g_stream_warps = value;
        return LEMOQ_OK;
    }
    if (key == 4 && (value == 0 || value == 1)) {
        g_step_use_whole = value;
        return LEMOQ_OK;
    }
    if (key == 5) return set_flag_spin_limit(value);
    return set_error(LEMOQ_ERR_INVALID, "set_tuning: unknown key %d or value %d out of range", key, value);
}

bool stream_gemv_eligible(const GemvParams& p, int M) {
    if (M != 1 || p.K > 2048 || p.N % 2 != 0 || p.group_size % 16 != 0) return false;
    const int groups = p.K / p.group_size;
    return (2 * p.K) % 16 == 0 && (2 * groups * 2) % 16 == 0 && aligned16(p.codes) && aligned16(p.scale);
}

template <int NCH, int MODE>
static int launch_stream_gemv_mode(const GemvParams& p, bool norm, bool resid, const LaunchCfg& lc) {
    const int groups = p.K / p.group_size;
    const size_t stage = (2 * p.K + 2 * groups * 2 + 127) & ~size_t(127);
    const int warps = pick_warps(kStreamStages * (stage + 8), 0);
    const size_t smem = WarpRing<kStreamStages>::smem_bytes(warps, stage);
    dim3 grid(grid_for(p.N / 2, warps)), block(warps * 32);
#define LEMOQ_SG(NORM_, RESID_)                                      \
    {                                                                \
        auto kern = stream_gemv_w8_kernel<NCH, MODE, NORM_, RESID_>; \
        if (int rc = set_smem(kern, smem)) return rc;                \
        return launch_kernel(kern, grid, block, smem, lc, p);        \
    }
    if (norm && resid) LEMOQ_SG(true, true)
    if (norm) LEMOQ_SG(true, false)
    if (resid) LEMOQ_SG(false, true)
    LEMOQ_SG(false, false)
#undef LEMOQ_SG
}

template <int NCH>
static int launch_stream_gemv_nch(const GemvParams& p, bool norm, bool resid, const LaunchCfg& lc) {
    switch (g_dot_mode) {
        case DOT_F32_MAGIC: return launch_stream_gemv_mode<NCH, DOT_F32_MAGIC>(p, norm, resid, lc);
        case DOT_F16_CVT: return launch_stream_gemv_mode<NCH, DOT_F16_CVT>(p, norm, resid, lc);
        case DOT_F16_FOLD: return launch_stream_gemv_mode<NCH, DOT_F16_FOLD>(p, norm, resid, lc);
        default: return launch_stream_gemv_mode<NCH, DOT_F16_MIXED>(p, norm, resid, lc);
    }
}

int launch_stream_gemv_w8(const GemvParams& p, bool norm, bool resid, const LaunchCfg& lc) {
    switch ((p.K + 511) / 512) {
        case 1: return launch_stream_gemv_nch<1>(p, norm, resid, lc);
        case 2: return launch_stream_gemv_nch<2>(p, norm, resid, lc);
        case 3: return launch_stream_gemv_nch<3>(p, norm, resid, lc);
        case 4: return launch_stream_gemv_nch<4>(p, norm, resid, lc);
        default: break;
    }
    return set_error(LEMOQ_ERR_UNSUPPORTED, "streaming GEMV: K=%d above 2048", p.K);
}

bool stream_moe_eligible(const MoeParams& p) {
    if (p.T != 1 || p.H > 2048 || p.F > 2048 || p.group_size % 16 != 0) return false;
    const int gh = p.H / p.group_size, gf = p.F / p.group_size;
    return p.H % 16 == 0 && (gh * 2) % 16 == 0 && (2 * p.F) % 16 == 0 && (2 * gf * 2) % 16 == 0 && p.H % 2 == 0 &&
           aligned16(p.gate_up) && aligned16(p.gu_scale) && aligned16(p.down) && aligned16(p.dn_scale);
}

template <int NCH, int MODE>
static int launch_stream_gate_up_mode(const MoeParams& p, const LaunchCfg& lc) {
    const int groups = p.H / p.group_size;
    const size_t stage = (2 * p.H + 2 * groups * 2 + 127) & ~size_t(127);
    const int warps = pick_warps(kStreamStages * (stage + 8), 0);
    const size_t smem = WarpRing<kStreamStages>::smem_bytes(warps, stage);
    dim3 grid(grid_for(p.K * p.F, warps)), block(warps * 32);
    auto kern = stream_gate_up_kernel<NCH, MODE>;
    if (int rc = set_smem(kern, smem)) return rc;
    return launch_kernel(kern, grid, block, smem, lc, p);
}

template <int NCH>
static int launch_stream_gate_up_nch(const MoeParams& p, const LaunchCfg& lc) {
    switch (g_dot_mode) {
        case DOT_F32_MAGIC: return launch_stream_gate_up_mode<NCH, DOT_F32_MAGIC>(p, lc);
        case DOT_F16_CVT: return launch_stream_gate_up_mode<NCH, DOT_F16_CVT>(p, lc);
        case DOT_F16_FOLD: return launch_stream_gate_up_mode<NCH, DOT_F16_FOLD>(p, lc);
        default: return launch_stream_gate_up_mode<NCH, DOT_F16_MIXED>(p, lc);
    }
}

int launch_stream_gate_up(const MoeParams& p, const LaunchCfg& lc) {
    switch ((p.H + 511) / 512) {
        case 1: return launch_stream_gate_up_nch<1>(p, lc);
        case 2: return launch_stream_gate_up_nch<2>(p, lc);
        case 3: return launch_stream_gate_up_nch<3>(p, lc);
        case 4: return launch_stream_gate_up_nch<4>(p, lc);
        default: break;
    }
    return set_error(LEMOQ_ERR_UNSUPPORTED, "streaming gate/up: hidden=%d above 2048", p.H);
}

template <int NCHF, int MODE>
static int launch_stream_down_mode(const MoeParams& p, const LaunchCfg& lc) {
    const int groups = p.F / p.group_size;
    const size_t stage = (2 * p.F + 2 * groups * 2 + 127) & ~size_t(127);
    const size_t act_bytes = static_cast<size_t>(p.K) * NCHF * 512 * (MODE == DOT_F16_MIXED ? 2 : 4);
    const int warps = pick_warps(kDownStages * (stage + 8), act_bytes + 128);
    const size_t ring = (WarpRing<kDownStages>::smem_bytes(warps, stage) + 127) & ~size_t(127);
    const size_t smem = ring + act_bytes;
    dim3 grid(grid_for(p.H / 2, warps)), block(warps * 32);
    if (p.resid) {
        auto kern = stream_down_kernel<NCHF, MODE, true>;
        if (int rc = set_smem(kern, smem)) return rc;
        return launch_kernel(kern, grid, block, smem, lc, p);
    }
    auto kern = stream_down_kernel<NCHF, MODE, false>;
    if (int rc = set_smem(kern, smem)) return rc;
    return launch_kernel(kern, grid, block, smem, lc, p);
}

template <int NCHF>
static int launch_stream_down_nchf(const MoeParams& p, const LaunchCfg& lc) {
    switch (g_dot_mode) {
        case DOT_F32_MAGIC: return launch_stream_down_mode<NCHF, DOT_F32_MAGIC>(p, lc);
        case DOT_F16_CVT: return launch_stream_down_mode<NCHF, DOT_F16_CVT>(p, lc);
        case DOT_F16_FOLD: return launch_stream_down_mode<NCHF, DOT_F16_FOLD>(p, lc);
        default: return launch_stream_down_mode<NCHF, DOT_F16_MIXED>(p, lc);
    }
}

int launch_stream_down(const MoeParams& p, const LaunchCfg& lc) {
    switch ((p.F + 511) / 512) {
        case 1: return launch_stream_down_nchf<1>(p, lc);
        case 2: return launch_stream_down_nchf<2>(p, lc);
        case 3: return launch_stream_down_nchf<3>(p, lc);
        case 4: return launch_stream_down_nchf<4>(p, lc);
        default: break;
    }
    return set_error(LEMOQ_ERR_UNSUPPORTED, "streaming down: ffn=%d above 2048", p.F);
}

}  // namespace lemoq
