// Grouped expert GEMV for decode: the expert id only enters pointer arithmetic.
//   gate_up : act[t,i,n] = silu(Wg[e,n,:].x_t) * (Wu[e,n,:].x_t)        -> fp16
//   down    : out[t,n]   = sum_i w[t,i] * (Wd[e,n,:].act[t,i,:])          -> fp16 (+ residual)
// Weights are int8 codes with per-group fp16 scales (dequantised in registers) or
// plain fp16.  HBM-bound streaming kernels: 128-bit coalesced loads, fp32 FMA,
// warp-shuffle reductions; no tensor cores.
#include "gemv_common.cuh"
#include "kernels.h"

namespace lemoq {

__device__ __forceinline__ int clamp_expert(int64_t e, int E, int* err_flag) {
    if (e < 0 || e >= E) {
        if (err_flag) atomicOr(err_flag, LEMOQ_FLAG_BAD_EXPERT);
        return e < 0 ? 0 : E - 1;
    }
    return static_cast<int>(e);
}

// grid = (ceil(F / warps), K, T), block = warps*32; one warp per (slot, n): it streams
// the gate row n and the up row n of expert ids[t, slot].
template <int NCH, bool W8>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(MoeParams p) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    const int n = blockIdx.x * warps + warp;
    const int slot = blockIdx.y;
    const int t = blockIdx.z;

    // The expert ids come from the router kernel: nothing can be fetched before it ends.
    pdl_wait();
    pdl_trigger();
    if (n >= p.F) return;

    const int e = clamp_expert(p.ids[static_cast<int64_t>(t) * p.K + slot], p.E, p.err_flag);
    const int64_t row_g = static_cast<int64_t>(e) * 2 * p.F + n;
    const int64_t row_u = row_g + p.F;
    WRow<NCH, W8> wg, wu;
    wg.load(p.gate_up, row_g, p.gu_scale, p.H, p.group_size, lane);
    wu.load(p.gate_up, row_u, p.gu_scale, p.H, p.group_size, lane);

    float xr[NCH][16];
    load_x_plain<NCH>(xr, p.x + static_cast<int64_t>(t) * p.H, p.H, lane);

    const float g = warp_sum(wg.dot(xr));
    const float u = warp_sum(wu.dot(xr));
    if (lane == 0) {
        const float a = g * (1.0f / (1.0f + expf(-g))) * u;
        p.act[(static_cast<int64_t>(t) * p.K + slot) * p.F + n] = __float2half_rn(a);
    }
}

// grid = (ceil(H / (warps*R)), T), block = warps*32, dynamic smem = K * NCHF*512 floats.
// One warp owns R output rows and walks the K routed experts; the K activation
// vectors of the token sit in shared memory in a lane-major layout
// ((((slot*NCHF + chunk)*4 + q)*32 + lane)*4 + r  <->  k = chunk*512 + lane*16 + q*4 + r)
// so that each lane reads its 16 values with four conflict-free 128-bit loads.
template <int NCHF, int R, bool W8, bool RESID>
__global__ void __launch_bounds__(256) moe_down_kernel(MoeParams p) {
    extern __shared__ float s_act[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    const int t = blockIdx.y;
    const int n0 = (blockIdx.x * warps + warp) * R;
    const int64_t* ids = p.ids + static_cast<int64_t>(t) * p.K;

    // ids / routing weights were written two kernels upstream, so the first expert's
    // rows can be requested before the dependency wait.
    WRow<NCHF, W8> buf0[R], buf1[R];
    auto load_slot = [&](WRow<NCHF, W8>(&buf)[R], int slot) {
        const int e = clamp_expert(ids[slot], p.E, p.err_flag);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = min(n0 + r, p.H - 1);
            buf[r].load(p.down, static_cast<int64_t>(e) * p.H + n, p.dn_scale, p.F, p.group_size, lane);
        }
    };
    load_slot(buf0, 0);

    pdl_wait();
    pdl_trigger();

    // stage the K activation vectors (fp16 -> fp32) into shared memory
    {
        const __half* act = p.act + static_cast<int64_t>(t) * p.K * p.F;
        const int per_slot = p.F / 8;  // 128-bit words per slot
        for (int idx = threadIdx.x; idx < p.K * per_slot; idx += blockDim.x) {
            const int slot = idx / per_slot;
            const int k = (idx - slot * per_slot) * 8;
            float f[8];
            unpack8_h(ld_cg16(act + static_cast<int64_t>(slot) * p.F + k), f);
            const int c = k >> 9, l = (k & 511) >> 4, q = (k & 15) >> 2;  // q in {0, 2}
            float* dst = s_act + ((((slot * NCHF + c) * 4 + q) * 32 + l) << 2);
            *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4*>(dst + 128) = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
    __syncthreads();

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;

    auto compute_slot = [&](const WRow<NCHF, W8>(&buf)[R], int slot) {
        float a[NCHF][16];
#pragma unroll
        for (int c = 0; c < NCHF; ++c) {
            if (c * 512 + lane * 16 < p.F) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 v =
                        *reinterpret_cast<const float4*>(s_act + ((((slot * NCHF + c) * 4 + q) * 32 + lane) << 2));
                    a[c][4 * q + 0] = v.x;
                    a[c][4 * q + 1] = v.y;
                    a[c][4 * q + 2] = v.z;
                    a[c][4 * q + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) a[c][j] = 0.f;
            }
        }
        const float w = __half2float(p.top_w[static_cast<int64_t>(t) * p.K + slot]);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = fmaf(w, buf[r].dot(a), acc[r]);
    };

    for (int i = 0; i < p.K; i += 2) {
        if (i + 1 < p.K) load_slot(buf1, i + 1);
        compute_slot(buf0, i);
        if (i + 1 < p.K) {
            if (i + 2 < p.K) load_slot(buf0, i + 2);
            compute_slot(buf1, i + 1);
        }
    }

#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float v = warp_sum(acc[r]);
        const int n = n0 + r;
        if (lane == 0 && n < p.H) {
            __half h = __float2half_rn(v);
            if (RESID) h = __hadd(h, p.resid[static_cast<int64_t>(t) * p.H + n]);
            p.out[static_cast<int64_t>(t) * p.H + n] = h;
        }
    }
}

int launch_moe_gate_up(const MoeParams& p, bool w8, const LaunchCfg& lc) {
    if (w8 && stream_moe_eligible(p)) return launch_stream_gate_up(p, lc);
    const int warps = 8;
    dim3 grid((p.F + warps - 1) / warps, p.K, p.T), block(warps * 32);
    const int nch = (p.H + 511) / 512;
#define LEMOQ_GU_CASE(N)                                                                              \
    case N:                                                                                           \
        return w8 ? launch_kernel(moe_gate_up_kernel<N, true>, grid, block, 0, lc, p)                 \
                  : launch_kernel(moe_gate_up_kernel<N, false>, grid, block, 0, lc, p);
    switch (nch) {
        LEMOQ_GU_CASE(1)
        LEMOQ_GU_CASE(2)
        LEMOQ_GU_CASE(3)
        LEMOQ_GU_CASE(4)
        default: break;
    }
#undef LEMOQ_GU_CASE
    return set_error(LEMOQ_ERR_UNSUPPORTED, "expert hidden size %d exceeds 2048", p.H);
}

template <int NCHF, bool W8>
static int launch_down_nchf(const MoeParams& p, const LaunchCfg& lc) {
    constexpr int R = 2;
    const int warps = 4;
    dim3 grid((p.H + warps * R - 1) / (warps * R), p.T), block(warps * 32);
    const size_t smem = static_cast<size_t>(p.K) * NCHF * 512 * sizeof(float);
    if (smem > 200 * 1024) return set_error(LEMOQ_ERR_UNSUPPORTED, "top_k*ffn too large for the down kernel");
    auto kern = p.resid ? moe_down_kernel<NCHF, R, W8, true> : moe_down_kernel<NCHF, R, W8, false>;
    if (smem > 48 * 1024) {
        const cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(err));
    }
    return launch_kernel(kern, grid, block, smem, lc, p);
}

int launch_moe_down(const MoeParams& p, bool w8, const LaunchCfg& lc) {
    if (w8 && stream_moe_eligible(p)) return launch_stream_down(p, lc);
    const int nchf = (p.F + 511) / 512;
#define LEMOQ_DN_CASE(N) \
    case N:              \
        return w8 ? launch_down_nchf<N, true>(p, lc) : launch_down_nchf<N, false>(p, lc);
    switch (nchf) {
        LEMOQ_DN_CASE(1)
        LEMOQ_DN_CASE(2)
        LEMOQ_DN_CASE(3)
        LEMOQ_DN_CASE(4)
        default: break;
    }
#undef LEMOQ_DN_CASE
    return set_error(LEMOQ_ERR_UNSUPPORTED, "expert ffn size %d exceeds 2048", p.F);
}

}  // namespace lemoq
