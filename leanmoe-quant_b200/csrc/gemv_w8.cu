// Dense W8 dequant GEMV (q.k.v / o_proj / lm_head) with optional fused RMSNorm
// prologue and fp16 residual epilogue, and the router GEMV with fused
// softmax/top-k.  HBM-bound: one warp streams RPW weight rows with 128-bit loads,
// dequantises in registers, reduces with shuffles.  No tensor cores.
#include "gemv_common.cuh"
#include "kernels.h"

namespace lemoq {

// ---------------------------------------------------------------------------
// y[m, n] = fp16( sum_k xin[m,k] * codes[n,k] * scale[n,k/g] ) (+ resid[m,n])
//   NORM : xin = RMSNorm(x[m,:]) * norm_w  (HF rounding chain), else xin = x
//   RESID: y = fp16(acc) + resid           (fp16 add, as the model's residual add)
// token != nullptr: row 0 of x (and of resid) is taken at x + *token * K (embedding
// gather fused into the first layer's kernels).
// grid = (ceil(N / (warps*RPW)), M), block = warps*32.
// ---------------------------------------------------------------------------
template <int NCH, int RPW, bool NORM, bool RESID, bool OUT_F32>
__global__ void __launch_bounds__(256) gemv_w8_kernel(GemvParams p) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    const int m = blockIdx.y;
    const int row0 = (blockIdx.x * warps + warp) * RPW;
    const int groups = p.K / p.group_size;

    // Weights do not depend on the previous kernel: get them in flight first.
    RowW8<NCH> rows[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int n = row0 + r;
        if (n < p.N) {
            load_row_w8<NCH>(rows[r], p.codes + static_cast<int64_t>(n) * p.K,
                             p.scale + static_cast<int64_t>(n) * groups, p.K, p.group_size, lane);
        } else {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                rows[r].w[c] = make_uint4(0, 0, 0, 0);
                rows[r].s[c] = __float2half_rn(0.f);
            }
        }
    }

    pdl_wait();
    pdl_trigger();

    int64_t x_off = static_cast<int64_t>(m) * p.x_stride;
    if (p.x_token != nullptr) x_off = checked_token(p.x_token, p.token_rows, p.err_flag) * static_cast<int64_t>(p.K);
    float xr[NCH][16];
    if (NORM) {
        load_x_rmsnorm<NCH>(xr, p.x + x_off, p.norm_w, p.eps, p.K, lane, nullptr);
    } else {
        load_x_plain<NCH>(xr, p.x + x_off, p.K, lane);
    }

#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int n = row0 + r;
        float acc = warp_sum(dot_row_w8<NCH>(rows[r], xr));
        if (lane == 0 && n < p.N) {
            const int64_t yo = static_cast<int64_t>(m) * p.y_stride + n;
            if (OUT_F32) {
                reinterpret_cast<float*>(p.y)[yo] = acc;
            } else {
                __half h = __float2half_rn(acc);
                if (RESID) {
                    int64_t ro = static_cast<int64_t>(m) * p.resid_stride + n;
                    if (p.resid_token != nullptr) ro = checked_token(p.resid_token, p.token_rows, nullptr) * static_cast<int64_t>(p.N) + n;
                    h = __hadd(h, p.resid[ro]);
                }
                reinterpret_cast<__half*>(p.y)[yo] = h;
            }
        }
    }
}

template <int NCH, int RPW>
static int launch_gemv_nch(const GemvParams& p, int M, bool norm, bool resid, bool out_f32, const LaunchCfg& lc) {
    const int warps = p.N >= 4096 ? 8 : 4;
    dim3 grid((p.N + warps * RPW - 1) / (warps * RPW), M), block(warps * 32);
    if (out_f32) {
        if (norm || resid) return set_error(LEMOQ_ERR_UNSUPPORTED, "fp32 output has no fused prologue/epilogue");
        return launch_kernel(gemv_w8_kernel<NCH, RPW, false, false, true>, grid, block, 0, lc, p);
    }
    if (norm && resid) return launch_kernel(gemv_w8_kernel<NCH, RPW, true, true, false>, grid, block, 0, lc, p);
    if (norm) return launch_kernel(gemv_w8_kernel<NCH, RPW, true, false, false>, grid, block, 0, lc, p);
    if (resid) return launch_kernel(gemv_w8_kernel<NCH, RPW, false, true, false>, grid, block, 0, lc, p);
    return launch_kernel(gemv_w8_kernel<NCH, RPW, false, false, false>, grid, block, 0, lc, p);
}

int launch_gemv_w8(const GemvParams& p, int M, bool norm, bool resid, bool out_f32, const LaunchCfg& lc) {
    if (!out_f32 && stream_gemv_eligible(p, M)) return launch_stream_gemv_w8(p, norm, resid, lc);
    const int nch = (p.K + 511) / 512;
    switch (nch) {
        case 1: return launch_gemv_nch<1, 2>(p, M, norm, resid, out_f32, lc);
        case 2: return launch_gemv_nch<2, 2>(p, M, norm, resid, out_f32, lc);
        case 3: return launch_gemv_nch<3, 2>(p, M, norm, resid, out_f32, lc);
        case 4: return launch_gemv_nch<4, 2>(p, M, norm, resid, out_f32, lc);
        default: break;
    }
    if (nch <= 8) return launch_gemv_nch<8, 1>(p, M, norm, resid, out_f32, lc);
    if (nch <= 16) return launch_gemv_nch<16, 1>(p, M, norm, resid, out_f32, lc);
    return set_error(LEMOQ_ERR_UNSUPPORTED, "K=%d exceeds the GEMV register tiling (max 8192)", p.K);
}

// ---------------------------------------------------------------------------
// Router: logits[e] = fp16( h . Wr[e,:] ) with h = RMSNorm(x)*w (NORM) or h = x;
// one warp per expert row (fp16 weights, 32 bytes per lane and chunk).  The last
// block to finish runs softmax + top-k over the E logits (one warp).
// When h_out != nullptr block 0 also writes h (fp16) for the expert kernels.
// ---------------------------------------------------------------------------
__device__ void softmax_topk_warp(const float* __restrict__ logit_s, int E, int top_k, bool norm, float* w_out,
                                  int64_t* i_out, float* scratch /* E floats */) {
    const int lane = threadIdx.x & 31;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, logit_s[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float pe = expf(logit_s[e] - mx);
        scratch[e] = pe;
        sum += pe;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) scratch[e] = scratch[e] / sum;
    __syncwarp();
    float wsum = 0.f;
    for (int k = 0; k < top_k; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = scratch[e];
            if (v > best) {  // ascending e inside a lane: the first maximum wins
                best = v;
                bi = e;
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
        if (lane == 0) {
            w_out[k] = best;
            i_out[k] = bi;
            scratch[bi] = -1.0e30f;
        }
        __syncwarp();
    }
    if (norm) {
        for (int k = lane; k < top_k; k += 32) w_out[k] = w_out[k] / wsum;
    }
    __syncwarp();
}

template <int NCH, bool NORM>
__global__ void __launch_bounds__(256) route_kernel(RouteParams p) {
    __shared__ float s_logit[kMaxExperts];
    __shared__ float s_prob[kMaxExperts];
    __shared__ int s_last;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    const int e = blockIdx.x * warps + warp;

    // fp16 router row: chunk c, lane l owns 16 halves = two 128-bit words.
    uint4 wq[NCH][2];
    if (e < p.E) {
        const __half* wr = p.router_w + static_cast<int64_t>(e) * p.H;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int k0 = c * 512 + lane * 16;
            if (k0 < p.H) {
                wq[c][0] = ld_stream16(wr + k0);
                wq[c][1] = ld_stream16(wr + k0 + 8);
            } else {
                wq[c][0] = wq[c][1] = make_uint4(0, 0, 0, 0);
            }
        }
    }

    pdl_wait();
    pdl_trigger();

    float xr[NCH][16];
    if (NORM) {
        load_x_rmsnorm<NCH>(xr, p.x, p.norm_w, p.eps, p.H, lane, nullptr);
    } else {
        load_x_plain<NCH>(xr, p.x, p.H, lane);
    }
    if (p.h_out != nullptr && blockIdx.x == 0 && warp == 0) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int k0 = c * 512 + lane * 16;
            if (k0 < p.H) {
                __align__(16) __half hv[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) hv[j] = __float2half_rn(xr[c][j]);  // exact: values are fp16
                *reinterpret_cast<uint4*>(p.h_out + k0) = *reinterpret_cast<const uint4*>(&hv[0]);
                *reinterpret_cast<uint4*>(p.h_out + k0 + 8) = *reinterpret_cast<const uint4*>(&hv[8]);
            }
        }
    }
    if (e < p.E) {
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            acc += dot8_h(wq[c][0], &xr[c][0]);
            acc += dot8_h(wq[c][1], &xr[c][8]);
        }
        acc = warp_sum(acc);
        if (lane == 0) p.logits_out[e] = __float2half_rn(acc);
    }

    // last-block election
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(p.counter, 1u);
        s_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < p.E; i += blockDim.x) {
        s_logit[i] = __half2float(__ldcg(p.logits_out + i));
    }
    __syncthreads();
    if (warp == 0) {
        __shared__ float s_w[kMaxTopK];
        softmax_topk_warp(s_logit, p.E, p.top_k, p.norm_topk_prob != 0, s_w, p.top_i, s_prob);
        __syncwarp();
        for (int k = lane; k < p.top_k; k += 32) p.top_w[k] = __float2half_rn(s_w[k]);
        if (lane == 0) *p.counter = 0u;
    }
}

int launch_route(const RouteParams& p, bool norm, const LaunchCfg& lc) {
    const int warps = 8;
    dim3 grid((p.E + warps - 1) / warps), block(warps * 32);
    const int nch = (p.H + 511) / 512;
#define LEMOQ_ROUTE_CASE(N)                                                                       \
    case N:                                                                                       \
        return norm ? launch_kernel(route_kernel<N, true>, grid, block, 0, lc, p)                 \
                    : launch_kernel(route_kernel<N, false>, grid, block, 0, lc, p);
    switch (nch) {
        LEMOQ_ROUTE_CASE(1)
        LEMOQ_ROUTE_CASE(2)
        LEMOQ_ROUTE_CASE(3)
        LEMOQ_ROUTE_CASE(4)
        default: break;
    }
#undef LEMOQ_ROUTE_CASE
    return set_error(LEMOQ_ERR_UNSUPPORTED, "router hidden size %d exceeds 2048", p.H);
}

// ---------------------------------------------------------------------------
// Stand-alone softmax + top-k over (T, E) logits, one warp per token.
// ---------------------------------------------------------------------------
template <typename TL>
__global__ void __launch_bounds__(32) routing_topk_kernel(const TL* __restrict__ logits, int64_t row_stride, int E,
                                                          int top_k, int norm, float* __restrict__ top_w,
                                                          int64_t* __restrict__ top_i) {
    extern __shared__ float sm[];
    float* s_logit = sm;
    float* s_prob = sm + E;
    float* s_w = sm + 2 * E;
    const int t = blockIdx.x;
    for (int e = threadIdx.x; e < E; e += 32) s_logit[e] = to_float(logits[t * row_stride + e]);
    __syncwarp();
    softmax_topk_warp(s_logit, E, top_k, norm != 0, s_w, top_i + static_cast<int64_t>(t) * top_k, s_prob);
    __syncwarp();
    for (int k = threadIdx.x; k < top_k; k += 32) top_w[static_cast<int64_t>(t) * top_k + k] = s_w[k];
}

int launch_routing_topk(const void* logits, int dtype, int64_t row_stride, int T, int E, int top_k, int norm,
                        float* top_w, int64_t* top_i, const LaunchCfg& lc) {
    const size_t smem = (2 * static_cast<size_t>(E) + top_k) * sizeof(float);
    if (dtype == LEMOQ_DTYPE_F16)
        return launch_kernel(routing_topk_kernel<__half>, dim3(T), dim3(32), smem, lc,
                             reinterpret_cast<const __half*>(logits), row_stride, E, top_k, norm, top_w, top_i);
    return launch_kernel(routing_topk_kernel<float>, dim3(T), dim3(32), smem, lc,
                         reinterpret_cast<const float*>(logits), row_stride, E, top_k, norm, top_w, top_i);
}

}  // namespace lemoq
