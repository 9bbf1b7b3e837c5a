// Internal (C++) launch interface between the C ABI / step engine and the kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace lemoq {

constexpr int kMaxExperts = 2048;
constexpr int kMaxTopK = 64;

struct LaunchCfg {
    cudaStream_t stream = nullptr;
    bool pdl = false;        // attach the programmatic-stream-serialization attribute
    int* launch_count = nullptr;
};

// Launch through cudaLaunchKernelEx so that the PDL attribute can be attached.
template <typename... KArgs, typename... Args>
int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, const LaunchCfg& lc, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = lc.stream;
    cudaLaunchAttribute attr[1];
    if (lc.pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (err != cudaSuccess) return set_error(LEMOQ_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(err));
    if (lc.launch_count) ++*lc.launch_count;
    return LEMOQ_OK;
}

// ---- dense GEMV -------------------------------------------------------------------
struct GemvParams {
    const __half* x = nullptr;       // (M, K), row stride x_stride
    int64_t x_stride = 0;
    const int64_t* x_token = nullptr;  // optional: row = x + *x_token * K
    int64_t token_rows = 0;          // rows behind x / resid when a token selects the row: ids outside [0, token_rows) are clamped and flagged
    const __half* norm_w = nullptr;  // (K) for the fused RMSNorm prologue
    float eps = 0.f;
    const int8_t* codes = nullptr;   // (N, K)
    const __half* scale = nullptr;   // (N, K/group_size)
    int N = 0, K = 0, group_size = 128;
    void* y = nullptr;               // (M, N) fp16 or fp32
    int64_t y_stride = 0;
    const __half* resid = nullptr;   // (M, N) fp16 for the residual epilogue
    int64_t resid_stride = 0;
    const int64_t* resid_token = nullptr;
    int* err_flag = nullptr;
};
int launch_gemv_w8(const GemvParams& p, int M, bool norm, bool resid, bool out_f32, const LaunchCfg& lc);
// persistent bulk-copy streaming variants (stream_gemv.cu); the *_eligible predicates state their shape rules
bool stream_gemv_eligible(const GemvParams& p, int M);
int set_stream_tuning(int key, int value);
int launch_stream_gemv_w8(const GemvParams& p, bool norm, bool resid, const LaunchCfg& lc);

// ---- router ----------------------------------------------------------------------
struct RouteParams {
    const __half* x = nullptr;       // (H) input (raw residual stream when norm is fused)
    const __half* norm_w = nullptr;
    float eps = 0.f;
    const __half* router_w = nullptr;  // (E, H) fp16
    int E = 0, H = 0, top_k = 0, norm_topk_prob = 0;
    __half* h_out = nullptr;         // optional (H): the normalised activations
    __half* logits_out = nullptr;    // (E)
    __half* top_w = nullptr;         // (top_k)
    int64_t* top_i = nullptr;        // (top_k)
    unsigned int* counter = nullptr; // zero-initialised arrival counter
};
int launch_route(const RouteParams& p, bool norm, const LaunchCfg& lc);
int launch_routing_topk(const void* logits, int dtype, int64_t row_stride, int T, int E, int top_k, int norm,
                        float* top_w, int64_t* top_i, const LaunchCfg& lc);

// ---- grouped experts ----------------------------------------------------------------
struct MoeParams {
    const __half* x = nullptr;       // (T, H) normalised activations
    const void* gate_up = nullptr;   // (E, 2F, H) int8 codes or fp16 weights
    const __half* gu_scale = nullptr;
    const void* down = nullptr;      // (E, H, F)
    const __half* dn_scale = nullptr;
    const int64_t* ids = nullptr;    // (T, K)
    const __half* top_w = nullptr;   // (T, K)
    int T = 1, K = 0, E = 0, H = 0, F = 0, group_size = 128;
    __half* act = nullptr;           // (T, K, F)
    __half* out = nullptr;           // (T, H)
    const __half* resid = nullptr;   // optional (T, H): out = fp16(acc) + resid
    int* err_flag = nullptr;
};
int launch_moe_gate_up(const MoeParams& p, bool w8, const LaunchCfg& lc);
int launch_moe_down(const MoeParams& p, bool w8, const LaunchCfg& lc);
bool stream_moe_eligible(const MoeParams& p);
int launch_stream_gate_up(const MoeParams& p, const LaunchCfg& lc);
int launch_stream_down(const MoeParams& p, const LaunchCfg& lc);

// ---- attention --------------------------------------------------------------------
struct AttnParams {
    // q source: either a finished (H, D) fp16 q (fused == 0), or the raw packed qkv
    // projection row (3*H*D) on which the kernel applies q/k RMSNorm + RoPE itself and
    // writes the new K/V row into the caches (fused == 1).
    const __half* q = nullptr;
    const __half* qkv = nullptr;
    const __half* q_norm_w = nullptr;
    const __half* k_norm_w = nullptr;
    const __half* rope_cos = nullptr;  // (max_len, D)
    const __half* rope_sin = nullptr;
    const int64_t* cache_position = nullptr;
    float eps = 0.f;
    // caches
    const void* k = nullptr;  // fp16 (H, S, D) or int8 codes
    const void* v = nullptr;
    const __half* ks = nullptr;  // (H, S) int8 mode
    const __half* vs = nullptr;
    __half* keys_fp16 = nullptr;  // fused: fp16 static cache to write the new row into
    __half* values_fp16 = nullptr;
    int64_t kv_head_stride = 0;   // elements between heads in k / v
    const int32_t* filled = nullptr;
    __half* out = nullptr;  // (H, D)
    int heads = 0, S = 0, D = 0, num_splits = 1;
    float qk_scale_log2 = 0.f;  // scale * log2(e)
    float* part = nullptr;      // (H, splits, D + 2) fp32 partials
    unsigned int* counters = nullptr;  // (H)
    int* err_flag = nullptr;
};
int launch_attn_decode(const AttnParams& p, bool int8_kv, bool fused, const LaunchCfg& lc);

// ---- small ops ---------------------------------------------------------------------
int launch_rms_norm(const __half* x, const __half* w, __half* y, int64_t rows, int H, float eps, const LaunchCfg& lc);
int launch_rope_qk(const __half* q, int64_t q_hs, int heads_q, const __half* k, int64_t k_hs, int heads_k,
                   const __half* cos, const __half* sin, int D, __half* q_out, __half* k_out, const LaunchCfg& lc);
int launch_kv_direct_write(const __half* k_row, const __half* v_row, int64_t src_hs, __half* k_cache, __half* v_cache,
                           const int64_t* pos, int heads, int max_len, int D, int* err_flag, const LaunchCfg& lc);
int launch_kv_int8_cache_write(const __half* k_row, const __half* v_row, int8_t* kc, __half* ks, int8_t* vc,
                               __half* vs, const int64_t* pos, int heads, int S, int D, int* err_flag,
                               const LaunchCfg& lc);
int launch_kv_int8_bulk(const __half* keys, const __half* values, int8_t* kc, __half* ks, int8_t* vc, __half* vs,
                        int heads, int S, int D, int filled, const LaunchCfg& lc);
int launch_rtn_quantize(const void* w, int w_dtype, int64_t rows, int in_features, int group_size, int8_t* codes,
                        __half* scale, const LaunchCfg& lc);

}  // namespace lemoq
