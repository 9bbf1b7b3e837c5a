// extern "C" entry points: argument validation + launch.  No allocation, no sync.
#include <cstdarg>
#include <cstdio>

#include "kernels.h"

namespace lemoq {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static LaunchCfg cfg_of(void* stream) {
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    return lc;
}

}  // namespace lemoq

using namespace lemoq;

extern "C" const char* lemoq_version(void) { return "lemoq_b200 0.1 (sm_100a)"; }
extern "C" const char* lemoq_last_error(void) { return g_err; }
extern "C" int lemoq_set_tuning(int key, int value) { return set_stream_tuning(key, value); }

extern "C" int lemoq_rtn_quantize_w8(const void* w, int w_dtype, int64_t rows, int in_features, int group_size,
                                     int8_t* codes, void* scale, void* stream) {
    LEMOQ_REQUIRE(w && codes && scale, LEMOQ_ERR_INVALID, "rtn_quantize_w8: null pointer");
    LEMOQ_REQUIRE(w_dtype == LEMOQ_DTYPE_F16 || w_dtype == LEMOQ_DTYPE_F32, LEMOQ_ERR_UNSUPPORTED,
                  "rtn_quantize_w8: weights must be fp16 or fp32");
    LEMOQ_REQUIRE(rows >= 0 && in_features > 0 && group_size > 0, LEMOQ_ERR_INVALID,
                  "rtn_quantize_w8: group_size must be > 0 and sizes non-negative");
    LEMOQ_REQUIRE(in_features % group_size == 0, LEMOQ_ERR_UNSUPPORTED,
                  "rtn_quantize_w8: in_features=%d is not a multiple of group_size=%d (no zero padding on this path)",
                  in_features, group_size);
    return launch_rtn_quantize(w, w_dtype, rows, in_features, group_size, codes, reinterpret_cast<__half*>(scale),
                               cfg_of(stream));
}

extern "C" int lemoq_dequant_gemv_w8(const void* x, int M, const int8_t* codes, const void* scale, int N, int K,
                                     int group_size, void* y, int out_dtype, void* stream) {
    LEMOQ_REQUIRE(x && codes && scale && y, LEMOQ_ERR_INVALID, "dequant_gemv_w8: null pointer");
    LEMOQ_REQUIRE(M >= 0 && N > 0 && K > 0, LEMOQ_ERR_INVALID, "dequant_gemv_w8: bad shape M=%d N=%d K=%d", M, N, K);
    LEMOQ_REQUIRE(group_size > 0 && group_size % 16 == 0, LEMOQ_ERR_UNSUPPORTED,
                  "dequant_gemv_w8: group_size=%d must be a positive multiple of 16", group_size);
    LEMOQ_REQUIRE(K % group_size == 0, LEMOQ_ERR_INVALID, "dequant_gemv_w8: K=%d is not a multiple of group_size=%d", K,
                  group_size);
    LEMOQ_REQUIRE(out_dtype == LEMOQ_DTYPE_F16 || out_dtype == LEMOQ_DTYPE_F32, LEMOQ_ERR_UNSUPPORTED,
                  "dequant_gemv_w8: out_dtype must be fp16 or fp32");
    LEMOQ_REQUIRE(aligned16(x) && aligned16(codes), LEMOQ_ERR_INVALID, "dequant_gemv_w8: x and codes must be 16-byte aligned");
    LEMOQ_REQUIRE(M <= 65535, LEMOQ_ERR_UNSUPPORTED, "dequant_gemv_w8: M=%d too large for a GEMV", M);
    if (M == 0) return LEMOQ_OK;
    GemvParams p;
    p.x = reinterpret_cast<const __half*>(x);
    p.x_stride = K;
    p.codes = codes;
    p.scale = reinterpret_cast<const __half*>(scale);
    p.N = N;
    p.K = K;
    p.group_size = group_size;
    p.y = y;
    p.y_stride = N;
    return launch_gemv_w8(p, M, false, false, out_dtype == LEMOQ_DTYPE_F32, cfg_of(stream));
}

extern "C" int lemoq_rms_norm(const void* x, const void* w, void* y, int64_t rows, int H, float eps, void* stream) {
    LEMOQ_REQUIRE(x && w && y, LEMOQ_ERR_INVALID, "rms_norm: null pointer");
    LEMOQ_REQUIRE(rows >= 0 && H > 0, LEMOQ_ERR_INVALID, "rms_norm: bad shape");
    LEMOQ_REQUIRE(H % 8 == 0 && H <= 8192, LEMOQ_ERR_UNSUPPORTED, "rms_norm: H=%d must be a multiple of 8 and <= 8192", H);
    LEMOQ_REQUIRE(aligned16(x) && aligned16(w) && aligned16(y), LEMOQ_ERR_INVALID, "rms_norm: pointers must be 16-byte aligned");
    LEMOQ_REQUIRE(rows <= 0x7fffffffll, LEMOQ_ERR_INVALID, "rms_norm: too many rows");
    return launch_rms_norm(reinterpret_cast<const __half*>(x), reinterpret_cast<const __half*>(w),
                           reinterpret_cast<__half*>(y), rows, H, eps, cfg_of(stream));
}

extern "C" int lemoq_rope_qk(const void* q, int64_t q_head_stride, int heads_q, const void* k, int64_t k_head_stride,
                             int heads_k, const void* cos, const void* sin, int D, void* q_out, void* k_out,
                             void* stream) {
    LEMOQ_REQUIRE(q && k && cos && sin && q_out && k_out, LEMOQ_ERR_INVALID, "rope_qk: null pointer");
    LEMOQ_REQUIRE(heads_q > 0 && heads_k > 0 && D >= 2 && D % 2 == 0, LEMOQ_ERR_INVALID, "rope_qk: bad shape");
    return launch_rope_qk(reinterpret_cast<const __half*>(q), q_head_stride, heads_q, reinterpret_cast<const __half*>(k),
                          k_head_stride, heads_k, reinterpret_cast<const __half*>(cos),
                          reinterpret_cast<const __half*>(sin), D, reinterpret_cast<__half*>(q_out),
                          reinterpret_cast<__half*>(k_out), cfg_of(stream));
}

extern "C" int lemoq_kv_direct_write(const void* k_row, const void* v_row, int64_t src_head_stride, void* k_cache,
                                     void* v_cache, const int64_t* pos, int heads, int max_len, int D, int* err_flag,
                                     void* stream) {
    LEMOQ_REQUIRE(k_row && v_row && k_cache && v_cache && pos, LEMOQ_ERR_INVALID, "kv_direct_write: null pointer");
    LEMOQ_REQUIRE(heads > 0 && max_len > 0 && D > 0, LEMOQ_ERR_INVALID, "kv_direct_write: bad shape");
    return launch_kv_direct_write(reinterpret_cast<const __half*>(k_row), reinterpret_cast<const __half*>(v_row),
                                  src_head_stride, reinterpret_cast<__half*>(k_cache),
                                  reinterpret_cast<__half*>(v_cache), pos, heads, max_len, D, err_flag, cfg_of(stream));
}

extern "C" int lemoq_kv_int8_cache_write(const void* k_row, const void* v_row, int8_t* kc, void* ks, int8_t* vc,
                                         void* vs, const int64_t* pos, int heads, int S, int D, int* err_flag,
                                         void* stream) {
    LEMOQ_REQUIRE(k_row && v_row && kc && ks && vc && vs, LEMOQ_ERR_INVALID, "kv_int8_cache_write: null pointer");
    LEMOQ_REQUIRE(heads > 0 && S > 0 && D > 0, LEMOQ_ERR_INVALID, "kv_int8_cache_write: bad shape");
    LEMOQ_REQUIRE(pos != nullptr || S == 1, LEMOQ_ERR_INVALID, "kv_int8_cache_write: pos may be NULL only when S == 1");
    return launch_kv_int8_cache_write(reinterpret_cast<const __half*>(k_row), reinterpret_cast<const __half*>(v_row), kc,
                                      reinterpret_cast<__half*>(ks), vc, reinterpret_cast<__half*>(vs), pos, heads, S, D,
                                      err_flag, cfg_of(stream));
}

extern "C" int lemoq_kv_int8_bulk_quantize(const void* keys, const void* values, int8_t* kc, void* ks, int8_t* vc,
                                           void* vs, int heads, int S, int D, int filled, void* stream) {
    LEMOQ_REQUIRE(keys && values && kc && ks && vc && vs, LEMOQ_ERR_INVALID, "kv_int8_bulk_quantize: null pointer");
    LEMOQ_REQUIRE(heads > 0 && S > 0 && D > 0, LEMOQ_ERR_INVALID, "kv_int8_bulk_quantize: bad shape");
    if (filled > S) filled = S;
    return launch_kv_int8_bulk(reinterpret_cast<const __half*>(keys), reinterpret_cast<const __half*>(values), kc,
                               reinterpret_cast<__half*>(ks), vc, reinterpret_cast<__half*>(vs), heads, S, D, filled,
                               cfg_of(stream));
}

extern "C" size_t lemoq_attn_workspace_bytes(int heads, int D, int num_splits) {
    if (heads <= 0 || D <= 0 || num_splits <= 0) return 0;
    // counters first (256-byte slot), then the fp32 partials
    const size_t counters = (sizeof(unsigned int) * heads + 255) / 256 * 256;
    return counters + sizeof(float) * heads * num_splits * (D + 2);
}

static int attn_common(AttnParams& p, const void* q, const int32_t* filled, void* out, int heads, int S, int D,
                       int num_splits, float scale, void* workspace, int* err_flag) {
    LEMOQ_REQUIRE(q && filled && out && workspace, LEMOQ_ERR_INVALID, "attn_decode: null pointer");
    LEMOQ_REQUIRE(heads > 0 && S > 0, LEMOQ_ERR_INVALID, "attn_decode: heads and cache capacity must be positive");
    LEMOQ_REQUIRE(D == 64 || D == 128, LEMOQ_ERR_UNSUPPORTED, "attn_decode: head_dim=%d, built for 64 and 128", D);
    LEMOQ_REQUIRE(num_splits >= 1 && num_splits <= 4096, LEMOQ_ERR_INVALID, "attn_decode: num_splits must be >= 1");
    LEMOQ_REQUIRE(aligned16(workspace), LEMOQ_ERR_INVALID, "attn_decode: workspace must be 16-byte aligned");
    p.q = reinterpret_cast<const __half*>(q);
    p.filled = filled;
    p.out = reinterpret_cast<__half*>(out);
    p.heads = heads;
    p.S = S;
    p.D = D;
    p.num_splits = num_splits;
    p.qk_scale_log2 = scale * 1.4426950408889634f;
    const size_t counters = (sizeof(unsigned int) * heads + 255) / 256 * 256;
    p.counters = reinterpret_cast<unsigned int*>(workspace);
    p.part = reinterpret_cast<float*>(static_cast<char*>(workspace) + counters);
    p.err_flag = err_flag;
    return LEMOQ_OK;
}

extern "C" int lemoq_attn_decode_fp16(const void* q, const void* k, const void* v, int64_t kv_head_stride,
                                      const int32_t* filled, void* out, int heads, int S, int D, int num_splits,
                                      float scale, void* workspace, int* err_flag, void* stream) {
    AttnParams p;
    if (int rc = attn_common(p, q, filled, out, heads, S, D, num_splits, scale, workspace, err_flag)) return rc;
    LEMOQ_REQUIRE(k && v, LEMOQ_ERR_INVALID, "attn_decode_fp16: null cache pointer");
    LEMOQ_REQUIRE(aligned16(k) && aligned16(v) && kv_head_stride % 8 == 0, LEMOQ_ERR_INVALID,
                  "attn_decode_fp16: caches must be 16-byte aligned with a head stride that is a multiple of 8");
    LEMOQ_REQUIRE(kv_head_stride >= static_cast<int64_t>(S) * D, LEMOQ_ERR_INVALID,
                  "attn_decode_fp16: heads overlap (head stride < S*D)");
    p.k = k;
    p.v = v;
    p.kv_head_stride = kv_head_stride;
    return launch_attn_decode(p, false, false, cfg_of(stream));
}

extern "C" int lemoq_attn_decode_int8(const void* q, const int8_t* kc, const void* ks, const int8_t* vc, const void* vs,
                                      int64_t kv_head_stride, const int32_t* filled, void* out, int heads, int S, int D,
                                      int num_splits, float scale, void* workspace, int* err_flag, void* stream) {
    AttnParams p;
    if (int rc = attn_common(p, q, filled, out, heads, S, D, num_splits, scale, workspace, err_flag)) return rc;
    LEMOQ_REQUIRE(kc && ks && vc && vs, LEMOQ_ERR_INVALID, "attn_decode_int8: null cache pointer");
    LEMOQ_REQUIRE(aligned16(kc) && aligned16(vc) && kv_head_stride % 16 == 0, LEMOQ_ERR_INVALID,
                  "attn_decode_int8: codes must be 16-byte aligned with a head stride that is a multiple of 16");
    LEMOQ_REQUIRE(kv_head_stride >= static_cast<int64_t>(S) * D, LEMOQ_ERR_INVALID,
                  "attn_decode_int8: heads overlap (head stride < S*D)");
    p.k = kc;
    p.v = vc;
    p.ks = reinterpret_cast<const __half*>(ks);
    p.vs = reinterpret_cast<const __half*>(vs);
    p.kv_head_stride = kv_head_stride;
    return launch_attn_decode(p, true, false, cfg_of(stream));
}

extern "C" int lemoq_routing_softmax_topk(const void* logits, int logits_dtype, int64_t row_stride, int T, int E,
                                          int top_k, int norm_topk_prob, float* top_w, int64_t* top_i, void* stream) {
    LEMOQ_REQUIRE(T >= 0 && E > 0, LEMOQ_ERR_INVALID, "routing_softmax_topk: bad shape");
    LEMOQ_REQUIRE(top_k > 0 && top_k <= E, LEMOQ_ERR_INVALID, "routing_softmax_topk: top_k=%d must be in (0, %d]", top_k, E);
    LEMOQ_REQUIRE(E <= kMaxExperts, LEMOQ_ERR_UNSUPPORTED, "routing_softmax_topk: E=%d above %d", E, kMaxExperts);
    LEMOQ_REQUIRE(logits_dtype == LEMOQ_DTYPE_F16 || logits_dtype == LEMOQ_DTYPE_F32, LEMOQ_ERR_UNSUPPORTED,
                  "routing_softmax_topk: logits must be fp16 or fp32");
    if (T == 0) return LEMOQ_OK;
    LEMOQ_REQUIRE(logits && top_w && top_i, LEMOQ_ERR_INVALID, "routing_softmax_topk: null pointer");
    return launch_routing_topk(logits, logits_dtype, row_stride, T, E, top_k, norm_topk_prob, top_w, top_i,
                               cfg_of(stream));
}

extern "C" int lemoq_route(const void* h, const void* router_w, int E, int H, int top_k, int norm_topk_prob,
                           void* logits_out, void* top_w, int64_t* top_i, void* workspace, void* stream) {
    LEMOQ_REQUIRE(h && router_w && logits_out && top_w && top_i && workspace, LEMOQ_ERR_INVALID, "route: null pointer");
    LEMOQ_REQUIRE(E > 0 && E <= kMaxExperts && top_k > 0 && top_k <= E && top_k <= kMaxTopK, LEMOQ_ERR_INVALID,
                  "route: experts/top_k out of range");
    LEMOQ_REQUIRE(H > 0 && H % 16 == 0 && H <= 2048, LEMOQ_ERR_UNSUPPORTED, "route: H=%d must be a multiple of 16, <= 2048", H);
    LEMOQ_REQUIRE(aligned16(h) && aligned16(router_w), LEMOQ_ERR_INVALID, "route: pointers must be 16-byte aligned");
    RouteParams p;
    p.x = reinterpret_cast<const __half*>(h);
    p.router_w = reinterpret_cast<const __half*>(router_w);
    p.E = E;
    p.H = H;
    p.top_k = top_k;
    p.norm_topk_prob = norm_topk_prob;
    p.logits_out = reinterpret_cast<__half*>(logits_out);
    p.top_w = reinterpret_cast<__half*>(top_w);
    p.top_i = top_i;
    p.counter = reinterpret_cast<unsigned int*>(workspace);
    return launch_route(p, false, cfg_of(stream));
}

static int moe_common(MoeParams& p, const void* x, const int64_t* ids, const void* top_w, int T, int K, int E, int H,
                      int F, void* act, void* out, int* err_flag) {
    LEMOQ_REQUIRE(x && ids && top_w && act && out, LEMOQ_ERR_INVALID, "moe_grouped: null pointer");
    LEMOQ_REQUIRE(T >= 0 && K > 0 && E > 0 && H > 0 && F > 0, LEMOQ_ERR_INVALID, "moe_grouped: bad shape");
    LEMOQ_REQUIRE(K <= kMaxTopK, LEMOQ_ERR_UNSUPPORTED, "moe_grouped: K=%d slots above %d", K, kMaxTopK);
    LEMOQ_REQUIRE(H % 16 == 0 && F % 16 == 0, LEMOQ_ERR_INVALID, "moe_grouped: hidden and ffn must be multiples of 16");
    LEMOQ_REQUIRE(T <= 65535, LEMOQ_ERR_UNSUPPORTED, "moe_grouped: T=%d tokens above the grid limit", T);
    LEMOQ_REQUIRE(aligned16(x) && aligned16(act), LEMOQ_ERR_INVALID, "moe_grouped: x and act must be 16-byte aligned");
    p.x = reinterpret_cast<const __half*>(x);
    p.ids = ids;
    p.top_w = reinterpret_cast<const __half*>(top_w);
    p.T = T;
    p.K = K;
    p.E = E;
    p.H = H;
    p.F = F;
    p.act = reinterpret_cast<__half*>(act);
    p.out = reinterpret_cast<__half*>(out);
    p.err_flag = err_flag;
    return LEMOQ_OK;
}

extern "C" int lemoq_moe_grouped_w8(const void* x, const int8_t* gu_codes, const void* gu_scale, const int8_t* dn_codes,
                                    const void* dn_scale, const int64_t* ids, const void* top_w, int T, int K, int E,
                                    int H, int F, int group_size, void* act, void* out, int* err_flag, void* stream) {
    MoeParams p;
    if (int rc = moe_common(p, x, ids, top_w, T, K, E, H, F, act, out, err_flag)) return rc;
    LEMOQ_REQUIRE(gu_codes && gu_scale && dn_codes && dn_scale, LEMOQ_ERR_INVALID, "moe_grouped_w8: null weight pointer");
    LEMOQ_REQUIRE(group_size > 0 && group_size % 16 == 0, LEMOQ_ERR_UNSUPPORTED,
                  "moe_grouped_w8: group_size=%d must be a positive multiple of 16", group_size);
    LEMOQ_REQUIRE(H % group_size == 0 && F % group_size == 0, LEMOQ_ERR_INVALID,
                  "moe_grouped_w8: hidden=%d / ffn=%d not divisible by group_size=%d", H, F, group_size);
    LEMOQ_REQUIRE(aligned16(gu_codes) && aligned16(dn_codes), LEMOQ_ERR_INVALID, "moe_grouped_w8: codes must be 16-byte aligned");
    if (T == 0) return LEMOQ_OK;
    p.gate_up = gu_codes;
    p.gu_scale = reinterpret_cast<const __half*>(gu_scale);
    p.down = dn_codes;
    p.dn_scale = reinterpret_cast<const __half*>(dn_scale);
    p.group_size = group_size;
    const LaunchCfg lc = cfg_of(stream);
    if (int rc = launch_moe_gate_up(p, true, lc)) return rc;
    return launch_moe_down(p, true, lc);
}

extern "C" int lemoq_moe_grouped_fp16(const void* x, const void* gate_up, const void* down, const int64_t* ids,
                                      const void* top_w, int T, int K, int E, int H, int F, void* act, void* out,
                                      int* err_flag, void* stream) {
    MoeParams p;
    if (int rc = moe_common(p, x, ids, top_w, T, K, E, H, F, act, out, err_flag)) return rc;
    LEMOQ_REQUIRE(gate_up && down, LEMOQ_ERR_INVALID, "moe_grouped_fp16: null weight pointer");
    LEMOQ_REQUIRE(aligned16(gate_up) && aligned16(down), LEMOQ_ERR_INVALID, "moe_grouped_fp16: weights must be 16-byte aligned");
    if (T == 0) return LEMOQ_OK;
    p.gate_up = gate_up;
    p.down = down;
    const LaunchCfg lc = cfg_of(stream);
    if (int rc = launch_moe_gate_up(p, false, lc)) return rc;
    return launch_moe_down(p, false, lc);
}

extern "C" int lemoq_moe_gate_up_w8(const void* x, const int8_t* gu_codes, const void* gu_scale, const int64_t* ids, int T,
                                    int K, int E, int H, int F, int group_size, void* act, int* err_flag, void* stream) {
    MoeParams p;
    // top_w / out are unused by this launch; pass act for both so that the common checks hold
    if (int rc = moe_common(p, x, ids, act, T, K, E, H, F, act, act, err_flag)) return rc;
    LEMOQ_REQUIRE(gu_codes && gu_scale, LEMOQ_ERR_INVALID, "moe_gate_up_w8: null weight pointer");
    LEMOQ_REQUIRE(group_size > 0 && group_size % 16 == 0 && H % group_size == 0, LEMOQ_ERR_INVALID,
                  "moe_gate_up_w8: hidden=%d / group_size=%d", H, group_size);
    if (T == 0) return LEMOQ_OK;
    p.gate_up = gu_codes;
    p.gu_scale = reinterpret_cast<const __half*>(gu_scale);
    p.group_size = group_size;
    return launch_moe_gate_up(p, true, cfg_of(stream));
}

extern "C" int lemoq_moe_down_w8(const void* act, const int8_t* dn_codes, const void* dn_scale, const int64_t* ids,
                                 const void* top_w, int T, int K, int E, int H, int F, int group_size, void* out,
                                 int* err_flag, void* stream) {
    MoeParams p;
    if (int rc = moe_common(p, act, ids, top_w, T, K, E, H, F, const_cast<void*>(act), out, err_flag)) return rc;
    LEMOQ_REQUIRE(dn_codes && dn_scale, LEMOQ_ERR_INVALID, "moe_down_w8: null weight pointer");
    LEMOQ_REQUIRE(group_size > 0 && group_size % 16 == 0 && F % group_size == 0, LEMOQ_ERR_INVALID,
                  "moe_down_w8: ffn=%d / group_size=%d", F, group_size);
    if (T == 0) return LEMOQ_OK;
    p.down = dn_codes;
    p.dn_scale = reinterpret_cast<const __half*>(dn_scale);
    p.group_size = group_size;
    return launch_moe_down(p, true, cfg_of(stream));
}
