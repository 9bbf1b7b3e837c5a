// Whole decode step: a fixed chain of 6 kernels per layer plus the lm_head GEMV.
//
//   K1  q.k.v GEMV        input RMSNorm fused as prologue                 -> qkv (3A)
//   K2  attention         q/k RMSNorm + RoPE + KV write/quantise fused    -> attn (A)
//   K3  o_proj GEMV       residual add fused as epilogue                  -> x1 (H)
//   K4  router            post-attention RMSNorm prologue, softmax/top-k  -> h2, ids, weights
//   K5  expert gate/up    SwiGLU epilogue                                 -> act (K, F)
//   K6  expert down       routing-weighted sum + residual add             -> x2 (H)
//   ..  lm_head GEMV      final RMSNorm prologue                          -> logits (V)
//
// Every kernel prefetches the weights it can address before griddepcontrol.wait and
// releases its successor right after, so with programmatic dependent launch the
// HBM stream of kernel n+1 overlaps the dependent tail of kernel n.
#include <new>

#include "kernels.h"
#include <cstdio>
#include <cstdlib>

#include "step_kernel.h"

struct lemoq_step {
    lemoq_step_desc d;
    lemoq_layer_desc* layers;
    int splits;
    // workspace carve-up
    int* err_flag;
    unsigned int* attn_counters;
    unsigned int* route_counter;
    __half* qkv;
    __half* attn;
    __half* xa;
    __half* xb;
    __half* h2;
    __half* act;
    __half* router_logits;  // (layers, experts)
    __half* top_w;          // (top_k)
    int64_t* top_i;         // (layers, top_k)
    float* attn_part;
    // whole-step cooperative kernel
    unsigned int* bar_counter;
    unsigned int* bar_epoch;
    lemoq::StepLayer* whole_layers;  // device copy of the layer descriptors
    int whole_grid;                  // blocks of the whole-step kernel; 0 = chained kernels
    unsigned long long* flagged;    // flagged-word exchange buffers of the whole-step kernel
    unsigned long long* stamps;     // phase time stamps of the whole-step kernel
};

namespace lemoq {

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// words of the flagged exchange buffers: x 4*2048, q.k.v 2*6144, sums of squares 2*2048, logits 2*128, activations 2*4096
constexpr size_t kFlX = 0, kFlQkv = kFlX + 4 * 2048, kFlStats = kFlQkv + 2 * 6144, kFlLogits = kFlStats + 2 * 2048,
                 kFlAct = kFlLogits + 2 * 128, kFlaggedWords = kFlAct + 2 * 4096;

static int resolve_splits(const lemoq_step_desc& d) {
    if (d.attn_splits > 0) return d.attn_splits;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
    }
    int s = (2 * sms + d.heads - 1) / d.heads;
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    return s;
}

struct Carve {
    size_t off = 0;
    size_t take(size_t bytes) {
        const size_t o = off;
        off = align_up(off + bytes, 256);
        return o;
    }
};

static size_t carve(const lemoq_step_desc& d, int splits, lemoq_step* s) {
    Carve c;
    char* base = s ? static_cast<char*>(d.workspace) : nullptr;
    const int A = d.heads * d.head_dim;
#define LEMOQ_TAKE(field, type, bytes)                     \
    {                                                      \
        const size_t o = c.take(bytes);                    \
        if (s) s->field = reinterpret_cast<type>(base + o); \
    }
    LEMOQ_TAKE(err_flag, int*, sizeof(int));
    LEMOQ_TAKE(attn_counters, unsigned int*, sizeof(unsigned int) * d.heads);
    LEMOQ_TAKE(route_counter, unsigned int*, sizeof(unsigned int));
    LEMOQ_TAKE(qkv, __half*, sizeof(__half) * 3 * A);
    LEMOQ_TAKE(attn, __half*, sizeof(__half) * A);
    LEMOQ_TAKE(xa, __half*, sizeof(__half) * d.hidden);
    LEMOQ_TAKE(xb, __half*, sizeof(__half) * d.hidden);
    LEMOQ_TAKE(h2, __half*, sizeof(__half) * d.hidden);
    LEMOQ_TAKE(act, __half*, sizeof(__half) * d.top_k * d.ffn);
    LEMOQ_TAKE(router_logits, __half*, sizeof(__half) * d.layers * d.experts);
    LEMOQ_TAKE(top_w, __half*, sizeof(__half) * d.top_k);
    LEMOQ_TAKE(top_i, int64_t*, sizeof(int64_t) * d.layers * d.top_k);
    LEMOQ_TAKE(attn_part, float*, sizeof(float) * d.heads * splits * (d.head_dim + 2));
    LEMOQ_TAKE(flagged, unsigned long long*, sizeof(unsigned long long) * kFlaggedWords);
    LEMOQ_TAKE(bar_counter, unsigned int*, sizeof(unsigned int));
    LEMOQ_TAKE(bar_epoch, unsigned int*, sizeof(unsigned int));
    LEMOQ_TAKE(whole_layers, lemoq::StepLayer*, sizeof(lemoq::StepLayer) * (d.layers + 1));
    LEMOQ_TAKE(stamps, unsigned long long*, sizeof(unsigned long long) * (6 * d.layers + 2));
#undef LEMOQ_TAKE
    return c.off;
}

static int validate(const lemoq_step_desc& d) {
    LEMOQ_REQUIRE(d.layers > 0 && d.hidden > 0 && d.heads > 0 && d.experts > 0 && d.top_k > 0 && d.ffn > 0 &&
                      d.vocab > 0 && d.max_len > 0,
                  LEMOQ_ERR_INVALID, "step: all sizes must be positive");
    LEMOQ_REQUIRE(d.head_dim == 64 || d.head_dim == 128, LEMOQ_ERR_UNSUPPORTED, "step: head_dim must be 64 or 128");
    LEMOQ_REQUIRE(d.group_size > 0 && d.group_size % 16 == 0, LEMOQ_ERR_INVALID,
                  "step: group_size must be a positive multiple of 16");
    const int A = d.heads * d.head_dim;
    LEMOQ_REQUIRE(d.hidden % d.group_size == 0 && d.ffn % d.group_size == 0 && A % d.group_size == 0,
                  LEMOQ_ERR_INVALID, "step: hidden, ffn and heads*head_dim must be multiples of group_size");
    LEMOQ_REQUIRE(d.hidden <= 2048 && d.ffn <= 2048 && A <= 2048, LEMOQ_ERR_UNSUPPORTED,
                  "step: hidden/ffn/attention width above 2048 is not built");
    LEMOQ_REQUIRE(d.top_k <= d.experts && d.top_k <= kMaxTopK && d.experts <= kMaxExperts, LEMOQ_ERR_INVALID,
                  "step: top_k/experts out of range");
    LEMOQ_REQUIRE(d.embed && d.final_norm && d.lm_head_codes && d.lm_head_scale && d.rope_cos && d.rope_sin &&
                      d.token && d.cache_position && d.filled_len && d.logits && d.workspace,
                  LEMOQ_ERR_INVALID, "step: null pointer in descriptor");
    LEMOQ_REQUIRE(!d.self_feed || d.next_token, LEMOQ_ERR_INVALID, "step: self_feed needs next_token");
    return LEMOQ_OK;
}

}  // namespace lemoq

namespace lemoq {
// argmax(logits) -> *next_token, first maximal index (one block)
__global__ void greedy_pick_kernel(const __half* logits, int n, int64_t* next_token, int64_t* token, int64_t* cache_position,
                                   int32_t* filled, int64_t* token_log, int max_len) {
    __shared__ float rv[32];
    __shared__ int ri[32];
    const int tok = block_argmax_f16(logits, n, rv, ri);
    if (threadIdx.x == 0) {
        *next_token = tok;
        const int64_t pos = *cache_position;
        if (token_log != nullptr && pos >= 0 && pos < max_len) token_log[pos] = tok;
        if (token != nullptr) {  // self-feeding step: the pick is the next step's input
            *token = tok;
            *cache_position += 1;
            *filled += 1;
        }
    }
}

int g_step_use_whole = 1;  // lemoq_set_tuning key 4: run the step as one cooperative kernel when the shapes allow it
}

using namespace lemoq;

extern "C" size_t lemoq_step_workspace_bytes(const lemoq_step_desc* desc) {
    if (!desc) return 0;
    return carve(*desc, resolve_splits(*desc), nullptr);
}

extern "C" int lemoq_step_create(const lemoq_step_desc* desc, const lemoq_layer_desc* layers, lemoq_step** out) {
    LEMOQ_REQUIRE(desc && layers && out, LEMOQ_ERR_INVALID, "step_create: null argument");
    if (int rc = validate(*desc)) return rc;
    const int splits = resolve_splits(*desc);
    const size_t need = carve(*desc, splits, nullptr);
    LEMOQ_REQUIRE(desc->workspace_bytes >= need, LEMOQ_ERR_INVALID, "step_create: workspace has %zu bytes, %zu needed",
                  desc->workspace_bytes, need);
    LEMOQ_REQUIRE(reinterpret_cast<uintptr_t>(desc->workspace) % 32 == 0, LEMOQ_ERR_INVALID,
                  "step_create: workspace must be 32-byte aligned");
    for (int l = 0; l < desc->layers; ++l) {
        const lemoq_layer_desc& L = layers[l];
        LEMOQ_REQUIRE(L.ln1 && L.ln2 && L.q_norm && L.k_norm && L.qkv_codes && L.qkv_scale && L.o_codes && L.o_scale &&
                          L.router && L.gu_codes && L.gu_scale && L.dn_codes && L.dn_scale && L.keys && L.values,
                      LEMOQ_ERR_INVALID, "step_create: null pointer in layer %d", l);
        LEMOQ_REQUIRE(!desc->kv_int8 || (L.kc && L.ks && L.vc && L.vs), LEMOQ_ERR_INVALID,
                      "step_create: layer %d has no int8 KV mirror", l);
    }
    lemoq_step* s = new (std::nothrow) lemoq_step();
    LEMOQ_REQUIRE(s, LEMOQ_ERR_CUDA, "step_create: out of host memory");
    s->d = *desc;
    s->layers = new (std::nothrow) lemoq_layer_desc[desc->layers];
    if (!s->layers) {
        delete s;
        return set_error(LEMOQ_ERR_CUDA, "step_create: out of host memory");
    }
    for (int l = 0; l < desc->layers; ++l) s->layers[l] = layers[l];
    s->splits = splits;
    carve(*desc, splits, s);
    s->whole_grid = 0;
    const bool want_whole = g_step_use_whole != 0 && tile_eligible(*desc);
    if (getenv("LEMOQ_VERBOSE")) fprintf(stderr, "lemoq: whole-step kernel eligible: %d\n", (int)want_whole);
    if (want_whole) {
        const int tgrid = tile_grid(*desc);
        const int grid = tgrid <= 1024 ? tgrid : 0;
        if (grid > 0) {
            // attention units are (head, split) blocks: at most one per resident block
            int ms = tile_attention_splits(*desc, grid);
            if (desc->attn_splits > 0 && desc->attn_splits < ms) ms = desc->attn_splits;
            // (the partials buffer doubles as the per-block candidate list of the greedy pick: 2 floats per block)
            if (desc->heads * ms <= grid && ms <= splits && desc->heads * splits * (desc->head_dim + 2) >= 2 * grid) {
                StepLayer* host = new (std::nothrow) StepLayer[desc->layers + 1]();
                if (host) {
                    for (int l = 0; l < desc->layers; ++l) {
                        const lemoq_layer_desc& L = layers[l];
                        StepLayer& m = host[l];
                        m.ln1 = reinterpret_cast<const __half*>(L.ln1);
                        m.ln2 = reinterpret_cast<const __half*>(L.ln2);
                        m.q_norm = reinterpret_cast<const __half*>(L.q_norm);
                        m.k_norm = reinterpret_cast<const __half*>(L.k_norm);
                        m.qkv_codes = L.qkv_codes;
                        m.qkv_scale = reinterpret_cast<const __half*>(L.qkv_scale);
                        m.o_codes = L.o_codes;
                        m.o_scale = reinterpret_cast<const __half*>(L.o_scale);
                        m.router = reinterpret_cast<const __half*>(L.router);
                        m.gu_codes = L.gu_codes;
                        m.gu_scale = reinterpret_cast<const __half*>(L.gu_scale);
                        m.dn_codes = L.dn_codes;
                        m.dn_scale = reinterpret_cast<const __half*>(L.dn_scale);
                        m.keys = reinterpret_cast<__half*>(L.keys);
                        m.values = reinterpret_cast<__half*>(L.values);
                        m.kc = L.kc;
                        m.ks = reinterpret_cast<__half*>(L.ks);
                        m.vc = L.vc;
                        m.vs = reinterpret_cast<__half*>(L.vs);
                    }
                    // pseudo layer after the last one: the lm_head rows stream like q.k.v rows behind the final norm
                    host[desc->layers].ln1 = reinterpret_cast<const __half*>(desc->final_norm);
                    host[desc->layers].qkv_codes = desc->lm_head_codes;
                    host[desc->layers].qkv_scale = reinterpret_cast<const __half*>(desc->lm_head_scale);
                    // set-up time only: the descriptors move to the device once (synchronous copy)
                    const cudaError_t err = cudaMemcpy(s->whole_layers, host, sizeof(StepLayer) * (desc->layers + 1), cudaMemcpyHostToDevice);
                    delete[] host;
                    if (err == cudaSuccess) {
                        s->whole_grid = grid;
                        s->splits = ms;
                    }
                }
            }
        }
    }
    *out = s;
    return LEMOQ_OK;
}

extern "C" void lemoq_step_destroy(lemoq_step* s) {
    if (!s) return;
    delete[] s->layers;
    delete s;
}

extern "C" int* lemoq_step_error_flag(lemoq_step* s) { return s ? s->err_flag : nullptr; }
extern "C" const int64_t* lemoq_step_topk_ids(lemoq_step* s) { return s ? s->top_i : nullptr; }
extern "C" const void* lemoq_step_router_logits(lemoq_step* s) { return s ? s->router_logits : nullptr; }
extern "C" const char* lemoq_step_engine(lemoq_step* s) {
    return (s && s->whole_grid > 0) ? "whole-step" : "chained";
}
extern "C" const unsigned long long* lemoq_step_phase_stamps(lemoq_step* s) { return (s && s->whole_grid > 0) ? s->stamps : nullptr; }

extern "C" int lemoq_step_run(lemoq_step* s, void* stream, int* launches) {
    LEMOQ_REQUIRE(s, LEMOQ_ERR_INVALID, "step_run: null step");
    const lemoq_step_desc& d = s->d;
    const int A = d.heads * d.head_dim;
    int count = 0;
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    lc.pdl = d.use_pdl != 0;
    lc.launch_count = &count;
    const float qk = (1.0f / sqrtf(static_cast<float>(d.head_dim))) * 1.4426950408889634f;

    if (s->whole_grid > 0) {
        StepParams p;
        p.layers = d.layers; p.H = d.hidden; p.heads = d.heads; p.D = d.head_dim; p.E = d.experts; p.K = d.top_k;
        p.F = d.ffn; p.V = d.vocab; p.group = d.group_size; p.S = d.max_len; p.splits = s->splits;
        p.kv_int8 = d.kv_int8; p.norm_topk = d.norm_topk_prob; p.eps = d.eps; p.qk_scale_log2 = qk;
        p.embed = reinterpret_cast<const __half*>(d.embed);
        p.final_norm = reinterpret_cast<const __half*>(d.final_norm);
        p.lm_scale = reinterpret_cast<const __half*>(d.lm_head_scale);
        p.rope_cos = reinterpret_cast<const __half*>(d.rope_cos);
        p.rope_sin = reinterpret_cast<const __half*>(d.rope_sin);
        p.lm_codes = d.lm_head_codes;
        p.token = d.token; p.cache_position = d.cache_position; p.filled = d.filled_len;
        p.logits = reinterpret_cast<__half*>(d.logits);
        p.next_token = d.next_token;
        p.self_feed = d.self_feed != 0 && d.next_token != nullptr;
        p.token_log = d.token_log;
        p.L = s->whole_layers;
        p.err_flag = s->err_flag; p.bar_counter = s->bar_counter; p.bar_epoch = s->bar_epoch;
        p.fl_x = s->flagged + kFlX; p.fl_qkv = s->flagged + kFlQkv; p.fl_stats = s->flagged + kFlStats;
        p.fl_logits = s->flagged + kFlLogits; p.fl_act = s->flagged + kFlAct;
        p.router_logits = s->router_logits; p.top_w = s->top_w; p.top_i = s->top_i; p.attn_part = s->attn_part;
        p.barriers_per_launch = d.layers + 1;  // attention -> o_proj in every layer, and the end of the step
        p.stamps = s->stamps;
        if (int rc = launch_step_tile(p, s->whole_grid, static_cast<cudaStream_t>(stream))) return rc;
        if (launches) *launches = 1;
        return LEMOQ_OK;
    }

    const __half* x_prev = reinterpret_cast<const __half*>(d.embed);
    const int64_t* x_token = d.token;  // layer 0 reads the embedding row of *token
    for (int l = 0; l < d.layers; ++l) {
        const lemoq_layer_desc& L = s->layers[l];
        // K1: qkv = W8(qkv) . RMSNorm(x_prev)
        {
            GemvParams p;
            p.x = x_prev;
            p.x_token = x_token;
            p.token_rows = d.vocab;
            p.norm_w = reinterpret_cast<const __half*>(L.ln1);
            p.eps = d.eps;
            p.codes = L.qkv_codes;
            p.scale = reinterpret_cast<const __half*>(L.qkv_scale);
            p.N = 3 * A;
            p.K = d.hidden;
            p.group_size = d.group_size;
            p.y = s->qkv;
            p.err_flag = s->err_flag;
            if (int rc = launch_gemv_w8(p, 1, true, false, false, lc)) return rc;
        }
        // K2: attention with fused q/k norm, RoPE, KV write
        {
            AttnParams p;
            p.qkv = s->qkv;
            p.q_norm_w = reinterpret_cast<const __half*>(L.q_norm);
            p.k_norm_w = reinterpret_cast<const __half*>(L.k_norm);
            p.rope_cos = reinterpret_cast<const __half*>(d.rope_cos);
            p.rope_sin = reinterpret_cast<const __half*>(d.rope_sin);
            p.cache_position = d.cache_position;
            p.eps = d.eps;
            p.keys_fp16 = reinterpret_cast<__half*>(L.keys);
            p.values_fp16 = reinterpret_cast<__half*>(L.values);
            if (d.kv_int8) {
                p.k = L.kc;
                p.v = L.vc;
                p.ks = reinterpret_cast<const __half*>(L.ks);
                p.vs = reinterpret_cast<const __half*>(L.vs);
            } else {
                p.k = L.keys;
                p.v = L.values;
            }
            p.kv_head_stride = static_cast<int64_t>(d.max_len) * d.head_dim;
            p.filled = d.filled_len;
            p.out = s->attn;
            p.heads = d.heads;
            p.S = d.max_len;
            p.D = d.head_dim;
            p.num_splits = s->splits;
            p.qk_scale_log2 = qk;
            p.part = s->attn_part;
            p.counters = s->attn_counters;
            p.err_flag = s->err_flag;
            if (int rc = launch_attn_decode(p, d.kv_int8 != 0, true, lc)) return rc;
        }
        // K3: x1 = x_prev + W8(o) . attn
        {
            GemvParams p;
            p.x = s->attn;
            p.codes = L.o_codes;
            p.scale = reinterpret_cast<const __half*>(L.o_scale);
            p.N = d.hidden;
            p.K = A;
            p.group_size = d.group_size;
            p.y = s->xa;
            p.err_flag = s->err_flag;
            p.resid = x_prev;
            p.resid_token = x_token;
            p.token_rows = d.vocab;
            if (int rc = launch_gemv_w8(p, 1, false, true, false, lc)) return rc;
        }
        // K4: h2 = RMSNorm(x1); router logits, softmax, top-k
        {
            RouteParams p;
            p.x = s->xa;
            p.norm_w = reinterpret_cast<const __half*>(L.ln2);
            p.eps = d.eps;
            p.router_w = reinterpret_cast<const __half*>(L.router);
            p.E = d.experts;
            p.H = d.hidden;
            p.top_k = d.top_k;
            p.norm_topk_prob = d.norm_topk_prob;
            p.h_out = s->h2;
            p.logits_out = s->router_logits + static_cast<int64_t>(l) * d.experts;
            p.top_w = s->top_w;
            p.top_i = s->top_i + static_cast<int64_t>(l) * d.top_k;
            p.counter = s->route_counter;
            if (int rc = launch_route(p, true, lc)) return rc;
        }
        // K5 + K6: grouped experts, x2 = x1 + moe
        {
            MoeParams p;
            p.x = s->h2;
            p.gate_up = L.gu_codes;
            p.gu_scale = reinterpret_cast<const __half*>(L.gu_scale);
            p.down = L.dn_codes;
            p.dn_scale = reinterpret_cast<const __half*>(L.dn_scale);
            p.ids = s->top_i + static_cast<int64_t>(l) * d.top_k;
            p.top_w = s->top_w;
            p.T = 1;
            p.K = d.top_k;
            p.E = d.experts;
            p.H = d.hidden;
            p.F = d.ffn;
            p.group_size = d.group_size;
            p.act = s->act;
            p.out = s->xb;
            p.resid = s->xa;
            p.err_flag = s->err_flag;
            if (int rc = launch_moe_gate_up(p, true, lc)) return rc;
            if (int rc = launch_moe_down(p, true, lc)) return rc;
        }
        x_prev = s->xb;
        x_token = nullptr;
    }
    // lm_head
    {
        GemvParams p;
        p.x = x_prev;
        p.x_token = x_token;
        p.token_rows = d.vocab;
        p.norm_w = reinterpret_cast<const __half*>(d.final_norm);
        p.eps = d.eps;
        p.codes = d.lm_head_codes;
        p.scale = reinterpret_cast<const __half*>(d.lm_head_scale);
        p.N = d.vocab;
        p.K = d.hidden;
        p.group_size = d.group_size;
        p.y = d.logits;
        p.err_flag = s->err_flag;
        if (int rc = launch_gemv_w8(p, 1, true, false, false, lc)) return rc;
    }
    if (d.next_token != nullptr) {
        LaunchCfg plain = lc;
        plain.pdl = false;
        const bool feed = d.self_feed != 0;
        if (int rc = launch_kernel(greedy_pick_kernel, dim3(1), dim3(1024), 0, plain, reinterpret_cast<const __half*>(d.logits), d.vocab,
                                   d.next_token, feed ? const_cast<int64_t*>(d.token) : static_cast<int64_t*>(nullptr),
                                   const_cast<int64_t*>(d.cache_position), const_cast<int32_t*>(d.filled_len), d.token_log, d.max_len))
            return rc;
    }
    if (launches) *launches = count;
    return LEMOQ_OK;
}
