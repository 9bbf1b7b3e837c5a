/*
 * lemoq_b200 - C ABI of the B200 (sm_100a) kernels for the LeanMoE-Quant batch-1
 * decode step.
 *
 * Conventions shared by every entry point
 *   - plain C: device pointers, sizes and a CUDA stream handle (`cudaStream_t`
 *     passed as `void*`; NULL = the legacy default stream);
 *   - no allocation, no synchronisation, no host<->device copies: work is only
 *     enqueued on `stream`, so every call is legal under stream capture;
 *   - tensors are contiguous unless a stride argument says otherwise; weight,
 *     cache and activation base pointers must be 16-byte aligned;
 *   - return value: LEMOQ_OK, or an error code with a message available from
 *     lemoq_last_error() (thread-local).  LEMOQ_ERR_INVALID maps to the
 *     reference's ValueError, LEMOQ_ERR_UNSUPPORTED to NotImplementedError and
 *     LEMOQ_ERR_CUDA to RuntimeError;
 *   - "ref:" lines name the reference interface (file:line inside the
 *     LeanMoE-Quant tree) that the entry point replaces.
 *
 * Data types: activations, norm weights, router weights, scales and caches are
 * IEEE fp16; weight and KV codes are int8; expert ids are int64; positions are
 * int64 (`cache_position`) and the filled length is int32, both read from
 * device memory so one captured launch serves every step.
 */
#ifndef LEMOQ_B200_H
#define LEMOQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LEMOQ_API __attribute__((visibility("default")))
#else
#define LEMOQ_API
#endif

#define LEMOQ_OK 0
#define LEMOQ_ERR_INVALID 1
#define LEMOQ_ERR_UNSUPPORTED 2
#define LEMOQ_ERR_CUDA 3

#define LEMOQ_DTYPE_F16 0
#define LEMOQ_DTYPE_F32 1

/* Library / build identification and the last error message of this thread. */
LEMOQ_API const char* lemoq_version(void);
LEMOQ_API const char* lemoq_last_error(void);

/* Kernel tuning knobs for benchmarking (process-wide, not thread-safe; defaults are the measured
 * best).  Returns LEMOQ_ERR_INVALID for an unknown key or a value out of range.
 *   key 0  int8 dot-product variant of the streaming GEMV kernels: 0 fp32 magic number, 1 exact fp16
 *          codes widened to fp32, 2 exact fp16 codes with mixed-precision FMA, 3 (default) fp16 codes
 *          with the offset folded into one correction per 16 codes
 *   key 1  warps per block of the streaming kernels (1..16)
 *   key 4  step engine: 1 (default) the whole-step cooperative kernel when the shapes allow it,
 *          0 chained per-op kernels; takes effect at the next lemoq_step_create
 *   key 5  whole-step kernel, current device: polls of a flagged word before a wait gives up with
 *          LEMOQ_FLAG_WAIT_TIMEOUT (1 .. 2^24, default 2^21).  A step whose wait ran out has gone on with
 *          stale values: its results are void, the flag says so, the next step is unaffected.  Exists so
 *          that the time-out path can be exercised (value 1) without anything hanging.
 * Keys 0, 1 and 4 give the same results up to fp32 summation order.
 * No counterpart in the reference, whose tile configs are module dicts
 * (ref: src/lemoq/kernels/moe_grouped.py:78, src/lemoq/kernels/_dequant_triton.py:83).
 */
LEMOQ_API int lemoq_set_tuning(int key, int value);

/* ---------------------------------------------------------------------------
 * Weight quantisation: per-row, per-group symmetric RTN to int8.
 * ref: src/lemoq/quant/rtn.py:38 (quantize_rtn, symmetric 8-bit branch),
 *      src/lemoq/kernels/moe_grouped_quant.py:191 (quantize_fused_experts),
 *      src/lemoq/quant/linear.py:253 (QuantLinear.__init__: fp16 scale buffer).
 * w: (rows, in_features) fp16 or fp32 (w_dtype); in_features % group_size == 0.
 * codes: (rows, in_features) int8; scale: (rows, in_features/group_size) fp16.
 */
LEMOQ_API int lemoq_rtn_quantize_w8(const void* w, int w_dtype, int64_t rows, int in_features, int group_size,
                          int8_t* codes, void* scale, void* stream);

/* ---------------------------------------------------------------------------
 * Dense W8 dequant GEMV: y[m, n] = sum_k x[m, k] * codes[n, k] * scale[n, k/g].
 * ref: src/lemoq/kernels/_dequant_triton.py:155 (dequant_gemm_fused, symmetric
 *      8-bit), called from src/lemoq/quant/linear.py:446 (QuantLinear fused arm)
 *      and src/lemoq/kernels/packed_qkv.py:78 (PackedQKV.project).
 * x: (M, K) fp16; codes: (N, K) int8; scale: (N, K/g) fp16; y: (M, N) fp16 or
 * fp32 (out_dtype).  K % group_size == 0, group_size % 16 == 0, K <= 8192.
 */
LEMOQ_API int lemoq_dequant_gemv_w8(const void* x, int M, const int8_t* codes, const void* scale, int N, int K,
                          int group_size, void* y, int out_dtype, void* stream);

/* ---------------------------------------------------------------------------
 * W8 rows against many tokens (batched decode, prefill: tens of tokens per
 * call): every weight byte is read once per block of 16 tokens.  Two calls: the
 * activations are first turned into integer digit planes
 * (lemoq_w8_quantise_tokens; planes of lemoq_w8_token_planes_bytes(T, K) bytes,
 * caller-provided, layout private to the library), then lemoq_w8_rows_tokens
 * computes y[t, n] = fp16(sum_k x[t, k] * codes[e, n, k] * scale[e, n, k/g]) with
 * exact integer partial sums per group of 128 on the int8 tensor-core tile.
 * ref: the batched (T > 1) arms of the reference dequantise the weights and call
 *      a dense matmul: src/lemoq/quant/linear.py:365 (QuantLinear separate arm) and
 *      src/lemoq/kernels/moe_static.py:329 (_prefill_forward); same arithmetic,
 *      fp32 accumulation, fp16 result.
 * codes: (E, N, K) int8, scale: (E, N, K/g) fp16.  seg_offsets: (E + 1) int32 device
 * array, tokens [seg[e], seg[e+1]) use expert e (tokens sorted by expert); NULL
 * with E == 1 means all T tokens.  gate_up != 0: N = 2F rows are gate [0, F) and up
 * [F, 2F); y is (T, F) = silu(gate) * up.  Otherwise y is (T, N).
 * K % 128 == 0, K <= 4096, N even, group_size % 128 == 0.
 */
LEMOQ_API size_t lemoq_w8_token_planes_bytes(int T, int K);
LEMOQ_API int lemoq_w8_quantise_tokens(const void* x, int T, int K, void* planes, void* stream);
LEMOQ_API int lemoq_w8_rows_tokens(const void* planes, int T, const int8_t* codes, const void* scale, int N, int K,
                         int group_size, const int32_t* seg_offsets, int E, int gate_up, void* y, void* stream);

/* ---------------------------------------------------------------------------
 * Row bookkeeping of the expert-parallel exchange (batched decode over several
 * GPUs, benchmark configuration 5).  These have no counterpart in the reference
 * (it has no multi-GPU code).  The contract: expert e lives on rank e / (experts / world),
 * rows travel sorted by (expert id, pair index), every peer gets a fixed block of
 * P = T * K row slots, a row is H fp16 activations + 8 fp16 of which the first is
 * the expert id, unused slots carry the id `experts`.  All arrays are device
 * memory; nothing is read on the host (legal under stream capture).
 *   lemoq_ep_dispatch: h (T, H) fp16, top_i (T, K) int64 -> send (world, P, H + 8) fp16,
 *       slot (P) int32 = send slot of pair (t, k), src (world * P) int32 scratch.
 *   lemoq_ep_regroup:  recv (R = world * P, H + 8) fp16 as received -> x_sorted (R, H)
 *       fp16 rows in local-expert order (zeros behind the real rows), perm (R) int32,
 *       seg (experts / world + 1) int32 segment offsets for lemoq_w8_rows_tokens.
 *   lemoq_ep_return:   y_sorted (R, H) -> y (R, H) in slot order (rows of unused slots untouched).
 *   lemoq_ep_combine:  back (world * P, H) fp16, slot, top_w (T, K) fp16 -> out (T, H) fp16,
 *       out[t] = sum_k top_w[t, k] * back[slot[t * K + k]] in slot order, fp32.
 * T * K <= 4096, R <= 4096, experts <= 2048, H % 8 == 0.  err_flag (may be NULL):
 * LEMOQ_FLAG_BAD_EXPERT for an id outside its range (clamped / treated as padding).
 */
LEMOQ_API int lemoq_ep_dispatch(const void* h, const int64_t* top_i, int T, int K, int H, int experts, int world, void* send,
                      int32_t* slot, int32_t* src, int* err_flag, void* stream);
LEMOQ_API int lemoq_ep_regroup(const void* recv, int R, int H, int experts, int world, int rank, void* x_sorted, int32_t* perm,
                     int32_t* seg, int* err_flag, void* stream);
LEMOQ_API int lemoq_ep_return(const void* y_sorted, const int32_t* perm, const int32_t* seg, int R, int H, int epr, void* y, void* stream);
LEMOQ_API int lemoq_ep_combine(const void* back, const int32_t* slot, const void* top_w, int T, int K, int H, void* out, void* stream);

/* ---------------------------------------------------------------------------
 * RMSNorm, HF-OLMoE rounding: y = fp16(x * rsqrt(mean(x^2) + eps)) * w (fp16 mul).
 * ref: src/lemoq/kernels/rmsnorm.py:102 (rms_norm_fused).
 * x, y: (rows, H) fp16; w: (H,) fp16.  H % 8 == 0, H <= 8192.
 */
LEMOQ_API int lemoq_rms_norm(const void* x, const void* w, void* y, int64_t rows, int H, float eps, void* stream);

/* ---------------------------------------------------------------------------
 * Half-split RoPE on the decode q and k rows: out = x*cos + rotate_half(x)*sin in
 * fp32, one rounding to fp16.
 * ref: src/lemoq/kernels/rope.py:160 (apply_rotary_pos_emb_fused).
 * q: heads_q rows of D fp16, row h at q + h*q_head_stride (elements); likewise k.
 * cos, sin: (D,) fp16.  q_out/k_out: contiguous (heads, D).
 */
LEMOQ_API int lemoq_rope_qk(const void* q, int64_t q_head_stride, int heads_q, const void* k, int64_t k_head_stride,
                  int heads_k, const void* cos, const void* sin, int D, void* q_out, void* k_out, void* stream);

/* ---------------------------------------------------------------------------
 * KV direct write: bit copy of the new (1,H,1,D) K and V rows into the static
 * fp16 cache (1,H,max_len,D) at slot *pos; no other slot is touched.
 * ref: src/lemoq/kernels/kv_direct.py:110 (kv_direct_write),
 *      contract src/lemoq/kernels/kv_write.py:28 (write_kv_slot).
 * pos: device int64 scalar.  A position outside [0, max_len) writes nothing and
 * sets *err_flag (device int32, may be NULL) to 1.
 */
LEMOQ_API int lemoq_kv_direct_write(const void* k_row, const void* v_row, int64_t src_head_stride, void* k_cache,
                          void* v_cache, const int64_t* pos, int heads, int max_len, int D, int* err_flag,
                          void* stream);

/* ---------------------------------------------------------------------------
 * Per-token symmetric int8 KV quantisation of the new K and V rows into the
 * int8 mirror cache at slot *pos: amax/127 in fp32 (1.0 for a zero row), true
 * division, round half to even, clamp to +-127, scale stored as fp16.
 * ref: src/lemoq/kernels/kv_int8.py:219 (kv_int8_cache_write); with pos == NULL
 *      and S == 1 it is src/lemoq/kernels/kv_int8.py:314 (kv_int8_write).
 * k_row, v_row: (H, D) fp16 contiguous; kc, vc: (H, S, D) int8; ks, vs: (H, S) fp16.
 */
LEMOQ_API int lemoq_kv_int8_cache_write(const void* k_row, const void* v_row, int8_t* kc, void* ks, int8_t* vc, void* vs,
                              const int64_t* pos, int heads, int S, int D, int* err_flag, void* stream);

/* Bulk quantisation of a whole fp16 cache into the mirror; slots at or beyond
 * `filled` get code 0 / scale 1 (filled < 0 quantises every slot; filled == 0
 * writes code 0 / scale 1 everywhere).  The reference's Python function treats a
 * zero length like "no length" (kv_int8.py:147); the host mirror passes -1 for it.
 * ref: src/lemoq/kernels/kv_int8.py:127 (kv_int8_bulk_quantize).
 */
LEMOQ_API int lemoq_kv_int8_bulk_quantize(const void* keys, const void* values, int8_t* kc, void* ks, int8_t* vc, void* vs,
                                int heads, int S, int D, int filled, void* stream);

/* ---------------------------------------------------------------------------
 * Split-KV decode attention over positions [0, *filled): per-split online softmax
 * (base 2), partials (m, l, acc[D]) in fp32, deterministic fixed-order merge done
 * by the last block of each head; *filled == 0 gives zeros.
 * ref: src/lemoq/kernels/attn_decode.py:496 (attn_decode_forward, fp16 K/V) and
 *      src/lemoq/kernels/attn_decode.py:627 (attn_decode_forward_int8: int8 codes
 *      with per-token fp16 scales folded into the scores / weights).
 * q: (H, D) fp16; k, v: head h at base + h*kv_head_stride elements, (S, D) each;
 * ks, vs: (H, S) fp16; out: (H, D) fp16; filled: device int32 scalar, clamped to
 * [0, S] (a value outside sets *err_flag).  D in {64, 128}.  num_splits >= 1.
 * workspace: lemoq_attn_workspace_bytes() bytes, zero-initialised once by the
 * caller before first use (it holds arrival counters that every launch leaves at
 * zero); launches sharing a workspace must not overlap on the GPU.
 */
LEMOQ_API size_t lemoq_attn_workspace_bytes(int heads, int D, int num_splits);
LEMOQ_API int lemoq_attn_decode_fp16(const void* q, const void* k, const void* v, int64_t kv_head_stride,
                           const int32_t* filled, void* out, int heads, int S, int D, int num_splits, float scale,
                           void* workspace, int* err_flag, void* stream);
LEMOQ_API int lemoq_attn_decode_int8(const void* q, const int8_t* kc, const void* ks, const int8_t* vc, const void* vs,
                           int64_t kv_head_stride, const int32_t* filled, void* out, int heads, int S, int D,
                           int num_splits, float scale, void* workspace, int* err_flag, void* stream);

/* ---------------------------------------------------------------------------
 * lemoq_attn_decode_int8 for callers that cannot allocate: no workspace argument.
 * This entry point has no counterpart in the reference; results equal those of
 * lemoq_attn_decode_int8 on the same inputs.
 * The split partials and arrival counters live in a fixed array inside the library
 * (lemoq_attn_static_scratch_bytes() = 1 MiB per device).  The call allocates and
 * frees nothing, and neither does anything it calls.  The first 16 KiB of the array
 * are the arrival counters (at most 4096 heads), the partials follow: sizes with
 * 16384 + 4*heads*num_splits*(D+2) bytes above the array's size are refused with
 * LEMOQ_ERR_INVALID and a message in lemoq_last_error().  Each call clears its
 * counters on the stream ahead of its kernel; the partials keep the last call's
 * contents and are written before they are read.
 * The first call on a device looks the array's address up (once per device, with
 * that device current); make that first call outside any stream capture.
 * All calls on a device share the array: calls whose kernels may overlap on the
 * device (different streams or threads) race on it - keep them on one stream.
 */
LEMOQ_API size_t lemoq_attn_static_scratch_bytes(void);
LEMOQ_API int lemoq_attn_decode_int8_static(const void* q, const int8_t* kc, const void* ks, const int8_t* vc,
                                  const void* vs, int64_t kv_head_stride, const int32_t* filled, void* out, int heads,
                                  int S, int D, int num_splits, float scale, int* err_flag, void* stream);

/* ---------------------------------------------------------------------------
 * Router softmax + top-k: fp32 softmax over E logits, top_k rounds of arg-max
 * (lowest index wins ties), optional renormalisation.
 * ref: src/lemoq/kernels/_routing_triton.py:88 (routing_softmax_topk).
 * logits: (T, E) fp16 or fp32, row stride in elements; top_w: (T, K) fp32;
 * top_i: (T, K) int64.  E <= 1024.
 */
LEMOQ_API int lemoq_routing_softmax_topk(const void* logits, int logits_dtype, int64_t row_stride, int T, int E, int top_k,
                               int norm_topk_prob, float* top_w, int64_t* top_i, void* stream);

/* Router linear + softmax/top-k for one token: logits = fp16(h . Wr^T) with fp32
 * accumulation, then as above; top_w is rounded to fp16.
 * ref: src/lemoq/kernels/moe_static.py:262 (_route).
 * h: (H,) fp16; router_w: (E, H) fp16; logits_out: (E,) fp16; top_w: (K,) fp16;
 * top_i: (K,) int64.  E <= 64*32, H % 8 == 0.  workspace: 16 bytes, zeroed once.
 */
LEMOQ_API int lemoq_route(const void* h, const void* router_w, int E, int H, int top_k, int norm_topk_prob,
                void* logits_out, void* top_w, int64_t* top_i, void* workspace, void* stream);

/* ---------------------------------------------------------------------------
 * Grouped expert GEMV, W8 weights dequantised in registers:
 *   act[t,i,n] = silu(Wg[e,n,:].x_t) * (Wu[e,n,:].x_t), rounded to fp16;
 *   out[t,n]   = fp16( sum_i top_w[t,i] * (Wd[e,n,:].act[t,i,:]) ),  e = ids[t,i].
 * ref: src/lemoq/kernels/moe_grouped_quant.py:411 (grouped_moe_forward_quant) and
 *      its kernels src/lemoq/kernels/_grouped_triton.py:249,335,197.
 * x: (T, H) fp16; gu_codes: (E, 2F, H) int8 (gate rows [0,F), up rows [F,2F));
 * gu_scale: (E, 2F, H/g) fp16; dn_codes: (E, H, F) int8; dn_scale: (E, H, F/g) fp16;
 * ids: (T, K) int64; top_w: (T, K) fp16; act: (T, K, F) fp16 workspace (also an
 * output); out: (T, H) fp16.  H, F multiples of 128 and <= 2048 / 8192; K <= 16.
 * An expert id outside [0, E) is clamped and sets *err_flag.
 */
LEMOQ_API int lemoq_moe_grouped_w8(const void* x, const int8_t* gu_codes, const void* gu_scale, const int8_t* dn_codes,
                         const void* dn_scale, const int64_t* ids, const void* top_w, int T, int K, int E, int H,
                         int F, int group_size, void* act, void* out, int* err_flag, void* stream);

/* The two launches of lemoq_moe_grouped_w8 on their own (same arguments; gate_up reads x and
 * writes act, down reads act and writes out).
 * ref: src/lemoq/kernels/_grouped_triton.py:249 (_gate_up_act_kernel_q) and
 *      src/lemoq/kernels/_grouped_triton.py:335 (_down_sum_kernel_q).
 */
LEMOQ_API int lemoq_moe_gate_up_w8(const void* x, const int8_t* gu_codes, const void* gu_scale, const int64_t* ids, int T,
                         int K, int E, int H, int F, int group_size, void* act, int* err_flag, void* stream);
LEMOQ_API int lemoq_moe_down_w8(const void* act, const int8_t* dn_codes, const void* dn_scale, const int64_t* ids,
                      const void* top_w, int T, int K, int E, int H, int F, int group_size, void* out, int* err_flag,
                      void* stream);

/* Same contract on unquantised fp16 expert weights.
 * ref: src/lemoq/kernels/moe_grouped.py:315 (grouped_moe_forward) and
 *      src/lemoq/kernels/_grouped_triton.py:55,139.
 */
LEMOQ_API int lemoq_moe_grouped_fp16(const void* x, const void* gate_up, const void* down, const int64_t* ids,
                           const void* top_w, int T, int K, int E, int H, int F, void* act, void* out,
                           int* err_flag, void* stream);

/* ---------------------------------------------------------------------------
 * Whole decode step (one token, all layers, lm_head) as a fixed chain of fused
 * kernels; the host captures one lemoq_step_run() call into a CUDA graph.
 * ref: the forward captured by benchmarks/cudagraph.py:713 (StaticCacheDecodeSession
 *      .capture) with every FUSION_DEFAULTS switch on
 *      (src/lemoq/kernels/fusion_switches.py:50), i.e. per layer
 *      src/lemoq/kernels/attn_decode.py:836 (_decode_forward_impl) followed by
 *      src/lemoq/kernels/moe_grouped_quant.py:562 (static_moe_forward_grouped_quant).
 */
typedef struct lemoq_layer_desc {
    const void* ln1;        /* (hidden) fp16 input_layernorm weight            */
    const void* ln2;        /* (hidden) fp16 post_attention_layernorm weight   */
    const void* q_norm;     /* (heads*head_dim) fp16                           */
    const void* k_norm;     /* (heads*head_dim) fp16                           */
    const int8_t* qkv_codes;/* (3*heads*head_dim, hidden) int8, rows [q;k;v]   */
    const void* qkv_scale;  /* (3*heads*head_dim, hidden/g) fp16               */
    const int8_t* o_codes;  /* (hidden, heads*head_dim) int8                   */
    const void* o_scale;    /* (hidden, heads*head_dim/g) fp16                 */
    const void* router;     /* (experts, hidden) fp16                          */
    const int8_t* gu_codes; /* (experts, 2*ffn, hidden) int8                   */
    const void* gu_scale;   /* (experts, 2*ffn, hidden/g) fp16                 */
    const int8_t* dn_codes; /* (experts, hidden, ffn) int8                     */
    const void* dn_scale;   /* (experts, hidden, ffn/g) fp16                   */
    void* keys;             /* (heads, max_len, head_dim) fp16 static cache    */
    void* values;           /* (heads, max_len, head_dim) fp16 static cache    */
    int8_t* kc;             /* (heads, max_len, head_dim) int8 mirror (kv_int8)*/
    void* ks;               /* (heads, max_len) fp16                           */
    int8_t* vc;
    void* vs;
} lemoq_layer_desc;

typedef struct lemoq_step_desc {
    int layers, hidden, heads, head_dim, experts, top_k, ffn, vocab, group_size, max_len;
    float eps;
    int norm_topk_prob;
    int kv_int8;            /* 1: attention reads the int8 mirror; 0: the fp16 cache       */
    int attn_splits;        /* 0 = choose from the SM count and max_len; > 0: this many (whole-step kernel: at most) */
    int use_pdl;            /* 1: programmatic dependent launch between the step's kernels  */
    const void* embed;      /* (vocab, hidden) fp16                                         */
    const void* final_norm; /* (hidden) fp16                                                */
    const int8_t* lm_head_codes; /* (vocab, hidden) int8                                    */
    const void* lm_head_scale;   /* (vocab, hidden/g) fp16                                  */
    const void* rope_cos;   /* (max_len, head_dim) fp16                                     */
    const void* rope_sin;
    const int64_t* token;          /* device scalar: id of the token being decoded          */
    const int64_t* cache_position; /* device scalar: its cache slot                         */
    const int32_t* filled_len;     /* device scalar: cache_position + 1                     */
    void* logits;           /* (vocab) fp16 output                                          */
    void* workspace;        /* lemoq_step_workspace_bytes() bytes, 32-byte aligned, zeroed once by the caller */
    size_t workspace_bytes;
    int64_t* next_token;    /* optional device scalar: the step also writes argmax(logits) here (the
                               first maximal index, as the reference's greedy loop picks it:
                               ref benchmarks/cudagraph.py:756-762); NULL = not wanted          */
    int self_feed;          /* 1 (needs next_token): at its very end the step also stores the picked token
                               into *token and adds 1 to *cache_position and *filled_len, so that K
                               launches in a row decode K tokens greedily with no host work in between
                               (the reference's loop syncs and reads the token back per step:
                               ref benchmarks/cudagraph.py:756-762).  A host that sets the three
                               scalars before every launch, as the reference does, is not affected. */
    int64_t* token_log;     /* optional device array of max_len entries (needs next_token): the step also
                               stores its pick at token_log[*cache_position], so a host that launched K
                               steps in a row reads the K tokens back with one copy; NULL = not wanted */
} lemoq_step_desc;

typedef struct lemoq_step lemoq_step; /* host-side plan, owns no device memory */

LEMOQ_API size_t lemoq_step_workspace_bytes(const lemoq_step_desc* desc);
LEMOQ_API int lemoq_step_create(const lemoq_step_desc* desc, const lemoq_layer_desc* layers, lemoq_step** out);
LEMOQ_API void lemoq_step_destroy(lemoq_step* step);
/* Enqueue one decode step.  Returns the number of kernels launched through
 * *launches when it is not NULL. */
LEMOQ_API int lemoq_step_run(lemoq_step* step, void* stream, int* launches);
/* Device int32 inside the workspace: 0, or a bit mask of LEMOQ_FLAG_* set by a
 * kernel that had to clamp a position, a length or an expert id. */
LEMOQ_API int* lemoq_step_error_flag(lemoq_step* step);
/* Device pointers to per-layer routing results of the last step (for parity
 * checks): top_i (layers, top_k) int64 and router logits (layers, experts) fp16. */
LEMOQ_API const int64_t* lemoq_step_topk_ids(lemoq_step* step);
LEMOQ_API const void* lemoq_step_router_logits(lemoq_step* step);
/* Name of the form the plan runs as: "whole-step" (one cooperative kernel per step on 8-row weight tiles and the
 * int8 tensor-core dot product) or "chained" (6 kernels per layer).  Static string.  No counterpart in the
 * reference (ref for the step itself: benchmarks/cudagraph.py:713). */
LEMOQ_API const char* lemoq_step_engine(lemoq_step* step);
/* Device pointer to 6*layers + 2 global-timer stamps (ns) of the last step, taken by block 0 of the whole-step
 * kernel: at its start, where it begins each phase of each layer (the phases of different blocks overlap, so
 * these are one block's view), and at its end; NULL when the step runs as chained kernels. */
LEMOQ_API const unsigned long long* lemoq_step_phase_stamps(lemoq_step* step);

#define LEMOQ_FLAG_BAD_POSITION 1
#define LEMOQ_FLAG_BAD_LENGTH 2
#define LEMOQ_FLAG_BAD_EXPERT 4
#define LEMOQ_FLAG_WAIT_TIMEOUT 8 /* a bounded wait on an async copy gave up */
#define LEMOQ_FLAG_BAD_TOKEN 16   /* *token outside [0, vocab): clamped */

#ifdef __cplusplus
}
#endif
#endif /* LEMOQ_B200_H */
