// Parameter block of the whole-step cooperative kernel (step_tile.cu), shared with the step engine.
#pragma once

#include "kernels.h"

namespace lemoq {

struct StepLayer {
    const __half *ln1, *ln2, *q_norm, *k_norm;
    const int8_t* qkv_codes;
    const __half* qkv_scale;
    const int8_t* o_codes;
    const __half* o_scale;
    const __half* router;
    const int8_t* gu_codes;
    const __half* gu_scale;
    const int8_t* dn_codes;
    const __half* dn_scale;
    __half *keys, *values;
    int8_t* kc;
    __half* ks;
    int8_t* vc;
    __half* vs;
};

struct StepParams {
    int layers, H, heads, D, E, K, F, V, group, S, splits, kv_int8, norm_topk;
    float eps, qk_scale_log2;
    const __half *embed, *final_norm, *lm_scale, *rope_cos, *rope_sin;
    const int8_t* lm_codes;
    const int64_t *token, *cache_position;
    const int32_t* filled;
    __half* logits;
    int64_t* next_token;  // optional: argmax(logits)
    int64_t* token_log;   // optional: token_log[position] = the pick
    int self_feed;        // the step ends by making its pick the next step's input (token, position + 1, length + 1)
    const StepLayer* L;   // device array: the layers, then a pseudo layer whose q.k.v rows are the lm_head
    int* err_flag;
    unsigned int *bar_counter, *bar_epoch;
    __half *router_logits, *top_w;
    // flagged-word buffers (8-byte words {data, tag}), two parities each: layer outputs [2][2048] then post-attention
    // streams [2][2048]; q.k.v rows [2][3*2048]; q/k sums of squares per block [2][2][1024]; router logits [2][128];
    // expert activations, two per word [2][4096]
    unsigned long long *fl_x, *fl_qkv, *fl_stats, *fl_logits, *fl_act;
    int64_t* top_i;
    float* attn_part;            // (m, l, acc[D]) partial of every (head, split) unit; at the end the per-block greedy candidates
    int barriers_per_launch;
    unsigned long long* stamps;  // optional: 6*layers + 2 phase time stamps of the last step
};

size_t tile_smem_bytes();
int set_flag_spin_limit(int polls);  // lemoq_set_tuning key 5 (current device)
bool tile_eligible(const lemoq_step_desc& d);
int tile_grid(const lemoq_step_desc& d);  // blocks to launch (one per SM), 0 = unavailable
int tile_attention_splits(const lemoq_step_desc& d, int grid);
int launch_step_tile(const StepParams& p, int grid, cudaStream_t stream);

}  // namespace lemoq
