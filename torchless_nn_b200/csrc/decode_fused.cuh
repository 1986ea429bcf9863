// Interface between the decoder (decode.cu) and the persistent decode kernel (decode_fused.cu).
#pragma once

#include "common.cuh"
#include <vector>

enum { DF_QKV = 0, DF_OUT = 1, DF_FFN1 = 2, DF_FFN2 = 3, DF_HEAD = 4 };

// One work item of a step: `rows` output features starting at n0 of one product, over the K range [k0, k0 + d).
struct df_item {
    int kind, layer, n0, rows, k0, pad0, pad1, pad2;
};

struct df_layer {
    const float *ln1_g, *ln1_b, *bqkv, *bo, *ln2_g, *ln2_b, *b1, *b2;
    const __nv_bfloat16 *wqkv, *wo, *w1, *w2;      // prepared (out, in) weights
    __nv_bfloat16 *kcache, *vcache;                // (B, max_len, d)
};

struct df_params {
    int B, d, H, L, V, max_len, act, n_steps;
    int slot_bytes, items_pitch, n_cols, pad;
    const df_layer* layers;                        // device array of L entries
    const df_item* items;                          // device: (grid, items_pitch)
    const int* item_counts;                        // device: (grid)
    const float *tok_table, *pos_table, *lnf_g, *lnf_b, *head_bias;
    const __nv_bfloat16* head;                     // (V, d)
    float* x;                                      // (B, d) residual stream
    __nv_bfloat16 *qkv, *att, *hid;                // (B, 3d), (B, d), (B, 4d)
    float2* cand;                                  // (grid, 64) arg-max candidates (value, index bits)
    int32_t* cur;                                  // (B) current tokens: input of the first step, output of the last
    int* len;                                      // device: position of the first step; advanced by n_steps
    int32_t* tokens_out;                           // (B, n_cols) or null
    unsigned* bar_count;                           // arrival counter followed by the abort flag (8 bytes, zeroed per launch)
    int* abort_flag;
    tlnn_dev_err* err;
    unsigned long long* prof;                      // optional phase timers (14 counters), null when off
};

struct tl_decode_fused_plan_t {
    bool ok = false;
    int ns = 0, slot_bytes = 0, grid = 0, items_pitch = 0, hd = 0;
    size_t smem = 0;
    std::vector<df_item> items;
    std::vector<int> counts;
};

// Decides whether the persistent kernel serves this model and batch (bf16, at most 64 rows, width a multiple of 128 up
// to 1024, head dimension 32 / 64 / 128, scores of max_len keys per warp fit the operand buffer) and builds the item table.
int tl_decode_fused_plan(tlnn_ctx* ctx, const tlnn_gpt_model& m, int B, int max_len, tl_decode_fused_plan_t* plan);
int tl_decode_fused_launch(tlnn_ctx* ctx, const tl_decode_fused_plan_t& plan, const df_params& params);
