// Interface between the decoder (decode.cu) and the persistent decode kernel (decode_fused.cu).
#pragma once

#include "common.cuh"
#include <vector>

enum { DF_QKV = 0, DF_OUT = 1, DF_FFN1 = 2, DF_FFN2 = 3, DF_HEAD = 4 };

// One work item of a step: `rows` output features starting at n0 of one product, over the K range [k0, k0 + d).
// The table is built on the host with every pointer resolved, so that the kernel never chases a pointer in global
// memory on its critical path.
struct df_item {
    int kind, layer, n0, rows, k0, ldw;            // ldw: row pitch of the weight in elements
    int pad0, pad1;
    const __nv_bfloat16* w;                        // first weight row of the item (at column k0)
    const float* bias;                             // bias of the product (whole vector, indexed by feature) or null
    const float* gamma;                            // LayerNorm in front of the product (QKV, first feed-forward, head) or null
    const float* beta;
};
static_assert(sizeof(df_item) == 64, "the kernel copies items as 64-byte records");

struct df_params {
    int B, d, H, L, V, max_len, act, n_steps;
    int slot_bytes, items_pitch, n_cols, a_region; // a_region: bytes at the start of shared memory for operand rows / attention ring
    int att_ck, ns, hd, pad2;                      // keys per chunk of the attention ring; features per item; head dimension
    const df_item* items;                          // device: (grid, items_pitch)
    const int* item_counts;                        // device: (grid)
    const float *tok_table, *pos_table;
    __nv_bfloat16 *kcache, *vcache;                // (L, B, max_len, d)
    float* x;                                      // (B, d) residual stream
    __nv_bfloat16 *qkv, *att, *hid;                // (B, 3d), (B, d), (B, 4d)
    float2* cand;                                  // (grid, 64) arg-max candidates (value, index bits)
    int32_t* cur;                                  // (B) current tokens: input of the first step, output of the last
    int* len;                                      // device: position of the first step; advanced by n_steps
    int32_t* tokens_out;                           // (B, n_cols) or null
    unsigned* bar_flags;                           // grid barrier: arrival counter (first word of a 4 KB block zeroed per launch)
    int* abort_flag;                               // last word of that block
    tlnn_dev_err* err;
    unsigned long long* prof;                      // optional phase timers, null when off
};

// One strided copy that brings a weight matrix (or one K range of it) into the decoder's packed copy.
struct df_pack_job {
    const void* src;
    size_t src_pitch, dst_off, width, rows;
};

struct tl_decode_fused_plan_t {
    bool ok = false;
    size_t pack_bytes = 0;                         // size of the packed weight copy (see tl_decode_fused_plan)
    std::vector<df_pack_job> pack_jobs;
    int ns = 0, slot_bytes = 0, grid = 0, items_pitch = 0, hd = 0, att_ck = 0, a_region = 0;
    size_t smem = 0;
    std::vector<df_item> items;
    std::vector<int> counts;
};

// Decides whether the persistent kernel serves this model and batch (bf16, at most 64 rows, width a multiple of 128 up
// to 1024, head dimension 32 / 64 / 128) and builds the item table from the model description (pointers into the
// caller's prepared weights).
// The kernel streams weights from a packed copy owned by the decoder: every matrix (every K range of the second
// feed-forward matrix) stored with rows of d + 8 elements, the pitch the rows have in shared memory, so that the rows
// of an item are one contiguous block and arrive with a single bulk copy.  Call once with pack_base == nullptr to learn
// pack_bytes, allocate, call again with the allocation, then run the pack_jobs (cudaMemcpy2DAsync each).  With
// pack_base == nullptr on the second call too (allocation failed) the items point at the caller's weights and their
// rows are copied one by one.
int tl_decode_fused_plan(tlnn_ctx* ctx, const tlnn_gpt_model& m, const tlnn_block_params* blocks, int B, int max_len,
                         char* pack_base, bool use_pack, tl_decode_fused_plan_t* plan);
int tl_decode_fused_launch(tlnn_ctx* ctx, const tl_decode_fused_plan_t& plan, const df_params& params);
