// Composite layer calls: each one enqueues the kernel sequence of one reference layer's forward on the context's
// stream, using the context's scratch arena for intermediates.  In bf16 mode every GEMM operand is bf16 and the
// residual stream stays float32; in TF32 mode operands are float32 rounded to nearest TF32 by their producer.
#include "common.cuh"

namespace {

inline int op_kind(int prec) { return prec == TLNN_PREC_BF16 ? TL_OUT_BF16 : TL_OUT_TF32; }
inline size_t op_size(int prec) { return prec == TLNN_PREC_BF16 ? 2 : 4; }
inline bool prec_ok(int prec) { return prec == TLNN_PREC_BF16 || prec == TLNN_PREC_TF32; }

// Token rows have a pitch of ldt >= p0 * p1 * C elements; the columns past the patch features are written as zeros
// (the GEMM operand rows must be a multiple of 16 bytes).
__global__ void patchify_kernel(const float* __restrict__ img, void* __restrict__ tokens, int out_kind, int B, int C,
                                int H, int W, int p0, int p1, int ldt) {
    const int nph = H / p0, npw = W / p1;
    const int tdim = p0 * p1 * C;
    const long long total = (long long)B * nph * npw * ldt;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int f = (int)(i % ldt);
        long long tok = i / ldt;
        int c = f % C, j = (f / C) % p1, ii = f / (C * p1);
        int pc = (int)(tok % npw), pr = (int)((tok / npw) % nph);
        long long b = tok / ((long long)npw * nph);
        float v = f < tdim ? img[((b * C + c) * H + (pr * p0 + ii)) * W + (pc * p1 + j)] : 0.f;
        if (out_kind == TL_OUT_BF16) {
            reinterpret_cast<__nv_bfloat16*>(tokens)[i] = __float2bfloat16_rn(v);
        } else {
            uint32_t u = __float_as_uint(v);
            if ((u & 0x7f800000u) != 0x7f800000u) { u += 0x00000fffu + ((u >> 13) & 1u); u &= 0xffffe000u; }
            reinterpret_cast<float*>(tokens)[i] = __uint_as_float(u);
        }
    }
}

// dst (rows, ldd) <- src (rows, cols) with zero columns appended; elements of `esz` bytes (2 or 4)
__global__ void pad_rows_kernel(const void* __restrict__ src, void* __restrict__ dst, int rows, int cols, int ldd, int esz) {
    const long long total = (long long)rows * ldd;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = (int)(i % ldd);
        const long long r = i / ldd;
        if (esz == 2) {
            reinterpret_cast<uint16_t*>(dst)[i] = c < cols ? reinterpret_cast<const uint16_t*>(src)[r * cols + c] : (uint16_t)0;
        } else {
            reinterpret_cast<uint32_t*>(dst)[i] = c < cols ? reinterpret_cast<const uint32_t*>(src)[r * cols + c] : 0u;
        }
    }
}

// out[b, r, :] = cls[r, :] + pos[r, :] for the class / register rows in front of the patch tokens
__global__ void cls_rows_kernel(const float* __restrict__ cls, const float* __restrict__ pos, float* __restrict__ out,
                                int B, int T, int d, int n_cls) {
    const long long total = (long long)B * n_cls * d;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int c = (int)(i % d);
        int r = (int)((i / d) % n_cls);
        long long b = i / ((long long)d * n_cls);
        out[(b * T + r) * d + c] = cls[r * d + c] + pos[r * d + c];
    }
}

size_t block_ws_bytes(int prec, long long M, int d) {
    const size_t es = op_size(prec);
    return tl_ws_round((size_t)M * d * es)            // normalised rows (GEMM operand)
         + tl_ws_round((size_t)M * 3 * d * es)        // packed q, k, v
         + tl_ws_round((size_t)M * d * es)            // merged attention output
         + tl_ws_round((size_t)M * d * 4)             // residual stream after attention
         + tl_ws_round((size_t)M * 4 * d * es);       // feed-forward hidden
}

// One pre-LN block on rows already resident in float32.  `cur` is advanced past the pieces taken.
int run_block(tlnn_ctx* ctx, int prec, const float* x, const tlnn_block_params* p, int act, float* out, int B, int T,
              int d, int heads, int causal, tl_ws_cursor cur, void* kcache = nullptr, void* vcache = nullptr,
              int cache_len = 0) {
    const long long M = (long long)B * T;
    const int kind = op_kind(prec);
    const int accurate = prec == TLNN_PREC_TF32;
    void* a = cur.take<char>((size_t)M * d * op_size(prec));
    void* qkv = cur.take<char>((size_t)M * 3 * d * op_size(prec));
    void* att = cur.take<char>((size_t)M * d * op_size(prec));
    // out == x: the caller owns x and wants the block applied in place.  Both residual additions then accumulate into
    // x itself (the GEMM adds its tile to the buffer through the memory system), and no second stream buffer is needed.
    const bool in_place = out == x;
    float* y = in_place ? out : cur.take<float>((size_t)M * d);
    void* hid = cur.take<char>((size_t)M * 4 * d * op_size(prec));

    TL_TRY(tl_layernorm(ctx, x, p->ln1_gamma, p->ln1_beta, 1e-5f, a, kind, M, d));
    tl_gemm_epilogue e1;
    e1.bias = p->bqkv; e1.out = qkv; e1.ldo = 3 * d;
    // the exact float32 attention kernels read unrounded q, k, v; the tensor-core one wants them rounded to TF32
    e1.out_kind = prec == TLNN_PREC_BF16 ? TL_OUT_BF16 : (tl_attention_tf32_applies(T, d / heads) ? TL_OUT_TF32 : TL_OUT_F32);
    TL_TRY(tl_gemm(ctx, prec, a, d, p->wqkv_t, d, (int)M, 3 * d, d, e1));
    if (kcache) TL_TRY(tl_kv_store(ctx, prec, qkv, kcache, vcache, B, T, d, heads, cache_len));
    TL_TRY(tl_attention_core(ctx, prec, qkv, att, kind, B, T, heads, d / heads, causal));
    tl_gemm_epilogue e2;
    e2.bias = p->bo; e2.residual = x; e2.ldr = d; e2.out = y; e2.ldo = d; e2.out_kind = TL_OUT_F32;
    TL_TRY(tl_gemm(ctx, prec, att, d, p->wo_t, d, (int)M, d, d, e2));
    TL_TRY(tl_layernorm(ctx, y, p->ln2_gamma, p->ln2_beta, 1e-5f, a, kind, M, d));
    tl_gemm_epilogue e3;
    e3.bias = p->b1; e3.act = act; e3.accurate_math = accurate; e3.out = hid; e3.ldo = 4 * d; e3.out_kind = kind;
    TL_TRY(tl_gemm(ctx, prec, a, d, p->w1_t, d, (int)M, 4 * d, d, e3));
    tl_gemm_epilogue e4;
    e4.bias = p->b2; e4.residual = y; e4.ldr = d; e4.out = out; e4.ldo = d; e4.out_kind = TL_OUT_F32;
    TL_TRY(tl_gemm(ctx, prec, hid, 4 * d, p->w2_t, 4 * d, (int)M, d, 4 * d, e4));
    return TLNN_OK;
}

int check_block_shape(int B, int T, int d, int heads) {
    TL_REQUIRE(B >= 0 && T >= 0 && d > 0 && heads > 0 && d % heads == 0, "bad shape B=%d T=%d d=%d heads=%d", B, T, d, heads);
    TL_REQUIRE((long long)B * T < (1ll << 31) / 4, "too many rows (%lld)", (long long)B * T);
    TL_REQUIRE(d % 8 == 0, "the model width %d must be a multiple of 8", d);
    return TLNN_OK;
}

size_t head_ws_bytes(tlnn_ctx* ctx, int prec, long long rows, int d, int vocab, bool want_tokens) {
    size_t n = tl_ws_round((size_t)rows * d * op_size(prec));
    if (want_tokens) {
        n += tl_ws_round((size_t)rows * tl_gemm_argmax_parts(prec, (int)rows, vocab, ctx->sm_count) * sizeof(float2));
    }
    return n;
}

// Head GEMM on operand rows `a` (already in the mode's operand type) with optional logits and fused arg-max.
int run_head(tlnn_ctx* ctx, int prec, const void* a, const void* table_t, const float* bias, float* logits,
             int32_t* tokens, long long rows, int d, int vocab, tl_ws_cursor cur) {
    tl_gemm_epilogue e;
    e.bias = bias; e.out = logits; e.ldo = vocab; e.out_kind = TL_OUT_F32;
    int n_parts = 0;
    if (tokens) {
        n_parts = tl_gemm_argmax_parts(prec, (int)rows, vocab, ctx->sm_count);
        e.argmax_partials = cur.take<float2>((size_t)rows * n_parts);
    }
    TL_TRY(tl_gemm(ctx, prec, a, d, table_t, d, (int)rows, vocab, d, e));
    if (tokens) TL_TRY(tl_argmax_partials(ctx, e.argmax_partials, n_parts, tokens, rows));
    return TLNN_OK;
}

}  // namespace

// Shared with the decode path: one causal block over a prompt, also copying the block's keys and values into the
// layer's cache (rows [0, T) of every sequence; the cache holds cache_len rows per sequence).
int tl_run_block_kv(tlnn_ctx* ctx, int prec, const float* x, const tlnn_block_params* p, int act, float* out, int B, int T,
                    int d, int heads, char* ws_base, void* kcache, void* vcache, int cache_len) {
    tl_ws_cursor cur(ctx);
    cur.base = ws_base;
    return run_block(ctx, prec, x, p, act, out, B, T, d, heads, 1, cur, kcache, vcache, cache_len);
}
size_t tl_block_ws_bytes(int prec, long long M, int d) { return block_ws_bytes(prec, M, d); }

extern "C" int tlnn_linear_fwd(tlnn_ctx* ctx, int prec, const float* a, long long lda, const void* wt, const float* bias,
                               int act, const float* residual, long long ldr, float* out, long long ldo, int M, int N, int K) {
    TL_NOTNULL(ctx); TL_NOTNULL(wt); TL_NOTNULL(out);
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_REQUIRE(M >= 0 && N > 0 && K > 0 && lda >= K && ldo >= N, "linear: bad shape M=%d N=%d K=%d lda=%lld ldo=%lld", M, N, K, lda, ldo);
    TL_REQUIRE(act >= TLNN_ACT_NONE && act <= TLNN_ACT_RELU, "unknown activation %d", act);
    TL_REQUIRE(K % 8 == 0, "linear: the input width %d must be a multiple of 8", K);
    if (M == 0) return TLNN_OK;
    TL_NOTNULL(a);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_TRY(tl_ws_reserve(ctx, tl_ws_round((size_t)M * K * op_size(prec))));
    tl_ws_cursor cur(ctx);
    void* op = cur.take<char>((size_t)M * K * op_size(prec));
    TL_TRY(tl_convert(ctx, a, lda, op, op_kind(prec), M, K));
    tl_gemm_epilogue e;
    e.bias = bias; e.act = act; e.accurate_math = prec == TLNN_PREC_TF32;
    e.residual = residual; e.ldr = ldr; e.out = out; e.ldo = ldo; e.out_kind = TL_OUT_F32;
    return tl_gemm(ctx, prec, op, K, wt, K, M, N, K, e);
}

extern "C" int tlnn_attention_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* wqkv_t, const float* bqkv,
                                  const void* wo_t, const float* bo, float* out, int B, int T, int d, int heads, int causal) {
    TL_NOTNULL(ctx); TL_NOTNULL(wqkv_t); TL_NOTNULL(wo_t); TL_NOTNULL(out);
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_TRY(check_block_shape(B, T, d, heads));
    const long long M = (long long)B * T;
    if (M == 0) return TLNN_OK;
    TL_NOTNULL(x);
    TL_CUDA(cudaSetDevice(ctx->device));
    const size_t es = op_size(prec);
    TL_TRY(tl_ws_reserve(ctx, 2 * tl_ws_round((size_t)M * d * es) + tl_ws_round((size_t)M * 3 * d * es)));
    tl_ws_cursor cur(ctx);
    void* a = cur.take<char>((size_t)M * d * es);
    void* qkv = cur.take<char>((size_t)M * 3 * d * es);
    void* att = cur.take<char>((size_t)M * d * es);
    const int kind = op_kind(prec);
    TL_TRY(tl_convert(ctx, x, d, a, kind, M, d));
    tl_gemm_epilogue e1;
    e1.bias = bqkv; e1.out = qkv; e1.ldo = 3 * d;
    e1.out_kind = prec == TLNN_PREC_BF16 ? TL_OUT_BF16 : (tl_attention_tf32_applies(T, d / heads) ? TL_OUT_TF32 : TL_OUT_F32);
    TL_TRY(tl_gemm(ctx, prec, a, d, wqkv_t, d, (int)M, 3 * d, d, e1));
    TL_TRY(tl_attention_core(ctx, prec, qkv, att, kind, B, T, heads, d / heads, causal));
    tl_gemm_epilogue e2;
    e2.bias = bo; e2.out = out; e2.ldo = d; e2.out_kind = TL_OUT_F32;
    return tl_gemm(ctx, prec, att, d, wo_t, d, (int)M, d, d, e2);
}

extern "C" int tlnn_ffn_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* w1_t, const float* b1, const void* w2_t,
                            const float* b2, int act, float* out, long long rows, int d) {
    TL_NOTNULL(ctx); TL_NOTNULL(w1_t); TL_NOTNULL(w2_t); TL_NOTNULL(out);
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_REQUIRE(rows >= 0 && rows < (1ll << 29) && d > 0 && d % 8 == 0, "ffn: bad shape rows=%lld d=%d", rows, d);
    TL_REQUIRE(act >= TLNN_ACT_NONE && act <= TLNN_ACT_RELU, "unknown activation %d", act);
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(x);
    TL_CUDA(cudaSetDevice(ctx->device));
    const size_t es = op_size(prec);
    TL_TRY(tl_ws_reserve(ctx, tl_ws_round((size_t)rows * d * es) + tl_ws_round((size_t)rows * 4 * d * es)));
    tl_ws_cursor cur(ctx);
    void* a = cur.take<char>((size_t)rows * d * es);
    void* hid = cur.take<char>((size_t)rows * 4 * d * es);
    const int kind = op_kind(prec);
    TL_TRY(tl_convert(ctx, x, d, a, kind, rows, d));
    tl_gemm_epilogue e1;
    e1.bias = b1; e1.act = act; e1.accurate_math = prec == TLNN_PREC_TF32; e1.out = hid; e1.ldo = 4 * d; e1.out_kind = kind;
    TL_TRY(tl_gemm(ctx, prec, a, d, w1_t, d, (int)rows, 4 * d, d, e1));
    tl_gemm_epilogue e2;
    e2.bias = b2; e2.out = out; e2.ldo = d; e2.out_kind = TL_OUT_F32;
    return tl_gemm(ctx, prec, hid, 4 * d, w2_t, 4 * d, (int)rows, d, 4 * d, e2);
}

static int check_block_params(const tlnn_block_params* p) {
    TL_NOTNULL(p);
    TL_NOTNULL(p->ln1_gamma); TL_NOTNULL(p->ln1_beta); TL_NOTNULL(p->wqkv_t); TL_NOTNULL(p->wo_t);
    TL_NOTNULL(p->ln2_gamma); TL_NOTNULL(p->ln2_beta); TL_NOTNULL(p->w1_t); TL_NOTNULL(p->w2_t);
    return TLNN_OK;
}

extern "C" int tlnn_block_fwd(tlnn_ctx* ctx, int prec, const float* x, const tlnn_block_params* p, int act, float* out,
                              int B, int T, int d, int heads, int causal) {
    TL_NOTNULL(ctx); TL_NOTNULL(out);
    TL_TRY(check_block_params(p));
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_REQUIRE(act >= TLNN_ACT_NONE && act <= TLNN_ACT_RELU, "unknown activation %d", act);
    TL_TRY(check_block_shape(B, T, d, heads));
    const long long M = (long long)B * T;
    if (M == 0) return TLNN_OK;
    TL_NOTNULL(x);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_TRY(tl_ws_reserve(ctx, block_ws_bytes(prec, M, d)));
    return run_block(ctx, prec, x, p, act, out, B, T, d, heads, causal, tl_ws_cursor(ctx));
}

extern "C" int tlnn_logits_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* table_t, const float* bias,
                               float* logits, int32_t* tokens, long long rows, int d, int vocab) {
    TL_NOTNULL(ctx); TL_NOTNULL(table_t);
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_REQUIRE(rows >= 0 && rows < (1ll << 29) && d > 0 && d % 8 == 0 && vocab > 0, "logits: bad shape rows=%lld d=%d vocab=%d", rows, d, vocab);
    TL_REQUIRE(logits || tokens, "logits: neither logits nor tokens requested");
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(x);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_TRY(tl_ws_reserve(ctx, head_ws_bytes(ctx, prec, rows, d, vocab, tokens != nullptr)));
    tl_ws_cursor cur(ctx);
    void* a = cur.take<char>((size_t)rows * d * op_size(prec));
    TL_TRY(tl_convert(ctx, x, d, a, op_kind(prec), rows, d));
    return run_head(ctx, prec, a, table_t, bias, logits, tokens, rows, d, vocab, cur);
}

extern "C" int tlnn_norm_logits_fwd(tlnn_ctx* ctx, int prec, const float* x, const float* gamma, const float* beta,
                                    const void* table_t, const float* bias, float* logits, int32_t* tokens,
                                    long long rows, int d, int vocab) {
    TL_NOTNULL(ctx); TL_NOTNULL(table_t); TL_NOTNULL(gamma); TL_NOTNULL(beta);
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_REQUIRE(rows >= 0 && rows < (1ll << 29) && d > 0 && d % 8 == 0 && vocab > 0, "logits: bad shape rows=%lld d=%d vocab=%d", rows, d, vocab);
    TL_REQUIRE(logits || tokens, "logits: neither logits nor tokens requested");
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(x);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_TRY(tl_ws_reserve(ctx, head_ws_bytes(ctx, prec, rows, d, vocab, tokens != nullptr)));
    tl_ws_cursor cur(ctx);
    void* a = cur.take<char>((size_t)rows * d * op_size(prec));
    TL_TRY(tl_layernorm(ctx, x, gamma, beta, 1e-5f, a, op_kind(prec), rows, d));
    return run_head(ctx, prec, a, table_t, bias, logits, tokens, rows, d, vocab, cur);
}

namespace {

// Operand row pitch of the patch matrix: a patch feature width that is not a multiple of 8 (the demo's 2 x 2 x 3 = 12)
// is padded with zero columns on both operands, because the GEMM wants operand rows of a multiple of 16 bytes.
inline int vit_patch_pitch(int tdim) { return (tdim + 7) / 8 * 8; }

size_t vit_project_ws_bytes(int prec, long long M, int d, int tdim) {
    const int ldt = vit_patch_pitch(tdim);
    return tl_ws_round((size_t)M * ldt * op_size(prec)) + tl_ws_round((size_t)d * ldt * op_size(prec));
}

// Everything the projector enqueues; the pieces come from `cur`, which the caller has reserved.
int vit_project_enqueue(tlnn_ctx* ctx, int prec, const float* img, const void* proj_t, const float* cls_reg, const float* pos,
                        float* out, int B, int C, int H, int W, int ph, int pw, int d, int regs, tl_ws_cursor cur) {
    const int tdim = ph * pw * C, n_patch = (H / ph) * (W / pw), n_cls = 1 + regs, T = n_cls + n_patch;
    const long long M = (long long)B * n_patch;
    const int ldt = vit_patch_pitch(tdim);
    void* tok = cur.take<char>((size_t)M * ldt * op_size(prec));
    const void* weight = proj_t;
    if (ldt != tdim) {
        void* wp = cur.take<char>((size_t)d * ldt * op_size(prec));
        size_t n = (size_t)d * ldt;
        int grid = (int)((n + 255) / 256);
        if (grid > ctx->sm_count * 16) grid = ctx->sm_count * 16;
        TL_LAUNCH(ctx, "vit_pad_weight", pad_rows_kernel<<<grid, 256, 0, ctx->stream>>>(proj_t, wp, d, tdim, ldt, (int)op_size(prec)));
        weight = wp;
    }
    {
        size_t n = (size_t)M * ldt;
        int grid = (int)((n + 255) / 256);
        if (grid > ctx->sm_count * 16) grid = ctx->sm_count * 16;
        TL_LAUNCH(ctx, "vit_patchify", patchify_kernel<<<grid, 256, 0, ctx->stream>>>(img, tok, op_kind(prec), B, C, H, W, ph, pw, ldt));
    }
    tl_gemm_epilogue e;
    e.residual = pos; e.ldr = d; e.res_row_mod = n_patch; e.res_row_off = n_cls;     // + positional row of the patch
    e.out = out; e.ldo = d; e.out_kind = TL_OUT_F32;
    e.row_group = n_patch; e.out_group = T; e.out_off = n_cls;                        // patch rows sit behind the class rows
    TL_TRY(tl_gemm(ctx, prec, tok, ldt, weight, ldt, (int)M, d, ldt, e));
    {
        size_t n = (size_t)B * n_cls * d;
        int grid = (int)((n + 255) / 256);
        if (grid > ctx->sm_count * 16) grid = ctx->sm_count * 16;
        TL_LAUNCH(ctx, "vit_cls_rows", cls_rows_kernel<<<grid, 256, 0, ctx->stream>>>(cls_reg, pos, out, B, T, d, n_cls));
    }
    return TLNN_OK;
}

int check_vit_image(int B, int C, int H, int W, int ph, int pw, int d, int regs) {
    TL_REQUIRE(B >= 0 && C > 0 && H > 0 && W > 0 && ph > 0 && pw > 0 && d > 0 && regs >= 0, "vit_project: bad shape");
    TL_REQUIRE(H % ph == 0 && W % pw == 0, "vit_project: image %dx%d is not a multiple of the patch %dx%d", H, W, ph, pw);
    return TLNN_OK;
}

}  // namespace

extern "C" int tlnn_vit_project_fwd(tlnn_ctx* ctx, int prec, const float* img, const void* proj_t, const float* cls_reg,
                                    const float* pos, float* out, int B, int C, int H, int W, int ph, int pw, int d, int regs) {
    TL_NOTNULL(ctx); TL_NOTNULL(proj_t); TL_NOTNULL(cls_reg); TL_NOTNULL(pos); TL_NOTNULL(out);
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_TRY(check_vit_image(B, C, H, W, ph, pw, d, regs));
    if (B == 0) return TLNN_OK;
    TL_NOTNULL(img);
    TL_CUDA(cudaSetDevice(ctx->device));
    const long long M = (long long)B * (H / ph) * (W / pw);
    TL_TRY(tl_ws_reserve(ctx, vit_project_ws_bytes(prec, M, d, ph * pw * C)));
    return vit_project_enqueue(ctx, prec, img, proj_t, cls_reg, pos, out, B, C, H, W, ph, pw, d, regs, tl_ws_cursor(ctx));
}

extern "C" int tlnn_vit_head_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* w_t, const float* bias, float* out,
                                 int B, int T, int d, int n_out) {
    TL_NOTNULL(ctx); TL_NOTNULL(w_t); TL_NOTNULL(out);
    TL_REQUIRE(prec_ok(prec), "unknown precision %d", prec);
    TL_REQUIRE(B >= 0 && T > 0 && d > 0 && d % 8 == 0 && n_out > 0, "vit_head: bad shape B=%d T=%d d=%d out=%d", B, T, d, n_out);
    if (B == 0) return TLNN_OK;
    TL_NOTNULL(x);
    // the class token is row 0 of every sample: a (B, d) matrix with a pitch of T*d
    return tlnn_linear_fwd(ctx, prec, x, (long long)T * d, w_t, bias, TLNN_ACT_NONE, nullptr, 0, out, n_out, B, n_out, d);
}

namespace {

// Launches made inside the scope may carry the programmatic-dependent-launch attribute (honoured by the kernels that
// begin with a grid-dependency wait; the others are launched plainly and serialise as usual).
struct pdl_scope {
    tlnn_ctx* c; bool old;
    pdl_scope(tlnn_ctx* cc, bool on) : c(cc), old(cc->pdl) { c->pdl = on; }
    ~pdl_scope() { c->pdl = old; }
};

// Everything tlnn_gpt_prefill enqueues, given that the workspace is already reserved.
int prefill_enqueue(tlnn_ctx* ctx, const tlnn_gpt_model* m, const void* ids, int ids_type, int B, int T, float* logits,
                    int32_t* tokens) {
    const long long M = (long long)B * T;
    // Kernels that begin with a grid-dependency wait (LayerNorm, the GEMMs, the small attention kernels, the arg-max
    // reduction) may be launched while their predecessor still runs.  That pays for small shards, whose products run
    // on the one-CTA GEMM and are short next to a launch:
    // 0.201 -> 0.193 ms for a 10.8 M-parameter model on 32 x 128 tokens; with the CTA-pair GEMM of large shards it
    // costs 1 %.  TLNN_PDL_PREFILL=1 / 0 forces it on / off.
    static const int pdl_env = getenv("TLNN_PDL_PREFILL") ? (strcmp(getenv("TLNN_PDL_PREFILL"), "1") == 0 ? 1 : 0) : -1;
    const int d = m->d;
    const bool pdl_auto = !tl_gemm_uses_pair(m->prec, (int)M, 3 * d, ctx->sm_count) && !tl_gemm_uses_pair(m->prec, (int)M, 4 * d, ctx->sm_count);
    pdl_scope scope(ctx, (pdl_env < 0 ? pdl_auto : pdl_env == 1) && !ctx->prof_classes);
    const size_t stream_bytes = tl_ws_round((size_t)M * d * 4);
    const size_t tail = block_ws_bytes(m->prec, M, d);
    const size_t head = head_ws_bytes(ctx, m->prec, M, d, m->vocab, tokens != nullptr);
    if (ctx->ws_bytes < 2 * stream_bytes + (tail > head ? tail : head)) { tl_set_error("gpt_prefill: workspace not reserved"); return TLNN_ERR_VALUE; }
    tl_ws_cursor cur(ctx);
    float* xa = cur.take<float>((size_t)M * d);
    float* xb = cur.take<float>((size_t)M * d);
    TL_TRY(tl_embed(ctx, ids, ids_type, m->tok_table, m->pos_table, xa, B, T, d, m->vocab));
    for (int l = 0; l < m->layers; l++) {
        if (m->prec == TLNN_PREC_BF16) {
            TL_TRY(run_block(ctx, m->prec, xa, &m->blocks[l], m->act, xa, B, T, d, m->heads, 1, cur));     // in place
        } else {
            TL_TRY(run_block(ctx, m->prec, xa, &m->blocks[l], m->act, xb, B, T, d, m->heads, 1, cur));
            float* t = xa; xa = xb; xb = t;
        }
    }
    void* a = cur.take<char>((size_t)M * d * op_size(m->prec));
    TL_TRY(tl_layernorm(ctx, xa, m->lnf_gamma, m->lnf_beta, 1e-5f, a, op_kind(m->prec), M, d));
    return run_head(ctx, m->prec, a, m->head_t, m->head_bias, logits, tokens, M, d, m->vocab, cur);
}

// A repeated whole-model call (same model description, buffers and shape) replays a captured CUDA graph of the first
// repetition: a step of a small shard is a hundred or more kernels of tens of microseconds, and the gaps between plain
// launches add up.  The context keeps one such graph, keyed by the bytes of everything the enqueued work depends on.
// TLNN_PREFILL_GRAPH=0 switches this off; per-class profiling always uses plain launches.
struct replay_cache {
    std::vector<unsigned char> key;
    int seen = 0;                       // identical calls so far
    long long launches = 0;             // kernels per replay
    cudaGraphExec_t exec = nullptr;
};

struct replay_key {
    std::vector<unsigned char> bytes;
    template <typename V> replay_key& add(const V& v) {
        const unsigned char* p = reinterpret_cast<const unsigned char*>(&v);
        bytes.insert(bytes.end(), p, p + sizeof(V));
        return *this;
    }
    replay_key& add_block(const tlnn_block_params& b) {
        return add(b.ln1_gamma).add(b.ln1_beta).add(b.wqkv_t).add(b.bqkv).add(b.wo_t).add(b.bo).add(b.ln2_gamma).add(b.ln2_beta)
              .add(b.w1_t).add(b.b1).add(b.w2_t).add(b.b2);
    }
};

bool prefill_graph_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("TLNN_PREFILL_GRAPH");
        on = (e && strcmp(e, "0") == 0) ? 0 : 1;
    }
    return on == 1;
}

// Runs `enqueue` (which launches on ctx->stream and returns a status): plainly the first time a key is seen, as a stream
// capture that is instantiated and launched the second time, as a replay of that graph from then on.
template <typename F>
int replay_or_run(tlnn_ctx* ctx, const replay_key& key, F&& enqueue) {
    if (!prefill_graph_enabled() || ctx->prof_classes) return enqueue();
    replay_cache* c = static_cast<replay_cache*>(ctx->prefill_cache);
    if (c && c->key == key.bytes) {
        if (c->exec) {
            TL_CUDA(cudaGraphLaunch(c->exec, ctx->stream));
            ctx->launches += c->launches;
            return TLNN_OK;
        }
        if (++c->seen == 2) {
            const long long before = ctx->launches;
            TL_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
            const int st = enqueue();
            cudaGraph_t g = nullptr;
            const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &g);
            c->launches = ctx->launches - before;
            ctx->launches = before;
            if (st != TLNN_OK) { if (g) cudaGraphDestroy(g); return st; }
            if (ce != cudaSuccess) return tl_cuda_fail(ce, "cudaStreamEndCapture", __FILE__, __LINE__);
            const cudaError_t ie = cudaGraphInstantiate(&c->exec, g, 0);
            cudaGraphDestroy(g);
            if (ie != cudaSuccess) { c->exec = nullptr; return tl_cuda_fail(ie, "cudaGraphInstantiate", __FILE__, __LINE__); }
            TL_CUDA(cudaGraphLaunch(c->exec, ctx->stream));
            ctx->launches += c->launches;
            return TLNN_OK;
        }
        return enqueue();
    }
    // a new description: remember it, run it with plain launches
    tl_prefill_cache_free(ctx);
    c = new replay_cache();
    c->key = key.bytes;
    c->seen = 1;
    ctx->prefill_cache = c;
    return enqueue();
}

// Everything tlnn_vit_forward enqueues, given that the workspace is already reserved.
int vit_forward_enqueue(tlnn_ctx* ctx, const tlnn_vit_model* m, const float* img, int B, float* out) {
    static const bool pdl_off = getenv("TLNN_PDL_VIT") && strcmp(getenv("TLNN_PDL_VIT"), "0") == 0;
    pdl_scope scope(ctx, !pdl_off && !ctx->prof_classes);
    const int d = m->d, n_patch = (m->height / m->patch_h) * (m->width / m->patch_w), T = 1 + m->registers + n_patch;
    const long long M = (long long)B * T;
    tl_ws_cursor cur(ctx);
    float* xa = cur.take<float>((size_t)M * d);
    float* xb = cur.take<float>((size_t)M * d);
    TL_TRY(vit_project_enqueue(ctx, m->prec, img, m->proj_t, m->cls_reg, m->pos, xa, B, m->channels, m->height, m->width,
                               m->patch_h, m->patch_w, d, m->registers, cur));
    for (int l = 0; l < m->layers; l++) {
        if (m->prec == TLNN_PREC_BF16) {
            TL_TRY(run_block(ctx, m->prec, xa, &m->blocks[l], m->act, xa, B, T, d, m->heads, 0, cur));     // in place
        } else {
            TL_TRY(run_block(ctx, m->prec, xa, &m->blocks[l], m->act, xb, B, T, d, m->heads, 0, cur));
            float* t = xa; xa = xb; xb = t;
        }
    }
    // LayerNorm works row by row and the head reads the class row only: normalise that row of every image
    float* cls = cur.take<float>((size_t)B * d);
    void* a = cur.take<char>((size_t)B * d * op_size(m->prec));
    TL_TRY(tl_convert(ctx, xa, (long long)T * d, cls, TL_OUT_F32, B, d));
    TL_TRY(tl_layernorm(ctx, cls, m->lnf_gamma, m->lnf_beta, 1e-5f, a, op_kind(m->prec), B, d));
    tl_gemm_epilogue e;
    e.bias = m->head_bias; e.out = out; e.ldo = m->n_out; e.out_kind = TL_OUT_F32;
    return tl_gemm(ctx, m->prec, a, d, m->head_t, d, B, m->n_out, d, e);
}

}  // namespace

void tl_prefill_cache_free(tlnn_ctx* ctx) {
    replay_cache* c = static_cast<replay_cache*>(ctx->prefill_cache);
    if (!c) return;
    if (c->exec) cudaGraphExecDestroy(c->exec);
    delete c;
    ctx->prefill_cache = nullptr;
}

extern "C" int tlnn_gpt_prefill(tlnn_ctx* ctx, const tlnn_gpt_model* m, const void* ids, int ids_type, int B, int T,
                                float* logits, int32_t* tokens) {
    TL_NOTNULL(ctx); TL_NOTNULL(m); TL_NOTNULL(m->tok_table); TL_NOTNULL(m->pos_table); TL_NOTNULL(m->blocks);
    TL_NOTNULL(m->lnf_gamma); TL_NOTNULL(m->lnf_beta); TL_NOTNULL(m->head_t);
    TL_REQUIRE(prec_ok(m->prec), "unknown precision %d", m->prec);
    TL_REQUIRE(m->layers >= 0 && m->vocab > 0 && m->context > 0, "gpt_prefill: bad model description");
    TL_REQUIRE(T <= m->context, "gpt_prefill: sequence length %d exceeds the context length %d", T, m->context);
    TL_REQUIRE(ids_type == TLNN_I32 || ids_type == TLNN_I64 || ids_type == TLNN_U8, "token ids must be int32, int64 or uint8");
    TL_REQUIRE(logits || tokens, "gpt_prefill: neither logits nor tokens requested");
    TL_TRY(check_block_shape(B, T, m->d, m->heads));
    for (int l = 0; l < m->layers; l++) TL_TRY(check_block_params(&m->blocks[l]));
    const long long M = (long long)B * T;
    if (M == 0) return TLNN_OK;
    TL_NOTNULL(ids);
    TL_CUDA(cudaSetDevice(ctx->device));
    {
        const int d = m->d;
        const size_t stream_bytes = tl_ws_round((size_t)M * d * 4);
        const size_t tail = block_ws_bytes(m->prec, M, d);
        const size_t head = head_ws_bytes(ctx, m->prec, M, d, m->vocab, tokens != nullptr);
        TL_TRY(tl_ws_reserve(ctx, 2 * stream_bytes + (tail > head ? tail : head)));
    }
    replay_key key;
    key.add('G').add(m->vocab).add(m->context).add(m->d).add(m->heads).add(m->layers).add(m->act).add(m->prec)
       .add(m->tok_table).add(m->pos_table).add(m->lnf_gamma).add(m->lnf_beta).add(m->head_t).add(m->head_bias)
       .add(ids).add(ids_type).add(B).add(T).add(logits).add(tokens).add(ctx->ws);
    for (int l = 0; l < m->layers; l++) key.add_block(m->blocks[l]);
    return replay_or_run(ctx, key, [&] { return prefill_enqueue(ctx, m, ids, ids_type, B, T, logits, tokens); });
}

extern "C" int tlnn_vit_forward(tlnn_ctx* ctx, const tlnn_vit_model* m, const float* img, int B, float* out) {
    TL_NOTNULL(ctx); TL_NOTNULL(m); TL_NOTNULL(m->proj_t); TL_NOTNULL(m->cls_reg); TL_NOTNULL(m->pos); TL_NOTNULL(m->blocks);
    TL_NOTNULL(m->lnf_gamma); TL_NOTNULL(m->lnf_beta); TL_NOTNULL(m->head_t); TL_NOTNULL(out);
    TL_REQUIRE(prec_ok(m->prec), "unknown precision %d", m->prec);
    TL_REQUIRE(m->layers >= 0 && m->n_out > 0, "vit_forward: bad model description");
    TL_REQUIRE(m->act >= TLNN_ACT_NONE && m->act <= TLNN_ACT_RELU, "unknown activation %d", m->act);
    TL_TRY(check_vit_image(B, m->channels, m->height, m->width, m->patch_h, m->patch_w, m->d, m->registers));
    const int n_patch = (m->height / m->patch_h) * (m->width / m->patch_w), T = 1 + m->registers + n_patch;
    TL_TRY(check_block_shape(B, T, m->d, m->heads));
    for (int l = 0; l < m->layers; l++) TL_TRY(check_block_params(&m->blocks[l]));
    if (B == 0) return TLNN_OK;
    TL_NOTNULL(img);
    TL_CUDA(cudaSetDevice(ctx->device));
    const long long M = (long long)B * T;
    const int d = m->d;
    {
        const size_t stream_bytes = tl_ws_round((size_t)M * d * 4);
        const size_t proj = vit_project_ws_bytes(m->prec, (long long)B * n_patch, d, m->patch_h * m->patch_w * m->channels);
        const size_t tail = block_ws_bytes(m->prec, M, d);
        const size_t head = tl_ws_round((size_t)B * d * 4) + tl_ws_round((size_t)B * d * op_size(m->prec));
        size_t most = proj > tail ? proj : tail;
        if (head > most) most = head;
        TL_TRY(tl_ws_reserve(ctx, 2 * stream_bytes + most));
    }
    replay_key key;
    key.add('V').add(m->channels).add(m->height).add(m->width).add(m->patch_h).add(m->patch_w).add(m->d).add(m->heads)
       .add(m->layers).add(m->act).add(m->prec).add(m->registers).add(m->n_out).add(m->proj_t).add(m->cls_reg).add(m->pos)
       .add(m->lnf_gamma).add(m->lnf_beta).add(m->head_t).add(m->head_bias).add(img).add(B).add(out).add(ctx->ws);
    for (int l = 0; l < m->layers; l++) key.add_block(m->blocks[l]);
    return replay_or_run(ctx, key, [&] { return vit_forward_enqueue(ctx, m, img, B, out); });
}
