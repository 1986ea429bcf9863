// Arg-max head that allocates nothing: the same kernels as tlnn_logits_fwd with tokens requested, but with every
// intermediate placed in one array that is part of the loaded library image instead of the context's arena.
#include "common.cuh"

// The scratch lives in the module's global data: each GPU that loads libtlnn.so carries these bytes from the first
// use of the library on that GPU until the process exits, whether or not this entry point is ever called.
static __device__ __align__(256) unsigned char g_static_scratch[TLNN_NOALLOC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel may dereference.  The
// device address is looked up once per device, with that device current, and cached here.
static void* g_scratch_addr[64] = {nullptr};

static int static_scratch(tlnn_ctx* ctx, char** out) {
    TL_REQUIRE(ctx->device >= 0 && ctx->device < 64, "device index %d is out of range for the static scratch table", ctx->device);
    if (!g_scratch_addr[ctx->device]) {
        void* p = nullptr;
        TL_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        g_scratch_addr[ctx->device] = p;
    }
    *out = reinterpret_cast<char*>(g_scratch_addr[ctx->device]);
    return TLNN_OK;
}

extern "C" int tlnn_logits_tokens_noalloc(tlnn_ctx* ctx, int prec, const float* x, const void* table_t, const float* bias,
                                          int32_t* tokens, long long rows, int d, int vocab) {
    TL_NOTNULL(ctx); TL_NOTNULL(table_t); TL_NOTNULL(tokens);
    TL_REQUIRE(prec == TLNN_PREC_BF16 || prec == TLNN_PREC_TF32, "unknown precision %d", prec);
    TL_REQUIRE(rows >= 0 && rows < (1ll << 29) && d > 0 && d % 8 == 0 && vocab > 0,
               "logits_tokens_noalloc: bad shape rows=%lld d=%d vocab=%d", rows, d, vocab);
    if (rows == 0) return TLNN_OK;
    TL_NOTNULL(x);
    TL_CUDA(cudaSetDevice(ctx->device));
    const size_t esz = prec == TLNN_PREC_BF16 ? 2 : 4;
    const int n_parts = tl_gemm_argmax_parts(prec, (int)rows, vocab, ctx->sm_count);
    const size_t operand_bytes = tl_ws_round((size_t)rows * d * esz);
    const size_t partial_bytes = (size_t)rows * n_parts * sizeof(float2);
    if (operand_bytes + partial_bytes > (size_t)TLNN_NOALLOC_SCRATCH_BYTES) {
        tl_set_error("logits_tokens_noalloc: rows=%lld d=%d vocab=%d needs %zu bytes of scratch, the built-in array holds %zu; "
                     "use tlnn_logits_fwd or fewer rows per call",
                     rows, d, vocab, operand_bytes + partial_bytes, (size_t)TLNN_NOALLOC_SCRATCH_BYTES);
        return TLNN_ERR_VALUE;
    }
    char* base = nullptr;
    TL_TRY(static_scratch(ctx, &base));
    void* operand = base;
    float2* partials = reinterpret_cast<float2*>(base + operand_bytes);
    // Both pieces are written in full before they are read (every operand element by the conversion, every
    // (row, tile) pair by the GEMM epilogue), so what an earlier call left behind never needs clearing.
    TL_TRY(tl_convert(ctx, x, d, operand, prec == TLNN_PREC_BF16 ? TL_OUT_BF16 : TL_OUT_TF32, rows, d));
    tl_gemm_epilogue e;
    e.bias = bias;
    e.argmax_partials = partials;
    TL_TRY(tl_gemm(ctx, prec, operand, d, table_t, d, (int)rows, vocab, d, e));
    return tl_argmax_partials(ctx, partials, n_parts, tokens, rows);
}
