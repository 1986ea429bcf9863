// Shared declarations of libtlnn: context, error handling, launch bookkeeping, workspace arena.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>
#include <map>
#include <utility>

#include "../../include/tlnn.h"

// ---- device-side error word ------------------------------------------------------------------
// Kernels never trap.  A kernel that meets a bad index or gives up a bounded wait records the first such
// event here and carries on (or returns); the host reads the word at the next sync.
struct tlnn_dev_err {
    int code;      // 0, TLNN_ERR_INDEX or TLNN_ERR_TIMEOUT
    int where;     // kernel-specific site id
    long long detail;
};

__device__ __forceinline__ void tl_dev_fail(tlnn_dev_err* e, int code, int where, long long detail) {
    if (atomicCAS(&e->code, 0, code) == 0) {
        e->where = where;
        e->detail = detail;
    }
}

// Debug build (-DTLNN_DEBUG, `python -m torchless_nn_b200.build --debug` -> libtlnn_debug.so): stores of the large
// kernels check their linear offset against the extent of the output first; a violation is recorded in the error word
// (TLNN_ERR_INDEX with the site and the offending offset, reported at the next sync) and the store is skipped - the
// kernel never traps.  In the regular build the check compiles to nothing.
#ifdef TLNN_DEBUG
#define TL_DBG_IN_BOUNDS(err, cond, site, detail) ((cond) ? true : (tl_dev_fail((err), TLNN_ERR_INDEX, (site), (long long)(detail)), false))
#else
#define TL_DBG_IN_BOUNDS(err, cond, site, detail) (true)
#endif

// ---- profiling table ----------------------------------------------------------------------------
struct tl_prof_pending {
    const char* name;
    cudaEvent_t start, stop;
};

struct tlnn_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaMemPool_t pool = nullptr;
    tlnn_dev_err* d_err = nullptr;     // device memory
    tlnn_dev_err* h_err = nullptr;     // pinned host mirror
    int* d_sched = nullptr;            // device work counter of the persistent attention kernel (zeroed per launch)
    long long launches = 0;
    bool pdl = false;                  // launches made now may start before their predecessor has finished (see tl_launch_kernel)
    void* prefill_cache = nullptr;     // captured graph of the last repeated tlnn_gpt_prefill call (layers.cu)
    // grow-only scratch arena used by the composite layer calls (stream-ordered reuse)
    char* ws = nullptr;
    size_t ws_bytes = 0;

    // whole-interval timing
    cudaEvent_t prof_a = nullptr, prof_b = nullptr;
    // per-class timing
    bool prof_classes = false;
    std::vector<tl_prof_pending> pending;
    std::vector<cudaEvent_t> event_pool;
    std::map<std::string, std::pair<long long, double>> table;

    // canary mode (tlnn_debug_canaries): every tlnn_alloc is followed by TL_CANARY_BYTES of a known pattern, checked
    // when the block is freed and by tlnn_debug_check
    bool canaries = false;
    std::map<void*, size_t> live;      // user pointer -> user bytes
    long long canary_failures = 0;
};
constexpr size_t TL_CANARY_BYTES = 256;
constexpr int TL_CANARY_BYTE = 0xC5;

// ---- host-side error plumbing --------------------------------------------------------------------
void tl_set_error(const char* fmt, ...);
int tl_cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define TL_CUDA(call)                                                             \
    do {                                                                          \
        cudaError_t e_ = (call);                                                  \
        if (e_ != cudaSuccess) return tl_cuda_fail(e_, #call, __FILE__, __LINE__); \
    } while (0)

#define TL_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            tl_set_error(__VA_ARGS__);   \
            return TLNN_ERR_VALUE;       \
        }                                \
    } while (0)

#define TL_NOTNULL(p)                                     \
    do {                                                  \
        if ((p) == nullptr) {                             \
            tl_set_error("null pointer argument: %s", #p); \
            return TLNN_ERR_NULL;                         \
        }                                                 \
    } while (0)

#define TL_TRY(call)              \
    do {                          \
        int s_ = (call);          \
        if (s_ != TLNN_OK) return s_; \
    } while (0)

// Bracket one kernel launch: optional per-class events, launch counter, launch-error check.
int tl_launch_begin(tlnn_ctx* ctx, const char* name);
int tl_launch_end(tlnn_ctx* ctx, const char* name);

#define TL_LAUNCH(ctx, name, ...)            \
    do {                                     \
        TL_TRY(tl_launch_begin(ctx, name));  \
        __VA_ARGS__;                         \
        TL_TRY(tl_launch_end(ctx, name));    \
    } while (0)

void tl_prefill_cache_free(tlnn_ctx* ctx);     // layers.cu: drops the captured prefill graph

// ---- programmatic dependent launch ---------------------------------------------------------------------------------
// A kernel that begins with tl_grid_dependency_sync() may be launched while its predecessor in the stream is still
// running: the call lets the kernel's own successor start launching, then waits until every predecessor grid has
// completed and its memory is visible.  Launch latency and whatever the kernel does before the call (barrier set-up,
// TMEM allocation) overlap with the predecessor.  Without the launch attribute both instructions do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void tl_grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void tl_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void tl_grid_dependency_sync() { tl_grid_dependency_trigger(); tl_grid_dependency_wait(); }

template <typename... KArgs, typename... Args>
inline void tl_launch_kernel(tlnn_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);      // the launch status is read by tl_launch_end
}
#endif

// ---- scratch arena ---------------------------------------------------------------------------------
// A composite call reserves its total need up front (which may reallocate while the stream is idle), then
// carves aligned pieces.  Pieces stay valid until the next reserve on the same context.
int tl_ws_reserve(tlnn_ctx* ctx, size_t bytes);

struct tl_ws_cursor {
    char* base;
    size_t off = 0;
    explicit tl_ws_cursor(tlnn_ctx* ctx) : base(ctx->ws) {}
    template <typename T>
    T* take(size_t n) {
        T* p = reinterpret_cast<T*>(base + off);
        off += (n * sizeof(T) + 1023) & ~size_t(1023);
        return p;
    }
};
static inline size_t tl_ws_round(size_t bytes) { return (bytes + 1023) & ~size_t(1023); }

// ---- internal kernels' host launchers (shared across translation units) -------------------------------
// Output element kinds of the row kernels and the GEMM epilogue.
enum { TL_OUT_F32 = 0, TL_OUT_BF16 = 1, TL_OUT_TF32 = 2 /* float32 storage rounded to TF32 */ };

int tl_layernorm(tlnn_ctx* ctx, const float* x, const float* gamma, const float* beta, float eps,
                 void* out, int out_kind, long long rows, int d);
int tl_convert(tlnn_ctx* ctx, const float* x, long long ldx, void* out, int out_kind, long long rows, int cols);
int tl_embed(tlnn_ctx* ctx, const void* ids, int ids_type, const float* table, const float* pos, float* out,
             int B, int T, int d, int vocab);
int tl_argmax_partials(tlnn_ctx* ctx, const float2* partials, int n_parts, int32_t* tokens, long long rows);
// Inverse-CDF draw per row; `step` (device, may be null) selects the block of `rows` uniform numbers to use.
int tl_sample(tlnn_ctx* ctx, const float* probs, long long ldp, const double* uniforms, const int* step, int32_t* out,
              long long rows, int cols);

// Epilogue description of the tensor-core GEMM: out = act(acc + bias) + residual, with optional row remapping
// (used by the ViT projector to drop patch rows behind the class token) and optional per-tile arg-max.
struct tl_gemm_epilogue {
    const float* bias = nullptr;        // (N) or null
    int act = TLNN_ACT_NONE;
    const float* residual = nullptr;    // float32, pitch ldr, or null
    long long ldr = 0;
    int res_row_mod = 0;                // >0: residual row = res_row_off + row % res_row_mod
    int res_row_off = 0;
    void* out = nullptr;                // may be null when only argmax partials are wanted
    long long ldo = 0;
    int out_kind = TL_OUT_F32;
    int row_group = 0;                  // >0: out row = (row / row_group) * out_group + out_off + row % row_group
    int out_group = 0;
    int out_off = 0;
    float2* argmax_partials = nullptr;  // (M, tl_gemm_argmax_parts) of (max, index as float bits) or null
    int accurate_math = 0;              // 1: activation to a few float32 ulp, 0: hardware tanh approximation
    long long out_elems = 0;            // extent of `out` in elements, filled in by tl_gemm (checked by the debug build's stores)
};

// A (M,K) and W (N,K) both with the contraction dimension contiguous, of element kind `prec`
// (TLNN_PREC_BF16: __nv_bfloat16, TLNN_PREC_TF32: float).  lda / ldw in elements.
int tl_gemm(tlnn_ctx* ctx, int prec, const void* a, long long lda, const void* w, long long ldw,
            int M, int N, int K, const tl_gemm_epilogue& ep);
// Tile width the GEMM will pick for this problem, and the number of arg-max candidates it leaves per row
// (the partial buffer holds rows x tl_gemm_argmax_parts float2 entries).
int tl_gemm_bn(int M, int N, int sm_count);
// Whether tl_gemm runs this product on the CTA-pair kernel (256 x 256 tiles) rather than the one-CTA kernel.
bool tl_gemm_uses_pair(int prec, int M, int N, int sm_count);
int tl_gemm_argmax_parts(int prec, int M, int N, int sm_count);

// Fused attention on a packed projection buffer: qkv is (B, T, 3d) with columns [0,d) Q, [d,2d) K, [2d,3d) V
// and head h at columns h*hd..(h+1)*hd inside each third.  out is (B, T, d) of the same kind.
int tl_attention_core(tlnn_ctx* ctx, int prec, const void* qkv, void* out, int out_kind,
                      int B, int T, int heads, int hd, int causal);

// FP32/TF32-mode attention on the tensor cores (attention_tf32.cu): whether a shape takes it - its projection should then
// round q, k and v to TF32 - and the launcher.
bool tl_attention_tf32_applies(int T, int hd);
int tl_attention_tf32(tlnn_ctx* ctx, const float* qkv, float* out, int B, int T, int heads, int causal, int round_out);

// Copy the K and V thirds of a packed (B*T, 3d) projection into per-layer caches laid out (B, heads, cache_len, d / heads):
// the rows of one (sequence, head) are contiguous, which is how the single-query attention of a decode step reads them.
int tl_kv_store(tlnn_ctx* ctx, int prec, const void* qkv, void* kcache, void* vcache, int B, int T, int d, int heads, int cache_len);
int tl_run_block_kv(tlnn_ctx* ctx, int prec, const float* x, const tlnn_block_params* p, int act, float* out, int B, int T,
                    int d, int heads, char* ws_base, void* kcache, void* vcache, int cache_len);
size_t tl_block_ws_bytes(int prec, long long M, int d);

