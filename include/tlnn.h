/*
 * tlnn.h - C ABI of libtlnn.so, the sm_100a (B200) engine behind the transformer
 * forward path of luke-skynet/torchless-nn.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an
 * int status (0 = success, negative = error class below) and never throws or
 * aborts.  `tlnn_last_error` returns the text of the most recent failure on the
 * calling thread.  All device pointers are pointers obtained from `tlnn_alloc`
 * on the same context (or any device pointer valid on the context's device).
 * All work is enqueued on the context's compute stream; `tlnn_sync`, `tlnn_d2h`
 * and `tlnn_check` are the only calls that wait for the device.
 *
 * Each declaration cites the reference code (file:line in the reference
 * repository) whose array operations it replaces.
 */
#ifndef TLNN_H
#define TLNN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define TLNN_OK              0
#define TLNN_ERR_VALUE      -1   /* bad shape / size / option        -> ValueError   */
#define TLNN_ERR_INDEX      -2   /* token id outside the table       -> IndexError   */
#define TLNN_ERR_CUDA       -3   /* CUDA runtime / driver error      -> RuntimeError */
#define TLNN_ERR_NOMEM      -4   /* device allocation failed         -> MemoryError  */
#define TLNN_ERR_TIMEOUT    -5   /* a bounded device-side wait gave up -> RuntimeError */
#define TLNN_ERR_NULL       -6   /* null pointer argument            -> ValueError   */

/* ---- element types ------------------------------------------------------ */
#define TLNN_F32   0
#define TLNN_BF16  1
#define TLNN_I32   2
#define TLNN_I64   3
#define TLNN_U8    4

/* ---- arithmetic modes (backend.py:9,16 enables TF32 tensor-op math) ------ */
#define TLNN_PREC_TF32 0   /* fp32 storage, operands rounded to TF32, fp32 accumulate */
#define TLNN_PREC_BF16 1   /* bf16 weights and GEMM operands, fp32 accumulate, fp32 residual stream */

/* ---- activations (activations.py:10-13, 24-28, 41-45) ------------------- */
#define TLNN_ACT_NONE 0
#define TLNN_ACT_GELU 1   /* tanh approximation */
#define TLNN_ACT_SILU 2   /* x (1 + tanh(x/2)) / 2 */
#define TLNN_ACT_RELU 3

typedef struct tlnn_ctx tlnn_ctx;

/* ---- lifecycle ---------------------------------------------------------- */
/* Replaces the import-time device set-up of backend.py:7-18. One context per device. */
int  tlnn_version(void);
int  tlnn_init(int device, tlnn_ctx** out);
int  tlnn_shutdown(tlnn_ctx* ctx);
const char* tlnn_last_error(void);
/* Wait for the compute stream; reports asynchronous faults and device-side error words. */
int  tlnn_sync(tlnn_ctx* ctx);
/* Read (and clear) the device-side error word without a message: 0, TLNN_ERR_INDEX or TLNN_ERR_TIMEOUT. */
int  tlnn_check(tlnn_ctx* ctx);
/* The context's compute stream as a cudaStream_t, for interop (events, NCCL). */
void* tlnn_stream(tlnn_ctx* ctx);
int  tlnn_device_info(tlnn_ctx* ctx, int* sm_count, size_t* total_mem, size_t* free_mem);
/* Number of this library's kernels launched on the context since the last reset (reset != 0 clears). */
long long tlnn_launch_count(tlnn_ctx* ctx, int reset);

/* ---- memory: replaces xp.zeros / xp.array / ndarray.get (backend.py:33-34, demo.ipynb:1576,1707) */
int tlnn_alloc(tlnn_ctx* ctx, size_t bytes, void** dptr);
int tlnn_free(tlnn_ctx* ctx, void* dptr);
int tlnn_host_alloc(size_t bytes, void** hptr);          /* pinned host memory */
int tlnn_host_free(void* hptr);
int tlnn_h2d(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes);   /* asynchronous if src is pinned */
int tlnn_d2h(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes);   /* waits for the stream */
int tlnn_d2h_async(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes);
int tlnn_d2d(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes);
int tlnn_memset(tlnn_ctx* ctx, void* dst, int byte, size_t bytes);
/* In-place parameter arithmetic used by weight loading (demo.ipynb:1725-1726) and ndarray.fill (utils.py:45-52):
   x = x * alpha + beta * y (y may be NULL), over n float32 elements. */
int tlnn_axpby_f32(tlnn_ctx* ctx, float* x, float alpha, const float* y, float beta, size_t n);
/* out[i] = a[i] + b[i]  (Residual "add" mode, utils.py:84-85) */
int tlnn_add_f32(tlnn_ctx* ctx, const float* a, const float* b, float* out, size_t n);
/* dst[i] = src[index[i]]: basic-slicing support for device arrays (the [0,-1] / [:, -1] idiom, demo.ipynb:1530) */
int tlnn_gather_f32(tlnn_ctx* ctx, const float* src, const int64_t* index, float* dst, size_t n);

/* ---- weight preparation -------------------------------------------------- */
/* Re-lay-out a reference weight once after upload.  `w` is float32, `rows` x `cols` row-major
 * (the reference stores GEMM weights as (in, out): layers.py:200,269,272,356,359).  With transpose != 0
 * the result is (cols, rows) row-major, i.e. (out, in) with the contraction dimension contiguous, which is
 * what the tensor-core operand descriptors read; with transpose == 0 the layout is kept (the tied token
 * table (V, d) already is (out, in): transformer_adapters.py:113,176).  `prec` selects bf16 rounding or
 * float32 rounded to nearest-even TF32.  `out` holds rows*cols elements of the target type. */
int tlnn_weight_prepare(tlnn_ctx* ctx, const float* w, int rows, int cols, int transpose, int prec, void* out);

/* ---- linear: out = act(A @ W^T + bias) + residual ------------------------ */
/* Replaces `input @ W + b` (layers.py:208, 286, 306, 372-373; transformer_adapters.py:49, 93, 176).
 * A is (M, K) float32 with row pitch lda elements; `wt` is a prepared weight (N, K) in the mode's type.
 * bias (N) and residual (M, N, pitch ldr) are optional float32.  out is (M, N) float32 with pitch ldo. */
int tlnn_linear_fwd(tlnn_ctx* ctx, int prec, const float* a, long long lda, const void* wt,
                    const float* bias, int act, const float* residual, long long ldr,
                    float* out, long long ldo, int M, int N, int K);

/* ---- layers -------------------------------------------------------------- */
/* GPTEmbedFront.forward (transformer_adapters.py:148-153): out[b,t,:] = table[ids[b,t],:] + pos[t,:].
 * Bit-exact float32.  ids_type is TLNN_I32, TLNN_I64 or TLNN_U8; negative ids wrap once like NumPy;
 * an id outside [-vocab, vocab) sets the device error word (TLNN_ERR_INDEX at the next sync/check). */
int tlnn_embed_fwd(tlnn_ctx* ctx, const void* ids, int ids_type, const float* table, const float* pos,
                   float* out, int B, int T, int d, int vocab);

/* LayerNorm.forward (layers.py:415-428): per row mean, biased variance, (var+eps)^0.5, affine. */
int tlnn_layernorm_fwd(tlnn_ctx* ctx, const float* x, const float* gamma, const float* beta, float eps,
                       float* out, long long rows, int d);

/* Element-wise activation layers on their own (activations.py:10-13, 24-28, 41-45). */
int tlnn_activation_fwd(tlnn_ctx* ctx, int act, const float* x, float* out, size_t n);

/* SoftMax.forward (activations.py:57-64): exp((x - max) / temperature) / sum over the last axis. */
int tlnn_softmax_fwd(tlnn_ctx* ctx, const float* x, float* out, long long rows, int cols, float temperature);

/* xp.argmax(logits, axis=-1) (network.py:135,158): first index of the row maximum, int32. */
int tlnn_argmax_fwd(tlnn_ctx* ctx, const float* x, long long ldx, int32_t* out, long long rows, int cols);

/* One batch of Network.evaluate (network.py:145-160) on the device: for every row of probs (rows, V, pitch ldp)
 * adds -log(probs[row, label] + 1e-7) (CrossEntropy.loss, network.py:19-22) to *loss_sum and 1 to *correct when the
 * first index of the row maximum equals the label (xp.argmax, network.py:158).  Both accumulators live on the device
 * (double and 64-bit integer) and are not cleared by the call; labels are TLNN_I32, TLNN_I64 or TLNN_U8.  A label
 * outside [0, V) is reported as TLNN_ERR_INDEX at the next sync, as NumPy's indexing would raise. */
int tlnn_eval_batch_fwd(tlnn_ctx* ctx, const float* probs, long long ldp, const void* labels, int labels_type,
                        long long rows, int cols, double* loss_sum, long long* correct);

/* xp.random.choice(xp.arange(V), p=probs) (demo.ipynb:1530, GPT.generate) for given uniform numbers: row r draws the
 * first index i with cumsum(probs[r])[i] / sum(probs[r]) > uniforms[r] (NumPy's inverse-CDF rule, prefix sums in
 * double); probs (rows, V) float32 with row pitch ldp, uniforms (rows) double in [0, 1) on the device, out int32.
 * The random numbers are the caller's: the library keeps no generator state. */
int tlnn_sample_fwd(tlnn_ctx* ctx, const float* probs, long long ldp, const double* uniforms, int32_t* out,
                    long long rows, int cols);

/* MultiHeadAttention.forward (layers.py:281-307).  x, out: (B, T, d) float32.  wqkv_t (3d, d) and
 * wo_t (d, d) are prepared weights; causal != 0 applies the decoder mask of layers.py:254-256,295-296. */
int tlnn_attention_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* wqkv_t, const float* bqkv,
                       const void* wo_t, const float* bo, float* out, int B, int T, int d, int heads, int causal);

/* TransformerFeedForward.forward (layers.py:369-375); w1_t (4d, d), w2_t (d, 4d) prepared. */
int tlnn_ffn_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* w1_t, const float* b1,
                 const void* w2_t, const float* b2, int act, float* out, long long rows, int d);

/* TransformerBlock.forward (layers.py:463-467) as one call; parameters in the order of layers.py:458. */
typedef struct {
    const float* ln1_gamma; const float* ln1_beta;
    const void*  wqkv_t;    const float* bqkv;
    const void*  wo_t;      const float* bo;
    const float* ln2_gamma; const float* ln2_beta;
    const void*  w1_t;      const float* b1;
    const void*  w2_t;      const float* b2;
} tlnn_block_params;
int tlnn_block_fwd(tlnn_ctx* ctx, int prec, const float* x, const tlnn_block_params* p, int act,
                   float* out, int B, int T, int d, int heads, int causal);

/* GPTEmbedBack.forward (transformer_adapters.py:174-177) / Dense head: logits = x @ table^T (+ bias).
 * `logits` (rows, vocab) float32 may be NULL when only tokens are wanted; `tokens` (rows) int32 may be NULL.
 * With tokens != NULL the arg-max over the vocabulary is taken inside the GEMM epilogue. */
int tlnn_logits_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* table_t, const float* bias,
                    float* logits, int32_t* tokens, long long rows, int d, int vocab);

/* A final LayerNorm followed by the head in one call (demo.ipynb:1497-1498): the normalised rows go
 * straight to the GEMM operand type without a float32 round trip. */
int tlnn_norm_logits_fwd(tlnn_ctx* ctx, int prec, const float* x, const float* gamma, const float* beta,
                         const void* table_t, const float* bias, float* logits, int32_t* tokens,
                         long long rows, int d, int vocab);

/* Arg-max head for callers that must not allocate.  No counterpart in the reference: it computes what
 * tlnn_logits_fwd(ctx, prec, x, table_t, bias, NULL, tokens, rows, d, vocab) computes, but takes its intermediates
 * (the converted operand rows and the per-tile arg-max candidates) from a TLNN_NOALLOC_SCRATCH_BYTES array built into
 * the library image, so the call never reaches cudaMalloc, cudaFree, the context's scratch arena or any other
 * allocating routine.  It is meant for hosts where allocation is off the table at call time: a serving process whose
 * own memory manager has claimed the whole GPU up front and hands out sub-buffers (x and tokens come from there), or a
 * latency-critical loop that cannot afford the device-wide stall an allocation may cause.
 *  - Every GPU that loads libtlnn.so keeps the array resident until the process exits.
 *  - Shapes whose intermediates exceed the array are refused with TLNN_ERR_VALUE and a message that states the need.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress), and the first call for a
 *    given precision and shape class sets the attributes of the kernel variant it picks; make one call per precision
 *    and shape you will use during set-up, before any stream capture begins.  The address is cached in a plain
 *    per-device table written without a lock: two threads that race through their first call store the same value.
 *  - Keep per-class profiling (tlnn_prof_classes) off around this call: with it on, every launch takes CUDA events
 *    from a pool that creates new ones when it is empty.
 *  - All calls on a device share the one array and leave their data in it; nothing in it has to be zero on entry.
 *    Two calls whose kernels can overlap on the GPU (different contexts/streams on one device) race: serialise them. */
#define TLNN_NOALLOC_SCRATCH_BYTES (16u << 20)
int tlnn_logits_tokens_noalloc(tlnn_ctx* ctx, int prec, const float* x, const void* table_t, const float* bias,
                               int32_t* tokens, long long rows, int d, int vocab);

/* VitProjector.forward (transformer_adapters.py:34-55).  img (B, C, H, W) float32; proj_t prepared
 * (d, ph*pw*C); cls_reg (1+regs, d); pos (1+regs+N, d); out (B, 1+regs+N, d). */
int tlnn_vit_project_fwd(tlnn_ctx* ctx, int prec, const float* img, const void* proj_t, const float* cls_reg,
                         const float* pos, float* out, int B, int C, int H, int W, int ph, int pw, int d, int regs);

/* VitMLPHead.forward (transformer_adapters.py:89-95): x[:,0,:] @ W + b.  x (B, T, d); w_t prepared (n_out, d). */
int tlnn_vit_head_fwd(tlnn_ctx* ctx, int prec, const float* x, const void* w_t, const float* bias,
                      float* out, int B, int T, int d, int n_out);

/* ---- whole-model prefill -------------------------------------------------- */
/* Network.predict (network.py:33-39) for the GPT recipe: embedding, L blocks, final LayerNorm, head.
 * One call enqueues the whole forward.  `blocks` points to `layers` parameter structs.  head_bias may be
 * NULL (tied head).  logits and tokens as in tlnn_logits_fwd. */
typedef struct {
    int vocab, context, d, heads, layers, act, prec;
    const float* tok_table; const float* pos_table;
    const tlnn_block_params* blocks;
    const float* lnf_gamma; const float* lnf_beta;
    const void* head_t; const float* head_bias;
} tlnn_gpt_model;
int tlnn_gpt_prefill(tlnn_ctx* ctx, const tlnn_gpt_model* m, const void* ids, int ids_type, int B, int T,
                     float* logits, int32_t* tokens);

/* Network.predict (network.py:33-39) for the ViT recipe of the notebook (demo.ipynb, the ViT cell): VitProjector,
 * L encoder blocks, final LayerNorm, VitMLPHead.  One call enqueues the whole forward and writes the class scores
 * out (B, n_out) float32.  img (B, channels, height, width) float32; proj_t, cls_reg and pos as in
 * tlnn_vit_project_fwd; head_t prepared (n_out, d); head_bias (n_out) or NULL.  The final LayerNorm is applied to the
 * class row of every image only - LayerNorm works row by row and VitMLPHead (transformer_adapters.py:89-95) reads no
 * other row - so the scores equal those of the layer-by-layer calls.  A repeated identical call replays a captured
 * CUDA graph, like tlnn_gpt_prefill. */
typedef struct {
    int channels, height, width, patch_h, patch_w, d, heads, layers, act, prec, registers, n_out;
    const void* proj_t; const float* cls_reg; const float* pos;
    const tlnn_block_params* blocks;
    const float* lnf_gamma; const float* lnf_beta;
    const void* head_t; const float* head_bias;
} tlnn_vit_model;
int tlnn_vit_forward(tlnn_ctx* ctx, const tlnn_vit_model* m, const float* img, int B, float* out);

/* ---- greedy decode with a per-layer KV cache ------------------------------- */
/* Replaces the generation loop of demo.ipynb:1520-1535 (which re-runs the whole window for every token)
 * with arg-max sampling.  `tlnn_decode_begin` runs the prompts (B, T0) through the model, fills the cache
 * and writes the first new token per row; each `tlnn_decode_step` feeds the previous tokens and writes the
 * next ones (device int32, B).  max_len bounds prompt + new tokens and must not exceed the model context. */
typedef struct tlnn_decoder tlnn_decoder;
int tlnn_decode_begin(tlnn_ctx* ctx, const tlnn_gpt_model* m, const void* ids, int ids_type, int B, int T0,
                      int max_len, int32_t* first_tokens, tlnn_decoder** out);
int tlnn_decode_step(tlnn_decoder* dec, const int32_t* prev_tokens, int32_t* next_tokens);
/* Runs n_steps steps back to back; tokens_out is (B, n_steps) int32 row-major on the device, column 0
 * being the token that follows `prev_tokens`. */
int tlnn_decode_run(tlnn_decoder* dec, const int32_t* prev_tokens, int n_steps, int32_t* tokens_out);
/* Sampling forms (demo.ipynb:1530, `random.choice(arange(V), p=probs)` after the model's SoftMax layer): the token of
 * every row is drawn from softmax(logits / temperature) with the inverse-CDF rule of tlnn_sample_fwd.  `uniforms` is
 * HOST memory: (B) for the first token, (n_steps, B) row-major for a run.  tlnn_decode_first_sampled replaces the
 * arg-max first token of tlnn_decode_begin and must be called right after it. */
int tlnn_decode_first_sampled(tlnn_decoder* dec, float temperature, const double* uniforms, int32_t* first_tokens);
int tlnn_decode_run_sampled(tlnn_decoder* dec, const int32_t* prev_tokens, int n_steps, float temperature,
                            const double* uniforms, int32_t* tokens_out);
int tlnn_decode_end(tlnn_decoder* dec);

/* ---- multi-GPU: batch-sharded replicas ------------------------------------ */
/* The reference is single-device: Network.predict (network.py:33-39) runs the whole batch in one process.  Eval-mode
 * rows are independent (LayerNorm is per row, layers.py:419-420; attention is per sample, layers.py:293-304), so N
 * processes, one per GPU with its own context and a full copy of the weights, each run a contiguous slice of the batch
 * rows and exchange only results.  A communicator wraps NCCL (bound at run time: TLNN_NCCL_LIB, else libnccl.so.2;
 * a process without NCCL can use everything else in this header).
 *   tlnn_comm_unique_id  rank 0 creates TLNN_COMM_ID_BYTES opaque bytes and hands them to the other ranks by whatever
 *                        means the launcher offers (a file, a socket, MPI, a key-value store).
 *   tlnn_comm_init       every rank calls it with the same bytes, its rank and the world size; collective: returns
 *                        once all ranks have joined.  TLNN_COMM_FAIL_INIT=1 makes it fail before any GPU or network
 *                        work (host-side failure injection for tests).
 *   tlnn_allgather_tokens / tlnn_allgather_logits
 *                        `local` holds this rank's n_local results (arg-max tokens of its rows: xp.argmax,
 *                        network.py:135,158; or logits rows), `all` receives every rank's block in rank order.  counts
 *                        (host array of `world` entries, may be NULL when every rank passes the same n_local) allows
 *                        ragged shards.  Enqueued on the context's compute stream, after the kernels that write
 *                        `local`; `all` is valid after the next tlnn_sync / tlnn_d2h.
 *   tlnn_comm_barrier    a one-int all-reduce followed by tlnn_sync: every rank has finished its enqueued work.
 * Calls on a communicator must be made in the same order on every rank. */
#define TLNN_COMM_ID_BYTES 128
typedef struct tlnn_comm tlnn_comm;
int tlnn_comm_nccl_version(int* version);
int tlnn_comm_unique_id(void* id_bytes);
int tlnn_comm_init(tlnn_ctx* ctx, const void* id_bytes, int rank, int world, tlnn_comm** out);
int tlnn_comm_rank(tlnn_comm* comm, int* rank, int* world);
int tlnn_allgather_tokens(tlnn_comm* comm, const int32_t* local, int32_t* all, long long n_local, const long long* counts);
int tlnn_allgather_logits(tlnn_comm* comm, const float* local, float* all, long long n_local, const long long* counts);
int tlnn_comm_barrier(tlnn_comm* comm);
int tlnn_comm_destroy(tlnn_comm* comm);

/* ---- double-buffered host feed ------------------------------------------- */
/* The reference uploads every batch synchronously (`xp.array(batch)`, network.py:117,152).  A feeder owns two pinned
 * host buffers, two device buffers and a copy stream: while the compute stream works on the batch in one slot, the
 * next batch is written into the other slot's host buffer and copied.  Per batch: write into tlnn_feed_host(slot),
 * tlnn_feed_submit(slot, bytes) (asynchronous copy; waits, on the copy stream, until the compute stream has released
 * the slot's device buffer), later tlnn_feed_acquire(slot, &dev) (the compute stream waits for the copy), enqueue the
 * work that reads dev, tlnn_feed_release(slot).  Before rewriting a slot's HOST buffer call tlnn_feed_host_wait(slot),
 * which blocks the calling thread until that slot's last copy has left the buffer. */
typedef struct tlnn_feeder tlnn_feeder;
int tlnn_feed_create(tlnn_ctx* ctx, size_t bytes_per_batch, tlnn_feeder** out);
int tlnn_feed_host(tlnn_feeder* f, int slot, void** host);
int tlnn_feed_host_wait(tlnn_feeder* f, int slot);
int tlnn_feed_submit(tlnn_feeder* f, int slot, size_t bytes);
int tlnn_feed_acquire(tlnn_feeder* f, int slot, void** dev);
int tlnn_feed_release(tlnn_feeder* f, int slot);
int tlnn_feed_destroy(tlnn_feeder* f);

/* ---- failure handling self-test ------------------------------------------ */
/* No counterpart in the reference.  Every device-side wait of the library (TMA, tensor-core and hand-over barriers)
 * goes through one bounded-wait routine; this call launches a one-thread kernel that waits, through that routine, on
 * a barrier nothing arrives at, with a limit of limit_ms (1..1000).  The kernel returns normally; the next
 * tlnn_sync / tlnn_check reports TLNN_ERR_TIMEOUT, after which the context is clean and usable again. */
int tlnn_selftest_wait(tlnn_ctx* ctx, int limit_ms);

/* ---- memory-safety checks for test runs ------------------------------------------ */
/* No counterpart in the reference (NumPy checks every index; a CUDA kernel does not).  Two aids stand in for a memory
 * checker:
 *  - canaries: after tlnn_debug_canaries(ctx, 1) every tlnn_alloc places 256 bytes of a known pattern behind the block;
 *    tlnn_free verifies them (this waits for the stream) and tlnn_debug_check verifies every live guarded block,
 *    returning the number of blocks found overwritten so far and the number of live guarded blocks;
 *  - the debug build of the library (`python -m torchless_nn_b200.build --debug` -> libtlnn_debug.so, loaded by the
 *    Python package when TLNN_DEBUG=1): the stores of the GEMM, attention and decode kernels check their offset against
 *    the output's extent, record a violation as TLNN_ERR_INDEX (site 9xx, offending offset) and skip the store. */
int tlnn_debug_canaries(tlnn_ctx* ctx, int enable);
int tlnn_debug_check(tlnn_ctx* ctx, long long* corrupted, long long* guarded);

/* ---- profiling -------------------------------------------------------------- */
/* CUDA-event timing of everything enqueued between begin and end on the compute stream (milliseconds). */
int tlnn_prof_begin(tlnn_ctx* ctx);
int tlnn_prof_end(tlnn_ctx* ctx, float* ms);
/* Per-kernel-class timing: when enabled every launch is bracketed by events (this serialises launches).
 * tlnn_prof_table fills up to `cap` rows of (name, launches, total ms) and returns the row count. */
typedef struct { char name[48]; long long launches; double ms; } tlnn_prof_row;
int tlnn_prof_classes(tlnn_ctx* ctx, int enable);
int tlnn_prof_table(tlnn_ctx* ctx, tlnn_prof_row* rows, int cap);

#ifdef __cplusplus
}
#endif
#endif /* TLNN_H */
