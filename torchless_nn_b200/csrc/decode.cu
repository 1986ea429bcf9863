// Greedy decode with a per-layer KV cache.
//
// The reference generates by re-running the whole window for every new token (demo.ipynb:1526-1533).  Here the prompt
// is run once (filling a (B, max_len, d) key and value cache per layer) and every further token costs one pass with a
// single row per sequence: LayerNorm -> QKV GEMM -> append the row's K, V -> single-query attention over the cache ->
// output GEMM + residual -> LayerNorm -> GEMM + activation -> GEMM + residual, then the final LayerNorm and the head
// GEMM with fused arg-max.  The step is weight-streaming (HBM) bound.  The current length lives in device memory and
// every kernel of a step reads it from there, so the launch sequence of a step does not depend on the position.
#include "common.cuh"
#include "decode_fused.cuh"
#include <cstdlib>

namespace {

constexpr int kWarp = 32;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float round_tf32(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x00000fffu + ((u >> 13) & 1u);
    u &= 0xffffe000u;
    return __uint_as_float(u);
}

// qkv (B*T, 3d) -> kcache / vcache (B, heads, cache_len, hd), positions [0, T), 16 bytes per thread and copy
template <typename E>
__global__ void kv_store_kernel(const E* __restrict__ qkv, E* __restrict__ kc, E* __restrict__ vc, int B, int T, int d,
                                int hd, int cache_len) {
    constexpr int PER = 16 / sizeof(E);            // elements per 16-byte unit (hd and d are multiples of it)
    const long long total = (long long)B * T * (d / PER);
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int H = d / hd, upr = d / PER;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = (int)(i % upr) * PER;
        const long long row = i / upr;
        const int t = (int)(row % T);
        const long long b = row / T;
        const int h = c / hd;
        const long long dst = ((b * H + h) * cache_len + t) * hd + (c - h * hd);
        *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(qkv + row * 3 * d + d + c);
        *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(qkv + row * 3 * d + 2 * d + c);
    }
}

// x[b, :] = table[token[b], :] + pos_table[*len, :]
__global__ void decode_embed_kernel(const int32_t* __restrict__ tokens, const float* __restrict__ table,
                                    const float* __restrict__ pos, const int* __restrict__ len, float* __restrict__ out,
                                    int B, int d, int vocab, tlnn_dev_err* err) {
    tl_grid_dependency_sync();
    const int b = blockIdx.x;
    long long id = tokens[b];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) tl_dev_fail(err, TLNN_ERR_INDEX, 2, id);
        id = 0;
    }
    const int t = *len;
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[(long long)b * d + c] = __fadd_rn(table[id * d + c], pos[(long long)t * d + c]);
}

// Append the new row's K, V (from the packed (B, 3d) projection) at position *len, then attend the row's query over
// cache rows [0, *len].  One CTA per (sequence, head); a group of HD*sizeof(E)/16 threads covers one key row with
// 16-byte loads and the DA_THREADS threads cover DA_THREADS / group keys at a time.  One pass over the cache: a thread
// requests the key rows AND the value rows of four keys before it uses the first, and every group keeps its own running
// maximum, sum and weighted row (online softmax); the groups are merged through shared memory at the end.  Nothing in
// shared memory grows with the cache, so its length is bounded by the context only.  Measured on 64 sequences x 12
// heads of 64 at 128-383 cached positions: one 16-byte load in flight per thread is 20 % slower per decode step, two
// keys per round 9 % slower, eight 1.5 % slower; a two-pass form with a score buffer runs at the same speed.
constexpr int DA_THREADS = 128;
template <typename E, int HD>
__global__ void __launch_bounds__(DA_THREADS)
decode_attention_kernel(const E* __restrict__ qkv, E* __restrict__ kc, E* __restrict__ vc, E* __restrict__ out,
                        const int* __restrict__ len_ptr, int H, int cache_len, float inv_sqrt_hd, int round_out) {
    constexpr int PER = 16 / sizeof(E);            // elements per 16-byte load
    constexpr int TPR = HD / PER;                  // threads per key row
    constexpr int KPP = DA_THREADS / TPR;          // keys per round of one load each
    constexpr int UN = 4;                          // keys per thread and round
    __shared__ float gm[KPP], gl[KPP];             // per group: running maximum (scaled scores) and sum
    __shared__ float part[DA_THREADS * PER];       // KPP x HD weighted rows
    const int d = H * HD;
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    // a layer's cache is laid out (sequence, head, position, HD): the rows one CTA reads are contiguous in memory
    E* kbase = kc + ((long long)(b * H + h) * cache_len) * HD;
    E* vbase = vc + ((long long)(b * H + h) * cache_len) * HD;
    const int tid = threadIdx.x;
    tl_grid_dependency_sync();
    const int pos = *len_ptr;
    const int n = pos + 1;
    const E* row = qkv + (long long)b * 3 * d;
    const int sub = tid % TPR, grp = tid / TPR;    // 16-byte unit inside the row, key residue
    // this thread's slice of the query, and the append of the new row (first TPR threads, 16 bytes each)
    float q[PER];
    {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + h * HD + sub * PER);
        const E* e = reinterpret_cast<const E*>(&raw);
#pragma unroll
        for (int i = 0; i < PER; i++) q[i] = to_f<E>(e[i]);
        if (grp == 0) {
            *reinterpret_cast<uint4*>(kbase + (long long)pos * HD + sub * PER) = *reinterpret_cast<const uint4*>(row + d + h * HD + sub * PER);
            *reinterpret_cast<uint4*>(vbase + (long long)pos * HD + sub * PER) = *reinterpret_cast<const uint4*>(row + 2 * d + h * HD + sub * PER);
        }
    }
    __syncthreads();
    float m_run = -INFINITY, l_run = 0.f;
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) acc[i] = 0.f;
    for (int k0 = 0; k0 < n; k0 += KPP * UN) {
        uint4 kr[UN], vr[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int k = k0 + u * KPP + grp;
            if (k < n) {
                kr[u] = *reinterpret_cast<const uint4*>(kbase + (long long)k * HD + sub * PER);
                vr[u] = *reinterpret_cast<const uint4*>(vbase + (long long)k * HD + sub * PER);
            } else {
                kr[u] = make_uint4(0u, 0u, 0u, 0u);
                vr[u] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        // scores: partial dot products combined by shuffles inside the group (every thread of a group ends with the sum)
        float sc[UN];
        float mb = -INFINITY;
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int k = k0 + u * KPP + grp;
            const E* e = reinterpret_cast<const E*>(&kr[u]);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i++) s = fmaf(q[i], to_f<E>(e[i]), s);
#pragma unroll
            for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            sc[u] = k < n ? s * inv_sqrt_hd : -INFINITY;
            mb = fmaxf(mb, sc[u]);
        }
        const float m_new = fmaxf(m_run, mb);
        if (m_new > -INFINITY) {                   // the same for all threads of a group
            const float alpha = __expf(m_run - m_new);          // 0 while m_run is still -inf
            l_run *= alpha;
#pragma unroll
            for (int i = 0; i < PER; i++) acc[i] *= alpha;
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const float p = __expf(sc[u] - m_new);          // 0 for a key beyond the cache
                l_run += p;
                const E* e = reinterpret_cast<const E*>(&vr[u]);
#pragma unroll
                for (int i = 0; i < PER; i++) acc[i] = fmaf(p, to_f<E>(e[i]), acc[i]);
            }
            m_run = m_new;
        }
    }
    if (sub == 0) { gm[grp] = m_run; gl[grp] = l_run; }
#pragma unroll
    for (int i = 0; i < PER; i++) part[(grp * TPR + sub) * PER + i] = acc[i];
    __syncthreads();
    if (tid < HD) {
        float mx = gm[0];
#pragma unroll
        for (int g = 1; g < KPP; g++) mx = fmaxf(mx, gm[g]);
        float o = 0.f, den = 0.f;
#pragma unroll 4
        for (int g = 0; g < KPP; g++) {
            const float w = __expf(gm[g] - mx);               // 0 for a group that saw no key
            den = fmaf(w, gl[g], den);
            o = fmaf(w, part[g * HD + tid], o);
        }
        o /= den;
        if (round_out) o = round_tf32(o);
        out[(long long)b * d + h * HD + tid] = from_f<E>(o);
    }
}

struct decode_sink {          // lives in device memory so that a captured step does not depend on call arguments
    int32_t* tokens_out;      // (B, n_cols) or null
    int n_cols;
    int pad;
};

__global__ void decode_advance_kernel(const int32_t* __restrict__ next, int32_t* __restrict__ cur,
                                      const decode_sink* __restrict__ sink, int* len, int* step, int B) {
    tl_grid_dependency_sync();
    const int s = *step;
    int32_t* tokens_out = sink->tokens_out;
    const int n_cols = sink->n_cols;
    __syncthreads();
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const int32_t t = next[b];
        cur[b] = t;
        if (tokens_out) tokens_out[(long long)b * n_cols + s] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) { *len += 1; *step = s + 1; }
}

inline size_t esize(int prec) { return prec == TLNN_PREC_BF16 ? 2 : 4; }
inline int okind(int prec) { return prec == TLNN_PREC_BF16 ? TL_OUT_BF16 : TL_OUT_TF32; }

}  // namespace

int tl_kv_store(tlnn_ctx* ctx, int prec, const void* qkv, void* kcache, void* vcache, int B, int T, int d, int heads, int cache_len) {
    const size_t n = (size_t)B * T * d / (prec == TLNN_PREC_BF16 ? 8 : 4);     // 16-byte units
    if (n == 0) return TLNN_OK;
    int grid = (int)((n + 255) / 256);
    if (grid > ctx->sm_count * 16) grid = ctx->sm_count * 16;
    if (prec == TLNN_PREC_BF16)
        TL_LAUNCH(ctx, "kv_store", kv_store_kernel<__nv_bfloat16><<<grid, 256, 0, ctx->stream>>>(
                      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, B, T, d, d / heads, cache_len));
    else
        TL_LAUNCH(ctx, "kv_store", kv_store_kernel<float><<<grid, 256, 0, ctx->stream>>>(
                      (const float*)qkv, (float*)kcache, (float*)vcache, B, T, d, d / heads, cache_len));
    return TLNN_OK;
}

struct tlnn_decoder {
    tlnn_ctx* ctx = nullptr;
    tlnn_gpt_model m;                            // copy of the description (pointers stay owned by the caller)
    std::vector<tlnn_block_params> blocks;
    int B = 0, max_len = 0, host_len = 0;
    char* mem = nullptr;                         // one allocation for caches and per-step buffers
    void *kcache = nullptr, *vcache = nullptr;   // (layers, B, max_len, d)
    float *x0 = nullptr, *x1 = nullptr, *y = nullptr;
    void *a = nullptr, *qkv = nullptr, *att = nullptr, *hid = nullptr;
    float2* parts = nullptr;
    int32_t *cur = nullptr, *next = nullptr;
    int *d_len = nullptr, *d_step = nullptr;
    decode_sink* d_sink = nullptr;
    int n_parts = 0;
    cudaGraphExec_t step_graph = nullptr;        // one captured step, replayed by tlnn_decode_run
    // persistent one-launch-per-run kernel (bf16 arg-max decode, see decode_fused.cu); null pointers when it does not apply
    tl_decode_fused_plan_t fused;
    char* fused_mem = nullptr;
    char* fused_pack = nullptr;                  // the model's GEMM weights at the row pitch the kernel's shared-memory slots use
    df_params fused_params = {};
    long long launches_per_step = 0;
    // sampling (allocated by the first sampled call): logits and probabilities (B, vocab), uniform numbers (max_len, B)
    char* sample_mem = nullptr;
    float *logits = nullptr, *probs = nullptr;
    double* uniforms = nullptr;
    cudaGraphExec_t sample_graph = nullptr;      // one captured sampling step for sample_temperature
    float sample_temperature = 0.f;
    long long sample_launches_per_step = 0;
};

namespace {

int launch_decode_attention(tlnn_decoder* dec, int layer) {
    tlnn_ctx* ctx = dec->ctx;
    const int d = dec->m.d, H = dec->m.heads, hd = d / H, B = dec->B;
    const size_t layer_elems = (size_t)B * dec->max_len * d;
    const float inv = 1.f / sqrtf((float)hd);
    const size_t smem = 0;
    const int round_out = dec->m.prec == TLNN_PREC_TF32;
#define DA_CASE(E, HDV)                                                                                              \
    TL_LAUNCH(ctx, "decode_attention", tl_launch_kernel(ctx, decode_attention_kernel<E, HDV>, dim3(B * H), dim3(DA_THREADS), smem, \
                  (const E*)dec->qkv, (E*)dec->kcache + layer * layer_elems, (E*)dec->vcache + layer * layer_elems, \
                  (E*)dec->att, dec->d_len, H, dec->max_len, inv, round_out))
    if (dec->m.prec == TLNN_PREC_BF16) {
        if (hd == 32) DA_CASE(__nv_bfloat16, 32);
        else if (hd == 64) DA_CASE(__nv_bfloat16, 64);
        else DA_CASE(__nv_bfloat16, 128);
    } else {
        if (hd == 32) DA_CASE(float, 32);
        else if (hd == 64) DA_CASE(float, 64);
        else DA_CASE(float, 128);
    }
#undef DA_CASE
    return TLNN_OK;
}

// One token for every sequence: cur tokens at position *d_len -> next tokens; advances the device counters.
int decode_one(tlnn_decoder* dec, bool sample = false, float temperature = 1.f) {
    tlnn_ctx* ctx = dec->ctx;
    const tlnn_gpt_model& m = dec->m;
    const int B = dec->B, d = m.d, prec = m.prec, kind = okind(prec);
    // Inside a step every kernel may be launched while its predecessor still runs (each starts with a grid-dependency
    // wait): a step is 89 dependent kernels of 5-15 us, and launch latency is a large part of it.  TLNN_PDL=0 disables.
    static const bool pdl_allowed = !(getenv("TLNN_PDL") && strcmp(getenv("TLNN_PDL"), "0") == 0);
    struct pdl_scope {
        tlnn_ctx* c; bool old;
        pdl_scope(tlnn_ctx* cc, bool on) : c(cc), old(cc->pdl) { c->pdl = on; }
        ~pdl_scope() { c->pdl = old; }
    } scope(ctx, pdl_allowed && !ctx->prof_classes);
    TL_LAUNCH(ctx, "decode_embed", tl_launch_kernel(ctx, decode_embed_kernel, dim3(B), dim3(128), 0, dec->cur, m.tok_table, m.pos_table,
                                                    dec->d_len, dec->x0, B, d, m.vocab, ctx->d_err));
    float* x = dec->x0;
    float* xn = dec->x1;
    for (int l = 0; l < m.layers; l++) {
        const tlnn_block_params& p = dec->blocks[l];
        TL_TRY(tl_layernorm(ctx, x, p.ln1_gamma, p.ln1_beta, 1e-5f, dec->a, kind, B, d));
        tl_gemm_epilogue e1;
        e1.bias = p.bqkv; e1.out = dec->qkv; e1.ldo = 3 * d; e1.out_kind = prec == TLNN_PREC_BF16 ? TL_OUT_BF16 : TL_OUT_F32;
        TL_TRY(tl_gemm(ctx, prec, dec->a, d, p.wqkv_t, d, B, 3 * d, d, e1));
        TL_TRY(launch_decode_attention(dec, l));
        tl_gemm_epilogue e2;
        // bf16 mode keeps the residual stream in place: x += attention projection, x += feed-forward (the GEMM adds its
        // tiles into x, split over K ranges when there are few tiles)
        float* y = prec == TLNN_PREC_BF16 ? x : dec->y;
        e2.bias = p.bo; e2.residual = x; e2.ldr = d; e2.out = y; e2.ldo = d; e2.out_kind = TL_OUT_F32;
        TL_TRY(tl_gemm(ctx, prec, dec->att, d, p.wo_t, d, B, d, d, e2));
        TL_TRY(tl_layernorm(ctx, y, p.ln2_gamma, p.ln2_beta, 1e-5f, dec->a, kind, B, d));
        tl_gemm_epilogue e3;
        e3.bias = p.b1; e3.act = m.act; e3.accurate_math = prec == TLNN_PREC_TF32; e3.out = dec->hid; e3.ldo = 4 * d; e3.out_kind = kind;
        TL_TRY(tl_gemm(ctx, prec, dec->a, d, p.w1_t, d, B, 4 * d, d, e3));
        tl_gemm_epilogue e4;
        float* out = prec == TLNN_PREC_BF16 ? x : xn;
        e4.bias = p.b2; e4.residual = y; e4.ldr = d; e4.out = out; e4.ldo = d; e4.out_kind = TL_OUT_F32;
        TL_TRY(tl_gemm(ctx, prec, dec->hid, 4 * d, p.w2_t, 4 * d, B, d, 4 * d, e4));
        if (prec != TLNN_PREC_BF16) { float* t = x; x = xn; xn = t; }
    }
    TL_TRY(tl_layernorm(ctx, x, m.lnf_gamma, m.lnf_beta, 1e-5f, dec->a, kind, B, d));
    tl_gemm_epilogue eh;
    eh.bias = m.head_bias;
    if (sample) {
        // logits -> softmax(logits / temperature) -> draw with this step's uniform numbers
        eh.out = dec->logits; eh.ldo = m.vocab; eh.out_kind = TL_OUT_F32;
        TL_TRY(tl_gemm(ctx, prec, dec->a, d, m.head_t, d, B, m.vocab, d, eh));
        TL_TRY(tlnn_softmax_fwd(ctx, dec->logits, dec->probs, B, m.vocab, temperature));
        TL_TRY(tl_sample(ctx, dec->probs, m.vocab, dec->uniforms, dec->d_step, dec->next, B, m.vocab));
    } else {
        eh.argmax_partials = dec->parts;
        TL_TRY(tl_gemm(ctx, prec, dec->a, d, m.head_t, d, B, m.vocab, d, eh));
        TL_TRY(tl_argmax_partials(ctx, dec->parts, dec->n_parts, dec->next, B));
    }
    TL_LAUNCH(ctx, "decode_advance", tl_launch_kernel(ctx, decode_advance_kernel, dim3(1), dim3(256), 0, dec->next, dec->cur, dec->d_sink,
                                                      dec->d_len, dec->d_step, B));
    return TLNN_OK;
}

// n_steps greedy steps in one launch; tokens_out is (B, n_cols) with column s the token of step s.
int run_fused(tlnn_decoder* dec, int n_steps, int32_t* tokens_out, int n_cols) {
    df_params p = dec->fused_params;
    int done = 0;
    while (done < n_steps) {
        const int chunk = n_steps - done < 2048 ? n_steps - done : 2048;       // keeps the barrier counter far from wrapping
        p.n_steps = chunk;
        p.tokens_out = tokens_out + done;
        p.n_cols = n_cols;
        TL_TRY(tl_decode_fused_launch(dec->ctx, dec->fused, p));
        done += chunk;
    }
    return TLNN_OK;
}

int set_sink(tlnn_decoder* dec, int32_t* tokens_out, int n_cols) {
    decode_sink h;
    h.tokens_out = tokens_out; h.n_cols = n_cols; h.pad = 0;
    // a synchronous copy from a stack object; the stream is idle or ordered behind it either way
    TL_CUDA(cudaMemcpyAsync(dec->d_sink, &h, sizeof(h), cudaMemcpyHostToDevice, dec->ctx->stream));
    TL_CUDA(cudaStreamSynchronize(dec->ctx->stream));
    return TLNN_OK;
}

}  // namespace

extern "C" int tlnn_decode_begin(tlnn_ctx* ctx, const tlnn_gpt_model* m, const void* ids, int ids_type, int B, int T0,
                                 int max_len, int32_t* first_tokens, tlnn_decoder** out) {
    TL_NOTNULL(ctx); TL_NOTNULL(m); TL_NOTNULL(ids); TL_NOTNULL(first_tokens); TL_NOTNULL(out);
    TL_NOTNULL(m->tok_table); TL_NOTNULL(m->pos_table); TL_NOTNULL(m->lnf_gamma); TL_NOTNULL(m->lnf_beta); TL_NOTNULL(m->head_t);
    TL_REQUIRE(m->layers == 0 || m->blocks != nullptr, "decode: the model has layers but no block parameters");
    TL_REQUIRE(m->prec == TLNN_PREC_BF16 || m->prec == TLNN_PREC_TF32, "unknown precision %d", m->prec);
    TL_REQUIRE(B > 0 && B <= 1024 && T0 > 0, "decode: bad batch %d or prompt length %d", B, T0);
    TL_REQUIRE(max_len > T0 && max_len <= m->context, "decode: prompt %d + new tokens must fit max_len %d <= context %d", T0, max_len, m->context);
    TL_REQUIRE(m->d > 0 && m->heads > 0 && m->d % m->heads == 0 && m->d % 8 == 0, "decode: bad width %d / heads %d", m->d, m->heads);
    const int hd = m->d / m->heads;
    TL_REQUIRE(hd == 32 || hd == 64 || hd == 128, "decode: head dimension %d is not supported (32, 64 or 128)", hd);
    TL_REQUIRE((long long)B * m->heads <= 65535, "decode: batch x heads exceeds 65535");
    TL_REQUIRE(ids_type == TLNN_I32 || ids_type == TLNN_I64 || ids_type == TLNN_U8, "token ids must be int32, int64 or uint8");
    TL_CUDA(cudaSetDevice(ctx->device));

    tlnn_decoder* dec = new tlnn_decoder();
    dec->ctx = ctx;
    dec->m = *m;
    dec->blocks.assign(m->blocks, m->blocks + m->layers);
    dec->m.blocks = dec->blocks.data();
    dec->B = B;
    dec->max_len = max_len;
    const int d = m->d, prec = m->prec;
    const size_t es = esize(prec);
    dec->n_parts = tl_gemm_argmax_parts(prec, B, m->vocab, ctx->sm_count);
    // carve one allocation
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) & ~size_t(255); return o; };
    const size_t cache_bytes = (size_t)m->layers * B * max_len * d * es;
    const size_t o_k = take(cache_bytes), o_v = take(cache_bytes);
    const size_t o_x0 = take((size_t)B * d * 4), o_x1 = take((size_t)B * d * 4), o_y = take((size_t)B * d * 4);
    const size_t o_a = take((size_t)B * d * es), o_qkv = take((size_t)B * 3 * d * es), o_att = take((size_t)B * d * es);
    const size_t o_hid = take((size_t)B * 4 * d * es), o_parts = take((size_t)B * dec->n_parts * sizeof(float2));
    const size_t o_cur = take((size_t)B * 4), o_next = take((size_t)B * 4), o_cnt = take(16), o_sink = take(sizeof(decode_sink));
    // the decoder's buffers come from the context's stream-ordered pool (freed blocks stay cached there, so a caller that
    // decodes batch after batch does not pay the driver for 100s of MB of allocations each time)
    cudaError_t e = cudaMallocAsync((void**)&dec->mem, off, ctx->stream);
    if (e != cudaSuccess) { delete dec; return tl_cuda_fail(e, "cudaMalloc(decoder)", __FILE__, __LINE__); }
    char* base = dec->mem;
    dec->kcache = base + o_k; dec->vcache = base + o_v;
    dec->x0 = (float*)(base + o_x0); dec->x1 = (float*)(base + o_x1); dec->y = (float*)(base + o_y);
    dec->a = base + o_a; dec->qkv = base + o_qkv; dec->att = base + o_att; dec->hid = base + o_hid;
    dec->parts = (float2*)(base + o_parts);
    dec->cur = (int32_t*)(base + o_cur); dec->next = (int32_t*)(base + o_next);
    dec->d_len = (int*)(base + o_cnt); dec->d_step = dec->d_len + 1;
    dec->d_sink = (decode_sink*)(base + o_sink);

    // ---- the persistent decode kernel, where it applies: its tables and exchange buffers
    {
        // the plan is made twice: once to learn the size of the packed weight copy, once with the allocation
        int st = tl_decode_fused_plan(ctx, dec->m, dec->blocks.data(), B, max_len, nullptr, true, &dec->fused);
        if (st == TLNN_OK && dec->fused.ok) {
            bool packed = cudaMallocAsync((void**)&dec->fused_pack, dec->fused.pack_bytes, ctx->stream) == cudaSuccess;
            if (!packed) { cudaGetLastError(); dec->fused_pack = nullptr; }
            st = tl_decode_fused_plan(ctx, dec->m, dec->blocks.data(), B, max_len, dec->fused_pack, packed, &dec->fused);
            for (const df_pack_job& j : dec->fused.pack_jobs) {
                if (cudaMemcpy2DAsync(dec->fused_pack + j.dst_off, (size_t)(d + 8) * 2, j.src, j.src_pitch, j.width, j.rows,
                                      cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess) {
                    cudaGetLastError();
                    dec->fused.ok = false;
                    break;
                }
            }
        }
        if (st == TLNN_OK && dec->fused.ok) {
            const tl_decode_fused_plan_t& pl = dec->fused;
            size_t o2 = 0;
            auto take2 = [&](size_t bytes) { size_t o = o2; o2 += (bytes + 255) & ~size_t(255); return o; };
            const size_t f_items = take2(sizeof(df_item) * pl.items.size());
            const size_t f_counts = take2(sizeof(int) * pl.counts.size()), f_cand = take2(sizeof(float2) * 64 * pl.grid);
            const size_t f_bar = take2(4096);
            cudaError_t fe = cudaMallocAsync((void**)&dec->fused_mem, o2, ctx->stream);
            if (fe != cudaSuccess) { cudaGetLastError(); dec->fused.ok = false; }
            else {
                char* fb = dec->fused_mem;
                fe = cudaMemcpyAsync(fb + f_items, pl.items.data(), sizeof(df_item) * pl.items.size(), cudaMemcpyHostToDevice, ctx->stream);
                if (fe == cudaSuccess) fe = cudaMemcpyAsync(fb + f_counts, pl.counts.data(), sizeof(int) * pl.counts.size(), cudaMemcpyHostToDevice, ctx->stream);
                if (fe != cudaSuccess) { cudaGetLastError(); dec->fused.ok = false; }    // the plan's vectors outlive the copies: they belong to the decoder
                df_params& fp = dec->fused_params;
                fp.B = B; fp.d = d; fp.H = m->heads; fp.L = m->layers; fp.V = m->vocab; fp.max_len = max_len; fp.act = m->act;
                fp.slot_bytes = pl.slot_bytes; fp.items_pitch = pl.items_pitch; fp.a_region = pl.a_region; fp.att_ck = pl.att_ck; fp.ns = pl.ns; fp.hd = pl.hd;
                fp.items = (const df_item*)(fb + f_items);
                fp.item_counts = (const int*)(fb + f_counts);
                fp.tok_table = m->tok_table; fp.pos_table = m->pos_table;
                fp.kcache = (__nv_bfloat16*)dec->kcache; fp.vcache = (__nv_bfloat16*)dec->vcache;
                fp.x = dec->x0; fp.qkv = (__nv_bfloat16*)dec->qkv; fp.att = (__nv_bfloat16*)dec->att; fp.hid = (__nv_bfloat16*)dec->hid;
                fp.cand = (float2*)(fb + f_cand); fp.cur = dec->cur; fp.len = dec->d_len;
                fp.bar_flags = (unsigned*)(fb + f_bar); fp.abort_flag = (int*)(fb + f_bar) + 1023; fp.err = ctx->d_err;
            }
        }
    }

    // ---- prompt: the blocks of the prefill path, also filling the caches
    int status = TLNN_OK;
    do {
        const long long M = (long long)B * T0;
        const size_t stream_bytes = tl_ws_round((size_t)M * d * 4);
        const size_t head_bytes = tl_ws_round((size_t)B * d * 4);
        status = tl_ws_reserve(ctx, 2 * stream_bytes + tl_block_ws_bytes(prec, M, d) + head_bytes);
        if (status) break;
        float* xa = (float*)ctx->ws;
        float* xb = (float*)(ctx->ws + stream_bytes);
        char* tail = ctx->ws + 2 * stream_bytes;
        status = tl_embed(ctx, ids, ids_type, m->tok_table, m->pos_table, xa, B, T0, d, m->vocab);
        if (status) break;
        const size_t layer_bytes = (size_t)B * max_len * d * es;
        for (int l = 0; l < m->layers && !status; l++) {
            status = tl_run_block_kv(ctx, prec, xa, &dec->blocks[l], m->act, xb, B, T0, d, m->heads, tail,
                                     (char*)dec->kcache + l * layer_bytes, (char*)dec->vcache + l * layer_bytes, max_len);
            float* t = xa; xa = xb; xb = t;
        }
        if (status) break;
        // last position of every prompt -> final LayerNorm -> head with arg-max
        float* last = (float*)(tail + tl_block_ws_bytes(prec, M, d));
        status = tl_convert(ctx, xa + (size_t)(T0 - 1) * d, (long long)T0 * d, last, TL_OUT_F32, B, d);
        if (status) break;
        status = tl_layernorm(ctx, last, m->lnf_gamma, m->lnf_beta, 1e-5f, dec->a, okind(prec), B, d);
        if (status) break;
        tl_gemm_epilogue eh;
        eh.bias = m->head_bias; eh.argmax_partials = dec->parts;
        status = tl_gemm(ctx, prec, dec->a, d, m->head_t, d, B, m->vocab, d, eh);
        if (status) break;
        status = tl_argmax_partials(ctx, dec->parts, dec->n_parts, dec->next, B);
        if (status) break;
        int init[2] = {T0, 0};
        cudaError_t ce = cudaMemcpyAsync(dec->d_len, init, sizeof(init), cudaMemcpyHostToDevice, ctx->stream);
        if (ce == cudaSuccess) ce = cudaMemcpyAsync(first_tokens, dec->next, (size_t)B * 4, cudaMemcpyDeviceToDevice, ctx->stream);
        if (ce == cudaSuccess) ce = cudaMemcpyAsync(dec->cur, dec->next, (size_t)B * 4, cudaMemcpyDeviceToDevice, ctx->stream);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(ctx->stream);      // `init` is a stack array
        if (ce != cudaSuccess) status = tl_cuda_fail(ce, "decode_begin copies", __FILE__, __LINE__);
        dec->host_len = T0;
    } while (0);
    if (status) {
        cudaFreeAsync(dec->mem, ctx->stream);
        if (dec->fused_mem) cudaFreeAsync(dec->fused_mem, ctx->stream);
        if (dec->fused_pack) cudaFreeAsync(dec->fused_pack, ctx->stream);
        delete dec;
        return status;
    }
    *out = dec;
    return TLNN_OK;
}

extern "C" int tlnn_decode_step(tlnn_decoder* dec, const int32_t* prev_tokens, int32_t* next_tokens) {
    TL_NOTNULL(dec); TL_NOTNULL(prev_tokens); TL_NOTNULL(next_tokens);
    tlnn_ctx* ctx = dec->ctx;
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_REQUIRE(dec->host_len < dec->max_len, "decode: the cache is full (%d positions)", dec->max_len);
    if (prev_tokens != dec->cur)
        TL_CUDA(cudaMemcpyAsync(dec->cur, prev_tokens, (size_t)dec->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (dec->fused.ok) {
        TL_TRY(run_fused(dec, 1, next_tokens, 1));
        dec->host_len++;
        return TLNN_OK;
    }
    TL_TRY(set_sink(dec, nullptr, 0));
    TL_TRY(decode_one(dec));
    dec->host_len++;
    TL_CUDA(cudaMemcpyAsync(next_tokens, dec->next, (size_t)dec->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return TLNN_OK;
}

extern "C" int tlnn_decode_run(tlnn_decoder* dec, const int32_t* prev_tokens, int n_steps, int32_t* tokens_out) {
    TL_NOTNULL(dec); TL_NOTNULL(prev_tokens); TL_NOTNULL(tokens_out);
    tlnn_ctx* ctx = dec->ctx;
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_REQUIRE(n_steps >= 0 && dec->host_len + n_steps <= dec->max_len, "decode: %d steps do not fit the cache (%d of %d used)",
               n_steps, dec->host_len, dec->max_len);
    if (n_steps == 0) return TLNN_OK;
    if (prev_tokens != dec->cur)
        TL_CUDA(cudaMemcpyAsync(dec->cur, prev_tokens, (size_t)dec->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (dec->fused.ok) {
        // all the steps in one launch of the persistent kernel
        TL_TRY(run_fused(dec, n_steps, tokens_out, n_steps));
        dec->host_len += n_steps;
        return TLNN_OK;
    }
    TL_TRY(set_sink(dec, tokens_out, n_steps));
    TL_CUDA(cudaMemsetAsync(dec->d_step, 0, sizeof(int), ctx->stream));
    // Every kernel of a step takes the position from device memory, so one step is captured once as a CUDA graph and
    // replayed; per-launch timing (tlnn_prof_classes) needs plain launches and bypasses the graph.
    if (!ctx->prof_classes && !dec->step_graph) {
        cudaGraph_t graph = nullptr;
        const long long before = ctx->launches;
        TL_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        const int st = decode_one(dec);
        dec->launches_per_step = ctx->launches - before;
        ctx->launches = before;                  // capturing records launches without running them
        const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
        if (st != TLNN_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        if (ce != cudaSuccess) return tl_cuda_fail(ce, "cudaStreamEndCapture", __FILE__, __LINE__);
        const cudaError_t ie = cudaGraphInstantiate(&dec->step_graph, graph, 0);
        cudaGraphDestroy(graph);
        if (ie != cudaSuccess) return tl_cuda_fail(ie, "cudaGraphInstantiate", __FILE__, __LINE__);
    }
    for (int s = 0; s < n_steps; s++) {
        if (dec->step_graph && !ctx->prof_classes) {
            TL_CUDA(cudaGraphLaunch(dec->step_graph, ctx->stream));
            ctx->launches += dec->launches_per_step;
        } else {
            TL_TRY(decode_one(dec));
        }
        dec->host_len++;
    }
    return TLNN_OK;
}

namespace {
int ensure_sampling_buffers(tlnn_decoder* dec) {
    if (dec->sample_mem) return TLNN_OK;
    const size_t row = ((size_t)dec->B * dec->m.vocab * 4 + 255) & ~size_t(255);
    const size_t un = ((size_t)dec->max_len * dec->B * 8 + 255) & ~size_t(255);
    TL_CUDA(cudaMallocAsync((void**)&dec->sample_mem, 2 * row + un, dec->ctx->stream));
    dec->logits = (float*)dec->sample_mem;
    dec->probs = (float*)(dec->sample_mem + row);
    dec->uniforms = (double*)(dec->sample_mem + 2 * row);
    return TLNN_OK;
}
}  // namespace

extern "C" int tlnn_decode_first_sampled(tlnn_decoder* dec, float temperature, const double* uniforms, int32_t* first_tokens) {
    TL_NOTNULL(dec); TL_NOTNULL(uniforms); TL_NOTNULL(first_tokens);
    tlnn_ctx* ctx = dec->ctx;
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_REQUIRE(temperature > 0.f, "decode: the temperature must be positive");
    TL_REQUIRE(dec->host_len < dec->max_len && dec->step_graph == nullptr && dec->sample_graph == nullptr,
               "decode: the first token is drawn right after tlnn_decode_begin, before any step");
    TL_TRY(ensure_sampling_buffers(dec));
    const tlnn_gpt_model& m = dec->m;
    // dec->a still holds the normalised last prompt rows of tlnn_decode_begin
    TL_CUDA(cudaMemcpyAsync(dec->uniforms, uniforms, (size_t)dec->B * 8, cudaMemcpyHostToDevice, ctx->stream));
    tl_gemm_epilogue eh;
    eh.bias = m.head_bias; eh.out = dec->logits; eh.ldo = m.vocab; eh.out_kind = TL_OUT_F32;
    TL_TRY(tl_gemm(ctx, m.prec, dec->a, m.d, m.head_t, m.d, dec->B, m.vocab, m.d, eh));
    TL_TRY(tlnn_softmax_fwd(ctx, dec->logits, dec->probs, dec->B, m.vocab, temperature));
    TL_TRY(tl_sample(ctx, dec->probs, m.vocab, dec->uniforms, nullptr, dec->next, dec->B, m.vocab));
    TL_CUDA(cudaMemcpyAsync(dec->cur, dec->next, (size_t)dec->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    TL_CUDA(cudaMemcpyAsync(first_tokens, dec->next, (size_t)dec->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    TL_CUDA(cudaStreamSynchronize(ctx->stream));            // `uniforms` is the caller's host memory
    return TLNN_OK;
}

extern "C" int tlnn_decode_run_sampled(tlnn_decoder* dec, const int32_t* prev_tokens, int n_steps, float temperature,
                                       const double* uniforms, int32_t* tokens_out) {
    TL_NOTNULL(dec); TL_NOTNULL(prev_tokens); TL_NOTNULL(tokens_out); TL_NOTNULL(uniforms);
    tlnn_ctx* ctx = dec->ctx;
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_REQUIRE(temperature > 0.f, "decode: the temperature must be positive");
    TL_REQUIRE(n_steps >= 0 && dec->host_len + n_steps <= dec->max_len, "decode: %d steps do not fit the cache (%d of %d used)",
               n_steps, dec->host_len, dec->max_len);
    if (n_steps == 0) return TLNN_OK;
    TL_TRY(ensure_sampling_buffers(dec));
    if (prev_tokens != dec->cur)
        TL_CUDA(cudaMemcpyAsync(dec->cur, prev_tokens, (size_t)dec->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    TL_CUDA(cudaMemcpyAsync(dec->uniforms, uniforms, (size_t)n_steps * dec->B * 8, cudaMemcpyHostToDevice, ctx->stream));
    TL_CUDA(cudaStreamSynchronize(ctx->stream));            // `uniforms` is the caller's host memory
    TL_TRY(set_sink(dec, tokens_out, n_steps));
    TL_CUDA(cudaMemsetAsync(dec->d_step, 0, sizeof(int), ctx->stream));
    if (!ctx->prof_classes && (!dec->sample_graph || dec->sample_temperature != temperature)) {
        if (dec->sample_graph) { cudaGraphExecDestroy(dec->sample_graph); dec->sample_graph = nullptr; }
        cudaGraph_t graph = nullptr;
        const long long before = ctx->launches;
        TL_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        const int st = decode_one(dec, true, temperature);
        dec->sample_launches_per_step = ctx->launches - before;
        ctx->launches = before;
        const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
        if (st != TLNN_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        if (ce != cudaSuccess) return tl_cuda_fail(ce, "cudaStreamEndCapture", __FILE__, __LINE__);
        const cudaError_t ie = cudaGraphInstantiate(&dec->sample_graph, graph, 0);
        cudaGraphDestroy(graph);
        if (ie != cudaSuccess) { dec->sample_graph = nullptr; return tl_cuda_fail(ie, "cudaGraphInstantiate", __FILE__, __LINE__); }
        dec->sample_temperature = temperature;
    }
    for (int s = 0; s < n_steps; s++) {
        if (dec->sample_graph && !ctx->prof_classes) {
            TL_CUDA(cudaGraphLaunch(dec->sample_graph, ctx->stream));
            ctx->launches += dec->sample_launches_per_step;
        } else {
            TL_TRY(decode_one(dec, true, temperature));
        }
        dec->host_len++;
    }
    return TLNN_OK;
}

extern "C" int tlnn_decode_end(tlnn_decoder* dec) {
    if (!dec) return TLNN_OK;
    cudaSetDevice(dec->ctx->device);
    cudaStreamSynchronize(dec->ctx->stream);
    if (dec->step_graph) cudaGraphExecDestroy(dec->step_graph);
    if (dec->sample_graph) cudaGraphExecDestroy(dec->sample_graph);
    cudaStream_t st = dec->ctx->stream;
    if (dec->sample_mem) cudaFreeAsync(dec->sample_mem, st);
    if (dec->fused_mem) cudaFreeAsync(dec->fused_mem, st);
    if (dec->fused_pack) cudaFreeAsync(dec->fused_pack, st);
    cudaFreeAsync(dec->mem, st);
    delete dec;
    return TLNN_OK;
}
