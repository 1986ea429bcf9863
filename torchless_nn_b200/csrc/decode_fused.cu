// One persistent kernel for KV-cached greedy decode in bf16 mode: every step of tlnn_decode_run runs inside a single
// cooperative launch, one CTA per SM.
//
// A decode step has one row per sequence, so its products are tiny (64 x 768 x 2304 at the largest) and strictly
// dependent: the launch-per-operator form spends its time in launch gaps and pipeline fill, not in HBM traffic.  Here
// the CTAs stay resident and meet at grid-wide barriers instead:
//   per layer   LayerNorm + QKV product | single-query attention over the cache | output product, x += |
//               LayerNorm + first feed-forward product + activation | second product, x += (four K ranges, atomics)
//   per step    final LayerNorm + head product with a running arg-max | arg-max over the CTAs' candidates, next token,
//               its embedding row for the next step.
// Weights never depend on the previous phase, so each CTA streams the weight rows of its upcoming work items into a
// two-slot shared-memory ring with bulk asynchronous copies while it waits at barriers: the HBM reads of the weights
// overlap everything else.  A work item is `ns` output features (rows of a prepared (out, in) weight) by one K range of
// d; items are dealt round-robin over the CTAs by a table built on the host.  The products run on mma.sync m16n8k16
// (the batch is at most 64 rows: the step is bound by HBM and by the barrier latency, not by tensor throughput).
//
// Every wait is bounded: a grid barrier or a copy that does not complete within its limit raises an abort flag that all
// CTAs poll, the kernel returns, and the host reports TLNN_ERR_TIMEOUT.
#include "sm100_ptx.cuh"
#include "decode_fused.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int DF_THREADS = 256;
constexpr int DF_WARPS = DF_THREADS / 32;
constexpr int DF_MMA_WARPS = 8;                // warps that take output tiles of a work item (the others help load its operands)
constexpr int DF_NST = 3;                      // stages of the attention ring
constexpr int DF_ROUNDS = 4;                   // key rounds a warp takes per chunk of the ring (handled as one batch)
// bytes of the ring: stages x (keys, values) x keys per chunk x row bytes.  Keys per chunk = warps x (32 lanes / (hd / 8)
// lanes per key) x rounds and a row has 2 hd bytes, so a chunk of keys is warps x 512 x rounds bytes for every head size.
constexpr int DF_RING_BYTES = DF_NST * 2 * DF_WARPS * 512 * DF_ROUNDS;
constexpr int DF_ITEMS_SMEM = 48;              // a CTA's item list is kept in shared memory when it has at most this many entries
// tail of the dynamic shared memory: barriers | K-split partials / attention partials | per-warp arg-max rows |
// attention extras (q, new key, new value per unit in flight) | item list
constexpr int DF_OFF_RED = 64, DF_OFF_ROWBEST = DF_OFF_RED + 8192, DF_OFF_EXTRAS = DF_OFF_ROWBEST + 4096;
constexpr int DF_OFF_ITEMS = DF_OFF_EXTRAS + DF_NST * 3 * 256;
constexpr int DF_TAIL_BYTES = (DF_OFF_ITEMS + DF_ITEMS_SMEM * 64 + 127) / 128 * 128;
constexpr unsigned long long DF_WAIT_NS = 2000000000ull;
constexpr long long DF_WAIT_CYCLES = 4000000000ll;      // about two seconds of SM clock: the limit of a grid barrier wait

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float activate(int act, float v) {
    if (act == TLNN_ACT_GELU) return 0.5f * v * (1.f + tanh_fast(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    if (act == TLNN_ACT_SILU) return v * ((1.f + tanh_fast(0.5f * v)) * 0.5f);
    if (act == TLNN_ACT_RELU) return fmaxf(v, 0.f);
    return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// One instance per CTA, in shared memory: every field is uniform over the CTA.  (Kept in registers or on the per-thread
// stack it would spill to local memory, 256 copies of it, and with almost all of the SM's memory configured as shared
// memory those accesses miss L1: every field read then costs a trip to L2.)  Thread 0 is the only writer after set-up,
// always between two __syncthreads.
// Bounded mbarrier wait of this kernel, timed by the SM's cycle counter (reading the nanosecond timer costs far more than
// a probe of the barrier, and these waits sit on the critical path of every phase).  Returns false after recording the
// failure and raising the CTA's abort flag when the phase did not complete within the limit.
__device__ __noinline__ bool df_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag, tlnn_dev_err* err, int site) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 4096; i++)
            if (sm100::mbar_test_wait(bar, parity)) return true;      // plain probes: a suspended try_wait wakes late
        if (*abort_flag) return false;
        if (clock64() - t0 > 4000000000ll) {
            *abort_flag = 1;
            tl_dev_fail(err, TLNN_ERR_TIMEOUT, site, (long long)blockIdx.x);
            return false;
        }
    }
}
__device__ __forceinline__ bool df_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, tlnn_dev_err* err, int site) {
    if (sm100::mbar_test_wait(bar, parity)) return true;
    return df_wait_slow(bar, parity, abort_flag, err, site);
}

struct df_state {
    df_params p;
    bf16* A;                  // (64, lda) operand rows
    bf16* W[2];               // two weight slots: rows of lda elements, then the item's bias slice, LayerNorm gamma and beta
    int w_bytes;              // bytes of the weight rows of a slot (the side arrays follow)
    uint64_t* full;           // [2] "slot filled" barriers
    float* red;               // K-split partial accumulators
    float2* rowbest;          // [DF_WARPS][64] running (value, index bits) of the head product
    unsigned char* extras;    // attention: DF_NST slots of a unit's q, new-key and new-value rows
    uint64_t* att_full;       // [DF_NST] "stage filled" barriers of the attention ring
    long long att_count;      // chunks streamed through the attention ring so far (stage and parity continue across phases)
    const CUtensorMap *kmap, *vmap;   // the key and value caches as (layers x sequences x heads x positions, head dimension) matrices
    volatile int* s_abort;    // shared: a wait of this CTA gave up
    int* s_bcast;             // shared: one int handed from thread 0 to the CTA
    const df_item* items;     // this CTA's items of one step
    int n_items;              // per step
    long long total;          // items over the whole launch
    long long cons;           // items consumed so far
    long long prod;           // items whose copies were issued
    unsigned epoch;           // grid barrier target
    int lda;
    int a_tag;                // what A currently holds (kind, layer, k0, step), -1 = nothing
};

// ---- grid-wide barrier: monotonic arrival counter in global memory, bounded wait -------------------------------------
// (A variant without atomics - one flag word per CTA, every CTA watching all the words - measured slower: about 3 us
// per barrier against 2.2 us for the counter.)
__device__ bool grid_sync(df_state& s) {
    const df_params& p = s.p;
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        s.epoch += gridDim.x;
        const unsigned target = s.epoch;
        __threadfence();
        atomicAdd(p.bar_flags, 1u);
        if (ld_acquire_u32(p.bar_flags) < target) {
            const long long t0 = clock64();
            unsigned polls = 0;
            while (ld_acquire_u32(p.bar_flags) < target) {
                if ((++polls & 255u) == 0) {
                    if (*reinterpret_cast<volatile int*>(p.abort_flag)) { ok = 0; break; }
                    if (clock64() - t0 > DF_WAIT_CYCLES) {
                        tl_dev_fail(p.err, TLNN_ERR_TIMEOUT, 700, (long long)blockIdx.x);
                        ok = 0;
                        break;
                    }
                }
            }
        }
        if (*s.s_abort) ok = 0;
        if (!ok) { *s.s_abort = 1; atomicExch(p.abort_flag, 1); }
        *s.s_bcast = ok;
    }
    __syncthreads();
    return *s.s_bcast != 0;
}

// ---- weight ring -------------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool bias_staged(const df_item& it) { return it.bias != nullptr && (it.rows & 3) == 0; }
__device__ __forceinline__ float* slot_bias(const df_state& s, int slot) {
    return reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(s.W[slot]) + s.w_bytes);
}
__device__ __forceinline__ float* slot_gamma(const df_state& s, int slot) { return slot_bias(s, slot) + s.p.ns; }
__device__ __forceinline__ float* slot_beta(const df_state& s, int slot) { return slot_gamma(s, slot) + s.p.d; }

// Warp 0 issues the copies of item `g` (if any) into slot g & 1: its weight rows, its bias slice and, for a product
// that follows a LayerNorm, gamma and beta.  The slot's previous contents have been consumed (the caller passed a
// __syncthreads since the last read).
__device__ void issue_item(df_state& s, long long g) {
    if (g >= s.total || (threadIdx.x >> 5) != 0) return;
    const df_params& p = s.p;
    const df_item it = s.items[g % s.n_items];
    const int slot = (int)(g & 1);
    const int lane = threadIdx.x & 31;
    const uint32_t row_bytes = (uint32_t)p.d * 2u;
    const uint32_t bar = sm100::smem_u32(&s.full[slot]);
    const bool with_bias = bias_staged(it), with_norm = it.gamma != nullptr;
    if (lane == 0) {
        sm100::fence_async_smem();          // the slot was last read through the generic proxy
        sm100::mbar_expect_tx(&s.full[slot], (it.ldw == s.lda ? (uint32_t)s.lda * 2u : row_bytes) * (uint32_t)it.rows + (with_bias ? (uint32_t)it.rows * 4u : 0u) +
                                                 (with_norm ? (uint32_t)p.d * 8u : 0u));
    }
    __syncwarp();
    if (it.ldw == s.lda) {
        // packed weights: the item's rows are one block at the pitch they have in shared memory (the eight pad elements
        // of a row travel along and are never read)
        if (lane == 3) bulk_g2s(sm100::smem_u32(s.W[slot]), it.w, (uint32_t)it.rows * (uint32_t)s.lda * 2u, bar);
    } else {
        for (int r = lane; r < it.rows; r += 32)
            bulk_g2s(sm100::smem_u32(s.W[slot] + (size_t)r * s.lda), it.w + (size_t)r * it.ldw, row_bytes, bar);
    }
    if (lane == 0 && with_bias) bulk_g2s(sm100::smem_u32(slot_bias(s, slot)), it.bias + it.n0, (uint32_t)it.rows * 4u, bar);
    if (lane == 1 && with_norm) bulk_g2s(sm100::smem_u32(slot_gamma(s, slot)), it.gamma, (uint32_t)p.d * 4u, bar);
    if (lane == 2 && with_norm) bulk_g2s(sm100::smem_u32(slot_beta(s, slot)), it.beta, (uint32_t)p.d * 4u, bar);
}

// ---- operand rows -------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A[m, :] = LayerNorm(x[m, :]) as bf16, mean and biased variance in two passes over the row held in registers.
// A warp keeps R rows in flight: the loads of a row take a trip to L2, and eight rows one after the other per warp
// would make the phase eight such trips long.
template <int V4, int R>      // float4 loads per lane per row (d = 128 * V4), rows per round
__device__ __noinline__ void load_a_layernorm_t(df_state& s, const float* x, const float* __restrict__ gamma, const float* __restrict__ beta) {
    const df_params& p = s.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = p.d;
    const float inv_d = 1.f / (float)d;
    for (int m0 = warp * R; m0 < p.B; m0 += DF_WARPS * R) {
        float4 v[R][V4];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int m = m0 + r < p.B ? m0 + r : p.B - 1;            // a clamped row keeps the loop free of branches
            const float4* row = reinterpret_cast<const float4*>(x + (size_t)m * d);
#pragma unroll
            for (int i = 0; i < V4; i++) v[r][i] = __ldcg(row + lane + 32 * i);
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < V4; i++) sum += (v[r][i].x + v[r][i].y) + (v[r][i].z + v[r][i].w);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float mean = sum * inv_d;
            float sq = 0.f;
#pragma unroll
            for (int i = 0; i < V4; i++) {
                const float a = v[r][i].x - mean, b = v[r][i].y - mean, c = v[r][i].z - mean, e = v[r][i].w - mean;
                sq += (a * a + b * b) + (c * c + e * e);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            const float rstd = 1.f / sqrtf(sq * inv_d + 1e-5f);
            if (m0 + r < p.B) {
                bf16* dst = s.A + (size_t)(m0 + r) * s.lda;
#pragma unroll
                for (int i = 0; i < V4; i++) {
                    const int c = (lane + 32 * i) * 4;
                    const float4 g = *reinterpret_cast<const float4*>(gamma + c);      // shared memory (came with the item's weights)
                    const float4 b = *reinterpret_cast<const float4*>(beta + c);
                    uint2 o;
                    o.x = pack_bf16((v[r][i].x - mean) * rstd * g.x + b.x, (v[r][i].y - mean) * rstd * g.y + b.y);
                    o.y = pack_bf16((v[r][i].z - mean) * rstd * g.z + b.z, (v[r][i].w - mean) * rstd * g.w + b.w);
                    *reinterpret_cast<uint2*>(dst + c) = o;
                }
            }
        }
    }
}

__device__ void load_a_layernorm(df_state& s, const float* x, const float* gamma, const float* beta) {
    switch (s.p.d / 128) {
        case 1: load_a_layernorm_t<1, 4>(s, x, gamma, beta); break;
        case 2: load_a_layernorm_t<2, 4>(s, x, gamma, beta); break;
        case 3: load_a_layernorm_t<3, 4>(s, x, gamma, beta); break;
        case 4: load_a_layernorm_t<4, 4>(s, x, gamma, beta); break;
        case 5: load_a_layernorm_t<5, 2>(s, x, gamma, beta); break;
        case 6: load_a_layernorm_t<6, 2>(s, x, gamma, beta); break;
        case 7: load_a_layernorm_t<7, 2>(s, x, gamma, beta); break;
        default: load_a_layernorm_t<8, 2>(s, x, gamma, beta); break;
    }
}

// A[m, 0:d] = src[m, k0:k0+d] (bf16 rows of pitch lds) with 16-byte asynchronous copies, all in flight at once.
// The caller's __syncthreads after this call makes every thread's copies visible to the CTA.
__device__ __noinline__ void load_a_copy(df_state& s, const bf16* src, int lds, int k0) {
    const df_params& p = s.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = p.d / 8;                     // 16-byte chunks per row
    const uint32_t a_base = sm100::smem_u32(s.A);
#pragma unroll 1
    for (int m = warp; m < p.B; m += DF_WARPS) {
        const bf16* row = src + (size_t)m * lds + k0;
        const uint32_t dst = a_base + (uint32_t)(m * s.lda) * 2u;
#pragma unroll 1
        for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 16, row + c * 8);
    }
    cp_async_commit();
    cp_async_wait<0>();
}

// ---- one work item: (B x d) operand rows times `rows` weight rows --------------------------------------------------
// The kernel's code is kept small on purpose (helpers out of line, loops rolled): every phase runs its code once per
// layer, so straight-line code that does not fit the instruction cache is paid for as instruction fetches from L2.
struct tile8 { float v[2][4]; };       // a warp's 16 x 16 output tile: [n tile][mma accumulator register]

// Accumulate the 16 x 16 output tile (m_tile, npi) over K range [k_begin, k_begin + klen).
__device__ __noinline__ tile8 mma_task(uint32_t a_base, uint32_t w_base, uint32_t row_pitch, int m_tile, int npi, int k_begin, int klen, int lane) {
    float acc[2][2][4] = {};
    // ldmatrix rows: A  m_tile*16 + lane%16 at k + (lane/16)*8;  W  npi*16 + lane%8 + (lane/16)*8 at k + ((lane/8)&1)*8
    const uint32_t a_addr = a_base + (uint32_t)(m_tile * 16 + (lane & 15)) * row_pitch + (uint32_t)((lane >> 4) * 8 + k_begin) * 2u;
    const uint32_t w_addr = w_base + (uint32_t)(npi * 16 + (lane & 7) + (lane >> 4) * 8) * row_pitch + (uint32_t)(((lane >> 3) & 1) * 8 + k_begin) * 2u;
    // fragments of the next K step are requested before the products of the current one are issued; two accumulator
    // sets shorten the dependent chain.  klen is a multiple of 16.
    uint32_t a0[4], b0[4], a1[4], b1[4];
    ldmatrix_x4(a0, a_addr);
    ldmatrix_x4(b0, w_addr);
#pragma unroll 1
    for (int k = 0; k < klen; k += 32) {
        const bool second = k + 16 < klen;
        if (second) {
            ldmatrix_x4(a1, a_addr + (k + 16) * 2);
            ldmatrix_x4(b1, w_addr + (k + 16) * 2);
        }
        mma_16816(acc[0][0], a0, b0[0], b0[1]);
        mma_16816(acc[0][1], a0, b0[2], b0[3]);
        if (k + 32 < klen) {
            ldmatrix_x4(a0, a_addr + (k + 32) * 2);
            ldmatrix_x4(b0, w_addr + (k + 32) * 2);
        }
        if (second) {
            mma_16816(acc[1][0], a1, b1[0], b1[1]);
            mma_16816(acc[1][1], a1, b1[2], b1[3]);
        }
    }
    tile8 c;
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) c.v[j][i] = acc[0][j][i] + acc[1][j][i];
    return c;
}

// What happens to a finished 16 x 16 tile.  Called by whole warps (the head's arg-max uses shuffles).  The loops are
// rolled on purpose (the tile goes through a small local array): this code runs once per item.
__device__ __noinline__ void item_epilogue(df_state& s, const df_item& it, const float* bias, int m_tile, int npi, int warp, int lane,
                                           const tile8 tile) {
    // `bias` is indexed by the feature inside the item: the slot's staged slice, or the global vector moved to the item's
    // first feature when the slice could not be staged, or null
    const df_params& p = s.p;
    const int g = lane >> 2, q2 = (lane & 3) * 2;
    float cv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) cv[i] = tile.v[i >> 2][i & 3];
    const int kind = it.kind;
#pragma unroll 1
    for (int half = 0; half < 2; half++) {
        const int m = m_tile * 16 + g + half * 8;
        const bool row_ok = m < p.B;
        float best = -INFINITY;
        int best_n = 0x7fffffff;
#pragma unroll 1
        for (int j = 0; j < 2; j++) {
            const int nl = npi * 16 + j * 8 + q2;            // feature inside the item
            if (!row_ok || nl >= it.rows) continue;
            const int n = it.n0 + nl;
            const bool has1 = nl + 1 < it.rows;               // the last vocabulary slice may end on an odd row
            float v0 = cv[j * 4 + half * 2], v1 = cv[j * 4 + half * 2 + 1];
            if (bias) { v0 += bias[nl]; if (has1) v1 += bias[nl + 1]; }
            if (kind == DF_HEAD) {
                if (v0 > best) { best = v0; best_n = n; }
                if (has1 && v1 > best) { best = v1; best_n = n + 1; }
            } else if (!TL_DBG_IN_BOUNDS(p.err, n + 1 < (kind == DF_QKV ? 3 : kind == DF_FFN1 ? 4 : 1) * p.d, 930 + kind, n)) {
                // debug build only: a feature outside the product's width (recorded, store skipped)
            } else if (kind == DF_QKV) {
                *reinterpret_cast<uint32_t*>(p.qkv + (size_t)m * 3 * p.d + n) = pack_bf16(v0, v1);
            } else if (kind == DF_FFN1) {
                *reinterpret_cast<uint32_t*>(p.hid + (size_t)m * 4 * p.d + n) = pack_bf16(activate(p.act, v0), activate(p.act, v1));
            } else {
                // x += product.  The output product has one writer per element; the second feed-forward product is split
                // into four K ranges whose sums meet here in no fixed order.  The reduction form spares the read trip.
                atomicAdd(p.x + (size_t)m * p.d + n, v0);
                atomicAdd(p.x + (size_t)m * p.d + n + 1, v1);
            }
        }
        if (kind == DF_HEAD) {       // uniform over the warp
            // the four lanes of a row hold disjoint columns: keep the largest value, the lowest index among equals
#pragma unroll 1
            for (int o = 1; o <= 2; o <<= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int on = __shfl_xor_sync(0xffffffffu, best_n, o);
                if (ov > best || (ov == best && on < best_n)) { best = ov; best_n = on; }
            }
            if (row_ok && (lane & 3) == 0) {
                float2& rb = s.rowbest[warp * 64 + m];
                const int cur_n = __float_as_int(rb.y);
                if (best > rb.x || (best == rb.x && best_n < cur_n)) { rb.x = best; rb.y = __int_as_float(best_n); }
            }
        }
    }
}

__device__ __noinline__ bool run_item(df_state& s, const df_item& it, int step) {
    const df_params& p = s.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long cons = s.cons, prod = s.prod;         // nobody writes them before the barriers at the end of this item
    const int slot = (int)(cons & 1);
    // the item's weights, bias slice and LayerNorm vectors (issued one or two items ago)
    if (!df_wait(&s.full[slot], (uint32_t)((cons >> 1) & 1), s.s_abort, p.err, 701)) return false;
    // operand rows for this item (kept across consecutive items of one phase)
    const int tag = ((it.kind * 64 + it.layer) * 8 + (it.kind == DF_FFN2 ? it.k0 / p.d : 0)) * 4096 + (step & 4095);
    if (tag != s.a_tag) {
        if (it.gamma) load_a_layernorm(s, p.x, slot_gamma(s, slot), slot_beta(s, slot));
        else if (it.kind == DF_OUT) load_a_copy(s, p.att, p.d, 0);
        else load_a_copy(s, p.hid, 4 * p.d, it.k0);
        __syncthreads();
        if (threadIdx.x == 0) s.a_tag = tag;        // every thread compared against the old value before this barrier
    }
    const float* bias = bias_staged(it) ? slot_bias(s, slot) : (it.bias ? it.bias + it.n0 : nullptr);

    // 16 x 16 output tiles over the warps; with fewer tiles than warps the contraction is split over warps as well and
    // the partial sums meet in shared memory in a fixed order
    const int mt = (p.B + 15) >> 4;
    const int np = (it.rows + 15) >> 4;
    const int tasks = mt * np;
    const uint32_t a_base = sm100::smem_u32(s.A), w_base = sm100::smem_u32(s.W[slot]);
    const uint32_t row_pitch = (uint32_t)s.lda * 2u;
    int ksplit = 1, kpart = 0, first = warp < DF_MMA_WARPS ? warp : tasks, stride = DF_MMA_WARPS;
    if (tasks < DF_MMA_WARPS) {
        ksplit = DF_MMA_WARPS / tasks;
        while (ksplit & (ksplit - 1)) ksplit &= ksplit - 1;                   // round down to a power of two
        while (ksplit > 1 && (p.d / ksplit) % 16 != 0) ksplit >>= 1;
        kpart = warp / tasks;
        first = (warp < DF_MMA_WARPS && kpart < ksplit) ? warp % tasks : tasks;   // idle warps run no tile
        stride = tasks;                                                       // one tile per warp
    }
    const int klen = p.d / ksplit;
    tile8 c;
    int mine = -1;
    for (int t = first; t < tasks; t += stride) {
        c = mma_task(a_base, w_base, row_pitch, t % mt, t / mt, kpart * klen, klen, lane);
        if (ksplit == 1) item_epilogue(s, it, bias, t % mt, t / mt, warp, lane, c);
        mine = t;
    }
    if (ksplit > 1) {       // uniform over the CTA
        if (mine >= 0 && kpart > 0) {
            float* dst = s.red + ((size_t)(kpart - 1) * tasks + mine) * 256 + lane * 8;
#pragma unroll
            for (int i = 0; i < 8; i++) dst[i] = c.v[i >> 2][i & 3];
        }
        __syncthreads();
        if (mine >= 0 && kpart == 0) {
            for (int q = 1; q < ksplit; q++) {
                const float* r = s.red + ((size_t)(q - 1) * tasks + mine) * 256 + lane * 8;
#pragma unroll
                for (int i = 0; i < 8; i++) c.v[i >> 2][i & 3] += r[i];
            }
            item_epilogue(s, it, bias, mine % mt, mine / mt, warp, lane, c);
        }
    }
    __syncthreads();                                 // all reads of the slot (and of the partial sums) are done
    issue_item(s, prod);
    if (threadIdx.x == 0) { s.prod = prod + 1; s.cons = cons + 1; }
    __syncthreads();                                 // the counters are read again by the caller
    return true;
}

// All items of this CTA that belong to (kind, layer) at the head of its list.
__device__ bool run_phase(df_state& s, int kind, int layer, int step) {
    const long long step_end = (long long)(step + 1) * s.n_items;          // never run into the next step's items
    while (s.cons < step_end) {
        const df_item& it = s.items[s.cons % s.n_items];       // read in place (shared memory for all but the largest models)
        if (it.kind != kind || (kind != DF_HEAD && it.layer != layer)) break;
        if (!run_item(s, it, step)) return false;
    }
    return true;
}

// ---- attention over the cache ------------------------------------------------------------------------------------------
// A CTA takes (sequence, head) units blockIdx.x, blockIdx.x + grid, ...  The cached keys and values of a unit stream
// through a DF_NST-stage shared-memory ring in chunks of `att_ck` keys: one TMA tile load for the keys and one for the
// values of a chunk (a box of att_ck rows by the head's columns out of the (layers x sequences x positions, d) cache),
// DF_NST - 1 chunks always in flight, so the phase runs at the rate the memory system delivers the cache; the cache of
// a layer is also requested into L2 a few phases ahead (prefetch_cache).  Inside a chunk every warp owns a block of keys
// and keeps its own running maximum, sum and weighted value sum (HD / 8 lanes per key, eight dimensions per lane); at
// the end of a unit the eight partial results and this step's own key and value (taken from the projection row, and
// appended to the cache) are merged by warp 0.
template <int HD>
__device__ __noinline__ bool attention_phase(df_state& s, int layer, int pos) {
    constexpr int ROWB = HD * 2;                   // bytes of one key or value row of a head
    constexpr int TPR = HD / 8;                    // lanes per row (16 bytes each)
    constexpr int KPP = 32 / TPR;                  // keys per warp round
    const df_params& p = s.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % TPR, grp = lane / TPR;
    const int d = p.d, H = p.H, CK = p.att_ck;
    const size_t layer_off = (size_t)layer * p.B * p.max_len * d;
    bf16* const kcache = p.kcache + layer_off;
    bf16* const vcache = p.vcache + layer_off;
    const float inv = rsqrtf((float)HD);
    const int n_units_all = p.B * H;
    const int my_units = (int)blockIdx.x < n_units_all ? (n_units_all - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int nchunk = pos > 0 ? (pos + CK - 1) / CK : 1;          // a unit without cached keys still brings its extras
    const int F = my_units * nchunk;
    const long long base = s.att_count;                            // chunks this CTA has streamed before this phase
    const uint32_t ring = sm100::smem_u32(s.A);                    // DF_NST stages of 2 * CK rows (keys, then values)
    const uint32_t stage_bytes = 2u * (uint32_t)CK * ROWB;
    unsigned char* extras = s.extras;                              // DF_NST slots (unit index mod DF_NST) of q, new key, new value
                                                                   // rows: they arrive with the unit's first chunk, stay until its merge
    float* wpart = s.red;                                          // per warp: running maximum, sum, HD weighted sums
    bool ok = true;

    float m_run = -INFINITY, l_run = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    float q[8];
    int ui_issue = 0, j_issue = 0;                                 // (unit, chunk) of the next chunk to request
    int ui = 0, j = 0;                                             // (unit, chunk) being consumed
#pragma unroll 1
    for (int f = 1 - DF_NST; f < F; f++) {                         // the first DF_NST - 1 turns only fill the ring
        // request chunk f + DF_NST - 1 into the stage chunk f - 1 was read from (everyone is past the barrier below)
        if (threadIdx.x == 0 && f + DF_NST - 1 < F) {
            const long long g = base + f + DF_NST - 1;
            const int st = (int)(g % DF_NST);
            const int u = blockIdx.x + ui_issue * gridDim.x;
            const int b = u / H, h = u - b * H;
            uint64_t* bar = &s.att_full[st];
            sm100::fence_async_smem();
            sm100::mbar_expect_tx(bar, stage_bytes + (j_issue == 0 ? 3u * ROWB : 0u));
            const int row0 = ((layer * p.B + b) * H + h) * p.max_len + j_issue * CK;
            sm100::tma_load_2d(ring + st * stage_bytes, s.kmap, sm100::smem_u32(bar), 0, row0);
            sm100::tma_load_2d(ring + st * stage_bytes + (uint32_t)CK * ROWB, s.vmap, sm100::smem_u32(bar), 0, row0);
            if (j_issue == 0) {
                const bf16* row = p.qkv + (size_t)b * 3 * d + h * HD;
                for (int which = 0; which < 3; which++)
                    bulk_g2s(sm100::smem_u32(extras + ((ui_issue % DF_NST) * 3 + which) * ROWB), row + (size_t)which * d, ROWB, sm100::smem_u32(bar));
            }
        }
        if (f + DF_NST - 1 < F && ++j_issue == nchunk) { j_issue = 0; ui_issue++; }
        if (f < 0) continue;
        const long long g = base + f;
        const int st = (int)(g % DF_NST);
        if (!df_wait(&s.att_full[st], (uint32_t)((g / DF_NST) & 1), s.s_abort, p.err, 704)) { ok = false; break; }
        if (j == 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(extras + ((ui % DF_NST) * 3 + 0) * ROWB + sub * 16);
            const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = __bfloat162float(e[i]);
        }
        const unsigned char* kst = reinterpret_cast<const unsigned char*>(s.A) + (size_t)st * stage_bytes;
        const unsigned char* vst = kst + (size_t)CK * ROWB;
        const int per_warp = KPP * DF_ROUNDS;                       // CK / DF_WARPS
        const int k_first = j * CK + warp * per_warp;               // first key of this warp in the chunk
        if (k_first < pos) {
            // the warp's DF_ROUNDS x KPP keys of the chunk as one batch: independent dot products, one maximum, one rescale
            float sc[DF_ROUNDS];
            uint4 vraw[DF_ROUNDS];
#pragma unroll
            for (int r = 0; r < DF_ROUNDS; r++) {
                const int kl = warp * per_warp + r * KPP + grp;     // row inside the stage
                const uint4 kraw = *reinterpret_cast<const uint4*>(kst + (size_t)kl * ROWB + sub * 16);
                vraw[r] = *reinterpret_cast<const uint4*>(vst + (size_t)kl * ROWB + sub * 16);
                const bf16* ke = reinterpret_cast<const bf16*>(&kraw);
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) a = fmaf(q[i], __bfloat162float(ke[i]), a);
                sc[r] = a;
            }
#pragma unroll
            for (int o = TPR / 2; o > 0; o >>= 1)
#pragma unroll
                for (int r = 0; r < DF_ROUNDS; r++) sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], o);
            float rm = -INFINITY;
#pragma unroll
            for (int r = 0; r < DF_ROUNDS; r++) {
                const bool valid = k_first + r * KPP + grp < pos;   // rows past the end hold later positions or zeros
                sc[r] = valid ? sc[r] * inv : -INFINITY;
                rm = fmaxf(rm, sc[r]);
            }
#pragma unroll
            for (int o = TPR; o < 32; o <<= 1) rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, o));
            if (rm > m_run) {                                       // uniform over the warp; the warp's first key is valid
                const float scale = __expf(m_run - rm);
                l_run *= scale;
#pragma unroll
                for (int i = 0; i < 8; i++) acc[i] *= scale;
                m_run = rm;
            }
#pragma unroll
            for (int r = 0; r < DF_ROUNDS; r++) {
                if (sc[r] != -INFINITY) {                           // never multiply stale value rows, not even by zero
                    const float pr = __expf(sc[r] - m_run);
                    l_run += pr;
                    const bf16* ve = reinterpret_cast<const bf16*>(&vraw[r]);
#pragma unroll
                    for (int i = 0; i < 8; i++) acc[i] = fmaf(pr, __bfloat162float(ve[i]), acc[i]);
                }
            }
        }
        if (j == nchunk - 1) {
            // ---- end of a unit: sum over the key groups of a warp, then over the warps
#pragma unroll
            for (int o = TPR; o < 32; o <<= 1) {
                l_run += __shfl_xor_sync(0xffffffffu, l_run, o);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
            }
            if (grp == 0) {
                float* w = wpart + warp * (HD + 2);
                if (sub == 0) { w[0] = m_run; w[1] = l_run; }
#pragma unroll
                for (int i = 0; i < 8; i++) w[2 + sub * 8 + i] = acc[i];
            }
            __syncthreads();
            if (warp == 0) {
                const int u = blockIdx.x + ui * gridDim.x;
                const int b = u / H, h = u - b * H;
                const uint4 kn = *reinterpret_cast<const uint4*>(extras + ((ui % DF_NST) * 3 + 1) * ROWB + sub * 16);
                const uint4 vn = *reinterpret_cast<const uint4*>(extras + ((ui % DF_NST) * 3 + 2) * ROWB + sub * 16);
                const bf16* ke = reinterpret_cast<const bf16*>(&kn);
                const bf16* ve = reinterpret_cast<const bf16*>(&vn);
                float s_new = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) s_new = fmaf(q[i], __bfloat162float(ke[i]), s_new);
#pragma unroll
                for (int o = TPR / 2; o > 0; o >>= 1) s_new += __shfl_xor_sync(0xffffffffu, s_new, o);
                s_new *= inv;
                float mx = s_new;
#pragma unroll 1
                for (int w = 0; w < DF_WARPS; w++) mx = fmaxf(mx, wpart[w * (HD + 2)]);
                float l_tot = __expf(s_new - mx);
                float o8[8];
#pragma unroll
                for (int i = 0; i < 8; i++) o8[i] = l_tot * __bfloat162float(ve[i]);
#pragma unroll 1
                for (int w = 0; w < DF_WARPS; w++) {
                    const float* wp = wpart + w * (HD + 2);
                    const float sc = wp[0] == -INFINITY ? 0.f : __expf(wp[0] - mx);
                    l_tot += sc * wp[1];
#pragma unroll
                    for (int i = 0; i < 8; i++) o8[i] = fmaf(sc, wp[2 + sub * 8 + i], o8[i]);
                }
                if (grp == 0) {
                    const float rs = 1.f / l_tot;
                    uint4 o;
                    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                    for (int i = 0; i < 4; i++) ow[i] = pack_bf16(o8[2 * i] * rs, o8[2 * i + 1] * rs);
                    *reinterpret_cast<uint4*>(p.att + (size_t)b * d + h * HD + sub * 8) = o;
                    // append this step's key and value rows to the cache
                    *reinterpret_cast<uint4*>(kcache + (((size_t)b * H + h) * p.max_len + pos) * HD + sub * 8) = kn;
                    *reinterpret_cast<uint4*>(vcache + (((size_t)b * H + h) * p.max_len + pos) * HD + sub * 8) = vn;
                }
            }
            m_run = -INFINITY;
            l_run = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] = 0.f;
        }
        if (++j == nchunk) { j = 0; ui++; }
        __syncthreads();                            // this stage (and, after a merge, the partials) may be overwritten
    }
    if (threadIdx.x == 0) {
        s.att_count = base + F;                     // read again after the grid barrier
        s.a_tag = -1;                               // the ring overwrote the operand rows
    }
    return ok;
}

// Ask for the cached keys and values of `layer` (positions [0, pos) of every sequence) to be brought into L2.  A
// layer's cache is at most a few tens of MB and is read in full by that layer's attention phase; requested a few
// phases ahead, the HBM reads overlap the latency-bound products in between.  CTA c < 2 B takes (sequence c / 2, keys or
// values); one thread issues the requests, 64 KB apiece.
__device__ void prefetch_cache(const df_params& p, int layer, int pos) {
    if ((int)blockIdx.x >= 2 * p.B || threadIdx.x != 32 || pos <= 0) return;
    const int b = blockIdx.x >> 1;
    const bf16* seq = ((blockIdx.x & 1) ? p.vcache : p.kcache) + ((size_t)layer * p.B + b) * p.max_len * p.d;
    const size_t bytes = (size_t)pos * p.hd * 2;                   // the live rows of one head are contiguous
    for (int h = 0; h < p.H; h++) {
        const bf16* base = seq + (size_t)h * p.max_len * p.hd;
        for (size_t off = 0; off < bytes; off += 65536) {
            const unsigned n = (unsigned)(bytes - off < 65536 ? bytes - off : 65536);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const char*>(base) + off), "r"(n) : "memory");
        }
    }
}

// x[b, :] = table[token, :] + pos_table[position, :] by CTA b
__device__ void embed_row(const df_params& p, int b, int token, int position) {
    long long id = token;
    if (id < 0 || id >= p.V) {
        if (threadIdx.x == 0) tl_dev_fail(p.err, TLNN_ERR_INDEX, 2, id);
        id = 0;
    }
    const float* t = p.tok_table + (size_t)id * p.d;
    const float* ps = p.pos_table + (size_t)position * p.d;
    for (int c = threadIdx.x; c < p.d; c += DF_THREADS) p.x[(size_t)b * p.d + c] = __fadd_rn(__ldg(t + c), __ldg(ps + c));
}

__global__ void __launch_bounds__(DF_THREADS, 1) decode_fused_kernel(const df_params p_in, const __grid_constant__ CUtensorMap kmap,
                                                                        const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort_word, s_bcast_word;
    __shared__ df_state s;
    if (threadIdx.x == 0) {
        s.p = p_in;
        const df_params& p = s.p;
        s.lda = p.d + 8;
        const size_t a_bytes = (size_t)p.a_region;    // operand rows; the attention ring uses the same bytes
        s.A = reinterpret_cast<bf16*>(smem);
        s.W[0] = reinterpret_cast<bf16*>(smem + a_bytes);
        s.W[1] = reinterpret_cast<bf16*>(smem + a_bytes + p.slot_bytes);
        s.w_bytes = p.ns * s.lda * 2;
        unsigned char* tail = smem + a_bytes + 2 * (size_t)p.slot_bytes;
        s.full = reinterpret_cast<uint64_t*>(tail);
        s.att_full = reinterpret_cast<uint64_t*>(tail) + 2;
        s.att_count = 0;
        s.kmap = &kmap;
        s.vmap = &vmap;
        s.red = reinterpret_cast<float*>(tail + DF_OFF_RED);                       // (K ranges - 1) x tiles x 256 floats: 7 KB at most
        s.rowbest = reinterpret_cast<float2*>(tail + DF_OFF_ROWBEST);              // 8 x 64 x 8 bytes
        s.extras = tail + DF_OFF_EXTRAS;
        s.s_abort = &s_abort_word;
        s.s_bcast = &s_bcast_word;
        s.n_items = p.item_counts[blockIdx.x];
        s.items = p.items + (size_t)blockIdx.x * p.items_pitch;
        s.total = (long long)s.n_items * p.n_steps;
        s.cons = 0;
        s.prod = 2;                                    // items 0 and 1 are issued below
        s.epoch = 0;
        s.a_tag = -1;
        s_abort_word = 0;
        s_bcast_word = 1;
        sm100::mbar_init(&s.full[0], 1);
        sm100::mbar_init(&s.full[1], 1);
        for (int i = 0; i < DF_NST; i++) sm100::mbar_init(&s.att_full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const df_params& p = s.p;
    if (s.n_items <= DF_ITEMS_SMEM) {
        // the item list is read on every item's critical path: keep it next to the SM
        unsigned char* tail = smem + (size_t)p.a_region + 2 * (size_t)p.slot_bytes;
        uint4* dst = reinterpret_cast<uint4*>(tail + DF_OFF_ITEMS);
        const uint4* src = reinterpret_cast<const uint4*>(s.items);
        for (int i = threadIdx.x; i < s.n_items * 4; i += DF_THREADS) dst[i] = src[i];
        __syncthreads();
        if (threadIdx.x == 0) s.items = reinterpret_cast<const df_item*>(dst);
        __syncthreads();
    }
    issue_item(s, 0);
    issue_item(s, 1);

    const int len0 = *p.len;
    bool alive = true;
    // embedding rows of the tokens this launch starts from
    prefetch_cache(p, 0, len0);
    if ((int)blockIdx.x < p.B) embed_row(p, blockIdx.x, p.cur[blockIdx.x], len0);
    alive = grid_sync(s);

    // Optional phase timing (TLNN_DECODE_PROF=1): thread 0 of every CTA adds the nanoseconds it spent in each phase and
    // in the barrier that follows it to p.prof[phase * 2 + {0, 1}]; the host divides by the number of CTAs.
    long long t_mark = p.prof ? clock64() : 0ll;
    auto lap = [&](int slot) {
        if (p.prof && threadIdx.x == 0) {
            const long long now = clock64();
            atomicAdd(p.prof + slot, (unsigned long long)(now - t_mark));
            t_mark = now;
        }
    };
    for (int step = 0; step < p.n_steps && alive; step++) {
        const int pos = len0 + step;
        for (int l = 0; l < p.L && alive; l++) {
            alive = run_phase(s, DF_QKV, l, step);
            lap(0);
            alive = alive && grid_sync(s);
            lap(1);
            if (!alive) break;
            if (p.hd == 64) alive = attention_phase<64>(s, l, pos);
            else if (p.hd == 32) alive = attention_phase<32>(s, l, pos);
            else alive = attention_phase<128>(s, l, pos);
            lap(2);
            alive = alive && grid_sync(s);
            lap(3);
            if (!alive) break;
            alive = run_phase(s, DF_OUT, l, step);
            lap(4);
            alive = alive && grid_sync(s);
            lap(5);
            if (!alive) break;
            // the next attention phase's cache: the next layer's at this position, or layer 0's at the next position
            if (l + 1 < p.L) prefetch_cache(p, l + 1, pos);
            else if (step + 1 < p.n_steps) prefetch_cache(p, 0, pos + 1);
            alive = run_phase(s, DF_FFN1, l, step);
            lap(6);
            alive = alive && grid_sync(s);
            lap(7);
            if (!alive) break;
            alive = run_phase(s, DF_FFN2, l, step);
            lap(8);
            alive = alive && grid_sync(s);
            lap(9);
        }
        if (!alive) break;
        // head: running arg-max of this CTA's vocabulary slices
        for (int i = threadIdx.x; i < DF_MMA_WARPS * 64; i += DF_THREADS) s.rowbest[i] = make_float2(-INFINITY, __int_as_float(0x7fffffff));
        __syncthreads();
        alive = run_phase(s, DF_HEAD, 0, step);
        if (!alive) break;
        lap(10);
        if (threadIdx.x < p.B) {
            float best = -INFINITY;
            int best_n = 0x7fffffff;
            for (int w = 0; w < DF_MMA_WARPS; w++) {
                const float2 rb = s.rowbest[w * 64 + threadIdx.x];
                const int n = __float_as_int(rb.y);
                if (rb.x > best || (rb.x == best && n < best_n)) { best = rb.x; best_n = n; }
            }
            p.cand[(size_t)blockIdx.x * 64 + threadIdx.x] = make_float2(best, __int_as_float(best_n));
        }
        alive = grid_sync(s);
        lap(11);
        if (!alive) break;
        // CTA b: arg-max of row b over the CTAs' candidates, the next token and its embedding row
        if ((int)blockIdx.x < p.B) {
            const int b = blockIdx.x;
            if (threadIdx.x < 32) {
                float best = -INFINITY;
                int best_n = 0x7fffffff;
                for (int c = threadIdx.x; c < (int)gridDim.x; c += 32) {
                    const float2 cb = __ldcg(p.cand + (size_t)c * 64 + b);
                    const int n = __float_as_int(cb.y);
                    if (cb.x > best || (cb.x == best && n < best_n)) { best = cb.x; best_n = n; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const int on = __shfl_xor_sync(0xffffffffu, best_n, o);
                    if (ov > best || (ov == best && on < best_n)) { best = ov; best_n = on; }
                }
                if (threadIdx.x == 0) {
                    if (best_n == 0x7fffffff) best_n = 0;                   // a row of NaN logits: keep the id in range
                    p.cur[b] = best_n;
                    if (p.tokens_out) p.tokens_out[(size_t)b * p.n_cols + step] = best_n;
                    s_bcast_word = best_n;
                }
            }
            __syncthreads();
            const int tok = s_bcast_word;
            if (step + 1 < p.n_steps) embed_row(p, b, tok, pos + 1);
        }
        lap(12);
        alive = grid_sync(s);
        lap(13);
    }
    // leave no copy in flight: wait (bounded) for every slot that was issued and not consumed
    for (long long g = s.cons; g < s.prod && g < s.total; g++)
        df_wait(&s.full[g & 1], (uint32_t)((g >> 1) & 1), s.s_abort, p.err, 702);
    if (alive && blockIdx.x == 0 && threadIdx.x == 0) *p.len = len0 + p.n_steps;
}

}  // namespace

// ---- host side ------------------------------------------------------------------------------------------------------------
int tl_decode_fused_plan(tlnn_ctx* ctx, const tlnn_gpt_model& m, const tlnn_block_params* blocks, int B, int max_len,
                         char* pack_base, bool use_pack, tl_decode_fused_plan_t* plan) {
    plan->ok = false;
    plan->pack_jobs.clear();
    plan->pack_bytes = 0;
    const int d = m.d, hd = m.d / m.heads;
    if (m.prec != TLNN_PREC_BF16 || B < 1 || B > 64 || d % 128 != 0 || d > 1024) return TLNN_OK;
    if (hd != 32 && hd != 64 && hd != 128) return TLNN_OK;
    if (m.layers < 1 || m.layers > 63) return TLNN_OK;
    // Opt-in (TLNN_DECODE_FUSED=1): on the 12-layer, 768-wide configuration the kernel is correct but, at about 1 ms per
    // step, still slower than the captured-graph path (0.66 ms per step); its 62 grid barriers per step (2.2 us each) and
    // the operand rows every CTA of a phase reads again bound it from below at about 0.4 ms.
    const char* env = getenv("TLNN_DECODE_FUSED");
    if (!env || strcmp(env, "1") != 0) return TLNN_OK;
    int dev_smem = 0, coop = 0;
    TL_CUDA(cudaDeviceGetAttribute(&dev_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device));
    TL_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
    if (!coop) return TLNN_OK;
    const int lda = d + 8;
    size_t a_bytes = (size_t)64 * lda * 2;
    if (a_bytes < (size_t)DF_RING_BYTES) a_bytes = DF_RING_BYTES;            // the attention ring lives in the operand rows' bytes
    // keys per chunk of the attention ring: every warp takes DF_ROUNDS rounds of 32 / (hd / 8) keys
    const int ck = DF_WARPS * (32 / (hd / 8)) * DF_ROUNDS;
    if ((size_t)DF_NST * 2 * ck * hd * 2 > a_bytes) {         // the TMA loads of the ring must stay inside the region
        tl_set_error("decode: attention ring of %d bytes does not fit its %zu-byte region", DF_NST * 2 * ck * hd * 2, a_bytes);
        return TLNN_ERR_VALUE;
    }
    plan->att_ck = ck;
    plan->a_region = (int)a_bytes;
    // features per item: two slots of (ns weight rows + ns bias values + gamma + beta) beside the operand rows and the tail
    const long long budget = ((long long)dev_smem - 256 - DF_TAIL_BYTES - (long long)a_bytes) / 2 - (long long)d * 8;
    int ns = (int)(budget / (lda * 2 + 4) / 16) * 16;
    if (ns > 64) ns = 64;
    if (ns < 16) return TLNN_OK;
    plan->ns = ns;
    plan->slot_bytes = ns * lda * 2 + ns * 4 + d * 8;
    plan->smem = a_bytes + 2 * (size_t)plan->slot_bytes + DF_TAIL_BYTES;
    plan->grid = ctx->sm_count;
    // the work items of one step, dealt round-robin over the CTAs in phase order
    std::vector<std::vector<df_item>> per(plan->grid);
    long long next = 0;
    auto deal = [&](int kind, int layer, int N, int k_ranges, const void* w, int ldw, const float* bias, const float* gamma, const float* beta) {
        for (int kq = 0; kq < k_ranges; kq++) {
            // the K range kq of this matrix in the packed copy: N rows of lda elements
            const size_t pack_off = plan->pack_bytes;
            if (use_pack) {
                plan->pack_jobs.push_back({static_cast<const __nv_bfloat16*>(w) + (size_t)kq * d, (size_t)ldw * 2, pack_off, (size_t)d * 2, (size_t)N});
                plan->pack_bytes += (size_t)N * lda * 2;
            }
            for (int n0 = 0; n0 < N; n0 += ns) {
                df_item it = {};
                it.kind = kind; it.layer = layer; it.n0 = n0; it.rows = N - n0 < ns ? N - n0 : ns; it.k0 = kq * d;
                if (use_pack) {
                    it.ldw = lda;
                    it.w = reinterpret_cast<const __nv_bfloat16*>(pack_base + pack_off) + (size_t)n0 * lda;
                } else {
                    it.ldw = ldw;
                    it.w = static_cast<const __nv_bfloat16*>(w) + (size_t)n0 * ldw + it.k0;
                }
                it.bias = kq == 0 ? bias : nullptr;            // the bias of a product split over K ranges goes with the first
                it.gamma = gamma; it.beta = beta;
                per[next++ % plan->grid].push_back(it);
            }
        }
    };
    for (int l = 0; l < m.layers; l++) {
        const tlnn_block_params& bp = blocks[l];
        deal(DF_QKV, l, 3 * d, 1, bp.wqkv_t, d, bp.bqkv, bp.ln1_gamma, bp.ln1_beta);
        deal(DF_OUT, l, d, 1, bp.wo_t, d, bp.bo, nullptr, nullptr);
        deal(DF_FFN1, l, 4 * d, 1, bp.w1_t, d, bp.b1, bp.ln2_gamma, bp.ln2_beta);
        deal(DF_FFN2, l, d, 4, bp.w2_t, 4 * d, bp.b2, nullptr, nullptr);
    }
    deal(DF_HEAD, 0, m.vocab, 1, m.head_t, d, m.head_bias, m.lnf_gamma, m.lnf_beta);
    size_t pitch = 1;
    for (auto& v : per) pitch = v.size() > pitch ? v.size() : pitch;
    plan->items_pitch = (int)pitch;
    plan->items.assign(pitch * plan->grid, df_item{});
    plan->counts.assign(plan->grid, 0);
    for (int c = 0; c < plan->grid; c++) {
        plan->counts[c] = (int)per[c].size();
        for (size_t i = 0; i < per[c].size(); i++) plan->items[(size_t)c * pitch + i] = per[c][i];
    }
    plan->hd = hd;
    plan->ok = true;
    return TLNN_OK;
}

int tl_decode_fused_launch(tlnn_ctx* ctx, const tl_decode_fused_plan_t& plan, const df_params& params) {
    void (*kernel)(const df_params, const CUtensorMap, const CUtensorMap) = decode_fused_kernel;
    static bool configured[1] = {false};
    const int which = 0;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem));
    if (!configured[which]) {
        int per_sm = 0;
        TL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, DF_THREADS, plan.smem));
        TL_REQUIRE(per_sm >= 1, "decode: the fused kernel does not fit an SM (%zu bytes of shared memory)", plan.smem);
        configured[which] = true;
    }
    TL_CUDA(cudaMemsetAsync(params.bar_flags, 0, 4096, ctx->stream));      // barrier flags (one word per CTA) and the abort flag
    df_params p = params;
    CUtensorMap kmap, vmap;
    const long long cache_rows = (long long)p.L * p.B * p.H * p.max_len;
    TL_TRY(sm100::make_plain_map(&kmap, p.kcache, cache_rows, p.hd, p.hd, p.hd, p.att_ck));
    TL_TRY(sm100::make_plain_map(&vmap, p.vcache, cache_rows, p.hd, p.hd, p.hd, p.att_ck));
    static const bool want_prof = getenv("TLNN_DECODE_PROF") && strcmp(getenv("TLNN_DECODE_PROF"), "1") == 0;
    unsigned long long* d_prof = nullptr;
    if (want_prof) {
        TL_CUDA(cudaMalloc(&d_prof, 32 * sizeof(unsigned long long)));
        TL_CUDA(cudaMemsetAsync(d_prof, 0, 32 * sizeof(unsigned long long), ctx->stream));
    }
    p.prof = d_prof;
    void* args[] = {&p, &kmap, &vmap};
    TL_TRY(tl_launch_begin(ctx, "decode_fused"));
    cudaLaunchCooperativeKernel((const void*)kernel, dim3(plan.grid), dim3(DF_THREADS), args, plan.smem, ctx->stream);
    TL_TRY(tl_launch_end(ctx, "decode_fused"));
    if (want_prof) {
        // debugging aid: mean microseconds per step a CTA spends in each phase and in the barrier after it
        unsigned long long h[32];
        TL_CUDA(cudaMemcpyAsync(h, d_prof, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream));
        TL_CUDA(cudaStreamSynchronize(ctx->stream));
        cudaFree(d_prof);
        static const char* names[7] = {"qkv", "attention", "out", "ffn1", "ffn2", "head", "next-token"};
        int khz = 1965000;
        cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device);      // the counters are SM cycles: scaled by the peak clock
        const double us_per_cycle = 1e3 / (double)khz;
        const double scale = us_per_cycle / ((double)plan.grid * p.n_steps);
        fprintf(stderr, "decode_fused phases, us per step at the peak SM clock (work + barrier):");
        for (int i = 0; i < 7; i++) fprintf(stderr, " %s %.1f+%.1f", names[i], h[2 * i] * scale, h[2 * i + 1] * scale);
        fprintf(stderr, "\n");
    }
    return TLNN_OK;
}
