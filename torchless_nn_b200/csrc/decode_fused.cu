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
constexpr int DF_TAIL_BYTES = 16384;           // barriers, K-split partials, per-warp arg-max rows
constexpr unsigned long long DF_WAIT_NS = 2000000000ull;

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

struct df_state {
    const df_params* p;
    bf16* A;                  // (64, lda) operand rows
    bf16* W[2];               // two weight slots, rows of lda elements
    uint64_t* full;           // [2] "slot filled" barriers
    float* red;               // K-split partial accumulators
    float2* rowbest;          // [DF_WARPS][64] running (value, index bits) of the head product
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
__device__ bool grid_sync(df_state& s) {
    const df_params& p = *s.p;
    s.epoch += gridDim.x;
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        __threadfence();
        atomicAdd(p.bar_count, 1u);
        if (ld_acquire_u32(p.bar_count) < s.epoch) {
            const unsigned long long t0 = sm100::globaltimer_ns();
            unsigned polls = 0;
            while (ld_acquire_u32(p.bar_count) < s.epoch) {
                if ((++polls & 255u) == 0) {
                    if (*reinterpret_cast<volatile int*>(p.abort_flag)) { ok = 0; break; }
                    if (sm100::globaltimer_ns() - t0 > DF_WAIT_NS) {
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
__device__ __forceinline__ const bf16* item_weight(const df_params& p, const df_item& it, int* ldw) {
    if (it.kind == DF_HEAD) { *ldw = p.d; return p.head + (size_t)it.n0 * p.d; }
    const df_layer& L = p.layers[it.layer];
    switch (it.kind) {
        case DF_QKV: *ldw = p.d; return L.wqkv + (size_t)it.n0 * p.d;
        case DF_OUT: *ldw = p.d; return L.wo + (size_t)it.n0 * p.d;
        case DF_FFN1: *ldw = p.d; return L.w1 + (size_t)it.n0 * p.d;
        default: *ldw = 4 * p.d; return L.w2 + (size_t)it.n0 * 4 * p.d + it.k0;
    }
}

// Warp 0 issues the row copies of item `g` (if any) into slot g & 1.  The slot's previous contents have been consumed
// (the caller passed a __syncthreads since the last read).
__device__ void issue_item(df_state& s, long long g) {
    if (g >= s.total || (threadIdx.x >> 5) != 0) return;
    const df_params& p = *s.p;
    const df_item it = s.items[g % s.n_items];
    const int slot = (int)(g & 1);
    const int lane = threadIdx.x & 31;
    int ldw;
    const bf16* src = item_weight(p, it, &ldw);
    const uint32_t row_bytes = (uint32_t)p.d * 2u;
    const uint32_t bar = sm100::smem_u32(&s.full[slot]);
    if (lane == 0) {
        sm100::fence_async_smem();          // the slot was last read through the generic proxy
        sm100::mbar_expect_tx(&s.full[slot], row_bytes * (uint32_t)it.rows);
    }
    __syncwarp();
    for (int r = lane; r < it.rows; r += 32)
        bulk_g2s(sm100::smem_u32(s.W[slot] + (size_t)r * s.lda), src + (size_t)r * ldw, row_bytes, bar);
}

// ---- operand rows -------------------------------------------------------------------------------------------------------
// A[m, :] = LayerNorm(x[m, :]) as bf16, mean and biased variance in two passes over the row held in registers.
template <int V4>      // float4 loads per lane per row (d = 128 * V4)
__device__ void load_a_layernorm_t(df_state& s, const float* x, const float* __restrict__ gamma, const float* __restrict__ beta) {
    const df_params& p = *s.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = p.d;
    const float inv_d = 1.f / (float)d;
    for (int m = warp; m < p.B; m += DF_WARPS) {
        const float4* row = reinterpret_cast<const float4*>(x + (size_t)m * d);
        float4 v[V4];
#pragma unroll
        for (int i = 0; i < V4; i++) v[i] = __ldcg(row + lane + 32 * i);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < V4; i++) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum * inv_d;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < V4; i++) {
            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
            sq += (a * a + b * b) + (c * c + e * e);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float rstd = 1.f / sqrtf(sq * inv_d + 1e-5f);
        bf16* dst = s.A + (size_t)m * s.lda;
#pragma unroll
        for (int i = 0; i < V4; i++) {
            const int c = (lane + 32 * i) * 4;
            const float4 g = __ldg(reinterpret_cast<const float4*>(gamma + c));
            const float4 b = __ldg(reinterpret_cast<const float4*>(beta + c));
            uint2 o;
            o.x = pack_bf16((v[i].x - mean) * rstd * g.x + b.x, (v[i].y - mean) * rstd * g.y + b.y);
            o.y = pack_bf16((v[i].z - mean) * rstd * g.z + b.z, (v[i].w - mean) * rstd * g.w + b.w);
            *reinterpret_cast<uint2*>(dst + c) = o;
        }
    }
}

__device__ void load_a_layernorm(df_state& s, const float* x, const float* gamma, const float* beta) {
    switch (s.p->d / 128) {
        case 1: load_a_layernorm_t<1>(s, x, gamma, beta); break;
        case 2: load_a_layernorm_t<2>(s, x, gamma, beta); break;
        case 3: load_a_layernorm_t<3>(s, x, gamma, beta); break;
        case 4: load_a_layernorm_t<4>(s, x, gamma, beta); break;
        case 5: load_a_layernorm_t<5>(s, x, gamma, beta); break;
        case 6: load_a_layernorm_t<6>(s, x, gamma, beta); break;
        case 7: load_a_layernorm_t<7>(s, x, gamma, beta); break;
        default: load_a_layernorm_t<8>(s, x, gamma, beta); break;
    }
}

// A[m, 0:d] = src[m, k0:k0+d] (bf16 rows of pitch lds), 16 bytes per load, eight loads in flight per thread
__device__ void load_a_copy(df_state& s, const bf16* src, int lds, int k0) {
    const df_params& p = *s.p;
    const int chunks = p.d / 8;                     // 16-byte chunks per row
    const int total = p.B * chunks;
    for (int base = threadIdx.x; base < total; base += DF_THREADS * 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = base + u * DF_THREADS;
            if (i < total) {
                const int m = i / chunks, c = i % chunks;
                v[u] = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)m * lds + k0 + c * 8));
            }
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = base + u * DF_THREADS;
            if (i < total) {
                const int m = i / chunks, c = i % chunks;
                *reinterpret_cast<uint4*>(s.A + (size_t)m * s.lda + c * 8) = v[u];
            }
        }
    }
}

// ---- one work item: (B x d) operand rows times `rows` weight rows --------------------------------------------------
// Accumulate the 16 x 16 output tile (m_tile, npi) over K range [k_begin, k_begin + klen).
__device__ __forceinline__ void mma_task(uint32_t a_base, uint32_t w_base, uint32_t row_pitch, int m_tile, int npi, int k_begin,
                                         int klen, int lane, float (&c)[2][4]) {
    float acc[2][2][4] = {};
    // ldmatrix rows: A  m_tile*16 + lane%16 at k + (lane/16)*8;  W  npi*16 + lane%8 + (lane/16)*8 at k + ((lane/8)&1)*8
    const uint32_t a_addr = a_base + (uint32_t)(m_tile * 16 + (lane & 15)) * row_pitch + (uint32_t)((lane >> 4) * 8 + k_begin) * 2u;
    const uint32_t w_addr = w_base + (uint32_t)(npi * 16 + (lane & 7) + (lane >> 4) * 8) * row_pitch + (uint32_t)(((lane >> 3) & 1) * 8 + k_begin) * 2u;
#pragma unroll 4
    for (int k = 0; k < klen; k += 16) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, a_addr + k * 2);
        ldmatrix_x4(b, w_addr + k * 2);
        const int set = (k >> 4) & 1;               // two accumulator sets shorten the dependent chain
        mma_16816(acc[set][0], a, b[0], b[1]);
        mma_16816(acc[set][1], a, b[2], b[3]);
    }
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) c[j][i] = acc[0][j][i] + acc[1][j][i];
}

// What happens to a finished 16 x 16 tile.  Called by whole warps (the head's arg-max uses shuffles).
__device__ __forceinline__ void item_epilogue(df_state& s, const df_item& it, int m_tile, int npi, int warp, int lane, const float (&c)[2][4]) {
    const df_params& p = *s.p;
    const int g = lane >> 2, q2 = (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int m = m_tile * 16 + g + half * 8;
        const bool row_ok = m < p.B;
        float best = -INFINITY;
        int best_n = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int nl = npi * 16 + j * 8 + q2;            // feature inside the item
            if (!row_ok || nl >= it.rows) continue;
            const int n = it.n0 + nl;
            float v0 = c[j][half * 2], v1 = c[j][half * 2 + 1];
            if (it.kind == DF_HEAD) {
                const bool has1 = nl + 1 < it.rows;           // the last vocabulary slice may end on an odd row
                if (p.head_bias) { v0 += __ldg(p.head_bias + n); if (has1) v1 += __ldg(p.head_bias + n + 1); }
                if (v0 > best) { best = v0; best_n = n; }
                if (has1 && v1 > best) { best = v1; best_n = n + 1; }
                continue;
            }
            const df_layer& L = p.layers[it.layer];
            if (it.kind == DF_QKV) {
                if (L.bqkv) { v0 += __ldg(L.bqkv + n); v1 += __ldg(L.bqkv + n + 1); }
                *reinterpret_cast<uint32_t*>(p.qkv + (size_t)m * 3 * p.d + n) = pack_bf16(v0, v1);
            } else if (it.kind == DF_OUT) {
                if (L.bo) { v0 += __ldg(L.bo + n); v1 += __ldg(L.bo + n + 1); }
                float2* dst = reinterpret_cast<float2*>(p.x + (size_t)m * p.d + n);
                float2 old = __ldcg(dst);
                old.x += v0; old.y += v1;
                *dst = old;
            } else if (it.kind == DF_FFN1) {
                if (L.b1) { v0 += __ldg(L.b1 + n); v1 += __ldg(L.b1 + n + 1); }
                *reinterpret_cast<uint32_t*>(p.hid + (size_t)m * 4 * p.d + n) = pack_bf16(activate(p.act, v0), activate(p.act, v1));
            } else {   // DF_FFN2: one of the four K ranges of the product; the bias goes with range 0
                if (it.k0 == 0 && L.b2) { v0 += __ldg(L.b2 + n); v1 += __ldg(L.b2 + n + 1); }
                atomicAdd(p.x + (size_t)m * p.d + n, v0);
                atomicAdd(p.x + (size_t)m * p.d + n + 1, v1);
            }
        }
        if (it.kind == DF_HEAD) {       // uniform over the warp
            // the four lanes of a row hold disjoint columns: keep the largest value, the lowest index among equals
#pragma unroll
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

__device__ bool run_item(df_state& s, const df_item& it, int step) {
    const df_params& p = *s.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = (int)(s.cons & 1);
    // operand rows for this item (kept across consecutive items of one phase)
    const int tag = ((it.kind * 64 + it.layer) * 8 + (it.kind == DF_FFN2 ? it.k0 / p.d : 0)) * 4096 + (step & 4095);
    if (tag != s.a_tag) {
        if (it.kind == DF_HEAD) load_a_layernorm(s, p.x, p.lnf_g, p.lnf_b);
        else {
            const df_layer& L = p.layers[it.layer];
            if (it.kind == DF_QKV) load_a_layernorm(s, p.x, L.ln1_g, L.ln1_b);
            else if (it.kind == DF_FFN1) load_a_layernorm(s, p.x, L.ln2_g, L.ln2_b);
            else if (it.kind == DF_OUT) load_a_copy(s, p.att, p.d, 0);
            else load_a_copy(s, p.hid, 4 * p.d, it.k0);
        }
        s.a_tag = tag;
        __syncthreads();
    }
    // weights of this item
    if (!sm100::mbar_wait(&s.full[slot], (uint32_t)((s.cons >> 1) & 1), s.s_abort, p.err, 701, DF_WAIT_NS)) return false;

    const int mt = (p.B + 15) >> 4;
    const int np = (it.rows + 15) >> 4;
    const int tasks = mt * np;
    const uint32_t a_base = sm100::smem_u32(s.A), w_base = sm100::smem_u32(s.W[slot]);
    const uint32_t row_pitch = (uint32_t)s.lda * 2u;
    if (tasks >= DF_WARPS) {
        for (int t = warp; t < tasks; t += DF_WARPS) {
            float c[2][4];
            mma_task(a_base, w_base, row_pitch, t % mt, t / mt, 0, p.d, lane, c);
            item_epilogue(s, it, t % mt, t / mt, warp, lane, c);
        }
    } else {
        // fewer tiles than warps: the contraction is split over warps, partial sums meet in shared memory in a fixed order
        int ksplit = DF_WARPS / tasks;
        while (ksplit & (ksplit - 1)) ksplit &= ksplit - 1;                   // round down to a power of two
        while (ksplit > 1 && (p.d / ksplit) % 16 != 0) ksplit >>= 1;
        const int t = warp % tasks, kpart = warp / tasks;
        const bool active = kpart < ksplit;
        const int klen = p.d / ksplit;
        float c[2][4];
        if (active) mma_task(a_base, w_base, row_pitch, t % mt, t / mt, kpart * klen, klen, lane, c);
        if (ksplit > 1) {
            if (active && kpart > 0) {
                float* dst = s.red + ((size_t)(kpart - 1) * tasks + t) * 256 + lane * 8;
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) dst[j * 4 + i] = c[j][i];
            }
            __syncthreads();
            if (kpart == 0) {
                for (int q = 1; q < ksplit; q++) {
                    const float* r = s.red + ((size_t)(q - 1) * tasks + t) * 256 + lane * 8;
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int i = 0; i < 4; i++) c[j][i] += r[j * 4 + i];
                }
            }
        }
        if (kpart == 0) item_epilogue(s, it, t % mt, t / mt, warp, lane, c);
    }
    __syncthreads();                                 // all reads of the slot (and of the partial sums) are done
    issue_item(s, s.prod);
    s.prod++;
    s.cons++;
    return true;
}

// All items of this CTA that belong to (kind, layer) at the head of its list.
__device__ bool run_phase(df_state& s, int kind, int layer, int step) {
    const long long step_end = (long long)(step + 1) * s.n_items;          // never run into the next step's items
    while (s.cons < step_end) {
        const df_item it = s.items[s.cons % s.n_items];
        if (it.kind != kind || (kind != DF_HEAD && it.layer != layer)) break;
        if (!run_item(s, it, step)) return false;
    }
    return true;
}

// ---- attention over the cache: one warp per (sequence, head) ---------------------------------------------------------
template <int HD>
__device__ void attention_phase(df_state& s, int layer, int pos) {
    constexpr int TPR = HD / 8;                    // lanes per key row (16 bytes each)
    constexpr int KPP = 32 / TPR;                  // keys per warp-wide load
    constexpr int U = 8;                           // loads in flight per lane
    const df_params& p = *s.p;
    const df_layer& L = p.layers[layer];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % TPR, grp = lane / TPR;
    const int d = p.d, H = p.H;
    const float inv = rsqrtf((float)HD);
    float* sc = reinterpret_cast<float*>(s.A) + (size_t)warp * p.max_len;      // this warp's scores (A is idle here)
    for (int u = warp * gridDim.x + blockIdx.x; u < p.B * H; u += DF_WARPS * gridDim.x) {
        const int b = u / H, h = u % H;
        const bf16* row = p.qkv + (size_t)b * 3 * d + h * HD + sub * 8;
        bf16* kbase = L.kcache + (size_t)b * p.max_len * d + h * HD + sub * 8;
        bf16* vbase = L.vcache + (size_t)b * p.max_len * d + h * HD + sub * 8;
        const uint4 qraw = __ldcg(reinterpret_cast<const uint4*>(row));
        const uint4 kraw = __ldcg(reinterpret_cast<const uint4*>(row + d));
        const uint4 vraw = __ldcg(reinterpret_cast<const uint4*>(row + 2 * d));
        if (grp == 0) {                             // append this step's key and value rows
            *reinterpret_cast<uint4*>(kbase + (size_t)pos * d) = kraw;
            *reinterpret_cast<uint4*>(vbase + (size_t)pos * d) = vraw;
        }
        float q[8];
        {
            const bf16* e = reinterpret_cast<const bf16*>(&qraw);
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = __bfloat162float(e[i]);
        }
        auto dot8 = [&](const uint4& raw) {
            const bf16* e = reinterpret_cast<const bf16*>(&raw);
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) a = fmaf(q[i], __bfloat162float(e[i]), a);
#pragma unroll
            for (int o = TPR / 2; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            return a * inv;
        };
        const float s_new = dot8(kraw);
        float mx = s_new;
        // scores of the cached keys [0, pos)
        for (int k0 = 0; k0 < pos; k0 += KPP * U) {
            uint4 raw[U] = {};
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int k = k0 + j * KPP + grp;
                if (k < pos) raw[j] = __ldcg(reinterpret_cast<const uint4*>(kbase + (size_t)k * d));
            }
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int k = k0 + j * KPP + grp;
                const float v = dot8(raw[j]);        // every lane takes part in the shuffles; stale data past the end is discarded
                if (k < pos) {
                    if (sub == 0) sc[k] = v;
                    mx = fmaxf(mx, v);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        __syncwarp();
        float sum = 0.f;
        for (int k = lane; k < pos; k += 32) {
            const float e = __expf(sc[k] - mx);
            sc[k] = e;
            sum += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float p_new = __expf(s_new - mx);
        sum += p_new;
        __syncwarp();
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = 0.f;
        for (int k0 = 0; k0 < pos; k0 += KPP * U) {
            uint4 raw[U] = {};
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int k = k0 + j * KPP + grp;
                if (k < pos) raw[j] = __ldcg(reinterpret_cast<const uint4*>(vbase + (size_t)k * d));
            }
#pragma unroll
            for (int j = 0; j < U; j++) {
                const int k = k0 + j * KPP + grp;
                if (k < pos) {
                    const float w = sc[k];
                    const bf16* e = reinterpret_cast<const bf16*>(&raw[j]);
#pragma unroll
                    for (int i = 0; i < 8; i++) acc[i] = fmaf(w, __bfloat162float(e[i]), acc[i]);
                }
            }
        }
#pragma unroll
        for (int o = TPR; o < 32; o <<= 1)
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
        if (grp == 0) {
            const bf16* e = reinterpret_cast<const bf16*>(&vraw);
            const float rs = 1.f / sum;
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int i = 0; i < 4; i++)
                ow[i] = pack_bf16((acc[2 * i] + p_new * __bfloat162float(e[2 * i])) * rs,
                                  (acc[2 * i + 1] + p_new * __bfloat162float(e[2 * i + 1])) * rs);
            *reinterpret_cast<uint4*>(p.att + (size_t)b * d + h * HD + sub * 8) = o;
        }
        __syncwarp();
    }
    s.a_tag = -1;                                    // the scores overwrote the operand rows
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

template <int HD>
__global__ void __launch_bounds__(DF_THREADS, 1) decode_fused_kernel(const df_params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort_word, s_bcast_word;
    df_state s;
    s.p = &p;
    s.lda = p.d + 8;
    const size_t a_bytes = (size_t)64 * s.lda * 2;
    s.A = reinterpret_cast<bf16*>(smem);
    s.W[0] = reinterpret_cast<bf16*>(smem + a_bytes);
    s.W[1] = reinterpret_cast<bf16*>(smem + a_bytes + p.slot_bytes);
    unsigned char* tail = smem + a_bytes + 2 * (size_t)p.slot_bytes;
    s.full = reinterpret_cast<uint64_t*>(tail);
    s.red = reinterpret_cast<float*>(tail + 64);                              // (K ranges - 1) x tiles x 256 floats: 7 KB at most
    s.rowbest = reinterpret_cast<float2*>(tail + 64 + 8192);                  // 8 x 64 x 8 bytes
    s.s_abort = &s_abort_word;
    s.s_bcast = &s_bcast_word;
    s.items = p.items + (size_t)blockIdx.x * p.items_pitch;
    s.n_items = p.item_counts[blockIdx.x];
    s.total = (long long)s.n_items * p.n_steps;
    s.cons = 0;
    s.prod = 0;
    s.epoch = 0;
    s.a_tag = -1;
    if (threadIdx.x == 0) {
        s_abort_word = 0;
        s_bcast_word = 1;
        sm100::mbar_init(&s.full[0], 1);
        sm100::mbar_init(&s.full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    issue_item(s, 0);
    issue_item(s, 1);
    s.prod = 2;

    const int len0 = *p.len;
    bool alive = true;
    // embedding rows of the tokens this launch starts from
    if ((int)blockIdx.x < p.B) embed_row(p, blockIdx.x, p.cur[blockIdx.x], len0);
    alive = grid_sync(s);

    // Optional phase timing (TLNN_DECODE_PROF=1): thread 0 of every CTA adds the nanoseconds it spent in each phase and
    // in the barrier that follows it to p.prof[phase * 2 + {0, 1}]; the host divides by the number of CTAs.
    unsigned long long t_mark = p.prof ? sm100::globaltimer_ns() : 0ull;
    auto lap = [&](int slot) {
        if (p.prof && threadIdx.x == 0) {
            const unsigned long long now = sm100::globaltimer_ns();
            atomicAdd(p.prof + slot, now - t_mark);
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
            attention_phase<HD>(s, l, pos);
            lap(2);
            alive = grid_sync(s);
            lap(3);
            if (!alive) break;
            alive = run_phase(s, DF_OUT, l, step);
            lap(4);
            alive = alive && grid_sync(s);
            lap(5);
            if (!alive) break;
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
        for (int i = threadIdx.x; i < DF_WARPS * 64; i += DF_THREADS) s.rowbest[i] = make_float2(-INFINITY, __int_as_float(0x7fffffff));
        __syncthreads();
        alive = run_phase(s, DF_HEAD, 0, step);
        if (!alive) break;
        lap(10);
        if (threadIdx.x < p.B) {
            float best = -INFINITY;
            int best_n = 0x7fffffff;
            for (int w = 0; w < DF_WARPS; w++) {
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
        sm100::mbar_wait(&s.full[g & 1], (uint32_t)((g >> 1) & 1), s.s_abort, p.err, 702, DF_WAIT_NS);
    if (alive && blockIdx.x == 0 && threadIdx.x == 0) *p.len = len0 + p.n_steps;
}

}  // namespace

// ---- host side ------------------------------------------------------------------------------------------------------------
int tl_decode_fused_plan(tlnn_ctx* ctx, const tlnn_gpt_model& m, int B, int max_len, tl_decode_fused_plan_t* plan) {
    plan->ok = false;
    const int d = m.d, hd = m.d / m.heads;
    if (m.prec != TLNN_PREC_BF16 || B < 1 || B > 64 || d % 128 != 0 || d > 1024) return TLNN_OK;
    if (hd != 32 && hd != 64 && hd != 128) return TLNN_OK;
    if (m.layers < 1 || m.layers > 63) return TLNN_OK;
    const char* env = getenv("TLNN_DECODE_FUSED");
    if (env && strcmp(env, "0") == 0) return TLNN_OK;
    int dev_smem = 0, coop = 0;
    TL_CUDA(cudaDeviceGetAttribute(&dev_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device));
    TL_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
    if (!coop) return TLNN_OK;
    const int lda = d + 8;
    const size_t a_bytes = (size_t)64 * lda * 2;
    if ((size_t)DF_WARPS * max_len * 4 > a_bytes) return TLNN_OK;           // the attention scores live in the operand buffer
    const long long budget = (long long)dev_smem - DF_TAIL_BYTES - (long long)a_bytes - 1024;
    int ns = (int)(budget / 2 / (lda * 2) / 16) * 16;
    if (ns > 64) ns = 64;
    if (const char* e = getenv("TLNN_DF_NS")) { const int v = atoi(e); if (v >= 16 && v <= ns && v % 16 == 0) ns = v; }   // experiments
    if (ns < 16) return TLNN_OK;
    plan->ns = ns;
    plan->slot_bytes = ns * lda * 2;
    plan->smem = a_bytes + 2 * (size_t)plan->slot_bytes + DF_TAIL_BYTES;
    plan->grid = ctx->sm_count;
    if (const char* e = getenv("TLNN_DF_GRID")) { const int v = atoi(e); if (v >= 64 && v <= ctx->sm_count) plan->grid = v; }   // experiments
    // the work items of one step, dealt round-robin over the CTAs in phase order
    std::vector<std::vector<df_item>> per(plan->grid);
    long long next = 0;
    auto deal = [&](int kind, int layer, int N, int k_ranges) {
        for (int kq = 0; kq < k_ranges; kq++)
            for (int n0 = 0; n0 < N; n0 += ns) {
                df_item it = {};
                it.kind = kind; it.layer = layer; it.n0 = n0; it.rows = N - n0 < ns ? N - n0 : ns; it.k0 = kq * d;
                per[next++ % plan->grid].push_back(it);
            }
    };
    for (int l = 0; l < m.layers; l++) {
        deal(DF_QKV, l, 3 * d, 1);
        deal(DF_OUT, l, d, 1);
        deal(DF_FFN1, l, 4 * d, 1);
        deal(DF_FFN2, l, d, 4);
    }
    deal(DF_HEAD, 0, m.vocab, 1);
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
    void (*kernel)(const df_params) = plan.hd == 32 ? decode_fused_kernel<32> : plan.hd == 64 ? decode_fused_kernel<64> : decode_fused_kernel<128>;
    static bool configured[3] = {false, false, false};
    const int which = plan.hd == 32 ? 0 : plan.hd == 64 ? 1 : 2;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem));
    if (!configured[which]) {
        int per_sm = 0;
        TL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, DF_THREADS, plan.smem));
        TL_REQUIRE(per_sm >= 1, "decode: the fused kernel does not fit an SM (%zu bytes of shared memory)", plan.smem);
        configured[which] = true;
    }
    TL_CUDA(cudaMemsetAsync(params.bar_count, 0, 8, ctx->stream));          // arrival counter and abort flag
    df_params p = params;
    static const bool want_prof = getenv("TLNN_DECODE_PROF") && strcmp(getenv("TLNN_DECODE_PROF"), "1") == 0;
    unsigned long long* d_prof = nullptr;
    if (want_prof) {
        TL_CUDA(cudaMalloc(&d_prof, 16 * sizeof(unsigned long long)));
        TL_CUDA(cudaMemsetAsync(d_prof, 0, 16 * sizeof(unsigned long long), ctx->stream));
    }
    p.prof = d_prof;
    void* args[] = {&p};
    TL_TRY(tl_launch_begin(ctx, "decode_fused"));
    cudaLaunchCooperativeKernel((const void*)kernel, dim3(plan.grid), dim3(DF_THREADS), args, plan.smem, ctx->stream);
    TL_TRY(tl_launch_end(ctx, "decode_fused"));
    if (want_prof) {
        // debugging aid: mean microseconds per step a CTA spends in each phase and in the barrier after it
        unsigned long long h[16];
        TL_CUDA(cudaMemcpyAsync(h, d_prof, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream));
        TL_CUDA(cudaStreamSynchronize(ctx->stream));
        cudaFree(d_prof);
        static const char* names[7] = {"qkv", "attention", "out", "ffn1", "ffn2", "head", "next-token"};
        const double scale = 1e-3 / ((double)plan.grid * p.n_steps);
        fprintf(stderr, "decode_fused phases, us per step (work + barrier):");
        for (int i = 0; i < 7; i++) fprintf(stderr, " %s %.1f+%.1f", names[i], h[2 * i] * scale, h[2 * i + 1] * scale);
        fprintf(stderr, "\n");
    }
    return TLNN_OK;
}
