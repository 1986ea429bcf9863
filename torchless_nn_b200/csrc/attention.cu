// Fused attention: softmax(Q K^T / sqrt(hd) [+ causal mask]) V without materialising the score matrix.
//
// Input is the packed projection (B, T, 3d) produced by the QKV GEMM (columns [0,d) Q, [d,2d) K, [2d,3d) V; head h
// at columns h*hd inside each third), so no head-major copy is ever made; output is written merged as (B, T, d).
// The decoder mask of the reference (-1e9 above the diagonal, exp underflows to exactly 0 in float32) is applied as
// an index comparison.
//
//  * bf16 path: flash-style kernel, 128 queries x 64 keys per step, 8 warps, operands staged with cp.async into
//    XOR-swizzled shared memory, ldmatrix + mma.sync m16n8k16 (bf16 in, float32 accumulate), online softmax in
//    registers with quad shuffles, exp2 with the 1/sqrt(hd) scale folded in.
//  * float32 path: CUDA-core kernels in exact float32 arithmetic for the FP32/TF32 mode, where the shapes are small
//    (T <= 128 or a ViT's 65 / 257 tokens, hd 32) and operand rounding would eat the tolerance: head dimensions up to
//    64 keep each query in the registers of one thread (or of four lanes when the grid is small), 96 and 128 use one
//    warp per query with the keys across lanes.
#include "common.cuh"
#include <cstdlib>

namespace {

// ============================================================================================ bf16 flash kernel
constexpr int FA_BM = 128;   // queries per CTA
constexpr int FA_BN = 64;    // keys per step
constexpr int FA_THREADS = 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    int bytes = valid ? 16 : 0;   // src-size 0 zero-fills the 16 destination bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold HD bf16; the chunk index is XOR-ed
// with row bits so that the eight rows touched by one ldmatrix phase fall into distinct banks.
template <int HD>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    constexpr int ROWB = HD * 2;
    int sw = HD == 32 ? ((row >> 1) & 3) : (row & 7);
    return (uint32_t)(row * ROWB + ((chunk ^ sw) << 4));
}

template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst_base, const __nv_bfloat16* src, long long row_stride, int row0,
                                          int rows, int T) {
    constexpr int CPR = HD / 8;   // 16-byte chunks per row
    const uint32_t dst = smem_u32(dst_base);
    for (int i = threadIdx.x; i < rows * CPR; i += FA_THREADS) {
        int r = i / CPR, c = i % CPR;
        int t = row0 + r;
        bool ok = t < T;
        const __nv_bfloat16* p = src + (long long)(ok ? t : 0) * row_stride + c * 8;
        cp_async16(dst + swz<HD>(r, c), p, ok);
    }
}

template <int HD, bool CAUSAL>
__global__ void __launch_bounds__(FA_THREADS, HD <= 64 ? 2 : 1)
flash_bf16_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out, int T, int H, float scale_log2) {
    constexpr int KSTEPS = HD / 16;       // k-steps of the S = Q K^T product
    constexpr int DT = HD / 8;            // 8-wide output column tiles
    constexpr int NT = FA_BN / 8;         // 8-wide key tiles per step
    extern __shared__ __align__(128) uint8_t fa_smem[];
    uint8_t* sQ = fa_smem;
    uint8_t* sK = sQ + FA_BM * HD * 2;
    uint8_t* sV = sK + 2 * FA_BN * HD * 2;

    const int d = H * HD;
    const long long row_stride = 3ll * d;
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int q_tile = CAUSAL ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;   // longest causal tiles first
    const int q0 = q_tile * FA_BM;
    const __nv_bfloat16* qbase = qkv + (long long)b * T * row_stride + h * HD;
    const __nv_bfloat16* kbase = qbase + d;
    const __nv_bfloat16* vbase = qbase + 2 * d;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int wrow0 = warp * 16;                     // first query row of this warp inside the tile

    int kv_end = T;
    if (CAUSAL) kv_end = min(T, q0 + FA_BM);
    const int n_steps = (kv_end + FA_BN - 1) / FA_BN;

    load_tile<HD>(sQ, qbase, row_stride, q0, FA_BM, T);
    load_tile<HD>(sK, kbase, row_stride, 0, FA_BN, T);
    load_tile<HD>(sV, vbase, row_stride, 0, FA_BN, T);
    cp_async_commit();

    uint32_t qf[KSTEPS][4];
    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY;     // running maxima (already multiplied by scale_log2) of rows g and g+8
    float l0 = 0.f, l1 = 0.f;                 // running partial sums (this thread's columns only)

    for (int j = 0; j < n_steps; j++) {
        const int buf = j & 1;
        if (j + 1 < n_steps) {
            load_tile<HD>(sK + (buf ^ 1) * FA_BN * HD * 2, kbase, row_stride, (j + 1) * FA_BN, FA_BN, T);
            load_tile<HD>(sV + (buf ^ 1) * FA_BN * HD * 2, vbase, row_stride, (j + 1) * FA_BN, FA_BN, T);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (j == 0) {
            const uint32_t q_s = smem_u32(sQ);
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                int row = wrow0 + (lane & 7) + ((lane >> 3) & 1) * 8;
                int chunk = ks * 2 + (lane >> 4);
                ldmatrix_x4(q_s + swz<HD>(row, chunk), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
            }
        }
        const int key0 = j * FA_BN;
        // A warp whose every query precedes every key of this step has nothing to add (causal only).
        const bool active = !CAUSAL || key0 <= q0 + wrow0 + 15;
        if (active) {
            const uint32_t k_s = smem_u32(sK + buf * FA_BN * HD * 2);
            const uint32_t v_s = smem_u32(sV + buf * FA_BN * HD * 2);
            float s[NT][4];
#pragma unroll
            for (int i = 0; i < NT; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
                for (int nt = 0; nt < NT; nt += 2) {
                    uint32_t b0, b1, b2, b3;
                    int key = nt * 8 + (lane & 7) + (lane >> 4) * 8;
                    int chunk = ks * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(k_s + swz<HD>(key, chunk), b0, b1, b2, b3);
                    mma_bf16(s[nt], qf[ks], b0, b1);
                    mma_bf16(s[nt + 1], qf[ks], b2, b3);
                }
            }
            // masking: keys beyond the sequence end, and keys after the query for the decoder
            const bool need_mask = (key0 + FA_BN > T) || (CAUSAL && key0 + FA_BN - 1 > q0 + wrow0);
            if (need_mask) {
                const int r0 = q0 + wrow0 + g, r1 = r0 + 8;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    int c = key0 + nt * 8 + tq * 2;
                    bool dead0 = c >= T, dead1 = c + 1 >= T;
                    if ((CAUSAL && c > r0) || dead0) s[nt][0] = -INFINITY;
                    if ((CAUSAL && c + 1 > r0) || dead1) s[nt][1] = -INFINITY;
                    if ((CAUSAL && c > r1) || dead0) s[nt][2] = -INFINITY;
                    if ((CAUSAL && c + 1 > r1) || dead1) s[nt][3] = -INFINITY;
                }
            }
            // online softmax
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0 * scale_log2), mn1 = fmaxf(m1, mx1 * scale_log2);
            // a row with no live key yet keeps m = -inf; use 0 as the subtrahend there so exp2(-inf - 0) = 0
            const float sub0 = mn0 == -INFINITY ? 0.f : mn0, sub1 = mn1 == -INFINITY ? 0.f : mn1;
            const float a0 = exp2f(m0 - sub0), a1 = exp2f(m1 - sub1);
            m0 = mn0; m1 = mn1;
            l0 *= a0; l1 *= a1;
#pragma unroll
            for (int i = 0; i < DT; i++) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
            uint32_t pf[NT / 2][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float p0 = exp2f(fmaf(s[nt][0], scale_log2, -sub0));
                float p1 = exp2f(fmaf(s[nt][1], scale_log2, -sub0));
                float p2 = exp2f(fmaf(s[nt][2], scale_log2, -sub1));
                float p3 = exp2f(fmaf(s[nt][3], scale_log2, -sub1));
                l0 += p0 + p1;
                l1 += p2 + p3;
                pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < FA_BN / 16; kk++) {
#pragma unroll
                for (int dt = 0; dt < DT; dt += 2) {
                    uint32_t b0, b1, b2, b3;
                    int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    int chunk = dt + (lane >> 4);
                    ldmatrix_x4_trans(v_s + swz<HD>(key, chunk), b0, b1, b2, b3);
                    mma_bf16(o[dt], pf[kk], b0, b1);
                    mma_bf16(o[dt + 1], pf[kk], b2, b3);
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before the next prefetch overwrites it
    }

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
    const int r0 = q0 + wrow0 + g, r1 = r0 + 8;
    __nv_bfloat16* obase = out + (long long)b * T * d + h * HD;
#pragma unroll
    for (int dt = 0; dt < DT; dt++) {
        int c = dt * 8 + tq * 2;
        if (r0 < T) *reinterpret_cast<uint32_t*>(obase + (long long)r0 * d + c) = pack_bf16(o[dt][0] * inv0, o[dt][1] * inv0);
        if (r1 < T) *reinterpret_cast<uint32_t*>(obase + (long long)r1 * d + c) = pack_bf16(o[dt][2] * inv1, o[dt][3] * inv1);
    }
}

// ============================================================================================ float32 kernel
constexpr int F32_QPB = 16;     // queries per CTA (4 warps x 4 queries)

__device__ __forceinline__ float round_tf32(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x00000fffu + ((u >> 13) & 1u);
    u &= 0xffffe000u;
    return __uint_as_float(u);
}

template <int HD, bool CAUSAL>
__global__ void __launch_bounds__(128)
attention_f32_kernel(const float* __restrict__ qkv, float* __restrict__ out, int T, int H, float inv_sqrt_hd, int round_out) {
    constexpr int DPL = HD / 32;                 // output dims per lane
    constexpr int F32_KT = HD <= 64 ? 64 : 32;   // keys per shared-memory tile (static shared memory stays under 48 KB)
    __shared__ float sQ[F32_QPB][HD];
    __shared__ float sK[F32_KT][HD + 1];
    __shared__ float sV[F32_KT][HD];

    const int d = H * HD;
    const long long row_stride = 3ll * d;
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int q0 = blockIdx.x * F32_QPB;
    const float* qbase = qkv + (long long)b * T * row_stride + h * HD;
    const float* kbase = qbase + d;
    const float* vbase = qbase + 2 * d;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int i = threadIdx.x; i < F32_QPB * HD; i += 128) {
        int r = i / HD, c = i % HD;
        sQ[r][c] = (q0 + r < T) ? qbase[(long long)(q0 + r) * row_stride + c] : 0.f;
    }
    constexpr int QPW = F32_QPB / 4;
    float m[QPW], l[QPW], o[QPW][DPL];
#pragma unroll
    for (int q = 0; q < QPW; q++) {
        m[q] = -INFINITY; l[q] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) o[q][i] = 0.f;
    }
    int kv_end = CAUSAL ? min(T, q0 + F32_QPB) : T;
    for (int k0 = 0; k0 < kv_end; k0 += F32_KT) {
        __syncthreads();
        for (int i = threadIdx.x; i < F32_KT * HD; i += 128) {
            int r = i / HD, c = i % HD;
            bool ok = k0 + r < T;
            sK[r][c] = ok ? kbase[(long long)(k0 + r) * row_stride + c] : 0.f;
            sV[r][c] = ok ? vbase[(long long)(k0 + r) * row_stride + c] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < QPW; q++) {
            const int qi = warp * QPW + q;
            const int qrow = q0 + qi;
            if (qrow >= T) continue;              // uniform per warp
#pragma unroll
            for (int half = 0; half < F32_KT / 32; half++) {
                const int kbeg = k0 + half * 32;
                if (kbeg >= kv_end || (CAUSAL && kbeg > qrow)) break;     // uniform per warp
                const int kl = half * 32 + lane;
                const int key = k0 + kl;
                float s = 0.f;
#pragma unroll 8
                for (int c = 0; c < HD; c++) s = fmaf(sQ[qi][c], sK[kl][c], s);
                s *= inv_sqrt_hd;
                const bool live = key < T && (!CAUSAL || key <= qrow);
                if (!live) s = -INFINITY;
                float mx = s;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
                const float mn = fmaxf(m[q], mx);            // finite: key `kbeg` is live for this query
                const float alpha = expf(m[q] - mn);
                const float p = live ? expf(s - mn) : 0.f;
                float ps = p;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
                l[q] = l[q] * alpha + ps;
                m[q] = mn;
#pragma unroll
                for (int i = 0; i < DPL; i++) o[q][i] *= alpha;
#pragma unroll 8
                for (int jj = 0; jj < 32; jj++) {
                    const float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
                    for (int i = 0; i < DPL; i++) o[q][i] = fmaf(pj, sV[half * 32 + jj][i * 32 + lane], o[q][i]);
                }
            }
        }
    }
#pragma unroll
    for (int q = 0; q < QPW; q++) {
        const int qrow = q0 + warp * QPW + q;
        if (qrow >= T) continue;
        float* op = out + ((long long)b * T + qrow) * d + h * HD;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            float v = o[q][i] / l[q];
            op[i * 32 + lane] = round_out ? round_tf32(v) : v;
        }
    }
}

// Queries past the last full warp (T_main <= qi < T), one warp per query: the lanes split the keys for the scores and
// the output columns for the weighted sum of value rows, both read straight from global memory (the row threads of the
// neighbouring CTAs have just pulled the same rows through L2).  Two passes over the keys: the row maximum first, then
// exponentials and the weighted sum 32 keys at a time, so nothing per key is kept.
template <int HD, bool CAUSAL>
__device__ __forceinline__ void attention_f32_tail_rows(const float* __restrict__ qbase, const float* __restrict__ kbase,
                                                        const float* __restrict__ vbase, float* __restrict__ out_bh,
                                                        int T, int T_main, int d, long long row_stride,
                                                        float inv_sqrt_hd, int round_out) {
    constexpr int V4 = HD / 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int qi = T_main + warp; qi < T; qi += nwarps) {
        float q[HD];
#pragma unroll
        for (int c = 0; c < V4; c++) {
            const float4 t = *reinterpret_cast<const float4*>(qbase + (long long)qi * row_stride + 4 * c);
            q[4 * c] = t.x; q[4 * c + 1] = t.y; q[4 * c + 2] = t.z; q[4 * c + 3] = t.w;
        }
        auto score = [&](int key) {
            const float* kr = kbase + (long long)key * row_stride;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int c = 0; c < V4; c++) {
                const float4 kv = *reinterpret_cast<const float4*>(kr + 4 * c);
                a0 = fmaf(q[4 * c], kv.x, a0); a1 = fmaf(q[4 * c + 1], kv.y, a1);
                a2 = fmaf(q[4 * c + 2], kv.z, a2); a3 = fmaf(q[4 * c + 3], kv.w, a3);
            }
            return ((a0 + a1) + (a2 + a3)) * inv_sqrt_hd;
        };
        const int nkeys = CAUSAL ? qi + 1 : T;
        float mx = -INFINITY;
        for (int key = lane; key < nkeys; key += 32) mx = fmaxf(mx, score(key));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        float l = 0.f, o0 = 0.f, o1 = 0.f;                 // output columns lane and lane + 32
        for (int k0 = 0; k0 < nkeys; k0 += 32) {
            const int key = k0 + lane;
            const float p = key < nkeys ? __expf(score(key) - mx) : 0.f;
            l += p;
            const int cnt = min(32, nkeys - k0);
#pragma unroll 8
            for (int kk = 0; kk < cnt; kk++) {
                const float pk = __shfl_sync(0xffffffffu, p, kk);
                const float* vr = vbase + (long long)(k0 + kk) * row_stride;
                if (lane < HD) o0 = fmaf(pk, vr[lane], o0);
                if (HD > 32) o1 = fmaf(pk, vr[(lane + 32) % HD], o1);
            }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) l += __shfl_xor_sync(0xffffffffu, l, s);
        float* op = out_bh + (long long)qi * d;
        if (lane < HD) { const float v = o0 / l; op[lane] = round_out ? round_tf32(v) : v; }
        if (HD > 32) { const float v = o1 / l; op[(lane + 32) % HD] = round_out ? round_tf32(v) : v; }
    }
}

// Float32 attention with the queries in registers (head dimension 8 to 64): a thread owns a query, its running
// maximum, row sum and output row; key and value rows are read from shared memory as broadcasts (every thread of a
// warp reads the same 16 bytes).  Keys are taken eight at a time: eight scores, one maximum update and one rescale of
// the output row, then eight exponentials.  Exact float32 products and sums; the exponentials are ex2.approx of
// the argument times log2(e) (2 ulp, against a dozen instructions for libm's), far inside the 2e-3 budget of the
// float32 / TF32 mode.
// KS = 1: one thread per query, nothing exchanged between threads.  KS = 4 (grids that would not fill the GPU): four
// adjacent lanes share a query and take the keys with index = lane part (mod 4), each with its own maximum, sum and
// output row, merged by shuffles at the end; tile rows are padded by 16 bytes so that the four rows read by one
// instruction fall into different banks.  The serial chain per thread is a quarter as long and there are four times
// the warps.  (Two queries per thread, which halves the shared-memory bytes per multiply-add, was slower: too few
// warps at 250 registers.  256 images of 65 tokens, 6 heads of 32: 1.27 ms per forward against 1.12 ms.)
// T_main is the number of queries the row threads take; when it is below T the last CTA of each (batch, head) column
// handles the remaining T - T_main queries with attention_f32_tail_rows instead.
template <int HD, bool CAUSAL, int KS>
__global__ void __launch_bounds__(128)
attention_f32_rowthread_kernel(const float* __restrict__ qkv, float* __restrict__ out, int T, int T_main, int H,
                               float inv_sqrt_hd, int round_out) {
    constexpr int KT = 64;                         // keys per shared-memory tile
    constexpr int V4 = HD / 4;
    constexpr int HDP = HD + (KS > 1 ? 4 : 0);     // padded row
    constexpr int CH = 8 * KS;                     // keys per step of the CTA: eight for each part
    __shared__ __align__(16) float sK[KT][HDP];
    __shared__ __align__(16) float sV[KT][HDP];

    const int d = H * HD;
    const long long row_stride = 3ll * d;
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int qpb = blockDim.x / KS;                  // queries per CTA
    const int q0 = blockIdx.x * qpb;
    const int part = threadIdx.x % KS;
    const int qi = q0 + threadIdx.x / KS;
    const bool active = qi < T_main;
    const float* qbase = qkv + (long long)b * T * row_stride + h * HD;
    const float* kbase = qbase + d;
    const float* vbase = qbase + 2 * d;
    if (T_main < T && blockIdx.x == gridDim.x - 1) {               // uniform over the CTA, before any barrier
        attention_f32_tail_rows<HD, CAUSAL>(qbase, kbase, vbase, out + (long long)b * T * d + h * HD, T, T_main, d,
                                            row_stride, inv_sqrt_hd, round_out);
        return;
    }

    float q[HD], o[HD];
#pragma unroll
    for (int c = 0; c < V4; c++) {
        const float4 t = active ? *reinterpret_cast<const float4*>(qbase + (long long)qi * row_stride + 4 * c)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
        q[4 * c] = t.x; q[4 * c + 1] = t.y; q[4 * c + 2] = t.z; q[4 * c + 3] = t.w;
        o[4 * c] = 0.f; o[4 * c + 1] = 0.f; o[4 * c + 2] = 0.f; o[4 * c + 3] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int kv_end = CAUSAL ? min(T, q0 + qpb) : T;
    for (int k0 = 0; k0 < kv_end; k0 += KT) {
        __syncthreads();
        const int tile_rows = min(KT, (kv_end - k0 + CH - 1) / CH * CH);   // whole steps; rows past T are zeros
        for (int i = threadIdx.x; i < tile_rows * V4; i += blockDim.x) {
            const int r = i / V4, c = i % V4;
            const bool ok = k0 + r < T;
            const long long off = (long long)(ok ? k0 + r : 0) * row_stride + 4 * c;
            cp_async16(smem_u32(&sK[r][4 * c]), kbase + off, ok);      // all of a thread's copies are in flight at once
            cp_async16(smem_u32(&sV[r][4 * c]), vbase + off, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        if (!active) continue;
        const int nk = min(KT, kv_end - k0);
        for (int c0 = 0; c0 < nk; c0 += CH) {
            if (CAUSAL && k0 + c0 > qi) break;                     // every later key is masked for this query
            const int cw = KS == 1 ? nk - c0 : 8;                   // live keys of this step (uniform over the CTA)
            float sc[8];
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                if (kk >= cw) { sc[kk] = -INFINITY; continue; }
                const int r = c0 + kk * KS + part;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int c = 0; c < V4; c++) {
                    const float4 kv = *reinterpret_cast<const float4*>(&sK[r][4 * c]);
                    a0 = fmaf(q[4 * c], kv.x, a0); a1 = fmaf(q[4 * c + 1], kv.y, a1);
                    a2 = fmaf(q[4 * c + 2], kv.z, a2); a3 = fmaf(q[4 * c + 3], kv.w, a3);
                }
                const int key = k0 + r;
                const bool live = key < T && (!CAUSAL || key <= qi);
                sc[kk] = live ? ((a0 + a1) + (a2 + a3)) * inv_sqrt_hd : -INFINITY;
            }
            const float cm = fmaxf(fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3])), fmaxf(fmaxf(sc[4], sc[5]), fmaxf(sc[6], sc[7])));
            const float mn = fmaxf(m, cm);
            if (mn == -INFINITY) continue;                          // nothing visible yet
            const float alpha = __expf(m - mn);                        // 0 while m is still -inf
            l *= alpha;
#pragma unroll
            for (int c = 0; c < HD; c++) o[c] *= alpha;
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                if (kk >= cw) break;
                const int r = c0 + kk * KS + part;
                const float p = __expf(sc[kk] - mn);                   // 0 for masked keys
                l += p;
#pragma unroll
                for (int c = 0; c < V4; c++) {
                    const float4 vv = *reinterpret_cast<const float4*>(&sV[r][4 * c]);
                    o[4 * c] = fmaf(p, vv.x, o[4 * c]); o[4 * c + 1] = fmaf(p, vv.y, o[4 * c + 1]);
                    o[4 * c + 2] = fmaf(p, vv.z, o[4 * c + 2]); o[4 * c + 3] = fmaf(p, vv.w, o[4 * c + 3]);
                }
            }
            m = mn;
        }
    }
    if (KS > 1) {
        // merge the parts of a query (adjacent lanes); every thread of the warp takes part in the shuffles
#pragma unroll
        for (int s = 1; s < KS; s <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m, s);
            const float l_o = __shfl_xor_sync(0xffffffffu, l, s);
            const float m_n = fmaxf(m, m_o);
            const float fa = m == -INFINITY ? 0.f : __expf(m - m_n);
            const float fb = m_o == -INFINITY ? 0.f : __expf(m_o - m_n);
            l = l * fa + l_o * fb;
#pragma unroll
            for (int c = 0; c < HD; c++) o[c] = o[c] * fa + __shfl_xor_sync(0xffffffffu, o[c], s) * fb;
            m = m_n;
        }
    }
    if (active) {
        float* op = out + ((long long)b * T + qi) * d + h * HD;
#pragma unroll
        for (int c = 0; c < V4; c++) {
            if (KS > 1 && c % KS != part) continue;                 // the parts share the row's 16-byte stores
            float4 r = make_float4(o[4 * c] / l, o[4 * c + 1] / l, o[4 * c + 2] / l, o[4 * c + 3] / l);
            if (round_out) { r.x = round_tf32(r.x); r.y = round_tf32(r.y); r.z = round_tf32(r.z); r.w = round_tf32(r.w); }
            *reinterpret_cast<float4*>(op + 4 * c) = r;
        }
    }
}

template <int HD>
int launch_bf16(tlnn_ctx* ctx, const __nv_bfloat16* qkv, __nv_bfloat16* out, int B, int T, int H, int causal) {
    const size_t smem = (size_t)(FA_BM + 4 * FA_BN) * HD * 2;
    dim3 grid((T + FA_BM - 1) / FA_BM, B * H);
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
    if (causal) {
        auto k = flash_bf16_kernel<HD, true>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        TL_LAUNCH(ctx, "attention_bf16_causal", k<<<grid, FA_THREADS, smem, ctx->stream>>>(qkv, out, T, H, scale_log2));
    } else {
        auto k = flash_bf16_kernel<HD, false>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        TL_LAUNCH(ctx, "attention_bf16_full", k<<<grid, FA_THREADS, smem, ctx->stream>>>(qkv, out, T, H, scale_log2));
    }
    return TLNN_OK;
}

template <int HD>
int launch_f32(tlnn_ctx* ctx, const float* qkv, float* out, int B, int T, int H, int causal, int round_out) {
    const float inv = 1.f / sqrtf((float)HD);
    if constexpr (HD <= 64) {
        // the packed projection rows must allow 16-byte loads of a head's slice
        if ((reinterpret_cast<uintptr_t>(qkv) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
            // A few queries past a warp boundary (a ViT's class token: 65, 257 rows) would cost a whole warp of row
            // threads; they go to one extra CTA per (batch, head) that spends a warp per query instead.
            const int rem = T % 32;
            const int T_main = (T >= 32 && rem > 0 && rem <= 4) ? T - rem : T;
            const int tail_cta = T_main < T ? 1 : 0;
            int threads = T_main >= 128 ? 128 : ((T_main + 31) / 32) * 32;
            // a grid that would leave most SMs with a warp or two: four lanes per query instead
            const bool split = (long long)((T_main + threads - 1) / threads) * B * H * (threads / 32) < 8ll * ctx->sm_count;
            if (split) threads = 128;
            const int qpb = split ? threads / 4 : threads;
            dim3 grid((T_main + qpb - 1) / qpb + tail_cta, B * H);
            auto launch = [&](auto kern) -> int {
                TL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
                TL_LAUNCH(ctx, causal ? "attention_f32_causal" : "attention_f32_full", kern<<<grid, threads, 0, ctx->stream>>>(qkv, out, T, T_main, H, inv, round_out));
                return TLNN_OK;
            };
            // Tighter launch bounds (80 or 96 registers, so that all CTAs of the 65-token case are resident at once)
            // were slower: the few spilled values sit in the key loop.
            if (split) return causal ? launch(attention_f32_rowthread_kernel<HD, true, 4>) : launch(attention_f32_rowthread_kernel<HD, false, 4>);
            return causal ? launch(attention_f32_rowthread_kernel<HD, true, 1>) : launch(attention_f32_rowthread_kernel<HD, false, 1>);
        }
    }
    if constexpr (HD < 32) {
        TL_REQUIRE(false, "attention: head dimension %d in float32 mode needs 16-byte aligned buffers", HD);
    } else {
    dim3 grid((T + F32_QPB - 1) / F32_QPB, B * H);
    if (causal)
        TL_LAUNCH(ctx, "attention_f32_causal", attention_f32_kernel<HD, true><<<grid, 128, 0, ctx->stream>>>(qkv, out, T, H, inv, round_out));
    else
        TL_LAUNCH(ctx, "attention_f32_full", attention_f32_kernel<HD, false><<<grid, 128, 0, ctx->stream>>>(qkv, out, T, H, inv, round_out));
    return TLNN_OK;
    }
}

}  // namespace

int tl_attention_tcgen05(tlnn_ctx* ctx, const __nv_bfloat16* qkv, __nv_bfloat16* out, int B, int T, int heads, int causal);

// TLNN_ATTENTION=legacy forces the mma.sync kernel, =tcgen05 forces the TMEM kernel (head dimension 64 only);
// by default the TMEM kernel takes sequences of at least 192 tokens.
static int attention_choice() {
    static int choice = -1;
    if (choice < 0) {
        const char* e = getenv("TLNN_ATTENTION");
        choice = !e ? 0 : (strcmp(e, "legacy") == 0 ? 1 : (strcmp(e, "tcgen05") == 0 ? 2 : 0));
    }
    return choice;
}

int tl_attention_core(tlnn_ctx* ctx, int prec, const void* qkv, void* out, int out_kind, int B, int T, int heads, int hd,
                      int causal) {
    if (B == 0 || T == 0) return TLNN_OK;
    TL_REQUIRE((long long)B * heads <= 65535, "attention: batch x heads = %lld exceeds 65535", (long long)B * heads);
    if (prec == TLNN_PREC_BF16) {
        TL_REQUIRE(out_kind == TL_OUT_BF16, "attention: the bf16 path writes bf16");
        const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(qkv);
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
        const int choice = attention_choice();
        if (hd == 64 && choice != 1 && (choice == 2 || T >= 192)) return tl_attention_tcgen05(ctx, q, o, B, T, heads, causal);
        if (hd == 32) return launch_bf16<32>(ctx, q, o, B, T, heads, causal);
        if (hd == 64) return launch_bf16<64>(ctx, q, o, B, T, heads, causal);
        if (hd == 128) return launch_bf16<128>(ctx, q, o, B, T, heads, causal);
        TL_REQUIRE(false, "attention: head dimension %d is not supported in bf16 mode (32, 64 or 128)", hd);
    }
    TL_REQUIRE(out_kind != TL_OUT_BF16, "attention: the float32 path writes float32");
    const float* q = reinterpret_cast<const float*>(qkv);
    float* o = reinterpret_cast<float*>(out);
    const int round_out = out_kind == TL_OUT_TF32;
    if (tl_attention_tf32_applies(T, hd) && (reinterpret_cast<uintptr_t>(qkv) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0)
        return tl_attention_tf32(ctx, q, o, B, T, heads, causal, round_out);
    if (hd == 8) return launch_f32<8>(ctx, q, o, B, T, heads, causal, round_out);
    if (hd == 16) return launch_f32<16>(ctx, q, o, B, T, heads, causal, round_out);
    if (hd == 32) return launch_f32<32>(ctx, q, o, B, T, heads, causal, round_out);
    if (hd == 64) return launch_f32<64>(ctx, q, o, B, T, heads, causal, round_out);
    if (hd == 96) return launch_f32<96>(ctx, q, o, B, T, heads, causal, round_out);
    if (hd == 128) return launch_f32<128>(ctx, q, o, B, T, heads, causal, round_out);
    TL_REQUIRE(false, "attention: head dimension %d is not supported in float32 mode (8, 16, 32, 64, 96 or 128)", hd);
}
