// Attention of the FP32/TF32 mode on the sm_100a tensor cores: one (batch, head) of at most 128 tokens per CTA.
//
// The reference computes scores and weighted values as batched matrix products (layers.py:293, 303), which its CUDA
// runtime runs as TF32 tensor-core GEMMs (backend.py:9,16).  Here both products are tcgen05.mma kind::tf32 with float32
// accumulation in TMEM; the whole score matrix of a sequence of up to 128 tokens fits one 128 x 128 accumulator, so there
// is no key loop and no running maximum:
//   TMA        Q, K, V head slices (rows x 32 floats, 128-byte swizzle) out of the packed (B T, 3 d) projection
//   MMA 1      S = Q K^T  (128 x NK x 32, four K = 8 steps), NK = tokens rounded up to 32
//   threads    one thread per query row: scores from TMEM, mask (sequence end, decoder triangle), maximum,
//              2^(x - max), sum; probabilities rounded to TF32 and written back over the scores in TMEM.  Meanwhile
//              the V tile is transposed in shared memory (the second product wants its B operand K-major: keys
//              contiguous)
//   MMA 2      O = P V  (128 x 32 x NK) with P read from TMEM as the A operand
//   threads    O rows from TMEM, divided by the row sum, stored (rounded to TF32 when the output feeds a GEMM)
// q, k and v are expected rounded to nearest TF32 by the projection's epilogue (tensor cores truncate float32 operands).
// Two to four CTAs share an SM (128 or 256 TMEM columns each), which hides the dependent chain of one sequence behind
// the others.  Head dimension 32 only (the FP32/TF32 configurations: 128 / 4 and 192 / 6).  All waits are bounded.
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int HD = 32;                  // head dimension: one 128-byte swizzle row of float32
constexpr int ROWS = 128;               // query rows per tile (the MMA's M)
constexpr int THREADS = 128;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float to_tf32(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x00000fffu + ((u >> 13) & 1u);
    u &= 0xffffe000u;
    return __uint_as_float(u);
}
// D += A B with A in TMEM (32-bit elements, one column per K element), B a shared-memory descriptor
__device__ __forceinline__ void umma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ uint32_t idesc_tf32(int n) {       // D float32, A and B TF32, both K-major, M = 128
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
}

template <bool CAUSAL>
__global__ void __launch_bounds__(THREADS)
attention_tf32_kernel(const __grid_constant__ CUtensorMap tm, float* __restrict__ out, int T, int NK, int H, float scale_log2,
                      int round_out, uint32_t tmem_cols, tlnn_dev_err* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t tile_bytes = (uint32_t)NK * 128u;                   // NK rows of 32 floats
    uint8_t* q_s = smem;
    uint8_t* k_s = smem + tile_bytes;
    uint8_t* v_s = smem + 2 * tile_bytes;
    uint8_t* vt_s = smem + 3 * tile_bytes;                              // four tiles of 32 (head dim) x 32 keys
    uint64_t* bars = reinterpret_cast<uint64_t*>(vt_s + 4 * 4096);      // loads done, scores done, output done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.x;
    const int b = bh / H, h = bh - b * H;
    const int d = H * HD;
    const int row0 = b * T;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm);
        for (int i = 0; i < 3; i++) mbar_init(&bars[i], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t s_tmem = tmem_base;                                  // NK columns: scores, then probabilities
    const uint32_t o_tmem = tmem_base + (uint32_t)NK;                   // 32 columns
    tl_grid_dependency_sync();                                          // the projection that wrote q, k, v has finished

    bool ok = true;
    if (threadIdx.x == 0) {
        mbar_expect_tx(&bars[0], 3 * tile_bytes);
        tma_load_2d(smem_u32(q_s), &tm, smem_u32(&bars[0]), h * HD, row0);
        tma_load_2d(smem_u32(k_s), &tm, smem_u32(&bars[0]), d + h * HD, row0);
        tma_load_2d(smem_u32(v_s), &tm, smem_u32(&bars[0]), 2 * d + h * HD, row0);
    }
    ok = mbar_wait(&bars[0], 0, abort_flag, err, 300);
    if (ok && threadIdx.x == 0) {
        // S = Q K^T: four K = 8 steps, 32 bytes further into both operands' rows each
        tc_fence_after();
        const uint64_t q_desc = make_smem_desc(smem_u32(q_s)), k_desc = make_smem_desc(smem_u32(k_s));
        const uint32_t idesc = idesc_tf32(NK);
#pragma unroll
        for (int k = 0; k < HD / 8; k++) umma<true>(s_tmem, q_desc + 2 * k, k_desc + 2 * k, idesc, k != 0 ? 1u : 0u);
        umma_commit(&bars[1]);
    }
    if (ok) {
        // V^T for the second product while the first one runs: thread = key.  Source row (swizzled): 16-byte chunk c of
        // key t sits at chunk c ^ (t % 8).  Destination: tile t / 32, row = head dimension n, the key's float at chunk
        // ((t % 32) / 4) ^ (n % 8), word t % 4.
        const int t = threadIdx.x;
        if (t < NK) {
            const uint8_t* src = v_s + (size_t)t * 128;
            uint8_t* dst_tile = vt_s + (size_t)(t >> 5) * 4096;
            const int kc = (t & 31) >> 2, kw = t & 3;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float4 v4 = *reinterpret_cast<const float4*>(src + ((c ^ (t & 7)) << 4));
                const float vals[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int n = c * 4 + e;
                    *reinterpret_cast<float*>(dst_tile + n * 128 + ((kc ^ (n & 7)) << 4) + kw * 4) = vals[e];
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the transposed tile is read by the tensor core
    }

    // ---- softmax over the row this thread owns
    const int r = threadIdx.x;                                           // query index inside the sequence
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float l_sum = 1.f;
    if (ok) ok = mbar_wait(&bars[1], 0, abort_flag, err, 301);
    if (ok) {
        __syncwarp();
        tc_fence_after();
        const int n_chunks = (NK + 31) >> 5;
        const int last = CAUSAL ? min(r, T - 1) : T - 1;                 // last key this row attends
        float mx = -INFINITY;
        for (int c = 0; c < n_chunks; c++) {
            uint32_t sc[32];
            tmem_ld32_issue(s_tmem + lane_base + (uint32_t)(c * 32), sc);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++)
                if (c * 32 + i <= last) mx = fmaxf(mx, __uint_as_float(sc[i]));
        }
        const float m2 = mx * scale_log2;
        float l = 0.f;
        for (int c = 0; c < n_chunks; c++) {
            uint32_t sc[32];
            tmem_ld32_issue(s_tmem + lane_base + (uint32_t)(c * 32), sc);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) {
                float p = 0.f;
                if (c * 32 + i <= last) p = to_tf32(ex2(fmaf(__uint_as_float(sc[i]), scale_log2, -m2)));
                l += p;
                sc[i] = __float_as_uint(p);
            }
            tmem_st32(s_tmem + lane_base + (uint32_t)(c * 32), sc);
        }
        l_sum = l;
        tmem_st_wait();
        tc_fence_before();
    }
    __syncthreads();
    if (ok && threadIdx.x == 0) {
        // O = P V: K = 8 keys per step; P columns 8 j .. 8 j + 7, V^T 32 bytes further per step inside a 32-key tile
        tc_fence_after();
        const uint32_t idesc = idesc_tf32(HD);
        const int steps = NK / 8;
        for (int j = 0; j < steps; j++) {
            const uint64_t vt_desc = make_smem_desc(smem_u32(vt_s + (size_t)(j >> 2) * 4096)) + 2 * (j & 3);
            umma_ts_tf32(o_tmem, s_tmem + (uint32_t)(8 * j), vt_desc, idesc, j != 0 ? 1u : 0u);
        }
        umma_commit(&bars[2]);
    }
    if (ok) ok = mbar_wait(&bars[2], 0, abort_flag, err, 302);
    if (ok) {
        __syncwarp();
        tc_fence_after();
        uint32_t acc[32];
        tmem_ld32_issue(o_tmem + lane_base, acc);
        tmem_ld_wait();
        if (r < T) {
            const float inv = 1.f / l_sum;
            float* dst = out + ((long long)(row0 + r)) * d + h * HD;
#pragma unroll
            for (int u = 0; u < 8; u++) {
                float4 o;
                o.x = __uint_as_float(acc[4 * u]) * inv; o.y = __uint_as_float(acc[4 * u + 1]) * inv;
                o.z = __uint_as_float(acc[4 * u + 2]) * inv; o.w = __uint_as_float(acc[4 * u + 3]) * inv;
                if (round_out) { o.x = to_tf32(o.x); o.y = to_tf32(o.y); o.z = to_tf32(o.z); o.w = to_tf32(o.w); }
                *reinterpret_cast<float4*>(dst + 4 * u) = o;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

}  // namespace

// Whether the FP32/TF32-mode attention of this shape runs on the tensor cores (its projection should then round q, k, v
// to TF32).  TLNN_ATTENTION_TF32=0 keeps the exact float32 kernels.
bool tl_attention_tf32_applies(int T, int hd) {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("TLNN_ATTENTION_TF32");
        on = (e && strcmp(e, "0") == 0) ? 0 : 1;
    }
    return on == 1 && hd == HD && T >= 1 && T <= ROWS;
}

int tl_attention_tf32(tlnn_ctx* ctx, const float* qkv, float* out, int B, int T, int heads, int causal, int round_out) {
    const int d = heads * HD;
    const long long rows = (long long)B * T;
    TL_REQUIRE(rows < (1ll << 31), "attention: too many rows");
    TL_REQUIRE(((uintptr_t)qkv & 15u) == 0 && ((uintptr_t)out & 15u) == 0, "attention: buffers must be 16-byte aligned");
    // keys (and rows of the Q, K, V tiles) rounded up to 32: a row reads its scores and writes its probabilities in chunks
    // of 32 TMEM columns; masked keys get probability 0
    const int NK = (T + 31) & ~31;
    const uint32_t tmem_cols = NK + 32 <= 128 ? 128u : 256u;          // scores / probabilities, then the 32 output columns
    CUtensorMap tm;
    TL_TRY(sm100::make_tile_map(&tm, false, qkv, rows, 3ll * d, 3ll * d, NK));
    size_t smem = 3 * (size_t)NK * 128 + 4 * 4096 + 64 + 1024;
    // a CTA that needs 256 TMEM columns shares the SM with one other at most: ask for enough shared memory that a third
    // is never scheduled (its TMEM allocation would have to wait for one of the two to finish)
    if (tmem_cols == 256u && smem < 80 * 1024) smem = 80 * 1024;
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
    auto launch = [&](auto kern) -> int {
        TL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TL_LAUNCH(ctx, causal ? "attention_tf32_causal" : "attention_tf32_full",
                  tl_launch_kernel(ctx, kern, dim3((unsigned)(B * heads)), dim3(THREADS), smem, tm, out, T, NK, heads, scale_log2, round_out,
                                   tmem_cols, ctx->d_err));
        return TLNN_OK;
    };
    return causal ? launch(attention_tf32_kernel<true>) : launch(attention_tf32_kernel<false>);
}
