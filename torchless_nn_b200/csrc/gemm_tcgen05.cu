// Tensor-core GEMM for sm_100a: out = epilogue(A @ W^T), A (M,K) and W (N,K) with K contiguous.
//
// One persistent CTA per SM walks a static list of 128 x BN output tiles.  Inside a CTA the work is split by warp:
//   warp 0      - TMA producer: streams 128 x 128-byte A tiles and BN x 128-byte W tiles (128-byte swizzle) into a
//                 ring of shared-memory stages, signalling `full[stage]` by transaction count;
//   warp 1      - MMA issuer: one thread issues tcgen05.mma (kind::f16 for bf16 operands, kind::tf32 for float32
//                 operands) from shared memory into one of two TMEM accumulators (BN columns each), frees each stage
//                 with tcgen05.commit -> `empty[stage]`, and hands a finished accumulator over with
//                 tcgen05.commit -> `acc_full[buf]`;
//   warps 2..5  - epilogue: tcgen05.ld the accumulator (each warp owns the 32 TMEM lanes of its warp-id mod 4),
//                 apply bias / activation / residual / arg-max, store, then release the accumulator
//                 (`acc_empty[buf]`) so that the next tile's MMAs overlap this tile's epilogue.
// Every wait on an mbarrier is bounded by wall-clock time; on expiry the kernel records TLNN_ERR_TIMEOUT in the
// context's error word, raises a CTA-wide abort flag, and all roles fall through to the common exit, where the
// TMEM allocation is returned.
#include "common.cuh"

#include <cuda.h>   // CUtensorMap and enums only; the encode entry point is fetched through the runtime

namespace {

constexpr int BM = 128;             // UMMA M (cta_group::1)
constexpr int ROW_BYTES = 128;      // one swizzle-128B row of K: 64 bf16 or 32 float32
constexpr int MMA_K_BYTES = 32;     // K extent of one tcgen05.mma: 16 bf16 or 8 tf32
constexpr int GROUP_M = 8;          // rasterisation: tiles are walked in groups of GROUP_M row-blocks
constexpr int NUM_THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s

template <int BN> struct Cfg {
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr uint32_t A_BYTES = BM * ROW_BYTES;
    static constexpr uint32_t B_BYTES = BN * ROW_BYTES;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// ---- PTX wrappers -------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false (after recording the failure and raising the CTA's abort flag) when the barrier
// did not flip within WAIT_LIMIT_NS or another role of this CTA already gave up.
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                            tlnn_dev_err* err, int site) {
    unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 128; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            tl_dev_fail(err, TLNN_ERR_TIMEOUT, site, (long long)blockIdx.x);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          tlnn_dev_err* err, int site) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, err, site);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <bool TF32>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// Arrive on an mbarrier once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes
// apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                  // leading byte offset (ignored for swizzled K-major), canonical value 1
    d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset
    d |= (uint64_t)1 << 46;                  // version
    d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D float32, A/B bf16 (1) or tf32 (2), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
template <int BN, bool TF32>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
    uint32_t fmt = TF32 ? 2u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ float round_tf32(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x00000fffu + ((u >> 13) & 1u);
    u &= 0xffffe000u;
    return __uint_as_float(u);
}

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool ACCURATE>
__device__ __forceinline__ float apply_act(int act, float v) {
    if (act == TLNN_ACT_GELU) {
        float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
        float t = ACCURATE ? tanhf(u) : tanh_fast(u);
        return 0.5f * v * (1.f + t);
    }
    if (act == TLNN_ACT_SILU) {
        float t = ACCURATE ? tanhf(0.5f * v) : tanh_fast(0.5f * v);
        return v * ((1.f + t) * 0.5f);
    }
    if (act == TLNN_ACT_RELU) return fmaxf(v, 0.f);
    return v;
}

struct TileCoord { int m_blk, n_blk; };
__device__ __forceinline__ TileCoord tile_coord(int t, int m_tiles, int n_tiles) {
    int per_group = GROUP_M * n_tiles;
    int g = t / per_group;
    int first_m = g * GROUP_M;
    int gsize = min(m_tiles - first_m, GROUP_M);
    int r = t - g * per_group;
    TileCoord c;
    c.m_blk = first_m + r % gsize;
    c.n_blk = r / gsize;
    return c;
}

// ---- the kernel ---------------------------------------------------------------------------------------------------------
template <int BN, bool TF32>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const tl_gemm_epilogue ep, int M, int N, int K, int m_tiles, int n_tiles, tlnn_dev_err* err) {
    using C = Cfg<BN>;
    constexpr int STAGES = C::STAGES;
    constexpr int K_ELEMS = TF32 ? 32 : 64;       // elements per 128-byte row

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = m_tiles * n_tiles;
    const int num_k = (K + K_ELEMS - 1) / K_ELEMS;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);      // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                TileCoord tc = tile_coord(t, m_tiles, n_tiles);
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, err, 101)) { ok = false; break; }
                    uint32_t sa = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
                    uint32_t bar = smem_u32(&full_bar[stage]);
                    mbar_expect_tx(&full_bar[stage], C::STAGE_BYTES);
                    tma_load_2d(sa, &tmA, bar, kb * K_ELEMS, tc.m_blk * BM);
                    tma_load_2d(sa + C::A_BYTES, &tmB, bar, kb * K_ELEMS, tc.n_blk * BN);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc<BN, TF32>();
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, local++) {
                const int buf = local & 1;
                const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
                if (!mbar_wait(&acc_empty[buf], buf_phase ^ 1u, abort_flag, err, 102)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag, err, 103)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t sa = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
                    uint64_t a_desc = make_smem_desc(sa);
                    uint64_t b_desc = make_smem_desc(sa + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < ROW_BYTES / MMA_K_BYTES; k++) {
                        // advancing K inside the swizzle atom = advancing the start address by 32 bytes (>>4 = 2)
                        umma<TF32>(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                                   (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps, 128 rows)
        const int quarter = warp & 3;                 // TMEM lanes this warp may read: 32*quarter .. +31
        const int elem_out = ep.out_kind == TL_OUT_BF16 ? 2 : 4;
        const bool vec_out = ep.out != nullptr && ((reinterpret_cast<uintptr_t>(ep.out) & 15u) == 0) &&
                             ((ep.ldo * elem_out) % 16 == 0);
        const bool vec_res = ep.residual != nullptr && ((reinterpret_cast<uintptr_t>(ep.residual) & 15u) == 0) &&
                             (ep.ldr % 4 == 0);
        const bool vec_bias = ep.bias != nullptr && ((reinterpret_cast<uintptr_t>(ep.bias) & 15u) == 0);
        int local = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, local++) {
            TileCoord tc = tile_coord(t, m_tiles, n_tiles);
            const int buf = local & 1;
            const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
            if (!mbar_wait(&acc_full[buf], buf_phase, abort_flag, err, 104)) break;
            __syncwarp();
            tc_fence_after();
            const long long row = (long long)tc.m_blk * BM + quarter * 32 + lane;
            const bool row_ok = row < M;
            long long out_row = row, res_row = row;
            if (ep.row_group > 0) out_row = (row / ep.row_group) * ep.out_group + ep.out_off + row % ep.row_group;
            if (ep.res_row_mod > 0) res_row = ep.res_row_off + row % ep.res_row_mod;
            const int n0 = tc.n_blk * BN;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
            float best = -INFINITY;
            int best_i = 0x7fffffff;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const int col0 = n0 + c0;
                if (col0 >= N) break;                 // uniform over the CTA
                float v[32];
                __syncwarp();                         // tcgen05.ld is warp-collective: reconverge first
                tmem_ld32(taddr + (uint32_t)c0, v);
                if (row_ok) {
                const int ncols = min(32, N - col0);
                const bool full = ncols == 32;
                if (ep.bias) {
                    if (full && vec_bias) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 b = __ldg(reinterpret_cast<const float4*>(ep.bias + col0 + j));
                            v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) if (j < ncols) v[j] += __ldg(ep.bias + col0 + j);
                    }
                }
                if (ep.act != TLNN_ACT_NONE) {
                    if (ep.accurate_math) {
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = apply_act<true>(ep.act, v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = apply_act<false>(ep.act, v[j]);
                    }
                }
                if (ep.residual) {
                    const float* rp = ep.residual + res_row * ep.ldr + col0;
                    if (full && vec_res) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 r = *reinterpret_cast<const float4*>(rp + j);
                            v[j] += r.x; v[j + 1] += r.y; v[j + 2] += r.z; v[j + 3] += r.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) if (j < ncols) v[j] += rp[j];
                    }
                }
                if (ep.argmax_partials) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (j < ncols && v[j] > best) { best = v[j]; best_i = col0 + j; }
                }
                if (ep.out) {
                    if (ep.out_kind == TL_OUT_BF16) {
                        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(ep.out) + out_row * ep.ldo + col0;
                        if (full && vec_out) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 p;
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                p.x = *reinterpret_cast<uint32_t*>(&h0);
                                p.y = *reinterpret_cast<uint32_t*>(&h1);
                                p.z = *reinterpret_cast<uint32_t*>(&h2);
                                p.w = *reinterpret_cast<uint32_t*>(&h3);
                                *reinterpret_cast<uint4*>(op + j) = p;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) if (j < ncols) op[j] = __float2bfloat16_rn(v[j]);
                        }
                    } else {
                        if (ep.out_kind == TL_OUT_TF32) {
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = round_tf32(v[j]);
                        }
                        float* op = reinterpret_cast<float*>(ep.out) + out_row * ep.ldo + col0;
                        if (full && vec_out) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(op + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) if (j < ncols) op[j] = v[j];
                        }
                    }
                }
                }   // row_ok
            }
            if (ep.argmax_partials && row_ok)
                ep.argmax_partials[row * n_tiles + tc.n_blk] = make_float2(best, __int_as_float(best_i));
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D map over a (rows, K) matrix with K contiguous and a pitch of ld elements; box = 128 bytes of K x box_rows.
int make_map(CUtensorMap* map, int prec, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        tl_set_error("cuTensorMapEncodeTiled is not available from the driver");
        return TLNN_ERR_CUDA;
    }
    const int esz = prec == TLNN_PREC_BF16 ? 2 : 4;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(ld * esz)};
    cuuint32_t box[2] = {(cuuint32_t)(ROW_BYTES / esz), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, prec == TLNN_PREC_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                    2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_set_error("cuTensorMapEncodeTiled failed with %d (rows=%lld K=%lld ld=%lld box_rows=%d)", (int)r, rows, K, ld,
                     box_rows);
        return TLNN_ERR_CUDA;
    }
    return TLNN_OK;
}

int pick_bn(int M, int N, int sm_count) {
    const int m_tiles = (M + BM - 1) / BM;
    if (N > 128 && (long long)m_tiles * ((N + 255) / 256) >= sm_count) return 256;
    if (N > 64 && (long long)m_tiles * ((N + 127) / 128) >= sm_count) return 128;
    if (N > 128) return 128;
    return 64;
}

template <int BN, bool TF32>
int launch(tlnn_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const tl_gemm_epilogue& ep, int M, int N, int K) {
    auto kernel = gemm_tcgen05_kernel<BN, TF32>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::SMEM));
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const long long total = (long long)m_tiles * n_tiles;
    TL_REQUIRE(total < (1ll << 31), "gemm: too many tiles");
    const int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
    const char* name = TF32 ? (BN == 256 ? "gemm_tf32_n256" : BN == 128 ? "gemm_tf32_n128" : "gemm_tf32_n64")
                            : (BN == 256 ? "gemm_bf16_n256" : BN == 128 ? "gemm_bf16_n128" : "gemm_bf16_n64");
    TL_LAUNCH(ctx, name, kernel<<<grid, NUM_THREADS, Cfg<BN>::SMEM, ctx->stream>>>(ta, tb, ep, M, N, K, m_tiles, n_tiles,
                                                                                   ctx->d_err));
    return TLNN_OK;
}

}  // namespace

int tl_gemm_bn(int M, int N, int sm_count) { return pick_bn(M, N, sm_count); }

int tl_gemm(tlnn_ctx* ctx, int prec, const void* a, long long lda, const void* w, long long ldw, int M, int N, int K,
            const tl_gemm_epilogue& ep) {
    if (M == 0 || N == 0) return TLNN_OK;
    TL_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad shape M=%d N=%d K=%d", M, N, K);
    const int esz = prec == TLNN_PREC_BF16 ? 2 : 4;
    TL_REQUIRE((K * esz) % 16 == 0, "gemm: the contraction length %d must be a multiple of %d elements", K, 16 / esz);
    TL_REQUIRE((lda * esz) % 16 == 0 && (ldw * esz) % 16 == 0, "gemm: operand pitches must be multiples of 16 bytes");
    TL_REQUIRE(((uintptr_t)a & 15u) == 0 && ((uintptr_t)w & 15u) == 0, "gemm: operands must be 16-byte aligned");
    const int bn = pick_bn(M, N, ctx->sm_count);
    CUtensorMap ta, tb;
    TL_TRY(make_map(&ta, prec, a, M, K, lda, BM));
    TL_TRY(make_map(&tb, prec, w, N, K, ldw, bn));
    const bool tf32 = prec == TLNN_PREC_TF32;
    if (bn == 256) return tf32 ? launch<256, true>(ctx, ta, tb, ep, M, N, K) : launch<256, false>(ctx, ta, tb, ep, M, N, K);
    if (bn == 128) return tf32 ? launch<128, true>(ctx, ta, tb, ep, M, N, K) : launch<128, false>(ctx, ta, tb, ep, M, N, K);
    return tf32 ? launch<64, true>(ctx, ta, tb, ep, M, N, K) : launch<64, false>(ctx, ta, tb, ep, M, N, K);
}
