// Tensor-core GEMM for sm_100a: out = epilogue(A @ W^T), A (M,K) and W (N,K) with K contiguous.
//
// One persistent CTA per SM walks a static list of 128 x BN output tiles.  Inside a CTA the work is split by warp:
//   warp 0      - TMA producer: streams 128 x 128-byte A tiles and BN x 128-byte W tiles (128-byte swizzle) into a
//                 ring of shared-memory stages, signalling `full[stage]` by transaction count;
//   warp 1      - MMA issuer: one thread issues tcgen05.mma (kind::f16 for bf16 operands, kind::tf32 for float32
//                 operands) from shared memory into one of two TMEM accumulators (BN columns each), frees each stage
//                 with tcgen05.commit -> `empty[stage]`, and hands a finished accumulator over with
//                 tcgen05.commit -> `acc_full[buf]`;
//   warps 2..9  - epilogue: tcgen05.ld the accumulator (a warp may read the 32 TMEM lanes of its warp-id mod 4; two
//                 warps share a row quarter and split its columns), apply bias / activation / arg-max, transpose
//                 through shared memory, add the residual and store whole 128-byte row segments; the accumulator is
//                 released (`acc_empty[buf]`) as soon as its last chunk is in registers, so the next tile's MMAs
//                 overlap this tile's epilogue.
// Every wait on an mbarrier is bounded by wall-clock time; on expiry the kernel records TLNN_ERR_TIMEOUT in the
// context's error word, raises a CTA-wide abort flag, and all roles fall through to the common exit, where the
// TMEM allocation is returned.
#include "sm100_ptx.cuh"
#include <cstdlib>
#include <cstring>

namespace {

using namespace sm100;

constexpr int BM = 128;             // UMMA M (cta_group::1)
constexpr int ROW_BYTES = 128;      // one swizzle-128B row of K: 64 bf16 or 32 float32
constexpr int MMA_K_BYTES = 32;     // K extent of one tcgen05.mma: 16 bf16 or 8 tf32
constexpr int GROUP_M = 8;          // rasterisation: tiles are walked in groups of GROUP_M row-blocks
constexpr int NUM_THREADS = 320;          // TMA warp, MMA warp, eight epilogue warps
#ifndef PAIR_TMEM_COLS
#define PAIR_TMEM_COLS 512
#endif

template <int BN> struct Cfg {
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr uint32_t A_BYTES = BM * ROW_BYTES;
    static constexpr uint32_t B_BYTES = BN * ROW_BYTES;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr uint32_t BAR_BYTES = 2048;      // barriers, then eight 128-byte bias lines; keeps the staging tiles 1024-byte aligned (TMA swizzle phase)
    static constexpr uint32_t EPI_OFFSET = STAGES * STAGE_BYTES + BAR_BYTES;     // eight 4 KB staging tiles
    static constexpr size_t SMEM = (size_t)EPI_OFFSET + 8 * 4096 + 1024 /*alignment slack*/;
};

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

// x * sigmoid(2 u) = 0.5 x (1 + tanh(u)) without the cancellation of 1 + tanh(u) for negative u, given a = -2 u log2(e):
// one ex2 (2^-22 relative), one reciprocal (1 ulp) and two more operations instead of a libm tanh.  The quotient is 0
// where the exponential overflows, as the function itself is to float32 precision.
__device__ __forceinline__ float x_sigmoid_exp2(float x, float a) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
    return x * r;
}
// tanh-GeLU of the reference, 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), to a few float32 ulp
__device__ __forceinline__ float gelu_precise(float x) {
    return x_sigmoid_exp2(x, x * fmaf(x * x, -2.f * 0.0356774081f * 1.4426950409f, -2.f * 0.7978845608f * 1.4426950409f));
}
// x (1 + tanh(x / 2)) / 2 = x sigmoid(x)
__device__ __forceinline__ float silu_precise(float x) { return x_sigmoid_exp2(x, x * -1.4426950409f); }

template <bool ACCURATE>
__device__ __forceinline__ float apply_act(int act, float v) {
    if (act == TLNN_ACT_GELU) {
        if (ACCURATE) return gelu_precise(v);
        float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
        return 0.5f * v * (1.f + tanh_fast(u));
    }
    if (act == TLNN_ACT_SILU) {
        if (ACCURATE) return silu_precise(v);
        return v * ((1.f + tanh_fast(0.5f * v)) * 0.5f);
    }
    if (act == TLNN_ACT_RELU) return fmaxf(v, 0.f);
    return v;
}

// Activation over a 32-element chunk with the selector hoisted out of the element loop, so that the 32 independent
// chains are scheduled together.
template <bool ACCURATE>
__device__ __forceinline__ void apply_act_chunk(int act, float (&v)[32]) {
    if (act == TLNN_ACT_GELU) {
        if (ACCURATE) {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = gelu_precise(v[j]);
        } else {
            // 0.5 x (1 + tanh(x (c0 + c1 x^2))) on pairs of float32 (mul / fma .f32x2): five packed instructions and
            // two hardware tanh per pair
            uint64_t c0, c1, half2;
            asm("mov.b64 %0, {%1, %1};" : "=l"(c0) : "f"(0.7978845608f));
            asm("mov.b64 %0, {%1, %1};" : "=l"(c1) : "f"(0.0356774081f));
            asm("mov.b64 %0, {%1, %1};" : "=l"(half2) : "f"(0.5f));
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                uint64_t x, x2, w, u, h, t, r;
                float u0, u1;
                asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(v[j]), "f"(v[j + 1]));
                asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(x2) : "l"(x));
                asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(w) : "l"(x2), "l"(c1), "l"(c0));
                asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(u) : "l"(x), "l"(w));
                asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(h) : "l"(x), "l"(half2));
                asm("mov.b64 {%0, %1}, %2;" : "=f"(u0), "=f"(u1) : "l"(u));
                const float t0 = tanh_fast(u0), t1 = tanh_fast(u1);
                asm("mov.b64 %0, {%1, %2};" : "=l"(t) : "f"(t0), "f"(t1));
                asm("fma.rn.f32x2 %0, %1, %2, %1;" : "=l"(r) : "l"(h), "l"(t));
                asm("mov.b64 {%0, %1}, %2;" : "=f"(v[j]), "=f"(v[j + 1]) : "l"(r));
            }
        }
    } else if (act == TLNN_ACT_SILU) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float x = v[j];
            v[j] = ACCURATE ? silu_precise(x) : x * ((1.f + tanh_fast(0.5f * x)) * 0.5f);
        }
    } else if (act == TLNN_ACT_RELU) {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
    }
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

// ---- epilogue -------------------------------------------------------------------------------------------------------------
// Epilogue variants.  The specialised ones carry only the code of one fused pattern, which keeps the instruction
// footprint of the eight epilogue warps small (the generic variant with every option compiled in runs out of
// instruction cache); the host picks a specialised variant only when its alignment and shape conditions hold.
enum {
    EPI_GENERIC = 0,     // everything decided at run time; any alignment, ragged N, row remapping
    EPI_BF16 = 1,        // bf16 out (+bias)                         N % 32 == 0, 16-byte aligned rows
    EPI_BF16_GELU = 2,   // bf16 out, bias, tanh-GeLU (hardware tanh)  same conditions
    EPI_F32_RES = 3,     // float32 out (+bias) + float32 residual     same conditions, residual rows aligned too
    EPI_ARGMAX = 4,      // no output, (+bias), per-row arg-max candidates; ragged N allowed
    EPI_F32_ACCUM = 5,   // out += acc (+bias): the residual IS the output buffer (in-place residual stream)
    EPI_F32 = 6          // float32 out (+bias, +activation, optionally rounded to TF32), no residual
};
// EPI_BF16, EPI_BF16_GELU, EPI_F32 and EPI_F32_ACCUM leave the tile through TMA: the warp writes its 32-row slab into its
// staging tile in the 128-byte-swizzled layout and one lane issues a bulk tensor store (bf16: 64 columns at a time) or a
// bulk tensor reduce-add (float32: the memory system adds the tile to the residual in place, so the residual never
// travels to the SM).  No per-thread global loads or stores, no second pass over the staging tile.

// Two warps share each 32-row quarter of the tile (a warp may only read the TMEM lanes of its warp-id mod 4) and take
// the even / odd 32-column chunks.  Per chunk:
//   phase 1 (thread = row): accumulator chunk from TMEM, + bias, activation, arg-max, then into this warp's 32 x 32
//                           float staging tile in shared memory (16-byte units XOR-swizzled by row);
//   phase 2 (8 lanes = one 128-byte row segment): read the tile transposed, + residual, convert, store - every store
//                           instruction writes four whole row segments.
// The bias and the residual of a chunk are requested before its accumulator is waited for, and the accumulator
// buffer goes back to the MMA warp as soon as this warp's last chunk is in registers.
// PAIR: the CTA is one half of a cta_group::2 pair.  Tiles are walked per cluster over (row pairs, n_tiles); this CTA
// owns row block 2 * pair + rank, and the accumulator buffer is given back on the leader CTA's barrier.
template <int BN, int MODE, bool PAIR = false>
__device__ __forceinline__ void epilogue_warp(const tl_gemm_epilogue& ep, int M, int N, int m_tiles, int n_tiles,
                                              int total_tiles, int warp, int lane, uint32_t tmem_base, float* staging,
                                              uint64_t* acc_full, uint64_t* acc_empty, volatile int* abort_flag,
                                              tlnn_dev_err* err, const CUtensorMap* tm_out, int split_k = 1) {
    const int tile0 = PAIR ? (int)cluster_id_x() : (int)blockIdx.x;
    const int tile_step = PAIR ? (int)cluster_count_x() : (int)gridDim.x;
    const int cta_rank = PAIR ? (int)cluster_ctarank() : 0;
    uint32_t acc_empty_leader[2] = {0u, 0u};
    if (PAIR) {
        acc_empty_leader[0] = map_to_cta(smem_u32(&acc_empty[0]), 0);
        acc_empty_leader[1] = map_to_cta(smem_u32(&acc_empty[1]), 0);
    }
    constexpr int NCHUNK = BN / 32;
    constexpr bool GENERIC = MODE == EPI_GENERIC;
    constexpr bool HAS_OUT = MODE != EPI_ARGMAX;
    constexpr bool TMA_BF16 = MODE == EPI_BF16 || MODE == EPI_BF16_GELU;
    constexpr bool TMA_OUT = TMA_BF16 || MODE == EPI_F32_ACCUM || MODE == EPI_F32;
    const int ew = warp - 2;                        // 0..7
    const int quarter = warp & 3;
    const int half = ew >> 2;                       // 0: even chunks, 1: odd chunks
    float* stage_tile = staging + ew * 1024;
    float* bias_line = staging - 256 + ew * 32;          // eight 128-byte lines in the 1 KB below the staging tiles
    const int sub_row = lane >> 3;                  // phase 2: row inside a group of four
    const int c4 = lane & 7;                        // phase 2: 16-byte unit inside the 128-byte row segment

    const bool has_bias = ep.bias != nullptr;
    const bool has_res = MODE == EPI_F32_RES || (GENERIC && ep.residual != nullptr);
    const bool want_argmax = MODE == EPI_ARGMAX || (GENERIC && ep.argmax_partials != nullptr);
    const bool has_out = HAS_OUT && (!GENERIC || ep.out != nullptr);
    const bool out_bf16 = MODE == EPI_BF16 || MODE == EPI_BF16_GELU || (GENERIC && ep.out_kind == TL_OUT_BF16);
    const bool round_out = (GENERIC || MODE == EPI_F32) && ep.out_kind == TL_OUT_TF32;
    bool vec_ok = true;                              // specialised variants: guaranteed by the host
    if (GENERIC) {
        const int esz = out_bf16 ? 2 : 4;
        vec_ok = has_out && ((reinterpret_cast<uintptr_t>(ep.out) & 15u) == 0) && ((ep.ldo * esz) % 16 == 0) &&
                 (!has_res || (((reinterpret_cast<uintptr_t>(ep.residual) & 15u) == 0) && (ep.ldr % 4 == 0)));
    }

    int local = 0;
    // with split_k > 1 (in-place accumulation only) a work unit is one K range of one tile; the ranges of a tile add
    // their partial sums into the output independently, and only range 0 adds the bias
    for (int u = tile0; u < total_tiles * split_k; u += tile_step, local++) {
        const int t = u / split_k;
        const bool first_split = u - t * split_k == 0;
        TileCoord tc = tile_coord(t, m_tiles, n_tiles);
        if (PAIR) tc.m_blk = tc.m_blk * 2 + cta_rank;
        const int buf = local & 1;
        const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
        const int n0 = tc.n_blk * BN;
        const long long row_base = (long long)tc.m_blk * BM + quarter * 32;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
        // live chunks of this warp: half, half + 2, ... while the chunk starts inside N; with bf16 TMA stores a warp
        // takes pairs of adjacent chunks (64 columns = one 128-byte staging row): 2 half, 2 half + 1, 2 half + 4, ...
        auto chunk_of = [&](int i) { return TMA_BF16 ? 2 * half + (i & 1) + 4 * (i >> 1) : half + 2 * i; };
        int n_live = 0;
        while (chunk_of(n_live) < NCHUNK && n0 + chunk_of(n_live) * 32 < N) n_live++;

        float best = -INFINITY;
        int best_i = 0x7fffffff;
        bool waited = false;
#pragma unroll 1
        for (int i = 0; i < n_live; i++) {
            const int chunk = chunk_of(i);
            const int col0 = n0 + chunk * 32;
            const int ncols = min(32, N - col0);
            const bool full = ncols == 32;
            const bool fast = vec_ok && full;
            // requests that do not depend on the accumulator go out first
            // the chunk's 32 bias values go through a 128-byte line of shared memory: every thread (= row) needs all of
            // them, and eight broadcast reads are cheaper than 32 shuffles
            if (has_bias && first_split) {
                __syncwarp();                                  // the previous chunk's reads are done
                bias_line[lane] = lane < ncols ? __ldg(ep.bias + col0 + lane) : 0.f;
                __syncwarp();
            }
            float4 res[8];
            if (has_res && fast) {
#pragma unroll
                for (int it = 0; it < 8; it++) {
                    const long long row = row_base + it * 4 + sub_row;
                    long long rrow = row;
                    if (GENERIC && ep.res_row_mod > 0) rrow = ep.res_row_off + row % ep.res_row_mod;
                    res[it] = row < M ? *reinterpret_cast<const float4*>(ep.residual + rrow * ep.ldr + col0 + c4 * 4)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            if (!waited) {
                if (!mbar_wait(&acc_full[buf], buf_phase, abort_flag, err, 104)) {
                    if (TMA_OUT && lane == 0) tma_store_wait_all();
                    return;
                }
                __syncwarp();
                tc_fence_after();
                waited = true;
            }
            uint32_t acc[32];
            tmem_ld32_issue(taddr + (uint32_t)(chunk * 32), acc);
            tmem_ld_wait();
            if (i == n_live - 1) {
                // every accumulator column this warp needs is in registers: hand the buffer back
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(acc_empty_leader[buf]);
                    else mbar_arrive(&acc_empty[buf]);
                }
            }
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(acc[j]);
            // ---- phase 1
            if (has_bias && first_split) {
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bias_line + 4 * u);
                    v[4 * u] += b4.x; v[4 * u + 1] += b4.y; v[4 * u + 2] += b4.z; v[4 * u + 3] += b4.w;
                }
            }
            if (MODE == EPI_BF16_GELU) {
                apply_act_chunk<false>(TLNN_ACT_GELU, v);
            } else if ((GENERIC || MODE == EPI_F32) && ep.act != TLNN_ACT_NONE) {
                if (ep.accurate_math) apply_act_chunk<true>(ep.act, v);
                else apply_act_chunk<false>(ep.act, v);
            }
            if (want_argmax) {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (j < ncols && v[j] > best) { best = v[j]; best_i = col0 + j; }
            }
            if (TMA_OUT) {
                // the previous store may still be reading the staging tile
                const bool first_of_tile = TMA_BF16 ? (i & 1) == 0 : true;
                if (first_of_tile) {
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
                }
                if (TMA_BF16) {
                    // 32 columns = 64 bytes = units 4 (i & 1) .. + 3 of this thread's 128-byte staging row
                    uint8_t* row = reinterpret_cast<uint8_t*>(stage_tile) + lane * 128;
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        uint4 pk;
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk.x) : "f"(v[8 * u + 1]), "f"(v[8 * u + 0]));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk.y) : "f"(v[8 * u + 3]), "f"(v[8 * u + 2]));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk.z) : "f"(v[8 * u + 5]), "f"(v[8 * u + 4]));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk.w) : "f"(v[8 * u + 7]), "f"(v[8 * u + 6]));
                        *reinterpret_cast<uint4*>(row + ((((i & 1) * 4 + u) ^ (lane & 7)) << 4)) = pk;
                    }
                } else {
                    if (MODE == EPI_F32 && round_out) {
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = round_tf32(v[j]);
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++)
                        *reinterpret_cast<float4*>(stage_tile + lane * 32 + ((u ^ (lane & 7)) << 2)) =
                            make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
                }
                const bool last_of_store = TMA_BF16 ? ((i & 1) == 1 || i == n_live - 1) : true;
                if (last_of_store) {
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const int x0 = TMA_BF16 ? n0 + (chunk & ~1) * 32 : col0;
                        if (MODE == EPI_F32_ACCUM) tma_reduce_add_2d(tm_out, smem_u32(stage_tile), x0, (int)row_base);
                        else tma_store_2d(tm_out, smem_u32(stage_tile), x0, (int)row_base);
                        tma_store_commit();
                    }
                }
            } else if (has_out) {
#pragma unroll
                for (int u = 0; u < 8; u++)
                    *reinterpret_cast<float4*>(stage_tile + lane * 32 + ((u ^ (lane & 7)) << 2)) =
                        make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
                __syncwarp();
                // ---- phase 2
                if (fast) {
#pragma unroll
                    for (int it = 0; it < 8; it++) {
                        const int rr = it * 4 + sub_row;
                        const long long row = row_base + rr;
                        float4 o = *reinterpret_cast<const float4*>(stage_tile + rr * 32 + ((c4 ^ (rr & 7)) << 2));
                        if (has_res) { o.x += res[it].x; o.y += res[it].y; o.z += res[it].z; o.w += res[it].w; }
                        if (row < M) {
                            long long orow = row;
                            if (GENERIC && ep.row_group > 0)
                                orow = (row / ep.row_group) * ep.out_group + ep.out_off + row % ep.row_group;
                            const long long off = orow * ep.ldo + col0 + c4 * 4;
                            if (!TL_DBG_IN_BOUNDS(err, off >= 0 && off + 4 <= ep.out_elems, 910, off)) continue;
                            if (out_bf16) {
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(o.x, o.y);
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(o.z, o.w);
                                uint2 pk;
                                pk.x = *reinterpret_cast<uint32_t*>(&h0);
                                pk.y = *reinterpret_cast<uint32_t*>(&h1);
                                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ep.out) + off) = pk;
                            } else {
                                if (round_out) {
                                    o.x = round_tf32(o.x); o.y = round_tf32(o.y); o.z = round_tf32(o.z); o.w = round_tf32(o.w);
                                }
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(ep.out) + off) = o;
                            }
                        }
                    }
                } else if (GENERIC) {
                    // ragged or unaligned: one column per lane, one row per step - still whole row segments
                    const bool col_ok = lane < ncols;
#pragma unroll 1
                    for (int rr = 0; rr < 32; rr++) {
                        const long long row = row_base + rr;
                        if (row >= M) break;
                        float o = stage_tile[rr * 32 + ((((lane >> 2) ^ (rr & 7)) << 2) | (lane & 3))];
                        if (col_ok) {
                            if (has_res) {
                                const long long rrow = ep.res_row_mod > 0 ? ep.res_row_off + row % ep.res_row_mod : row;
                                o += ep.residual[rrow * ep.ldr + col0 + lane];
                            }
                            const long long orow = ep.row_group > 0
                                ? (row / ep.row_group) * ep.out_group + ep.out_off + row % ep.row_group : row;
                            const long long off = orow * ep.ldo + col0 + lane;
                            if (out_bf16) reinterpret_cast<__nv_bfloat16*>(ep.out)[off] = __float2bfloat16_rn(o);
                            else reinterpret_cast<float*>(ep.out)[off] = round_out ? round_tf32(o) : o;
                        }
                    }
                }
                __syncwarp();     // the staging tile is rewritten by the next chunk
            }
        }
        if (n_live == 0) {
            // no live chunk in this tile: the MMA warp still needs this warp's arrival for the buffer
            if (!mbar_wait(&acc_full[buf], buf_phase, abort_flag, err, 105)) {
                if (TMA_OUT && lane == 0) tma_store_wait_all();
                return;
            }
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(acc_empty_leader[buf]);
                else mbar_arrive(&acc_empty[buf]);
            }
        }
        if (want_argmax) {
            const long long my_row = row_base + lane;
            // two warps cover a row: each leaves its own candidate, the reduce kernel takes the better one
            if (my_row < M)
                ep.argmax_partials[(my_row * n_tiles + tc.n_blk) * 2 + half] = make_float2(best, __int_as_float(best_i));
        }
    }
    if (TMA_OUT && lane == 0) tma_store_wait_all();
}

// ---- the kernel ---------------------------------------------------------------------------------------------------------
template <int BN, bool TF32, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmOut, const tl_gemm_epilogue ep, int M, int N, int K, int m_tiles,
                    int n_tiles, int split_k, tlnn_dev_err* err) {
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

    tl_grid_dependency_trigger();            // the successor may start launching; it waits for this grid itself
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = m_tiles * n_tiles;
    const int num_k = (K + K_ELEMS - 1) / K_ELEMS;
    const int kb_per_split = (num_k + split_k - 1) / split_k;      // the host guarantees that no K range is empty
    const int total_units = total_tiles * split_k;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (MODE == EPI_BF16 || MODE == EPI_BF16_GELU || MODE == EPI_F32_ACCUM || MODE == EPI_F32) tma_prefetch_desc(&tmOut);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 8);      // one arrival per epilogue warp
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
    // barriers, TMEM and descriptors are ready; nothing below may touch global memory before the predecessor is done
    tl_grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                const int t = u / split_k;
                const int kb_lo = (u - t * split_k) * kb_per_split, kb_hi = min(num_k, kb_lo + kb_per_split);
                TileCoord tc = tile_coord(t, m_tiles, n_tiles);
                for (int kb = kb_lo; kb < kb_hi; kb++) {
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
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, local++) {
                const int kb_lo = (u % split_k) * kb_per_split, kb_hi = min(num_k, kb_lo + kb_per_split);
                const int buf = local & 1;
                const uint32_t buf_phase = (uint32_t)(local >> 1) & 1u;
                if (!mbar_wait(&acc_empty[buf], buf_phase ^ 1u, abort_flag, err, 102)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kb = kb_lo; kb < kb_hi; kb++) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag, err, 103)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t sa = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
                    uint64_t a_desc = make_smem_desc(sa);
                    uint64_t b_desc = make_smem_desc(sa + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < ROW_BYTES / MMA_K_BYTES; k++) {
                        // advancing K inside the swizzle atom = advancing the start address by 32 bytes (>>4 = 2)
                        umma<TF32>(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                                   (kb != kb_lo || k != 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (8 warps, 128 rows x BN columns)
        epilogue_warp<BN, MODE>(ep, M, N, m_tiles, n_tiles, total_tiles, warp, lane, tmem_base,
                                reinterpret_cast<float*>(smem + C::EPI_OFFSET), acc_full, acc_empty, abort_flag, err, &tmOut,
                                split_k);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

// ---- the pair kernel (bf16, 256 x 256 tiles over two SMs) ---------------------------------------------------------------
// A cluster of two CTAs computes a 256 x 256 tile: each CTA loads its own 128 rows of A and one half (128 rows) of
// the W tile, the leader CTA (rank 0) issues tcgen05.mma.cta_group::2, which reads both halves of W from both CTAs'
// shared memory, and each CTA ends up with its 128 x 256 accumulator in its own TMEM.  Per k-block a CTA writes and
// reads 32 KB of shared memory instead of 48 KB, which lifts the shared-memory bandwidth limit of the one-CTA tile.
// Barriers: `full` lives in the leader and counts the bytes of all four loads; `empty` and `acc_full` exist in both
// CTAs and the leader's MMA thread commits to each; `acc_empty` lives in the leader and collects the sixteen
// epilogue warps of the pair.  Both CTAs pass one cluster barrier after set-up and one before they return their
// TMEM; every role reaches the second one on every path, time-outs included.
struct PairCfg {
    static constexpr int BN = 256;
    static constexpr int STAGES = 6;
    static constexpr uint32_t A_BYTES = BM * ROW_BYTES;            // 16 KB: this CTA's rows of A
    static constexpr uint32_t B_BYTES = (BN / 2) * ROW_BYTES;      // 16 KB: this CTA's half of the W tile
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = PAIR_TMEM_COLS;
    static constexpr uint32_t BAR_BYTES = 2048;      // barriers, then eight 128-byte bias lines; keeps the staging tiles 1024-byte aligned (TMA swizzle phase)
    static constexpr uint32_t EPI_OFFSET = STAGES * STAGE_BYTES + BAR_BYTES;
    static constexpr size_t SMEM = (size_t)EPI_OFFSET + 8 * 4096 + 1024;
};

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmOut, const tl_gemm_epilogue ep, int M, int N, int K,
                         int m_pairs, int n_tiles, tlnn_dev_err* err) {
    using C = PairCfg;
    constexpr int STAGES = C::STAGES;
    constexpr int BN = C::BN;
    constexpr int K_ELEMS = 64;
    constexpr int ACC_BUFS = C::TMEM_COLS / BN;            // 2 (1 while the allocation semantics are being verified)

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    tl_grid_dependency_trigger();            // the successor may start launching; it waits for this grid itself
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int total_tiles = m_pairs * n_tiles;
    const int num_k = (K + K_ELEMS - 1) / K_ELEMS;
    const int tile0 = (int)cluster_id_x(), tile_step = (int)cluster_count_x();

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (MODE == EPI_BF16 || MODE == EPI_BF16_GELU || MODE == EPI_F32_ACCUM || MODE == EPI_F32) tma_prefetch_desc(&tmOut);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 16);     // one arrival per epilogue warp of the pair
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // barriers, TMEM and descriptors are ready; nothing below may touch global memory before the predecessor is done
    tl_grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one per CTA)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = tile0; t < total_tiles && ok; t += tile_step) {
                const TileCoord tc = tile_coord(t, m_pairs, n_tiles);
                const int row_a = (tc.m_blk * 2 + (int)rank) * BM;
                const int row_b = tc.n_blk * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, err, 111)) { ok = false; break; }
                    const uint32_t sa = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
                    const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
                    if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * C::STAGE_BYTES);
                    tma_load_2d_pair(sa, &tmA, bar, kb * K_ELEMS, row_a);
                    tma_load_2d_pair(sa + C::A_BYTES, &tmB, bar, kb * K_ELEMS, row_b);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            // D float32, A / B bf16 K-major, N = 256, M = 256 over the pair
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = tile0; t < total_tiles && ok; t += tile_step, local++) {
                const int buf = local % ACC_BUFS;
                const uint32_t buf_phase = (uint32_t)(local / ACC_BUFS) & 1u;
                if (!mbar_wait(&acc_empty[buf], buf_phase ^ 1u, abort_flag, err, 112)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag, err, 113)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
                    const uint64_t a_desc = make_smem_desc(sa);
                    const uint64_t b_desc = make_smem_desc(sa + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < ROW_BYTES / MMA_K_BYTES; k++)
                        umma_pair_f16(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
                    // the stage is free in both CTAs once these MMAs have read it
                    const uint32_t eb = smem_u32(&empty_bar[stage]);
                    umma_commit_pair(map_to_cta(eb, 0));
                    umma_commit_pair(map_to_cta(eb, 1));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) {
                    const uint32_t fb = smem_u32(&acc_full[buf]);
                    umma_commit_pair(map_to_cta(fb, 0));
                    umma_commit_pair(map_to_cta(fb, 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (8 warps per CTA, 128 rows x 256 columns)
        if (ACC_BUFS == 2) {
            epilogue_warp<BN, MODE, true>(ep, M, N, m_pairs, n_tiles, total_tiles, warp, lane, tmem_base,
                                          reinterpret_cast<float*>(smem + C::EPI_OFFSET), acc_full, acc_empty, abort_flag, err,
                                          &tmOut);
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       // nobody returns TMEM or leaves while the peer may still touch this CTA
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
int pick_bn(int M, int N, int sm_count) {
    // TLNN_GEMM_BN=64|128|256 forces the tile width (measurements only)
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("TLNN_GEMM_BN");
        forced = e ? atoi(e) : 0;
        if (forced != 64 && forced != 128 && forced != 256) forced = 0;
    }
    if (forced) return forced;
    const int m_tiles = (M + BM - 1) / BM;
    const long long t256 = (long long)m_tiles * ((N + 255) / 256), t128 = (long long)m_tiles * ((N + 127) / 128);
    if (N > 128 && t256 >= sm_count) return 256;
    // one round of 256-wide tiles on most of the SMs against two rounds of 128-wide ones (16640 x 192 outputs: 130
    // tiles against 260; 2.5 % of a whole ViT forward)
    if (N > 128 && t256 * 4 >= sm_count * 3ll && t128 > sm_count) return 256;
    if (N > 64 && t128 >= sm_count) return 128;
    // too few tiles to fill the SMs either way: the narrowest tile gives the most CTAs streaming the weight
    return 64;
}

template <int BN, bool TF32, int MODE>
int launch(tlnn_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const tl_gemm_epilogue& ep,
           int M, int N, int K) {
    auto kernel = gemm_tcgen05_kernel<BN, TF32, MODE>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::SMEM));
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    long long total = (long long)m_tiles * n_tiles;
    TL_REQUIRE(total < (1ll << 31), "gemm: too many tiles");
    // In-place accumulation with few tiles and a long contraction (the feed-forward output and attention output
    // products of a decode step): split K over several CTAs, each adding its partial tile into the output.  The order
    // of those float32 additions is not fixed from run to run.
    int split_k = 1;
    static const bool split_allowed = !(getenv("TLNN_GEMM_SPLITK") && strcmp(getenv("TLNN_GEMM_SPLITK"), "0") == 0);
    if (MODE == EPI_F32_ACCUM && split_allowed && total * 2 <= ctx->sm_count) {
        const int num_k = (K + (TF32 ? 32 : 64) - 1) / (TF32 ? 32 : 64);
        int want = (int)(ctx->sm_count / total);
        if (want > num_k / 3) want = num_k / 3;                 // at least three k-blocks per range
        if (want > 1) {
            const int per = (num_k + want - 1) / want;
            split_k = (num_k + per - 1) / per;                   // no empty range
        }
    }
    total *= split_k;
    const int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
    const char* name = TF32 ? (BN == 256 ? "gemm_tf32_n256" : BN == 128 ? "gemm_tf32_n128" : "gemm_tf32_n64")
                            : (BN == 256 ? "gemm_bf16_n256" : BN == 128 ? "gemm_bf16_n128" : "gemm_bf16_n64");
    TL_LAUNCH(ctx, name, tl_launch_kernel(ctx, kernel, dim3(grid), dim3(NUM_THREADS), Cfg<BN>::SMEM, ta, tb, to, ep, M, N, K, m_tiles,
                                          n_tiles, split_k, ctx->d_err));
    return TLNN_OK;
}

// Persistent clusters of the pair kernel that fit on the device at once (queried once per epilogue variant).
template <int MODE>
int launch_pair(tlnn_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const tl_gemm_epilogue& ep,
                int M, int N, int K) {
    auto kernel = gemm_tcgen05_pair_kernel<MODE>;
    const int m_pairs = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + PairCfg::BN - 1) / PairCfg::BN;
    const long long total = (long long)m_pairs * n_tiles;
    TL_REQUIRE(total < (1ll << 31), "gemm: too many tiles");
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;      // see tl_launch_kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = PairCfg::SMEM;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 2 : 1;
    static int max_clusters = 0;
    if (max_clusters == 0) {
        TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairCfg::SMEM));
        cfg.gridDim = dim3(2 * (ctx->sm_count / 2));
        int n = 0;
        TL_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        TL_REQUIRE(n > 0, "gemm: no cluster of two CTAs fits on this device");
        max_clusters = n < ctx->sm_count / 2 ? n : ctx->sm_count / 2;
    }
    const int clusters = (int)(total < max_clusters ? total : max_clusters);
    cfg.gridDim = dim3(2 * clusters);
    TL_LAUNCH(ctx, "gemm_bf16_pair", TL_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, to, ep, M, N, K, m_pairs, n_tiles, ctx->d_err)));
    return TLNN_OK;
}

int launch_pair_mode(tlnn_ctx* ctx, int mode, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to,
                     const tl_gemm_epilogue& ep, int M, int N, int K) {
    switch (mode) {
        case EPI_BF16: return launch_pair<EPI_BF16>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_BF16_GELU: return launch_pair<EPI_BF16_GELU>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_F32_RES: return launch_pair<EPI_F32_RES>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_F32_ACCUM: return launch_pair<EPI_F32_ACCUM>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_F32: return launch_pair<EPI_F32>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_ARGMAX: return launch_pair<EPI_ARGMAX>(ctx, ta, tb, to, ep, M, N, K);
        default: return launch_pair<EPI_GENERIC>(ctx, ta, tb, to, ep, M, N, K);
    }
}

// The pair kernel pays off when there are enough 256 x 256 tiles to keep every cluster busy for two rounds or more
// (measured at M = 16384, N = 1024: 8 % faster than the one-CTA tile at K = 4096, 3 % slower at K = 1024).
// TLNN_GEMM_PAIR=0 switches it off, =force uses it for every bf16 product.
bool use_pair(int sm_count, int prec, int M, int N) {
    static int policy = -1;
    if (policy < 0) {
        const char* e = getenv("TLNN_GEMM_PAIR");
        policy = e == nullptr ? 1 : (strcmp(e, "0") == 0 ? 0 : (strcmp(e, "force") == 0 ? 2 : 1));
    }
    if (prec != TLNN_PREC_BF16 || policy == 0) return false;
    if (policy == 2) return true;
    const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + PairCfg::BN - 1) / PairCfg::BN);
    // a pair needs rows for both of its CTAs
    return M > BM && pick_bn(M, N, sm_count) == 256 && tiles >= (long long)sm_count;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The specialised epilogue that matches this description exactly, or EPI_GENERIC.
int pick_mode(const tl_gemm_epilogue& ep, int N) {
    const bool plain_rows = ep.row_group == 0 && ep.res_row_mod == 0;
    if (ep.out == nullptr && ep.argmax_partials != nullptr && ep.residual == nullptr && ep.act == TLNN_ACT_NONE)
        return EPI_ARGMAX;
    if (!plain_rows || ep.argmax_partials != nullptr || ep.out == nullptr || N % 32 != 0 || !aligned16(ep.out))
        return EPI_GENERIC;
    if (ep.out_kind == TL_OUT_BF16 && ep.residual == nullptr && (ep.ldo * 2) % 16 == 0) {
        if (ep.act == TLNN_ACT_NONE) return EPI_BF16;
        if (ep.act == TLNN_ACT_GELU && !ep.accurate_math) return EPI_BF16_GELU;
    }
    // float32 out (as is, or rounded to TF32 for the next product), optional activation, no residual
    if ((ep.out_kind == TL_OUT_F32 || ep.out_kind == TL_OUT_TF32) && ep.residual == nullptr && (ep.ldo * 4) % 16 == 0)
        return EPI_F32;
    if (ep.out_kind == TL_OUT_F32 && ep.residual != nullptr && ep.act == TLNN_ACT_NONE && (ep.ldo * 4) % 16 == 0 &&
        aligned16(ep.residual) && ep.ldr % 4 == 0)
        return (ep.residual == ep.out && ep.ldr == ep.ldo) ? EPI_F32_ACCUM : EPI_F32_RES;
    return EPI_GENERIC;
}

template <int BN>
int launch_bn(tlnn_ctx* ctx, bool tf32, int mode, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to,
              const tl_gemm_epilogue& ep, int M, int N, int K) {
    if (tf32) {
        // float32 / TF32 operands: the variants whose output is plain float32
        switch (mode) {
            case EPI_F32: return launch<BN, true, EPI_F32>(ctx, ta, tb, to, ep, M, N, K);
            case EPI_F32_RES: return launch<BN, true, EPI_F32_RES>(ctx, ta, tb, to, ep, M, N, K);
            default: return launch<BN, true, EPI_GENERIC>(ctx, ta, tb, to, ep, M, N, K);
        }
    }
    switch (mode) {
        case EPI_F32: return launch<BN, false, EPI_F32>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_BF16: return launch<BN, false, EPI_BF16>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_BF16_GELU: return launch<BN, false, EPI_BF16_GELU>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_F32_RES: return launch<BN, false, EPI_F32_RES>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_F32_ACCUM: return launch<BN, false, EPI_F32_ACCUM>(ctx, ta, tb, to, ep, M, N, K);
        case EPI_ARGMAX: return launch<BN, false, EPI_ARGMAX>(ctx, ta, tb, to, ep, M, N, K);
        default: return launch<BN, false, EPI_GENERIC>(ctx, ta, tb, to, ep, M, N, K);
    }
}

}  // namespace

namespace {
// A wait that nothing will satisfy, through the same bounded-wait routine every kernel of the library uses: it gives
// up after limit_ns, records TLNN_ERR_TIMEOUT and the kernel returns normally.
__global__ void wait_selftest_kernel(unsigned long long limit_ns, tlnn_dev_err* err) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_wait(&bar, 0, &abort_flag, err, 900, limit_ns);
    }
}
}  // namespace

extern "C" int tlnn_selftest_wait(tlnn_ctx* ctx, int limit_ms) {
    TL_NOTNULL(ctx);
    TL_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, "selftest: the wait limit must lie between 1 and 1000 ms");
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_LAUNCH(ctx, "wait_selftest", wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>((unsigned long long)limit_ms * 1000000ull, ctx->d_err));
    return TLNN_OK;
}

int tl_gemm_bn(int M, int N, int sm_count) { return pick_bn(M, N, sm_count); }
bool tl_gemm_uses_pair(int prec, int M, int N, int sm_count) { return use_pair(sm_count, prec, M, N); }
int tl_gemm_argmax_parts(int prec, int M, int N, int sm_count) {
    const int bn = use_pair(sm_count, prec, M, N) ? PairCfg::BN : pick_bn(M, N, sm_count);
    return 2 * ((N + bn - 1) / bn);     // two epilogue warps cover each row of a tile
}

int tl_gemm(tlnn_ctx* ctx, int prec, const void* a, long long lda, const void* w, long long ldw, int M, int N, int K,
            const tl_gemm_epilogue& ep_in) {
    if (M == 0 || N == 0) return TLNN_OK;
    tl_gemm_epilogue ep = ep_in;
    {
        // extent of the output as the epilogue addresses it (rows may be remapped in groups): last row's end
        const long long out_rows = ep.row_group > 0 ? ((long long)(M - 1) / ep.row_group) * ep.out_group + ep.out_off + (M - 1) % ep.row_group + 1 : M;
        ep.out_elems = (out_rows - 1) * ep.ldo + N;
    }
    TL_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad shape M=%d N=%d K=%d", M, N, K);
    const int esz = prec == TLNN_PREC_BF16 ? 2 : 4;
    TL_REQUIRE((K * esz) % 16 == 0, "gemm: the contraction length %d must be a multiple of %d elements", K, 16 / esz);
    TL_REQUIRE((lda * esz) % 16 == 0 && (ldw * esz) % 16 == 0, "gemm: operand pitches must be multiples of 16 bytes");
    TL_REQUIRE(((uintptr_t)a & 15u) == 0 && ((uintptr_t)w & 15u) == 0, "gemm: operands must be 16-byte aligned");
    const bool tf32 = prec == TLNN_PREC_TF32;
    int mode = pick_mode(ep, N);
    if (tf32 && mode != EPI_F32 && mode != EPI_F32_RES) mode = EPI_GENERIC;
    // output tensor map of the epilogues that leave through TMA: 32 rows x 128 bytes (64 bf16 or 32 float32 columns)
    CUtensorMap ta, tb, to;
    memset(&to, 0, sizeof(to));
    if (mode == EPI_BF16 || mode == EPI_BF16_GELU) TL_TRY(make_tile_map(&to, true, ep.out, M, N, ep.ldo, 32));
    if (mode == EPI_F32_ACCUM || mode == EPI_F32) TL_TRY(make_tile_map(&to, false, ep.out, M, N, ep.ldo, 32));
    if (use_pair(ctx->sm_count, prec, M, N)) {
        TL_TRY(make_tile_map(&ta, true, a, M, K, lda, BM));
        TL_TRY(make_tile_map(&tb, true, w, N, K, ldw, PairCfg::BN / 2));
        return launch_pair_mode(ctx, mode, ta, tb, to, ep, M, N, K);
    }
    const int bn = pick_bn(M, N, ctx->sm_count);
    TL_TRY(make_tile_map(&ta, prec == TLNN_PREC_BF16, a, M, K, lda, BM));
    TL_TRY(make_tile_map(&tb, prec == TLNN_PREC_BF16, w, N, K, ldw, bn));
    if (bn == 256) return launch_bn<256>(ctx, tf32, mode, ta, tb, to, ep, M, N, K);
    if (bn == 128) return launch_bn<128>(ctx, tf32, mode, ta, tb, to, ep, M, N, K);
    return launch_bn<64>(ctx, tf32, mode, ta, tb, to, ep, M, N, K);
}

// ---- tensor-map encoding (shared with the attention kernel) ---------------------------------------------------------
namespace {
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

}  // namespace

int sm100::make_tile_map(CUtensorMap* map, bool bf16, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        tl_set_error("cuTensorMapEncodeTiled is not available from the driver");
        return TLNN_ERR_CUDA;
    }
    const int esz = bf16 ? 2 : 4;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(ld * esz)};
    cuuint32_t box[2] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                    2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_set_error("cuTensorMapEncodeTiled failed with %d (rows=%lld K=%lld ld=%lld box_rows=%d)", (int)r, rows, K, ld,
                     box_rows);
        return TLNN_ERR_CUDA;
    }
    return TLNN_OK;
}


// Row-major bf16 matrix, box of box_cols x box_rows elements, no swizzle: the tile lands in shared memory as box_rows
// dense rows of box_cols elements (used where a consumer reads whole rows with plain shared-memory loads).
int sm100::make_plain_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_cols, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        tl_set_error("cuTensorMapEncodeTiled is not available from the driver");
        return TLNN_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(ld * 2)};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_set_error("cuTensorMapEncodeTiled failed with %d (rows=%lld cols=%lld ld=%lld box=%dx%d)", (int)r, rows, cols, ld, box_cols, box_rows);
        return TLNN_ERR_CUDA;
    }
    return TLNN_OK;
}
