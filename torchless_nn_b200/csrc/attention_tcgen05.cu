// Fused attention on the sm_100a tensor cores (bf16, head dimension 64).
//
// One CTA owns 256 consecutive queries of one (batch, head) as two independent 128-row streams.  Roles by warp:
//   warps 0-3  softmax of stream 0 (thread = query row: a score row is read from TMEM by one thread, so the row
//              maximum and the row sum need no shuffles), warps 4-7 the same for stream 1;
//   warps 8-9  MMA issuers, one thread per stream: S_j = Q K_j^T (128 x 64 x 64) into one of the stream's two S
//              buffers in TMEM, and O += P_j V_j (128 x 64 x 64) with P taken from shared memory and V read as an
//              MN-major operand; S_{j+2} is issued as soon as S_j has been read, P_j V_j when P_j is complete;
//   warp 10    TMA producer: Q once, then K / V tiles of 64 keys through a six-stage ring.
// S is double-buffered per stream, so S_{j+1} and S_{j+2} are computed while the softmax warps work on S_j; the
// softmax of a tile waits only for its own S (and, rarely, for the accumulator to be quiescent), never for the P V
// product of the previous tile.  O accumulates in TMEM across tiles; probabilities are taken against a reference
// maximum that is moved (and O, l rescaled in TMEM) only when the true row maximum has grown by more than 2^8, which is
// exact after the final division by l.  The decoder mask is an index comparison.
// All waits are bounded in time; on expiry the kernel records TLNN_ERR_TIMEOUT and every role leaves.
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int HD = 64;                 // head dimension
constexpr int BQ = 128;                // query rows per stream
constexpr int BK = 64;                 // keys per tile
constexpr int KV_STAGES = 6;
constexpr int AT_THREADS = 352;        // 8 softmax warps, 2 MMA issuers, 1 TMA producer
constexpr uint32_t Q_BYTES = BQ * HD * 2;          // 16 KB per stream
constexpr uint32_t K_BYTES = BK * HD * 2;          // 8 KB
constexpr uint32_t V_BYTES = BK * HD * 2;          // 8 KB
constexpr uint32_t P_BYTES = BQ * BK * 2;          // 16 KB: 128 rows x 128 bytes, one swizzle block
constexpr uint32_t OFF_Q = 0;
constexpr uint32_t OFF_KV = OFF_Q + 2 * Q_BYTES;
constexpr uint32_t OFF_P = OFF_KV + KV_STAGES * (K_BYTES + V_BYTES);      // P[stream][buffer]
constexpr uint32_t OFF_BAR = OFF_P + 4 * P_BYTES;
constexpr size_t AT_SMEM = OFF_BAR + 512 + 1024;   // barriers + alignment slack
constexpr uint32_t TMEM_COLS = 512;                // S[s][b] at 128 s + 64 b, O[s] at 256 + 64 s

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two float32 -> packed bf16 pair, round to nearest (ties up) with integer adds and one byte permute, which keeps the
// conversions off the special-function unit.  Inputs are finite and non-negative.
__device__ __forceinline__ uint32_t pack_bf16_rn(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}

// Instruction descriptors: D float32, A and B bf16, M = 128, N = 64.  S: both operands K-major.  PV: A K-major (P),
// B MN-major (V rows are keys, the head dimension is contiguous).
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BK >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                              ((uint32_t)(BQ >> 4) << 24);

template <bool CAUSAL>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                         __nv_bfloat16* __restrict__ out, int T, int H, float scale_log2, tlnn_dev_err* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* kv_full = q_full + 1;                  // [KV_STAGES]
    uint64_t* kv_empty = kv_full + KV_STAGES;        // [KV_STAGES]
    uint64_t* s_full = kv_empty + KV_STAGES;         // [2][2] S_j is in TMEM buffer j & 1
    uint64_t* p_full = s_full + 4;                   // [2][2] P_j is in shared-memory buffer j & 1 (and S_j has been read)
    uint64_t* pv_done = p_full + 4;                  // [2][2] O includes P_j V_j (and P buffer j & 1 may be rewritten)
    uint64_t* s_free = pv_done + 4;                  // [2][2] S_j has been read into registers: its TMEM buffer may be rewritten
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = H * HD;
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int q_blk = CAUSAL ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;     // longest causal blocks first
    const int q0 = q_blk * 2 * BQ;
    const int row0 = b * T;                                // first row of this sequence in the packed (B*T, 3d) buffer
    const int tiles_all = (T + BK - 1) / BK;
    // key tiles per stream: causal rows q see keys <= q
    const int qs1 = q0 + BQ;
    const int nt0 = q0 >= T ? 0 : (CAUSAL ? min(tiles_all, (q0 + BQ - 1) / BK + 1) : tiles_all);
    const int nt1 = qs1 >= T ? 0 : (CAUSAL ? min(tiles_all, (qs1 + BQ - 1) / BK + 1) : tiles_all);
    const int n_max = max(nt0, nt1);

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_kv);
        mbar_init(q_full, 1);
        for (int i = 0; i < KV_STAGES; i++) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 2); }
        for (int i = 0; i < 4; i++) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&pv_done[i], 1); mbar_init(&s_free[i], 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 10) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, 2 * Q_BYTES);
            tma_load_2d(smem_u32(smem + OFF_Q), &tm_q, smem_u32(q_full), h * HD, row0 + q0);
            tma_load_2d(smem_u32(smem + OFF_Q + Q_BYTES), &tm_q, smem_u32(q_full), h * HD, row0 + q0 + BQ);
            int stage = 0;
            uint32_t phase = 0;
            for (int t = 0; t < n_max; t++) {
                if (!mbar_wait(&kv_empty[stage], phase ^ 1u, abort_flag, err, 201)) break;
                const uint32_t sk = smem_u32(smem + OFF_KV) + (uint32_t)stage * (K_BYTES + V_BYTES);
                const uint32_t bar = smem_u32(&kv_full[stage]);
                mbar_expect_tx(&kv_full[stage], K_BYTES + V_BYTES);
                tma_load_2d(sk, &tm_kv, bar, d + h * HD, row0 + t * BK);
                tma_load_2d(sk + K_BYTES, &tm_kv, bar, 2 * d + h * HD, row0 + t * BK);
                if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ MMA issuers: one thread per stream
        // Order per stream: S_0, S_1, then for every tile j: wait until S_j has been read -> S_{j+2}; wait P_j ->
        // O += P_j V_j -> give the key tile back.  Both issuers wait on the same kv_full phases; a key tile returns to the producer after two
        // arrivals on kv_empty, one per stream (a stream that does not need a tile arrives for it once it is loaded).
        if (lane == 0) {
            const int s = warp - 8;
            const int nt = s == 0 ? nt0 : nt1;
            bool ok = mbar_wait(q_full, 0, abort_flag, err, 202);
            tc_fence_after();
            const uint64_t q_desc = make_smem_desc(smem_u32(smem + OFF_Q + s * Q_BYTES));
            const uint64_t kv_desc0 = make_smem_desc(smem_u32(smem + OFF_KV));             // + stage * 1024 (16-byte units)
            const uint64_t p_desc0 = make_smem_desc(smem_u32(smem + OFF_P + s * 2 * P_BYTES));
            const uint32_t s_tmem0 = tmem_base + (uint32_t)(s * 128);
            const uint32_t o_tmem = tmem_base + 256u + (uint32_t)(s * HD);
            constexpr uint64_t STAGE_UNITS = (K_BYTES + V_BYTES) >> 4, V_UNITS = K_BYTES >> 4, P_UNITS = P_BYTES >> 4;
            int ld_stage = 0;            // stage / phase of the next tile whose S will be issued
            uint32_t ld_phase = 0;
            int use_stage = 0;           // stage of the next tile whose V will be consumed
            auto issue_s = [&](int j) -> bool {
                if (!mbar_wait(&kv_full[ld_stage], ld_phase, abort_flag, err, 203)) return false;
                tc_fence_after();
                const uint64_t k_desc = kv_desc0 + (uint64_t)ld_stage * STAGE_UNITS;
                const uint32_t s_tmem = s_tmem0 + (uint32_t)((j & 1) * 64);
#pragma unroll
                for (int k = 0; k < HD / 16; k++) umma<false>(s_tmem, q_desc + 2 * k, k_desc + 2 * k, IDESC_S, k != 0 ? 1u : 0u);
                umma_commit(&s_full[s * 2 + (j & 1)]);
                if (++ld_stage == KV_STAGES) { ld_stage = 0; ld_phase ^= 1u; }
                return true;
            };
            if (ok && nt > 0) ok = issue_s(0);
            if (ok && nt > 1) ok = issue_s(1);
            for (int j = 0; j < nt && ok; j++) {
                // the score buffer of tile j is free as soon as the softmax warps hold S_j in registers: compute S_{j+2}
                // into it right away, long before P_j is finished
                if (j + 2 < nt) {
                    if (!mbar_wait(&s_free[s * 2 + (j & 1)], (uint32_t)(j >> 1) & 1u, abort_flag, err, 210)) { ok = false; break; }
                    tc_fence_after();
                    ok = issue_s(j + 2);
                    if (!ok) break;
                }
                if (!mbar_wait(&p_full[s * 2 + (j & 1)], (uint32_t)(j >> 1) & 1u, abort_flag, err, 204)) { ok = false; break; }
                tc_fence_after();
                const uint64_t p_desc = p_desc0 + (uint64_t)(j & 1) * P_UNITS;
                const uint64_t v_desc = kv_desc0 + (uint64_t)use_stage * STAGE_UNITS + V_UNITS;
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++)
                    umma<false>(o_tmem, p_desc + 2 * kk, v_desc + 128 * kk, IDESC_PV, (j > 0 || kk != 0) ? 1u : 0u);
                umma_commit(&pv_done[s * 2 + (j & 1)]);
                umma_commit(&kv_empty[use_stage]);
                if (++use_stage == KV_STAGES) use_stage = 0;
            }
            // key tiles only the other stream needs: arrive for each once it is known to be loaded
            for (int t = nt; t < n_max && ok; t++) {
                if (!mbar_wait(&kv_full[ld_stage], ld_phase, abort_flag, err, 209)) { ok = false; break; }
                mbar_arrive(&kv_empty[ld_stage]);
                if (++ld_stage == KV_STAGES) { ld_stage = 0; ld_phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps (two streams of four warps)
        const int s = warp >> 2;                          // stream
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31
        const int r = quarter * 32 + lane;                // row inside the stream's tile
        const int q_row = q0 + s * BQ + r;                // query index in the sequence
        const int warp_row_lo = q0 + s * BQ + quarter * 32;
        const int nt = s == 0 ? nt0 : nt1;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t o_tmem = tmem_base + lane_base + 256u + (uint32_t)(s * HD);
        // Running statistics.  m_ref is the reference maximum the probabilities and the TMEM accumulator are currently
        // expressed against (log2 units); it moves - and O and l are rescaled - only when the true row maximum has
        // grown by more than 2^8 since, so most tiles do not touch O.
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < nt && ok; j++) {
            const int bsel = j & 1;
            const uint32_t par = (uint32_t)(j >> 1) & 1u;
            if (!mbar_wait(&s_full[s * 2 + bsel], par, abort_flag, err, 205)) { ok = false; break; }
            __syncwarp();
            tc_fence_after();
            const int k0 = j * BK;
            const bool need_mask = (k0 + BK > T) || (CAUSAL && k0 + BK - 1 > warp_row_lo);
            uint32_t sc[BK];
            const uint32_t s_tmem = tmem_base + lane_base + (uint32_t)(s * 128 + bsel * 64);
            tmem_ld32_issue(s_tmem, *reinterpret_cast<uint32_t(*)[32]>(&sc[0]));
            tmem_ld32_issue(s_tmem + 32u, *reinterpret_cast<uint32_t(*)[32]>(&sc[32]));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[s * 2 + bsel]);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < BK; i++) {
                    const int key = k0 + i;
                    if (key >= T || (CAUSAL && key > q_row)) sc[i] = 0xff800000u;      // -inf
                }
            }
            // eight independent partial maxima, then a tree: no 64-long dependency chain
            float mp[8];
#pragma unroll
            for (int i = 0; i < 8; i++) mp[i] = __uint_as_float(sc[i]);
#pragma unroll
            for (int i = 8; i < BK; i++) mp[i & 7] = fmaxf(mp[i & 7], __uint_as_float(sc[i]));
            const float mx = fmaxf(fmaxf(fmaxf(mp[0], mp[1]), fmaxf(mp[2], mp[3])), fmaxf(fmaxf(mp[4], mp[5]), fmaxf(mp[6], mp[7])));
            // tile 0 holds key 0, visible to every row, so m_ref is finite from the first tile on; a later tile whose
            // keys are all masked for this row leaves it unchanged
            const float m_new = fmaxf(m_ref, mx * scale_log2);
            const bool grow = m_new - m_ref > 8.f;                       // also true while m_ref is still -inf
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? ex2(m_ref - m_new) : 1.f;      // 0 on the first tile
                if (grow) m_ref = m_new;
                l_run *= alpha;
                if (j > 0) {
                    // the accumulator must be quiescent: P_{j-1} V_{j-1} is the last product issued for this stream
                    if (!mbar_wait(&pv_done[s * 2 + ((j - 1) & 1)], (uint32_t)((j - 1) >> 1) & 1u, abort_flag, err, 206)) { ok = false; break; }
                    __syncwarp();
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < HD / 32; c++) {
                        uint32_t acc[32];
                        tmem_ld32_issue(o_tmem + (uint32_t)(c * 32), acc);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) acc[i] = __float_as_uint(__uint_as_float(acc[i]) * alpha);
                        tmem_st32(o_tmem + (uint32_t)(c * 32), acc);
                    }
                    tmem_st_wait();
                }
            }
            // the P buffer of this parity was last read by P_{j-2} V_{j-2}
            if (j >= 2) {
                if (!mbar_wait(&pv_done[s * 2 + bsel], (uint32_t)((j - 2) >> 1) & 1u, abort_flag, err, 207)) { ok = false; break; }
            }
            // probabilities against the reference, row sum, bf16 P into the K-major 128-byte-swizzled operand layout
            uint8_t* p_row = smem + OFF_P + (s * 2 + bsel) * P_BYTES + r * 128;
            // (Packed ex2.approx.bf16x2 was measured slower than the float32 instruction here, and a P operand in f16
            // against V in bf16 is rejected by tcgen05.mma as an illegal instruction: A and B share one 16-bit format.)
            float lp[8];
#pragma unroll
            for (int g = 0; g < 8; g++) {
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; i++) pv[i] = ex2(fmaf(__uint_as_float(sc[g * 8 + i]), scale_log2, -m_ref));
                lp[g] = ((pv[0] + pv[1]) + (pv[2] + pv[3])) + ((pv[4] + pv[5]) + (pv[6] + pv[7]));
                uint4 pk;
                pk.x = pack_bf16_rn(pv[0], pv[1]);
                pk.y = pack_bf16_rn(pv[2], pv[3]);
                pk.z = pack_bf16_rn(pv[4], pv[5]);
                pk.w = pack_bf16_rn(pv[6], pv[7]);
                // keys 8g .. 8g+7: 16-byte unit g of the row, XOR-swizzled by the row
                *reinterpret_cast<uint4*>(p_row + ((g ^ (r & 7)) << 4)) = pk;
            }
            l_run += ((lp[0] + lp[1]) + (lp[2] + lp[3])) + ((lp[4] + lp[5]) + (lp[6] + lp[7]));
            // make P visible to the tensor core (async proxy), order the TMEM accesses, then hand over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[s * 2 + bsel]);
        }
        if (ok && nt > 0) {
            // the accumulator after the last product
            if (mbar_wait(&pv_done[s * 2 + ((nt - 1) & 1)], (uint32_t)((nt - 1) >> 1) & 1u, abort_flag, err, 208)) {
                __syncwarp();
                tc_fence_after();
                const float inv = 1.f / l_run;
                __nv_bfloat16* dst = out + ((long long)(row0 + q_row)) * d + h * HD;
#pragma unroll
                for (int c = 0; c < HD / 32; c++) {
                    uint32_t acc[32];
                    tmem_ld32_issue(o_tmem + (uint32_t)(c * 32), acc);
                    tmem_ld_wait();
                    if (q_row < T) {
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            uint4 pk;
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(acc[u * 8 + 0]) * inv, __uint_as_float(acc[u * 8 + 1]) * inv);
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(acc[u * 8 + 2]) * inv, __uint_as_float(acc[u * 8 + 3]) * inv);
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(acc[u * 8 + 4]) * inv, __uint_as_float(acc[u * 8 + 5]) * inv);
                            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(acc[u * 8 + 6]) * inv, __uint_as_float(acc[u * 8 + 7]) * inv);
                            pk.x = *reinterpret_cast<uint32_t*>(&h0);
                            pk.y = *reinterpret_cast<uint32_t*>(&h1);
                            pk.z = *reinterpret_cast<uint32_t*>(&h2);
                            pk.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(dst + c * 32 + u * 8) = pk;
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

// qkv: packed (B*T, 3d) bf16 projection; out: (B*T, d) bf16.  Head dimension 64 only.
int tl_attention_tcgen05(tlnn_ctx* ctx, const __nv_bfloat16* qkv, __nv_bfloat16* out, int B, int T, int heads, int causal) {
    const int d = heads * HD;
    const long long rows = (long long)B * T;
    TL_REQUIRE(rows < (1ll << 31), "attention: too many rows");
    TL_REQUIRE(((uintptr_t)qkv & 15u) == 0 && ((uintptr_t)out & 15u) == 0, "attention: buffers must be 16-byte aligned");
    CUtensorMap tq, tkv;
    TL_TRY(make_tile_map(&tq, true, qkv, rows, 3ll * d, 3ll * d, BQ));
    TL_TRY(make_tile_map(&tkv, true, qkv, rows, 3ll * d, 3ll * d, BK));
    dim3 grid((T + 2 * BQ - 1) / (2 * BQ), B * heads);
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
    if (causal) {
        auto k = attention_tcgen05_kernel<true>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM));
        TL_LAUNCH(ctx, "attention_tc_causal", k<<<grid, AT_THREADS, AT_SMEM, ctx->stream>>>(tq, tkv, out, T, heads, scale_log2, ctx->d_err));
    } else {
        auto k = attention_tcgen05_kernel<false>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM));
        TL_LAUNCH(ctx, "attention_tc_full", k<<<grid, AT_THREADS, AT_SMEM, ctx->stream>>>(tq, tkv, out, T, heads, scale_log2, ctx->d_err));
    }
    return TLNN_OK;
}
