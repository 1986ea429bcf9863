// Fused attention on the sm_100a tensor cores (bf16, head dimension 64).
//
// One CTA owns 256 consecutive queries of one (batch, head) as two independent 128-row streams.  Roles by warp:
//   warps 0-3  softmax of stream 0 (thread = query row: the S tile is read from TMEM one row per thread, so the row
//              maximum and the row sum need no shuffles), warps 4-7 the same for stream 1;
//   warp 8     MMA issuer (one thread): S = Q K^T with tcgen05.mma (128 x 128 x 64) into TMEM, and O_j = P V
//              (128 x 64 x 128) with P taken from shared memory and V read as an MN-major operand;
//   warp 9     TMA producer: Q once, then K / V tiles of 128 keys through a three-stage ring.
// Per stream and key tile j the tensor core runs [P_{j-1} V_{j-1}, Q K_j^T] and then the stream's softmax warps turn
// S_j into P_j (bf16, written straight into the swizzled operand layout) while folding the partial product O_{j-1}
// into their float32 running output: O = (O + O_{j-1}) * 2^(m_{j-1} - m_j).  The two streams alternate on the tensor
// core, so one stream's exponentials overlap the other stream's MMAs.  The decoder mask is an index comparison.
// All mbarrier waits are bounded in time; on expiry the kernel records TLNN_ERR_TIMEOUT and every role leaves.
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int HD = 64;                 // head dimension
constexpr int BQ = 128;                // query rows per stream
constexpr int BK = 128;                // keys per tile
constexpr int KV_STAGES = 3;
constexpr int AT_THREADS = 320;
constexpr uint32_t Q_BYTES = BQ * HD * 2;          // 16 KB per stream
constexpr uint32_t K_BYTES = BK * HD * 2;          // 16 KB
constexpr uint32_t V_BYTES = BK * HD * 2;          // 16 KB
constexpr uint32_t P_BYTES = BQ * BK * 2;          // 32 KB per stream: two 64-key blocks of 128 rows x 128 bytes
constexpr uint32_t OFF_Q = 0;
constexpr uint32_t OFF_KV = OFF_Q + 2 * Q_BYTES;
constexpr uint32_t OFF_P = OFF_KV + KV_STAGES * (K_BYTES + V_BYTES);
constexpr uint32_t OFF_BAR = OFF_P + 2 * P_BYTES;
constexpr size_t AT_SMEM = OFF_BAR + 256 + 1024;   // barriers + alignment slack
constexpr uint32_t TMEM_COLS = 512;                // S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Instruction descriptors: D float32, A and B bf16, M = 128.  S: N = 128, both operands K-major.  PV: N = 64, A
// K-major (P), B MN-major (V rows are keys, the head dimension is contiguous).
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BK >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                              ((uint32_t)(BQ >> 4) << 24);

template <bool CAUSAL>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_qkv, __nv_bfloat16* __restrict__ out, int T, int H,
                         float scale_log2, tlnn_dev_err* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* kv_full = q_full + 1;                  // [KV_STAGES]
    uint64_t* kv_empty = kv_full + KV_STAGES;        // [KV_STAGES]
    uint64_t* mma_done = kv_empty + KV_STAGES;       // [2] per stream: S_j (and O_{j-1}) are in TMEM
    uint64_t* p_full = mma_done + 2;                 // [2] per stream: P_j is in shared memory, S_j and O_{j-1} consumed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_full + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = H * HD;
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int q_blk = CAUSAL ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;     // longest causal blocks first
    const int q0 = q_blk * 2 * BQ;
    const int row0 = b * T;                                // first row of this sequence in the packed (B*T, 3d) buffer
    const int tiles_all = (T + BK - 1) / BK;
    // key tiles each stream needs: causal rows q see keys <= q
    int n_tiles[2];
#pragma unroll
    for (int s = 0; s < 2; s++) {
        const int qs = q0 + s * BQ;
        n_tiles[s] = qs >= T ? 0 : (CAUSAL ? min(tiles_all, qs / BK + 1) : tiles_all);
    }
    const int n_max = max(n_tiles[0], n_tiles[1]);

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_qkv);
        mbar_init(q_full, 1);
        for (int i = 0; i < KV_STAGES; i++) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&mma_done[s], 1); mbar_init(&p_full[s], 4); }
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

    if (warp == 9) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, 2 * Q_BYTES);
            tma_load_2d(smem_u32(smem + OFF_Q), &tm_qkv, smem_u32(q_full), h * HD, row0 + q0);
            tma_load_2d(smem_u32(smem + OFF_Q + Q_BYTES), &tm_qkv, smem_u32(q_full), h * HD, row0 + q0 + BQ);
            int stage = 0;
            uint32_t phase = 0;
            for (int j = 0; j < n_max; j++) {
                if (!mbar_wait(&kv_empty[stage], phase ^ 1u, abort_flag, err, 201)) break;
                const uint32_t sk = smem_u32(smem + OFF_KV + stage * (K_BYTES + V_BYTES));
                const uint32_t bar = smem_u32(&kv_full[stage]);
                mbar_expect_tx(&kv_full[stage], K_BYTES + V_BYTES);
                tma_load_2d(sk, &tm_qkv, bar, d + h * HD, row0 + j * BK);
                tma_load_2d(sk + K_BYTES, &tm_qkv, bar, 2 * d + h * HD, row0 + j * BK);
                if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = mbar_wait(q_full, 0, abort_flag, err, 202);
            tc_fence_after();
            int stage = 0, prev_stage = 0;
            uint32_t phase = 0;
            // iteration j issues, per stream, P_{j-1} V_{j-1} (if any) and then Q K_j^T (if any)
            for (int j = 0; j <= n_max && ok; j++) {
                if (j < n_max) {
                    if (!mbar_wait(&kv_full[stage], phase, abort_flag, err, 203)) { ok = false; break; }
                    tc_fence_after();
                }
                const uint32_t sk = smem_u32(smem + OFF_KV + stage * (K_BYTES + V_BYTES));
                const uint32_t sv_prev = smem_u32(smem + OFF_KV + prev_stage * (K_BYTES + V_BYTES) + K_BYTES);
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    if (j > n_tiles[s] || n_tiles[s] == 0) continue;
                    if (j > 0) {
                        // P_{j-1} of this stream is complete (which also means S_{j-1} and O_{j-2} have been consumed)
                        if (!mbar_wait(&p_full[s], (uint32_t)(j - 1) & 1u, abort_flag, err, 204)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t sp = smem_u32(smem + OFF_P + s * P_BYTES);
                        const uint32_t o_tmem = tmem_base + 256u + (uint32_t)(s * HD);
#pragma unroll
                        for (int kk = 0; kk < BK / 16; kk++) {
                            // A: P rows x 16 keys inside 64-key block kk / 4; B: 16 key rows of V (2048 bytes per step)
                            const uint64_t a_desc = make_smem_desc(sp + (uint32_t)(kk >> 2) * (BQ * 128) + (uint32_t)(kk & 3) * 32);
                            const uint64_t b_desc = make_smem_desc(sv_prev + (uint32_t)kk * 2048);
                            umma<false>(o_tmem, a_desc, b_desc, IDESC_PV, kk != 0 ? 1u : 0u);
                        }
                    }
                    if (j < n_tiles[s]) {
                        const uint32_t sq = smem_u32(smem + OFF_Q + s * Q_BYTES);
                        const uint32_t s_tmem = tmem_base + (uint32_t)(s * BK);
#pragma unroll
                        for (int k = 0; k < HD / 16; k++) {
                            umma<false>(s_tmem, make_smem_desc(sq + k * 32), make_smem_desc(sk + k * 32), IDESC_S, k != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(&mma_done[s]);
                }
                if (!ok) break;
                if (j > 0) umma_commit(&kv_empty[prev_stage]);      // K_{j-1} and V_{j-1} are no longer needed
                prev_stage = stage;
                if (j < n_max) { if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; } }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps (two streams of four warps)
        const int s = warp >> 2;                          // stream
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31
        const int r = quarter * 32 + lane;                // row inside the stream's tile
        const int q_row = q0 + s * BQ + r;                // query index in the sequence
        const int nt = n_tiles[s];
        const uint32_t s_tmem = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(s * BK);
        const uint32_t o_tmem = tmem_base + ((uint32_t)(quarter * 32) << 16) + 256u + (uint32_t)(s * HD);
        uint8_t* p_row = smem + OFF_P + s * P_BYTES + r * 128;
        float o_acc[HD];
#pragma unroll
        for (int i = 0; i < HD; i++) o_acc[i] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < nt && ok; j++) {
            if (!mbar_wait(&mma_done[s], (uint32_t)j & 1u, abort_flag, err, 205)) { ok = false; break; }
            __syncwarp();
            tc_fence_after();
            const int k0 = j * BK;
            const bool need_mask = (k0 + BK > T) || (CAUSAL && k0 + BK - 1 > q0 + s * BQ + quarter * 32);
            // pass 1: row maximum
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < BK / 32; c++) {
                uint32_t acc[32];
                tmem_ld32_issue(s_tmem + (uint32_t)(c * 32), acc);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int key = k0 + c * 32 + i;
                        const bool dead = key >= T || (CAUSAL && key > q_row);
                        mx = dead ? mx : fmaxf(mx, __uint_as_float(acc[i]));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(acc[i]));
                }
            }
            const float m_new = fmaxf(m_run, mx * scale_log2);     // finite: every processed tile has a live key per row
            const float alpha = ex2(m_run - m_new);
            // fold the previous tile's partial product, then rescale to the new maximum
            if (j > 0) {
#pragma unroll
                for (int c = 0; c < HD / 32; c++) {
                    uint32_t acc[32];
                    tmem_ld32_issue(o_tmem + (uint32_t)(c * 32), acc);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) o_acc[c * 32 + i] = (o_acc[c * 32 + i] + __uint_as_float(acc[i])) * alpha;
                }
            }
            l_run *= alpha;
            m_run = m_new;
            // pass 2: probabilities, row sum, bf16 P into the K-major 128-byte-swizzled operand layout
            float l_add = 0.f;
#pragma unroll 1
            for (int c = 0; c < BK / 32; c++) {
                uint32_t acc[32];
                tmem_ld32_issue(s_tmem + (uint32_t)(c * 32), acc);
                tmem_ld_wait();
                float p[32];
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float e = ex2(fmaf(__uint_as_float(acc[i]), scale_log2, -m_new));
                    if (need_mask) {
                        const int key = k0 + c * 32 + i;
                        if (key >= T || (CAUSAL && key > q_row)) e = 0.f;
                    }
                    p[i] = e;
                    l_add += e;
                }
                // keys c*32 .. c*32+31 live in 64-key block c / 2, 16-byte units (c & 1) * 4 .. + 3 of this row
                uint8_t* blk = p_row + (c >> 1) * (BQ * 128);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(p[8 * u + 0], p[8 * u + 1]);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(p[8 * u + 2], p[8 * u + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(p[8 * u + 4], p[8 * u + 5]);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(p[8 * u + 6], p[8 * u + 7]);
                    pk.x = *reinterpret_cast<uint32_t*>(&h0);
                    pk.y = *reinterpret_cast<uint32_t*>(&h1);
                    pk.z = *reinterpret_cast<uint32_t*>(&h2);
                    pk.w = *reinterpret_cast<uint32_t*>(&h3);
                    const int unit = ((c & 1) * 4 + u) ^ (r & 7);
                    *reinterpret_cast<uint4*>(blk + unit * 16) = pk;
                }
            }
            l_run += l_add;
            // make P visible to the tensor core (async proxy), order the TMEM reads, then hand over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[s]);
        }
        if (ok && nt > 0) {
            // the last partial product
            if (mbar_wait(&mma_done[s], (uint32_t)nt & 1u, abort_flag, err, 206)) {
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
                            float v[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) v[i] = (o_acc[c * 32 + u * 8 + i] + __uint_as_float(acc[u * 8 + i])) * inv;
                            uint4 pk;
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
                            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
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
    CUtensorMap tm;
    TL_TRY(make_tile_map(&tm, true, qkv, rows, 3ll * d, 3ll * d, BQ));
    dim3 grid((T + 2 * BQ - 1) / (2 * BQ), B * heads);
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
    if (causal) {
        auto k = attention_tcgen05_kernel<true>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM));
        TL_LAUNCH(ctx, "attention_tc_causal", k<<<grid, AT_THREADS, AT_SMEM, ctx->stream>>>(tm, out, T, heads, scale_log2, ctx->d_err));
    } else {
        auto k = attention_tcgen05_kernel<false>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM));
        TL_LAUNCH(ctx, "attention_tc_full", k<<<grid, AT_THREADS, AT_SMEM, ctx->stream>>>(tm, out, T, heads, scale_log2, ctx->d_err));
    }
    return TLNN_OK;
}
