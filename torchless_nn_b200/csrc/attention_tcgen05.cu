// Fused attention on the sm_100a tensor cores (bf16, head dimension 64).
//
// Work item: 128 consecutive queries of one (batch, head).  A CTA is persistent and runs three independent streams;
// each stream takes the next item from a global counter, so an SM always has three items in different phases in
// flight and the items balance dynamically.  Items are ordered in groups of 32 (batch, head) pairs, longest causal
// blocks first inside a group, which keeps the keys and values of the group in L2 while its query blocks are spread
// over the SMs.  Roles by warp:
//   warps 0-11   softmax, four warps per stream (thread = query row: a score row is read from TMEM by one thread, so
//                the row maximum and the row sum need no shuffles);
//   warps 12-14  MMA issuers, one thread per stream: S_j = Q K_j^T (128 x 64 x 64) into the stream's score buffer in
//                TMEM as soon as S_{j-1} has been read into registers, and O += P_j V_j (128 x 64 x 64) with P taken
//                from TMEM (A operand) and V from shared memory as an MN-major operand;
//   warps 16-18  TMA producers, one thread per stream: fetch the item, load Q, then K / V tiles of 64 keys through a
//                three-stage ring (warps 15 and 19 only complete the warpgroups that hand their registers over).
// Probabilities go from registers straight back to TMEM as packed bf16 (tcgen05.st), so neither the P tile nor its
// re-read by the tensor core touches shared memory: shared-memory bandwidth is what a 64-wide MMA is bound by.
// Three softmax warps per scheduler because one warp alone cannot issue fast enough to keep the special-function
// unit busy and two in lock-step leave it idle half of the time (measured: 1500 cycles per 64-key tile for a lone
// warp, of which 800 in the exponent loop).  O accumulates in TMEM across tiles; probabilities are taken against a
// reference maximum that is moved (and O, l rescaled in TMEM) only when the true row maximum has grown by more than
// 2^8, which is exact after the final division by l.  The decoder mask is an index comparison.
// All waits are bounded in time; on expiry the kernel records TLNN_ERR_TIMEOUT and every role leaves.
#define TLNN_INLINE_WAITS 1
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int HD = 64;                 // head dimension
constexpr int BQ = 128;                // query rows per item
constexpr int BK = 64;                 // keys per tile
constexpr int NS = 3;                  // streams per CTA
constexpr int KV_STAGES = 3;           // per stream
constexpr int GROUP_BH = 32;           // (batch, head) pairs whose items are interleaved
constexpr int AT_THREADS = 640;
// Register hand-over (setmaxnreg): the softmax warpgroups grow, the service warpgroups shrink.  The CTA owns what it
// was launched with - 96 registers per thread at 640 threads - and setmaxnreg.inc waits, without a limit, until the
// CTA's pool covers the request: the totals after the hand-over must not exceed the launch allocation (checked
// against the compiled kernel's register count before every first launch).
constexpr int LAUNCH_REGS = 96;
constexpr int SOFTMAX_REGS = 128;
constexpr int SERVICE_REGS = 48;
constexpr int REGS_AFTER = SOFTMAX_REGS * 384 + SERVICE_REGS * 256;
static_assert(REGS_AFTER <= LAUNCH_REGS * 640, "register hand-over exceeds the launch allocation");
constexpr int ISSUER_WARP0 = 12, PRODUCER_WARP0 = 16;
constexpr uint32_t Q_BYTES = BQ * HD * 2;          // 16 KB
constexpr uint32_t K_BYTES = BK * HD * 2;          // 8 KB
constexpr uint32_t V_BYTES = BK * HD * 2;          // 8 KB
constexpr uint32_t STAGE_BYTES = K_BYTES + V_BYTES;
constexpr uint32_t STREAM_BYTES = Q_BYTES + KV_STAGES * STAGE_BYTES;       // 64 KB: Q, then the K / V ring
constexpr uint32_t OFF_BAR = NS * STREAM_BYTES;
constexpr size_t AT_SMEM = OFF_BAR + 1024 + 1024;  // barriers and item slots + alignment slack
constexpr uint32_t TMEM_COLS = 512;
// TMEM columns of stream s: scores S at 64 s, accumulator O at 192 + 64 s, probabilities P (bf16 pairs) at 384 + 32 s
__device__ __forceinline__ constexpr uint32_t s_col(int s) { return (uint32_t)(64 * s); }
__device__ __forceinline__ constexpr uint32_t o_col(int s) { return (uint32_t)(192 + 64 * s); }
__device__ __forceinline__ constexpr uint32_t p_col(int s) { return (uint32_t)(384 + 32 * s); }

// per-stream barriers
struct stream_bars {
    uint64_t q_full, q_empty, s_full, s_free, p_full, pv_done;
    uint64_t kv_full[KV_STAGES], kv_empty[KV_STAGES];
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// O += A B with A (the probabilities) in TMEM: 128 lanes x 8 columns of bf16 pairs per K = 16 step.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Store 16 registers per thread to 32 lanes x 16 columns of TMEM.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Instruction descriptors: D float32, A and B bf16, M = 128, N = 64.  S: both operands K-major.  PV: A K-major (P),
// B MN-major (V rows are keys, the head dimension is contiguous).
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BK >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                              ((uint32_t)(BQ >> 4) << 24);

// Item number -> (batch * heads + head, query block).  Groups of GROUP_BH pairs; inside a group the query blocks run
// from the last (most keys under the causal mask) to the first, the pairs of the group interleaved.
__device__ __forceinline__ void decode_item(int idx, int n_bh, int n_qb, int& bh, int& qb) {
    const int per_group = GROUP_BH * n_qb;
    const int full = n_bh / GROUP_BH;
    int grp = idx / per_group;
    int members = GROUP_BH;
    if (grp >= full) { grp = full; members = n_bh - full * GROUP_BH; }
    const int rem = idx - grp * per_group;
    const int lvl = rem / members;
    qb = n_qb - 1 - lvl;
    bh = grp * GROUP_BH + (rem - lvl * members);
}

template <bool CAUSAL>
__device__ __forceinline__ int item_tiles(int qb, int T) {
    const int tiles_all = (T + BK - 1) / BK;
    return CAUSAL ? min(tiles_all, (qb * BQ + BQ - 1) / BK + 1) : tiles_all;
}

template <bool CAUSAL>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                         __nv_bfloat16* __restrict__ out, int T, int H, int n_bh, float scale_log2,
                         int* __restrict__ next_item, tlnn_dev_err* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    stream_bars* bars = reinterpret_cast<stream_bars*>(smem + OFF_BAR);
    volatile int* item_slot = reinterpret_cast<volatile int*>(bars + NS);          // [NS][2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_cast<int*>(item_slot) + NS * 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = H * HD;
    const int n_qb = (T + BQ - 1) / BQ;
    const int total = n_bh * n_qb;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_kv);
        for (int s = 0; s < NS; s++) {
            mbar_init(&bars[s].q_full, 1);
            mbar_init(&bars[s].q_empty, 1);
            mbar_init(&bars[s].s_full, 1);
            mbar_init(&bars[s].s_free, 4);
            mbar_init(&bars[s].p_full, 4);
            mbar_init(&bars[s].pv_done, 1);
            for (int i = 0; i < KV_STAGES; i++) { mbar_init(&bars[s].kv_full[i], 1); mbar_init(&bars[s].kv_empty[i], 1); }
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == ISSUER_WARP0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= ISSUER_WARP0) {
      // two warpgroups that hand registers over to the softmax warpgroups
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(SERVICE_REGS));
      if (warp >= PRODUCER_WARP0 && warp < PRODUCER_WARP0 + NS) {
        // ------------------------------------------------------------------ TMA producer of stream s
        if (lane == 0) {
            const int s = warp - PRODUCER_WARP0;
            stream_bars& bar = bars[s];
            const uint32_t q_smem = smem_u32(smem + s * STREAM_BYTES);
            int stage = 0;
            uint32_t phase = 0;
            for (uint32_t it = 0;; it++) {
                const int idx = atomicAdd(next_item, 1);
                // the previous item's last S product has read Q: the Q buffer and the older item slot are free
                if (it > 0 && !mbar_wait(&bar.q_empty, (it - 1) & 1u, abort_flag, err, 200)) break;
                if (idx >= total) {
                    item_slot[s * 2 + (it & 1u)] = -1;
                    mbar_arrive(&bar.q_full);                  // release: the slot is visible to whoever sees the phase
                    break;
                }
                item_slot[s * 2 + (it & 1u)] = idx;
                int bh, qb;
                decode_item(idx, n_bh, n_qb, bh, qb);
                const int b = bh / H, h = bh - b * H;
                const int row0 = b * T;
                const int nt = item_tiles<CAUSAL>(qb, T);
                mbar_expect_tx(&bar.q_full, Q_BYTES);
                tma_load_2d(q_smem, &tm_q, smem_u32(&bar.q_full), h * HD, row0 + qb * BQ);
                bool ok = true;
                for (int t = 0; t < nt; t++) {
                    if (!mbar_wait(&bar.kv_empty[stage], phase ^ 1u, abort_flag, err, 201)) { ok = false; break; }
                    const uint32_t sk = q_smem + Q_BYTES + (uint32_t)stage * STAGE_BYTES;
                    const uint32_t fb = smem_u32(&bar.kv_full[stage]);
                    mbar_expect_tx(&bar.kv_full[stage], STAGE_BYTES);
                    tma_load_2d(sk, &tm_kv, fb, d + h * HD, row0 + t * BK);
                    tma_load_2d(sk + K_BYTES, &tm_kv, fb, 2 * d + h * HD, row0 + t * BK);
                    if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
            }
        }
      } else if (warp < ISSUER_WARP0 + NS) {
        // ------------------------------------------------------------------ MMA issuer of stream s
        // g counts the stream's tiles across items: tile g uses phase g & 1 of s_full / s_free / p_full / pv_done.
        if (lane == 0) {
            const int s = warp - ISSUER_WARP0;
            stream_bars& bar = bars[s];
            const uint64_t q_desc = make_smem_desc(smem_u32(smem + s * STREAM_BYTES));
            const uint64_t kv_desc0 = make_smem_desc(smem_u32(smem + s * STREAM_BYTES + Q_BYTES));
            constexpr uint64_t STAGE_UNITS = STAGE_BYTES >> 4, V_UNITS = K_BYTES >> 4;
            const uint32_t s_tmem = tmem_base + s_col(s), o_tmem = tmem_base + o_col(s), p_tmem = tmem_base + p_col(s);
            int ld_stage = 0;            // stage / phase of the next tile whose S will be issued
            uint32_t ld_phase = 0;
            int use_stage = 0;           // stage of the next tile whose V will be consumed
            uint32_t g = 0;
            bool ok = true;
            auto issue_s = [&]() -> bool {
                if (!mbar_wait(&bar.kv_full[ld_stage], ld_phase, abort_flag, err, 203)) return false;
                tc_fence_after();
                const uint64_t k_desc = kv_desc0 + (uint64_t)ld_stage * STAGE_UNITS;
#pragma unroll
                for (int k = 0; k < HD / 16; k++) umma<false>(s_tmem, q_desc + 2 * k, k_desc + 2 * k, IDESC_S, k != 0 ? 1u : 0u);
                umma_commit(&bar.s_full);
                if (++ld_stage == KV_STAGES) { ld_stage = 0; ld_phase ^= 1u; }
                return true;
            };
            for (uint32_t it = 0; ok; it++) {
                if (!mbar_wait(&bar.q_full, it & 1u, abort_flag, err, 202)) break;
                const int idx = item_slot[s * 2 + (it & 1u)];
                if (idx < 0) break;
                int bh, qb;
                decode_item(idx, n_bh, n_qb, bh, qb);
                const int nt = item_tiles<CAUSAL>(qb, T);
                // S_0 goes into the score buffer once the last scores of the previous item are in registers
                if (g > 0 && !mbar_wait(&bar.s_free, (g - 1) & 1u, abort_flag, err, 210)) break;
                tc_fence_after();
                if (!issue_s()) break;
                if (nt == 1) umma_commit(&bar.q_empty);
                for (int j = 0; j < nt; j++) {
                    const uint32_t par = (g + (uint32_t)j) & 1u;
                    if (j + 1 < nt) {
                        // S_{j+1} while the softmax warps work on S_j
                        if (!mbar_wait(&bar.s_free, par, abort_flag, err, 211)) { ok = false; break; }
                        tc_fence_after();
                        if (!issue_s()) { ok = false; break; }
                        if (j + 2 == nt) umma_commit(&bar.q_empty);
                    }
                    if (!mbar_wait(&bar.p_full, par, abort_flag, err, 204)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t v_desc = kv_desc0 + (uint64_t)use_stage * STAGE_UNITS + V_UNITS;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++)
                        umma_ts(o_tmem, p_tmem + (uint32_t)(8 * kk), v_desc + 128 * kk, IDESC_PV, (j > 0 || kk != 0) ? 1u : 0u);
                    umma_commit(&bar.pv_done);
                    umma_commit(&bar.kv_empty[use_stage]);
                    if (++use_stage == KV_STAGES) use_stage = 0;
                }
                g += (uint32_t)nt;
            }
        }
      }
    } else {
        // ------------------------------------------------------------------ softmax warps (four per stream)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
        const int s = warp >> 2;                          // stream
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31
        const int r = quarter * 32 + lane;                // row inside the item
        stream_bars& bar = bars[s];
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_tmem = tmem_base + lane_base + s_col(s);
        const uint32_t o_tmem = tmem_base + lane_base + o_col(s);
        const uint32_t p_tmem = tmem_base + lane_base + p_col(s);
        uint64_t scale2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(scale2) : "f"(scale_log2));
        uint32_t g = 0;
        bool ok = true;
        for (uint32_t it = 0; ok; it++) {
            if (!mbar_wait(&bar.q_full, it & 1u, abort_flag, err, 212)) break;
            const int idx = item_slot[s * 2 + (it & 1u)];
            if (idx < 0) break;
            int bh, qb;
            decode_item(idx, n_bh, n_qb, bh, qb);
            const int b = bh / H, h = bh - b * H;
            const int nt = item_tiles<CAUSAL>(qb, T);
            const int q_row = qb * BQ + r;                  // query index in the sequence
            const int warp_row_lo = qb * BQ + quarter * 32;
            // Running statistics.  m_ref is the reference maximum the probabilities and the TMEM accumulator are
            // currently expressed against (log2 units); it moves - and O and l are rescaled - only when the true row
            // maximum has grown by more than 2^8 since, so most tiles do not touch O.
            float m_ref = -INFINITY, l_run = 0.f;
            for (int j = 0; j < nt; j++) {
                const uint32_t par = (g + (uint32_t)j) & 1u;
                if (!mbar_wait(&bar.s_full, par, abort_flag, err, 205)) { ok = false; break; }
                __syncwarp();
                tc_fence_after();
                const int k0 = j * BK;
                if (CAUSAL && k0 > warp_row_lo + 31) {
                    // every key of this tile lies beyond every row of this warp (upper half of the block's last tile):
                    // the probabilities are zero, nothing else changes
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar.s_free);
                    if (j > 0) {
                        if (!mbar_wait(&bar.pv_done, par ^ 1u, abort_flag, err, 207)) { ok = false; break; }
                        __syncwarp();
                        tc_fence_after();
                    }
                    uint32_t zero[BK / 4];
#pragma unroll
                    for (int i = 0; i < BK / 4; i++) zero[i] = 0u;
                    tmem_st16(p_tmem, zero);
                    tmem_st16(p_tmem + (uint32_t)(BK / 4), zero);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar.p_full);
                    continue;
                }
                uint32_t sc[BK];
                tmem_ld32_issue(s_tmem, *reinterpret_cast<uint32_t(*)[32]>(&sc[0]));
                tmem_ld32_issue(s_tmem + 32u, *reinterpret_cast<uint32_t(*)[32]>(&sc[32]));
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar.s_free);
                if ((k0 + BK > T) || (CAUSAL && k0 + BK - 1 > warp_row_lo)) {
#pragma unroll
                    for (int i = 0; i < BK; i++) {
                        const int key = k0 + i;
                        if (key >= T || (CAUSAL && key > q_row)) sc[i] = 0xff800000u;      // -inf
                    }
                }
                // eight independent partial maxima (three-input maximum: two new scores per instruction), then a tree
                float mp[8];
#pragma unroll
                for (int i = 0; i < 8; i++) mp[i] = __uint_as_float(sc[i]);
#pragma unroll
                for (int p = 0; p < (BK - 8) / 2; p++)
                    asm("max.f32 %0, %0, %1, %2;" : "+f"(mp[p & 7]) : "f"(__uint_as_float(sc[8 + 2 * p])), "f"(__uint_as_float(sc[9 + 2 * p])));
                const float mx = fmaxf(fmaxf(fmaxf(mp[0], mp[1]), fmaxf(mp[2], mp[3])), fmaxf(fmaxf(mp[4], mp[5]), fmaxf(mp[6], mp[7])));
                // tile 0 holds key 0, visible to every row, so m_ref is finite from the first tile on; a later tile
                // whose keys are all masked for this row leaves it unchanged
                const float m_new = fmaxf(m_ref, mx * scale_log2);
                const bool grow = m_new - m_ref > 8.f;                       // also true while m_ref is still -inf
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = grow ? ex2(m_ref - m_new) : 1.f;      // 0 on the first tile
                    if (grow) m_ref = m_new;
                    l_run *= alpha;
                    if (j > 0) {
                        // the accumulator must be quiescent: P_{j-1} V_{j-1} is the last product issued for this stream
                        if (!mbar_wait(&bar.pv_done, par ^ 1u, abort_flag, err, 206)) { ok = false; break; }
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
                // Probabilities against the reference, row sum, packed bf16 pairs.  Packed float32 pairs (fma.f32x2 /
                // add.f32x2) halve the instructions of the scaling and of the row sum and one cvt packs two
                // probabilities: the loop is bound by instruction issue as much as by the special-function unit.
                // (Packed ex2.approx.bf16x2 was measured slower than the float32 instruction here, and a P operand in
                // f16 against V in bf16 is rejected by tcgen05.mma as an illegal instruction: A and B share one format.)
                uint64_t negm2, ls[4];
                asm("mov.b64 %0, {%1, %1};" : "=l"(negm2) : "f"(-m_ref));
#pragma unroll
                for (int i = 0; i < 4; i++) ls[i] = 0ull;
                // The P columns were last read by P_{j-1} V_{j-1} (for j = 0 the previous item's epilogue waited).  P goes
                // to TMEM in two halves of 32 keys, so that the packed registers of the first half are free again
                // while the second half is computed.
                auto exp_half = [&](int h, uint32_t (&pk)[BK / 4]) {
#pragma unroll
                    for (int q = 0; q < BK / 4; q++) {
                        const int i = h * (BK / 4) + q;
                        uint64_t in, xs, pp;
                        float x0, x1;
                        asm("mov.b64 %0, {%1, %2};" : "=l"(in) : "r"(sc[2 * i]), "r"(sc[2 * i + 1]));
                        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(xs) : "l"(in), "l"(scale2), "l"(negm2));
                        asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(xs));
                        const float p0 = ex2(x0), p1 = ex2(x1);
                        asm("mov.b64 %0, {%1, %2};" : "=l"(pp) : "f"(p0), "f"(p1));
                        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(ls[i & 3]) : "l"(ls[i & 3]), "l"(pp));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk[q]) : "f"(p1), "f"(p0));      // key 2i in the low half
                    }
                };
                {
                    uint32_t pk[BK / 4];
                    exp_half(0, pk);
                    if (j > 0) {
                        if (!mbar_wait(&bar.pv_done, par ^ 1u, abort_flag, err, 207)) { ok = false; break; }
                        __syncwarp();
                        tc_fence_after();
                    }
                    tmem_st16(p_tmem, pk);
                }
                {
                    uint32_t pk[BK / 4];
                    exp_half(1, pk);
                    tmem_st16(p_tmem + (uint32_t)(BK / 4), pk);
                }
                {
                    float a0, a1, a2, a3, a4, a5, a6, a7;
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(ls[0]));
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(a2), "=f"(a3) : "l"(ls[1]));
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(a4), "=f"(a5) : "l"(ls[2]));
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(a6), "=f"(a7) : "l"(ls[3]));
                    l_run += ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar.p_full);
            }
            if (!ok) break;
            // the accumulator after the last product
            if (!mbar_wait(&bar.pv_done, (g + (uint32_t)nt - 1u) & 1u, abort_flag, err, 208)) break;
            __syncwarp();
            tc_fence_after();
            const float inv = 1.f / l_run;
            __nv_bfloat16* dst = out + ((long long)(b * T + q_row)) * d + h * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; c++) {
                uint32_t acc[32];
                tmem_ld32_issue(o_tmem + (uint32_t)(c * 32), acc);
                tmem_ld_wait();
                if (q_row < T && TL_DBG_IN_BOUNDS(err, (long long)(b * T + q_row) * d + h * HD + c * 32 + 32 <= (long long)n_bh / H * T * d, 920,
                                                  (long long)(b * T + q_row) * d + h * HD + c * 32)) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        uint4 pk4;
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk4.x) : "f"(__uint_as_float(acc[u * 8 + 1]) * inv), "f"(__uint_as_float(acc[u * 8 + 0]) * inv));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk4.y) : "f"(__uint_as_float(acc[u * 8 + 3]) * inv), "f"(__uint_as_float(acc[u * 8 + 2]) * inv));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk4.z) : "f"(__uint_as_float(acc[u * 8 + 5]) * inv), "f"(__uint_as_float(acc[u * 8 + 4]) * inv));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk4.w) : "f"(__uint_as_float(acc[u * 8 + 7]) * inv), "f"(__uint_as_float(acc[u * 8 + 6]) * inv));
                        *reinterpret_cast<uint4*>(dst + c * 32 + u * 8) = pk4;
                    }
                }
            }
            tc_fence_before();
            g += (uint32_t)nt;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == ISSUER_WARP0) {
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
    const long long items = (long long)B * heads * ((T + BQ - 1) / BQ);
    TL_REQUIRE(items < (1ll << 30), "attention: too many query blocks");
    CUtensorMap tq, tkv;
    TL_TRY(make_tile_map(&tq, true, qkv, rows, 3ll * d, 3ll * d, BQ));
    TL_TRY(make_tile_map(&tkv, true, qkv, rows, 3ll * d, 3ll * d, BK));
    const int grid = (int)std::min<long long>(ctx->sm_count, (items + NS - 1) / NS);
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
    TL_CUDA(cudaMemsetAsync(ctx->d_sched, 0, sizeof(int), ctx->stream));
    {
        // never launch a build whose register allocation cannot satisfy the hand-over (it would wait forever)
        static int regs_ok = -1;
        if (regs_ok < 0) {
            cudaFuncAttributes fa, fb;
            TL_CUDA(cudaFuncGetAttributes(&fa, attention_tcgen05_kernel<true>));
            TL_CUDA(cudaFuncGetAttributes(&fb, attention_tcgen05_kernel<false>));
            regs_ok = (fa.numRegs * AT_THREADS >= REGS_AFTER && fb.numRegs * AT_THREADS >= REGS_AFTER) ? 1 : 0;
        }
        TL_REQUIRE(regs_ok == 1, "attention: the kernel's launch register allocation does not cover its register hand-over");
    }
    if (causal) {
        auto k = attention_tcgen05_kernel<true>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM));
        TL_LAUNCH(ctx, "attention_tc_causal", k<<<grid, AT_THREADS, AT_SMEM, ctx->stream>>>(tq, tkv, out, T, heads, B * heads, scale_log2, ctx->d_sched, ctx->d_err));
    } else {
        auto k = attention_tcgen05_kernel<false>;
        TL_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM));
        TL_LAUNCH(ctx, "attention_tc_full", k<<<grid, AT_THREADS, AT_SMEM, ctx->stream>>>(tq, tkv, out, T, heads, B * heads, scale_log2, ctx->d_sched, ctx->d_err));
    }
    return TLNN_OK;
}
