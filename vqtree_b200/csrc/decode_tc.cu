// Decode (seqlen_q == 1) with the two contractions on the tensor cores, keys on the M axis.
//
// The decode step is a bandwidth-bound stream over the window rows (k, v) and the far rows
// (codebook, value sums, counts) of every (batch, kv head).  Here the arithmetic is taken off the
// SIMT pipes: for a tile of 128 rows
//   S^T [128 rows x 16]  = Ktile [128 x D] . Q^T        (tcgen05.mma, M = 128 rows, N = 16 query heads)
//   O^T [D x 16]        += Vtile^T [D x 128] . P        (tcgen05.mma, M = D, N = 16; P = exp2(S - m) in bf16)
// so a thread owns ONE row (its score sits in its own TMEM lane), and all the query heads of a kv
// head (up to 16) share one pass over the rows.  Roles in a CTA (one per SM):
//   warp 5  (one lane) producer: TMA tile loads (128-byte swizzle) of the key-like tile and the value
//           tile into a 3-stage ring, the counts of a far tile, and the query rows of a new unit;
//   warp 4  (one lane) issues the MMAs: scores of tile t+1 before the product of tile t;
//   warps 0-3 softmax: thread i reads the scores of row i, masks, exponentiates against a reference
//           maximum kept per head (raised, with O rescaled, only when a score exceeds it by 2^8 -
//           an OR over the four warps tells), adds to its partial denominators and writes P for the product;
//           at the end of a unit it hands the denominators to the write-out warps and goes on with the next
//           unit, which accumulates in the other of two O^T buffers;
//   warps 6-9 write-out: thread d reads column d of a finished unit's O^T buffer once the unit's last product
//           has completed, releases the buffer, and normalises and stores the output row - or, for a unit
//           shared with other CTAs, publishes this CTA's partial and merges the unit if it is the last contributor.
// The global list of tiles is split evenly over the CTAs (a range may start or end inside a unit);
// a CTA writes one partial (numerator, maximum, denominator) per unit it touched and the last CTA
// of a unit (atomic ticket) merges them - the same workspace protocol as the SIMT bulk kernel.
// Every wait is bounded; a failed wait raises the status word and the CTA leaves; TMEM is freed.
#include "decode_common.cuh"
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr int kDtRows = 128;       // rows per tile
constexpr int kDtStages = 3;
constexpr int kDtN = 16;           // query heads per MMA (columns of S^T and O^T)
constexpr int kDtThreads = 320;    // 4 softmax warps + MMA warp + TMA warp + 4 write-out warps
constexpr int kDtD = 128;
constexpr int kDtTile = kDtRows * kDtD * 2;             // 32 KB
constexpr int kDtStageBytes = 2 * kDtTile;              // key-like tile, value tile
constexpr int kDtQBytes = kDtN * kDtD * 2;              // 4 KB: 16 query rows
constexpr int kDtOffQ = kDtStages * kDtStageBytes;      // 2 slots x (q1, q2)
constexpr int kDtOffP = kDtOffQ + 2 * 2 * kDtQBytes;    // 2 x P [16 x 128 rows] bf16
constexpr int kDtOffCnt = kDtOffP + 2 * kDtQBytes;      // 3 x 128 counts
constexpr int kDtSmem = kDtOffCnt + kDtStages * kDtRows * 4 + 1024;
constexpr float kDtLazy = 8.f;
#ifndef VQ_DT_MIN_GROUP
#define VQ_DT_MIN_GROUP 1
#endif

struct DtParams {
    DecodeParams d;
    int tiles_wi;        // window items per unit (tiles, plus one when a tile straddles n_bd)
    int ts;              // the straddling tile or -1
    int tiles_f, TU, units, num_ctas;
    float *partial;      // [(num_ctas + units)][G][D+2]
    int *ticket;         // [units]
    int32_t *status;
    long long wait_limit;  // cycles a device-side wait may last before the kernel gives up
};

struct DtItem {
    int kind;            // 0: window rows scored q1.k1, 1: window rows scored q2.k3, 2: far rows (q2.codebook)
    int row0;            // first row of the tile in its source
    int lo, hi;          // valid rows of the tile: [lo, hi)
};

__device__ __forceinline__ DtItem dt_item(const DtParams &bp, int tt)
{
    const DecodeParams &p = bp.d;
    DtItem it;
    if (tt < bp.tiles_wi) {
        int t = tt;
        bool second = false;
        if (bp.ts >= 0 && tt > bp.ts) {
            t = tt - 1;
            second = tt == bp.ts + 1;
        }
        const int r0 = t * kDtRows, r1 = min(r0 + kDtRows, p.n_valid);
        it.row0 = r0;
        if (bp.ts >= 0 && t == bp.ts) {
            it.kind = second ? 0 : 1;
            it.lo = second ? p.n_bd - r0 : 0;
            it.hi = second ? r1 - r0 : p.n_bd - r0;
        } else {
            it.kind = r0 >= p.n_bd ? 0 : 1;
            it.lo = 0;
            it.hi = r1 - r0;
        }
    } else {
        it.kind = 2;
        it.row0 = (tt - bp.tiles_wi) * kDtRows;
        it.lo = 0;
        it.hi = kDtRows;
    }
    return it;
}

__device__ __forceinline__ void dt_bulk_copy(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__global__ void __launch_bounds__(kDtThreads, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k3,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_cb,
                 const __grid_constant__ CUtensorMap tm_vs, const __grid_constant__ CUtensorMap tm_q1,
                 const __grid_constant__ CUtensorMap tm_q2, DtParams bp)
{
    const DecodeParams &p = bp.d;
    constexpr int D = kDtD, NS = kDtStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full[NS], empty[NS], q_full[2], q_free[2], s_ready[2], p_ready[2], o_done[2];
    __shared__ __align__(8) uint64_t o_final[2], f_req[2], f_done[2];   // hand-offs with the write-out warps, one set per O^T buffer
    __shared__ float s_wlr[2][4][kDtN], s_mr[2][kDtN];                  // a finished unit's denominators (per softmax warp) and references
    __shared__ uint32_t s_tmem;
    __shared__ int s_err, s_last;
    __shared__ uint32_t s_flag[2][4];
    __shared__ float s_wm[4][kDtN];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.G, TU = bp.TU;
    const int64_t T = static_cast<int64_t>(bp.units) * TU;
    const int NC = bp.num_ctas, c = blockIdx.x;
    const int64_t g0 = static_cast<int64_t>(c) * T / NC, g1 = static_cast<int64_t>(c + 1) * T / NC;
    const int n_items = static_cast<int>(g1 - g0);
    // (unit, tile) of the first item; the roles step them item by item (no 64-bit divisions in the loops)
    const int ue0 = static_cast<int>(g0 / TU), tt0 = static_cast<int>(g0 % TU);

    // The producer lane initialises the barriers itself and starts the first tile loads at once; the
    // other roles see the barriers after the CTA-wide barrier below (TMEM is allocated meanwhile).
    if (tid == 5 * 32) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&q_free[i], 1);
            mbar_init(&s_ready[i], 1);
            mbar_init(&p_ready[i], 4);
            mbar_init(&o_done[i], 1);
            mbar_init(&o_final[i], 1);
            mbar_init(&f_req[i], 4);
            mbar_init(&f_done[i], 1);
        }
        fence_mbar_init();
        s_err = 0;
    }
    float *cnt_s = reinterpret_cast<float *>(smem + kDtOffCnt);
    // producer state (lane 0 of warp 5): position in the CTA's item list
    int pr_t = 0, pr_ue = ue0, pr_tt = tt0 - 1, pr_cur = -1, pr_seg = -1;
    bool pr_ok = true;
    auto produce = [&](int upto) {  // issue the loads of items [pr_t, upto)
        for (; pr_t < upto && pr_ok; ++pr_t) {
            const int t = pr_t, st = t % NS;
            if (++pr_tt == TU) {
                pr_tt = 0;
                ++pr_ue;
            }
            const int ue = pr_ue, tt = pr_tt;
            const int b = ue / p.Hkv, hk = ue % p.Hkv;
            if (t >= NS && !mbar_wait(&empty[st], ((t / NS) - 1) & 1, bp.wait_limit)) {
                pr_ok = false;
                break;
            }
            if (ue != pr_cur) {
                pr_cur = ue;
                ++pr_seg;
                const int slot = pr_seg & 1;
                if (pr_seg >= 2 && !mbar_wait(&q_free[slot], ((pr_seg >> 1) - 1) & 1, bp.wait_limit)) {
                    pr_ok = false;
                    break;
                }
                uint8_t *qd = smem + kDtOffQ + slot * 2 * kDtQBytes;
                mbar_expect_tx(&q_full[slot], 2 * kDtQBytes);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    tma_load_3d(qd + h * (kDtN * 128), &tm_q1, &q_full[slot], 64 * h, hk * G, b);
                    tma_load_3d(qd + kDtQBytes + h * (kDtN * 128), &tm_q2, &q_full[slot], 64 * h, hk * G, b);
                }
            }
            const DtItem it = dt_item(bp, tt);
            uint8_t *dst = smem + st * kDtStageBytes;
            mbar_expect_tx(&full[st], kDtStageBytes + (it.kind == 2 ? kDtRows * 4 : 0));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (it.kind == 2) {
                    tma_load_3d(dst + h * kHalfBytes, &tm_cb, &full[st], 64 * h, it.row0, hk);
                    tma_load_4d(dst + kDtTile + h * kHalfBytes, &tm_vs, &full[st], 64 * h, it.row0, hk, b);
                } else {
                    tma_load_4d(dst + h * kHalfBytes, it.kind == 0 ? &tm_k1 : &tm_k3, &full[st], 64 * h, it.row0, hk, b);
                    tma_load_4d(dst + kDtTile + h * kHalfBytes, &tm_v, &full[st], 64 * h, it.row0, hk, b);
                }
            }
            if (it.kind == 2)
                dt_bulk_copy(cnt_s + st * kDtRows, p.cnt + static_cast<int64_t>(ue) * p.MK + it.row0, kDtRows * 4, &full[st]);
        }
    };
    if (tid == 5 * 32) produce(min(n_items, NS));   // the ring is empty: no wait inside
    if (warp == 4) {
        __syncwarp();
        tmem_alloc(&s_tmem, 64);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;  // columns: S^T buffers at 0 and 16, O^T buffers at 32 and 48 (the unit segments alternate)

    if (warp == 5) {
        // ================================================================== producer (the first loads were issued above)
        if (lane == 0) {
            produce(n_items);
            if (!pr_ok) s_err = 1;
        }
    } else if (warp == 4) {
        // ================================================================== MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(128, kDtN, 0, 0);   // S^T = Ktile (K-major) . Q^T (K-major)
            constexpr uint32_t idesc_o = idesc_bf16(128, kDtN, 1, 0);   // O^T = Vtile^T (MN-major A) . P (K-major)
            const uint64_t d_ring = smem_desc_sw128(smem_u32(smem), 16, 1024);
            const uint64_t d_vring = smem_desc_sw128(smem_u32(smem + kDtTile), kHalfBytes, 1024);
            const uint64_t d_q = smem_desc_sw128(smem_u32(smem + kDtOffQ), 16, 1024);
            const uint64_t d_p = smem_desc_sw128(smem_u32(smem + kDtOffP), 16, 1024);
            bool ok = true;
            int seg = -1;                    // unit segment of the last issued score MMA
            int seg_p = -1;                  // unit segment of the last issued product: its parity selects the O^T buffer
            int tt_s = tt0 - 1, tt_p = tt0 - 1;  // tile inside its unit of the last score / product item
            auto scores = [&](int t) {
                if (!ok) return;
                const int st = t % NS, sb = t & 1;
                if (++tt_s == TU) tt_s = 0;
                const int tt = tt_s;
                if (t == 0 || tt == 0) {         // first item of a unit segment
                    ++seg;
                    if (!mbar_wait(&q_full[seg & 1], (seg >> 1) & 1, bp.wait_limit)) {
                        ok = false;
                        return;
                    }
                }
                if (!mbar_wait(&full[st], (t / NS) & 1, bp.wait_limit)) {
                    ok = false;
                    return;
                }
                tc_fence_after();
                const DtItem it = dt_item(bp, tt);
                const uint64_t da = d_ring + static_cast<uint64_t>((st * kDtStageBytes) >> 4);
                const uint64_t db = d_q + static_cast<uint64_t>(((seg & 1) * 2 * kDtQBytes + (it.kind == 0 ? 0 : kDtQBytes)) >> 4);
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)
                        mma_ss(tmem + 16 * sb, da + static_cast<uint64_t>((h * kHalfBytes + k4 * 32) >> 4),
                               db + static_cast<uint64_t>((h * (kDtN * 128) + k4 * 32) >> 4), idesc_s, (h | k4) ? 1u : 0u);
                tc_commit(&s_ready[sb]);
                // the query rows of a unit are free after its last score MMA in this CTA
                const bool last_of_seg = (t + 1 == n_items) || tt + 1 == TU;
                if (last_of_seg) tc_commit(&q_free[seg & 1]);
            };
            auto product = [&](int t) {
                if (!ok) return;
                const int st = t % NS, sb = t & 1;
                if (++tt_p == TU) tt_p = 0;
                const bool first_of_seg = (t == 0) || tt_p == 0;
                if (first_of_seg) {
                    ++seg_p;
                    // this segment's O^T buffer was used two segments ago: the write-out warps must have read it
                    if (seg_p >= 2 && !mbar_wait(&f_done[seg_p & 1], ((seg_p >> 1) - 1) & 1, bp.wait_limit)) {
                        ok = false;
                        return;
                    }
                }
                if (!mbar_wait(&p_ready[sb], (t >> 1) & 1, bp.wait_limit)) {
                    ok = false;
                    return;
                }
                tc_fence_after();
                const uint64_t da = d_vring + static_cast<uint64_t>((st * kDtStageBytes) >> 4);
                const uint64_t db = d_p + static_cast<uint64_t>((sb * kDtQBytes) >> 4);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // 16 rows per step: V rows advance 2048 B, P columns 32 B (second half of the rows: + 2048 B)
                    mma_ss(tmem + 32 + 16 * (seg_p & 1), da + static_cast<uint64_t>((kk * 2048) >> 4),
                           db + static_cast<uint64_t>(((kk >> 2) * (kDtN * 128) + (kk & 3) * 32) >> 4), idesc_o,
                           (!first_of_seg || kk) ? 1u : 0u);
                tc_commit(&empty[st]);
                tc_commit(&o_done[sb]);
                if (t + 1 == n_items || tt_p + 1 == TU) tc_commit(&o_final[seg_p & 1]);   // the segment's accumulator is complete
            };
            if (n_items > 0) scores(0);
            for (int t = 0; t < n_items; ++t) {
                if (t + 1 < n_items) scores(t + 1);
                product(t);
            }
            if (!ok) s_err = 1;
        }
    } else if (warp < 4) {
        // ================================================================== softmax (thread = row of a tile)
        constexpr unsigned kAll = 0xffffffffu;
        const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
        float m_ref[kDtN], l_part[kDtN];
#pragma unroll
        for (int g = 0; g < kDtN; ++g) {
            m_ref[g] = -INFINITY;
            l_part[g] = 0.f;
        }
        bool ok = true;
        int cur_ue = -1, obuf = 1;
        int req = 0;            // unit segments handed to the write-out warps so far
        uint32_t xph = 0;
        // Barrier of the 128 softmax threads (hardware barrier 1) that also ORs their failure flags: when a bounded wait
        // has expired in any of them, all four warps learn it at the same barrier and leave together - nobody is left
        // waiting at a barrier the others never reach.  (The waits that can fail are mbarrier waits on other roles; this
        // barrier itself only joins warps that are all on their way to it.)
        auto sync4 = [&]() {
            uint32_t failed;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.or.pred p, 1, 128, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(failed)
                : "r"(ok ? 0u : 1u)
                : "memory");
            ++xph;
            if (failed) ok = false;
            return failed == 0;
        };

        int ue = ue0, tt = tt0 - 1;
        for (int t = 0; t < n_items; ++t) {
            const int st = t % NS, sb = t & 1;
            if (++tt == TU) {
                tt = 0;
                ++ue;
            }
            const bool first_of_seg = ue != cur_ue;
            if (first_of_seg) {
                cur_ue = ue;
                obuf ^= 1;      // the unit segments alternate between the two O^T buffers
#pragma unroll
                for (int gg = 0; gg < kDtN; ++gg) {
                    m_ref[gg] = -INFINITY;
                    l_part[gg] = 0.f;
                }
            }
            const DtItem it = dt_item(bp, tt);
            // the counts of a far tile arrive with the tile; the scores once the MMAs have finished
            // a wait that expires marks this warp as failed; the four warps find out together at the next barrier
            if (!__all_sync(kAll, mbar_wait(&full[st], (t / NS) & 1, bp.wait_limit) && mbar_wait(&s_ready[sb], (t >> 1) & 1, bp.wait_limit)))
                ok = false;
            tc_fence_after();
            uint32_t sr[16];
            tmem_ld16(tmem + lane_off + 16 * sb, sr);
            tc_wait_ld();
            const float w = it.kind == 2 ? cnt_s[st * kDtRows + tid] : 1.f;
            const bool valid = tid >= it.lo && tid < it.hi && w > 0.f;
            float sc[kDtN];
            bool exceed = false;
#pragma unroll
            for (int gg = 0; gg < kDtN; ++gg) {
                sc[gg] = (valid && gg < G) ? __uint_as_float(sr[gg]) * p.scale_log2 : -INFINITY;
                exceed |= sc[gg] > m_ref[gg] + kDtLazy;   // also true for the first valid score (reference -inf)
            }
            {
                const unsigned bal = __ballot_sync(kAll, exceed);
                if (lane == 0) s_flag[xph & 1][warp] = bal;
            }
            const uint32_t fslot = xph & 1;
            if (!sync4()) break;
            if ((s_flag[fslot][0] | s_flag[fslot][1] | s_flag[fslot][2] | s_flag[fslot][3]) != 0) {
                // ---- raise the reference maxima (rare after the first tiles): tile maximum per head over the 128 rows
#pragma unroll
                for (int gg = 0; gg < kDtN; ++gg)
                    if (gg < G) {   // (G is the same in every thread: the shuffles stay warp-wide)
                        float v = sc[gg];
#pragma unroll
                        for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(kAll, v, off));
                        if (lane == 0) s_wm[warp][gg] = v;
                    }
                if (!sync4()) break;
                float alpha[kDtN];
                bool any_scale = false;
#pragma unroll
                for (int gg = 0; gg < kDtN; ++gg) {
                    alpha[gg] = 1.f;
                    if (gg < G) {
                        const float mt = fmaxf(fmaxf(s_wm[0][gg], s_wm[1][gg]), fmaxf(s_wm[2][gg], s_wm[3][gg]));
                        const float mn = fmaxf(m_ref[gg], mt);
                        alpha[gg] = (mn == m_ref[gg]) ? 1.f : ex2(m_ref[gg] - mn);   // reference -inf -> 0
                        any_scale |= alpha[gg] != 1.f;
                        l_part[gg] *= alpha[gg];
                        m_ref[gg] = mn;
                    }
                }
                if (!sync4()) break;  // s_wm may be rewritten
                if (any_scale && !first_of_seg) {
                    // O^T holds the products up to the previous tile: wait for the last one, then scale column g by alpha[g]
                    if (!__all_sync(kAll, mbar_wait(&o_done[(t - 1) & 1], ((t - 1) >> 1) & 1, bp.wait_limit))) ok = false;
                    tc_fence_after();
                    uint32_t o[16];
                    tmem_ld16(tmem + lane_off + 32 + 16 * obuf, o);
                    tc_wait_ld();
#pragma unroll
                    for (int gg = 0; gg < kDtN; ++gg) o[gg] = __float_as_uint(__uint_as_float(o[gg]) * alpha[gg]);
                    tmem_st16(tmem + lane_off + 32 + 16 * obuf, o);
                    tc_wait_st();
                }
            }
            // ---- P (bf16, row g of the B operand: 128-byte swizzled, rows 0-63 then 64-127) and the denominators
            uint8_t *pb = smem + kDtOffP + sb * kDtQBytes + (tid >> 6) * (kDtN * 128) + (tid & 7) * 2;
            const int chunk = (tid & 63) >> 3;
#pragma unroll
            for (int gg = 0; gg < kDtN; ++gg)
                if (gg < G) {
                    const float pv = sc[gg] == -INFINITY ? 0.f : ex2(sc[gg] - m_ref[gg]);
                    l_part[gg] = fmaf(pv, w, l_part[gg]);
                    *reinterpret_cast<__nv_bfloat16 *>(pb + gg * 128 + ((chunk ^ (gg & 7)) << 4)) = __float2bfloat16_rn(pv);
                }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[sb]);
            if (t + 1 == n_items || tt + 1 == TU) {
                // ---- the unit segment ends here: its denominators (summed over this warp's 32 rows) and references go to
                // the write-out warps, which wait for the segment's last product themselves; nothing here waits for them
                // except for the slot of the segment before last to be free again
                const int slot = req & 1;
                if (req >= 2 && !__all_sync(kAll, mbar_wait(&f_done[slot], ((req >> 1) - 1) & 1, bp.wait_limit))) ok = false;
#pragma unroll
                for (int gg = 0; gg < kDtN; ++gg)
                    if (gg < G) {
                        float v = l_part[gg];
#pragma unroll
                        for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(kAll, v, off);
                        if (lane == 0) {
                            s_wlr[slot][warp][gg] = v;
                            if (warp == 0) s_mr[slot][gg] = m_ref[gg];
                        }
                    }
                __syncwarp();
                if (lane == 0) mbar_arrive(&f_req[slot]);
                ++req;
            }
        }
        if (!ok) s_err = 1;
    } else if (warp >= 6) {
        // ================================================================== write-out (thread = column d of O^T)
        // Warps 6-9 take a finished unit segment off the softmax warps: they read its O^T buffer once the segment's
        // last product has finished, release the buffer, and then normalise and write the output row (a unit this CTA
        // processed alone) or publish this CTA's partial and, as the last contributor, merge the unit.
        constexpr unsigned kAll = 0xffffffffu;
        const int q = warp & 3;                              // the TMEM lane quarter this warp may read
        const int dcol = q * 32 + lane;                      // column of O^T = element d of the output rows
        const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
        const bool lead = warp == 6 && lane == 0;
        bool ok = true;
        auto syncf = [&]() {                                 // hardware barrier 2: the 128 write-out threads, failure flags ORed
            uint32_t failed;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.or.pred p, 2, 128, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(failed)
                : "r"(ok ? 0u : 1u)
                : "memory");
            if (failed) ok = false;
            return failed == 0;
        };
        const int nseg = n_items > 0 ? static_cast<int>((g1 - 1) / TU) - ue0 + 1 : 0;
#pragma unroll 1
        for (int r = 0; r < nseg; ++r) {
            const int slot = r & 1, ue = ue0 + r;
            const uint32_t par = static_cast<uint32_t>(r >> 1) & 1u;
            if (!__all_sync(kAll, mbar_wait(&f_req[slot], par, bp.wait_limit) && mbar_wait(&o_final[slot], par, bp.wait_limit))) ok = false;
            tc_fence_after();
            uint32_t o[16];
            tmem_ld16(tmem + lane_off + 32 + 16 * slot, o);
            tc_wait_ld();
            float den[kDtN], mr[kDtN];
#pragma unroll
            for (int g = 0; g < kDtN; ++g) {
                den[g] = g < G ? (s_wlr[slot][0][g] + s_wlr[slot][1][g]) + (s_wlr[slot][2][g] + s_wlr[slot][3][g]) : 1.f;
                mr[g] = g < G ? s_mr[slot][g] : 0.f;
            }
            tc_fence_before();
            if (!syncf()) break;
            if (lead) mbar_arrive(&f_done[slot]);            // buffer and sums have been read by all 128 threads
            if (static_cast<int64_t>(ue) * TU >= g0 && static_cast<int64_t>(ue + 1) * TU <= g1) {
                // the whole unit was processed by this CTA: normalise and write the output row directly
                const int b = ue / p.Hkv, hk = ue % p.Hkv;
#pragma unroll
                for (int g = 0; g < kDtN; ++g)
                    if (g < G)
                        static_cast<__nv_bfloat16 *>(p.out)[b * p.o_sb + (hk * G + g) * p.o_sh + dcol] =
                            __float2bfloat16_rn(__uint_as_float(o[g]) / den[g]);
                continue;
            }
            const int first_c = static_cast<int>(((static_cast<int64_t>(ue) * TU + 1) * NC - 1) / T);
            const int last_c = static_cast<int>(((static_cast<int64_t>(ue + 1) * TU) * NC - 1) / T);
            float *part = bp.partial + static_cast<int64_t>(c + ue) * G * (D + 2);
#pragma unroll
            for (int g = 0; g < kDtN; ++g)
                if (g < G) {
                    part[g * (D + 2) + dcol] = __uint_as_float(o[g]);
                    if (dcol == 0) {
                        part[g * (D + 2) + D] = mr[g];
                        part[g * (D + 2) + D + 1] = den[g];
                    }
                }
            // Publication: the barrier orders the 128 threads' partial stores before the lead thread's ticket increment,
            // whose release makes them visible device-wide together with it; the last contributor's acquire (the same
            // instruction) and the barrier after it order every thread's loads behind the other CTAs' partials.
            if (!syncf()) break;
            if (lead) {
                int tk;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(tk) : "l"(bp.ticket + ue) : "memory");
                s_last = (tk == last_c - first_c);
            }
            if (!syncf()) break;
            const bool last = s_last != 0;
            if (!syncf()) break;                             // s_last may be rewritten for the next segment
            if (last) {
                // merge of the contributors' partials, four heads at a time: one pass over the contributors with a
                // running maximum (all loads of a contributor are independent and in flight together)
                const int b = ue / p.Hkv, hk = ue % p.Hkv;
#pragma unroll 1
                for (int gq = 0; gq < G; gq += 4) {
                    float M[4], num[4], dd4[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        M[i] = -INFINITY;
                        num[i] = 0.f;
                        dd4[i] = 0.f;
                    }
#pragma unroll 2
                    for (int cc = first_c; cc <= last_c; ++cc) {
                        const float *pc = bp.partial + (static_cast<int64_t>(cc + ue) * G + gq) * (D + 2);
                        float ms[4], x[4], dd[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const bool on = gq + i < G;
                            ms[i] = on ? __ldcg(pc + i * (D + 2) + D) : -INFINITY;
                            x[i] = on ? __ldcg(pc + i * (D + 2) + dcol) : 0.f;
                            dd[i] = on ? __ldcg(pc + i * (D + 2) + D + 1) : 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float mn = fmaxf(M[i], ms[i]);
                            const float a = (M[i] == -INFINITY) ? 0.f : exp2f(M[i] - mn);
                            const float w = (ms[i] == -INFINITY) ? 0.f : exp2f(ms[i] - mn);
                            num[i] = fmaf(num[i], a, w * x[i]);
                            dd4[i] = fmaf(dd4[i], a, w * dd[i]);
                            M[i] = mn;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (gq + i < G)
                            static_cast<__nv_bfloat16 *>(p.out)[b * p.o_sb + (hk * G + gq + i) * p.o_sh + dcol] =
                                __float2bfloat16_rn(num[i] / dd4[i]);
                }
                if (lead) bp.ticket[ue] = 0;  // ready for the next call on this stream
            }
        }
        if (!ok) s_err = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (s_err && tid == 0) {
        if (bp.status) atomicExch(bp.status, VQ_WORD_TIMEOUT);
        // a bounded wait expired: give tile loads still in flight time to land before leaving
#pragma unroll 1
        for (int w = 0; w < (1 << 14); ++w) __nanosleep(256);
    }
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tmem_dealloc(tmem, 64);
    }
}

// ------------------------------------------------------------------------------------------ host side

// SM count of the current device; the answer is kept per device ordinal (this runs once per generated token)
static int dt_sm_count()
{
    static int cached[64] = {0};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

// bf16, D = 128, dense rows, 1 to 16 query heads per kv head, bf16 codebook, M*K a multiple of 128.
bool decode_tc_eligible(const VqDecodeArgs *a)
{
    const bool far = a->use_far != 0;
    const int64_t D = a->q1.shape[2], Hq = a->q1.shape[1], Hkv = a->k1_win.shape[1];
    if (a->q1.dtype != VQ_BF16 || D != kDtD || Hq / Hkv > kDtN || Hq / Hkv < VQ_DT_MIN_GROUP) return false;
    if (far && (a->codebook.dtype != VQ_BF16 || a->codebook.shape[1] % kDtRows != 0)) return false;
    const VqTensorDesc *w[] = {&a->k1_win, &a->k3_win, &a->v_win};
    for (auto t : w)
        if (t->stride[2] != D || t->stride[1] % 8 || t->stride[0] % 8) return false;
    if (a->q1.stride[1] != D || a->q2.stride[1] != D || a->q1.stride[0] % 8 || a->q2.stride[0] % 8) return false;
    if (reinterpret_cast<uintptr_t>(a->q1.ptr) % 16 || reinterpret_cast<uintptr_t>(a->q2.ptr) % 16) return false;
    if (far && reinterpret_cast<uintptr_t>(a->cnt.ptr) % 16) return false;
    return true;
}

size_t decode_tc_workspace_bytes(int64_t units, int64_t G, int64_t D, int num_ctas)
{
    const size_t tickets = (static_cast<size_t>(units) * sizeof(int) + 255) / 256 * 256;
    return tickets + (static_cast<size_t>(num_ctas) + units) * G * (D + 2) * sizeof(float);
}

// Returns VQ_EWORKSPACE when the caller's workspace is too small for this kernel (the caller then
// takes the SIMT kernel, whose need vqattn_decode_workspace_bytes reports).
int launch_decode_tc(const VqDecodeArgs *a, const DecodeParams &p, cudaStream_t s)
{
    const int64_t B = a->q1.shape[0], Hq = a->q1.shape[1], Hkv = a->k1_win.shape[1];
    DtParams bp{};
    bp.d = p;
    const int tiles_w = (p.n_valid + kDtRows - 1) / kDtRows;
    bp.ts = (p.n_bd % kDtRows != 0 && p.n_bd < p.n_valid) ? p.n_bd / kDtRows : -1;
    bp.tiles_wi = tiles_w + (bp.ts >= 0 ? 1 : 0);
    bp.tiles_f = p.use_far ? p.MK / kDtRows : 0;
    bp.TU = bp.tiles_wi + bp.tiles_f;
    bp.units = static_cast<int>(B * Hkv);
    const int64_t T = static_cast<int64_t>(bp.units) * bp.TU;
    int64_t nc = dt_sm_count();
    if (nc > T) nc = T;
    bp.num_ctas = static_cast<int>(nc);
    if (a->workspace_bytes < decode_tc_workspace_bytes(bp.units, p.G, kDtD, bp.num_ctas)) return VQ_EWORKSPACE;
    const size_t tickets = (static_cast<size_t>(bp.units) * sizeof(int) + 255) / 256 * 256;
    bp.ticket = static_cast<int *>(a->workspace);
    bp.partial = reinterpret_cast<float *>(static_cast<char *>(a->workspace) + tickets);
    bp.status = a->status_word;
    bp.wait_limit = wait_limit_cycles();

    CUtensorMap mk1, mk3, mv, mcb, mvs, mq1, mq2;
    auto win_map = [&](CUtensorMap *m, const VqTensorDesc &t) {
        const uint64_t dims[4] = {static_cast<uint64_t>(kDtD), static_cast<uint64_t>(p.n_valid > 0 ? p.n_valid : 1),
                                  static_cast<uint64_t>(Hkv), static_cast<uint64_t>(B)};
        const uint64_t str[4] = {1, static_cast<uint64_t>(t.stride[2]), static_cast<uint64_t>(t.stride[1]), static_cast<uint64_t>(t.stride[0])};
        return make_map(m, t.ptr, 4, dims, str);
    };
    auto q_map = [&](CUtensorMap *m, const VqTensorDesc &t) {
        const uint64_t dims[3] = {static_cast<uint64_t>(kDtD), static_cast<uint64_t>(Hq), static_cast<uint64_t>(B)};
        const uint64_t str[3] = {1, static_cast<uint64_t>(t.stride[1]), static_cast<uint64_t>(t.stride[0])};
        return make_map(m, t.ptr, 3, dims, str, kDtN);
    };
    if (!win_map(&mk1, a->k1_win) || !win_map(&mk3, a->k3_win) || !win_map(&mv, a->v_win) || !q_map(&mq1, a->q1) || !q_map(&mq2, a->q2))
        return VQ_ELAUNCH;
    if (p.use_far) {
        const uint64_t cd[3] = {static_cast<uint64_t>(kDtD), static_cast<uint64_t>(p.MK), static_cast<uint64_t>(Hkv)};
        const uint64_t cs[3] = {1, static_cast<uint64_t>(kDtD), static_cast<uint64_t>(p.MK) * kDtD};
        const uint64_t vd[4] = {static_cast<uint64_t>(kDtD), static_cast<uint64_t>(p.MK), static_cast<uint64_t>(Hkv), static_cast<uint64_t>(B)};
        const uint64_t vs[4] = {1, static_cast<uint64_t>(kDtD), static_cast<uint64_t>(p.MK) * kDtD, static_cast<uint64_t>(p.MK) * kDtD * Hkv};
        if (!make_map(&mcb, a->codebook.ptr, 3, cd, cs) || !make_map(&mvs, a->vsum.ptr, 4, vd, vs)) return VQ_ELAUNCH;
    } else {
        mcb = mv;
        mvs = mv;
    }
    {
        // the shared-memory opt-in is a per-device attribute of the kernel: set once per device
        static bool opted[64] = {false};
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess) return VQ_EDEVICE;
        if (dev < 0 || dev >= 64 || !opted[dev]) {
            if (cudaFuncSetAttribute(decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDtSmem) != cudaSuccess) return VQ_ELAUNCH;
            if (dev >= 0 && dev < 64) opted[dev] = true;
        }
    }
    decode_tc_kernel<<<bp.num_ctas, kDtThreads, kDtSmem, s>>>(mk1, mk3, mv, mcb, mvs, mq1, mq2, bp);
    return launch_status();
}

}  // namespace vq
