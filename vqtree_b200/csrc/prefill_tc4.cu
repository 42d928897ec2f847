// Fused VQ-attention prefill on the sm_100a tensor cores: one softmax thread per query row, three
// softmax warpgroups that take the work items of a query tile in turn.
//
// One CTA owns one 128-row query tile of one (batch, query head) and walks its work items (far
// codebook tiles, boundary block, interior blocks, causal diagonal - see TcWork) with ONE online
// softmax (this replaces the reference's two kernels and their log-sum-exp merge,
// ops/triton_fused_vq_attn.py:202-250).  Tensor memory holds three S/P buffers (128 columns each)
// and the O accumulator.  Roles:
//   warps 0-11  softmax: warpgroup g = warp / 4 owns score buffer g and the items j = g, g+3, ...;
//               inside it one thread per query row reads the row's 128 scores, so the row maximum
//               and the row sum need no exchange.  All rows of the tile share one reference maximum
//               per row, kept in shared memory and handed from item j to item j+1 through a
//               barrier chain: the thread of item j picks up the reference left by item j-1, raises
//               it only when its own maximum is more than 2^8 above it (then it rescales O once the
//               product of item j-1 has finished), publishes it, and only then exponentiates - so
//               the three warpgroups exponentiate three items at the same time and keep the
//               special-function unit busy while the tensor pipe works on the others' tiles.
//               Each thread keeps the partial denominator of its own items, scaled to the reference
//               it used last; the three partial sums are merged at the end.
//   warp 12     one thread issues every tcgen05.mma: S(j) = Q K(j)^T three items ahead (operands in
//               shared memory), O += P(j) V(j) (P from tensor memory, V MN-major in shared memory);
//   warp 13     one thread issues the TMA tile loads into a ring of three 32 KB slots in the order the
//               tensor pipe consumes them (K0 K1 K2 V0 K3 V1 ...).
// Hand-offs are mbarriers (tcgen05.commit arrives for the MMA side); every wait is bounded and a
// failed wait raises the status word; all roles meet at one final barrier and TMEM is freed.
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr int kT4Bufs = 3;        // S/P buffers = softmax warpgroups
constexpr float kT4Lazy = 8.f;    // log2 units: P stays below 2^8

template <int D>
struct T4Cfg {
    static constexpr int kWarps = 4 * kT4Bufs;                 // softmax warps
    static constexpr int kWarpMma = kWarps, kWarpTma = kWarps + 1;
    static constexpr int kThreads = (kWarps + 2) * 32;
    static constexpr int NH = D / 64;
    static constexpr int kTile = NH * kHalfBytes;             // 128 x D bf16
    static constexpr int kSlots = 3;                           // ring of K / V tiles (3 measured faster than 4 and 2)
    static constexpr int kQ1 = 0, kQ2 = kTile, kRing = 2 * kTile;
    static constexpr int kTotal = kRing + kSlots * kTile + 1024;  // + slack for 1024-byte alignment
    static constexpr uint32_t kColS = 0, kColO = 128 * kT4Bufs, kCols = 512;
    static constexpr int kOq = D / 2;                          // O columns written by one thread at the end
};

// MODE 0: no mask; 1: columns [lo, hi) valid (relative to the chunk's first column); 2: far tile in
// which every code has members (count-weighted sum, no mask); 3: far tile with empty codes: a code
// with cnt == 0 is excluded from the maximum and from P, as the reference does before its maximum
// (ops/triton_fused_vq_attn.py:44-46) - otherwise an unused codeword with a dominating score could
// push every real weight below the exponent range.  cw: the counts of the chunk's 32 columns.
template <int MODE>
__device__ __forceinline__ void t4_mask2(float &x0, float &x1, int c0, int lo, int hi, const float *cw)
{
    if (MODE == 1) {
        x0 = (c0 >= lo && c0 < hi) ? x0 : -INFINITY;
        x1 = (c0 + 1 >= lo && c0 + 1 < hi) ? x1 : -INFINITY;
    }
    if (MODE == 3) {
        const float2 w = *reinterpret_cast<const float2 *>(cw + c0);
        x0 = w.x > 0.f ? x0 : -INFINITY;
        x1 = w.y > 0.f ? x1 : -INFINITY;
    }
}

// maximum of 32 score columns of the thread's row
template <int MODE>
__device__ __forceinline__ float t4_max_pass(uint32_t s_addr, int lo, int hi, const float *cw = nullptr)
{
    uint32_t r[32];
    tmem_ld32(s_addr, r);
    tc_wait_ld();
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float a0 = __uint_as_float(r[2 * j]), a1 = __uint_as_float(r[2 * j + 1]);
        t4_mask2<MODE>(a0, a1, 2 * j, lo, hi, cw);
        mx[j & 3] = fmax3(mx[j & 3], a0, a1);
    }
    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// P = exp2(S * scale - m) for 32 columns, packed 16-bit floats written to 16 columns at p_addr; returns
// the (count-weighted for MODE 2 and 3) sum of the 32 values.
template <int MODE, bool F16>
__device__ __forceinline__ float t4_exp_pass(uint32_t s_addr, uint32_t p_addr, const float *cw, int lo, int hi,
                                             float scale_log2, float neg_m)
{
    uint32_t r[32], pk[16];
    tmem_ld32(s_addr, r);
    tc_wait_ld();
    float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int c0 = 2 * j;
        float x0 = __uint_as_float(r[c0]), x1 = __uint_as_float(r[c0 + 1]);
        float t0, t1;
        t4_mask2<MODE>(x0, x1, c0, lo, hi, cw);
        ffma2(t0, t1, x0, x1, scale_log2, scale_log2, neg_m, neg_m);
        const float p0 = ex2(t0), p1 = ex2(t1);
        if (MODE >= 2) ffma2(ls[2 * (j & 1)], ls[2 * (j & 1) + 1], p0, p1, cw[c0], cw[c0 + 1], ls[2 * (j & 1)], ls[2 * (j & 1) + 1]);
        else fadd2(ls[2 * (j & 1)], ls[2 * (j & 1) + 1], ls[2 * (j & 1)], ls[2 * (j & 1) + 1], p0, p1);
        pk[j] = pack16<F16>(p0, p1);
    }
    tmem_st16(p_addr, pk);
    return (ls[0] + ls[1]) + (ls[2] + ls[3]);
}

template <int D, bool F16>
__global__ void __launch_bounds__(T4Cfg<D>::kThreads, 1)
prefill_tc4_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                   const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k3,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_cb,
                   const __grid_constant__ CUtensorMap tm_vs, TcParams p)
{
    using C = T4Cfg<D>;
    constexpr int NH = C::NH, NS = C::kSlots, NB3 = kT4Bufs;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bar_q, kv_full[NS], kv_empty[NS], s_full[NB3], p_full[NB3], pv_done[NB3], refbar[NB3][4], endbar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;
    __shared__ __align__(16) float s_cw[C::kWarps][kBlock];  // [softmax warp][column]: counts of the far tile it works on
    __shared__ float s_ref[kBlock];                          // reference maximum of every query row (log2 units)
    __shared__ float s_lend[NB3][kBlock], s_mend[NB3][kBlock];  // partial denominators and the references they are scaled to

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // grid.x = (query tile, query head inside its kv-head group), grid.y = (batch, kv head): the query heads
    // that share a kv head run next to each other, so their K / V / value-sum tiles meet in L2
    const int G = p.Hq / p.Hkv;
    const int m = p.ntiles - 1 - static_cast<int>(blockIdx.x) / G;  // heavy tiles first
    const int u = blockIdx.y;
    const int b = u / p.Hkv, hk = u % p.Hkv;
    const int hq = hk * G + static_cast<int>(blockIdx.x) % G;
    const int bh = b * p.Hq + hq;
    const TcWork work(p, m);
    const int n = work.n_items;

    if (tid == 0) {
        mbar_init(&bar_q, 1);
        for (int i = 0; i < NS; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        for (int i = 0; i < NB3; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 4);  // one arrival per warp of the warpgroup
            mbar_init(&pv_done[i], 1);
            for (int g = 0; g < 4; ++g) mbar_init(&refbar[i][g], 1);
        }
        mbar_init(&endbar, C::kWarps);
        fence_mbar_init();
        s_err = 0;
    }
    if (tid < kBlock) s_ref[tid] = -INFINITY;
    if (warp == C::kWarpTma) {
        __syncwarp();
        tmem_alloc(&s_tmem, C::kCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp == C::kWarpTma) {
        // ================================================================== TMA producer
        if (lane == 0) {
            prefetch_tmap(&tm_q1); prefetch_tmap(&tm_k1); prefetch_tmap(&tm_v);
            mbar_expect_tx(&bar_q, (p.rerope ? 2 : 1) * C::kTile);
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                tma_load_4d(smem + C::kQ1 + h * kHalfBytes, &tm_q1, &bar_q, 64 * h, m * kBlock, hq, b);
                if (p.rerope) tma_load_4d(smem + C::kQ2 + h * kHalfBytes, &tm_q2, &bar_q, 64 * h, m * kBlock, hq, b);
            }
            bool ok = true;
            int slot = 0;               // ring slot of the next load (consumption sequence K0 K1 K2 V0 K3 V1 ...)
            uint32_t free_par = 1u;     // phase of kv_empty[slot] that frees it; the first round needs no wait
            bool first_round = true;
            auto load = [&](int it, bool is_v) {
                if (!ok) return;
                if (!first_round && !mbar_wait(&kv_empty[slot], free_par, p.wait_limit)) {
                    ok = false;
                    return;
                }
                const int kind = work.kind(it), blk = work.block(it);
                uint8_t *dst = smem + C::kRing + slot * C::kTile;
                mbar_expect_tx(&kv_full[slot], C::kTile);
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    if (kind == kFar) {
                        if (is_v) tma_load_3d(dst + h * kHalfBytes, &tm_vs, &kv_full[slot], 64 * h, blk * kBlock, u * p.NB + work.far_blk);
                        else tma_load_3d(dst + h * kHalfBytes, &tm_cb, &kv_full[slot], 64 * h, blk * kBlock, hk);
                    } else {
                        const CUtensorMap *tm = is_v ? &tm_v : (kind == kBdA ? &tm_k3 : &tm_k1);
                        tma_load_4d(dst + h * kHalfBytes, tm, &kv_full[slot], 64 * h, blk * kBlock, hk, b);
                    }
                }
                if (++slot == NS) {
                    slot = 0;
                    free_par ^= 1u;
                    first_round = false;
                }
            };
            for (int j = 0; j < NB3 && j < n; ++j) load(j, false);
            for (int j = 0; j < n; ++j) {
                load(j, true);
                if (j + NB3 < n) load(j + NB3, false);
            }
            if (!ok) s_err = 1;
        }
    } else if (warp == C::kWarpMma) {
        // ================================================================== MMA issuer
        // The tensor pipe's queue is shallow: whatever this thread does between two groups of MMAs is time the
        // pipe idles.  So the loop carries no divisions, no per-item classification and no 64-bit descriptor
        // arithmetic: ring slot, score buffer and their barrier phases are running counters, the operand
        // descriptors of the three slots are built once (only the low word of a descriptor depends on the
        // address), and an item needs the constant-position query exactly when it comes before `n_q2`.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_f16kind(128, 128, 0, 0, F16 ? 0u : 1u);
            constexpr uint32_t idesc_pv = idesc_f16kind(128, D, 0, 1, F16 ? 0u : 1u);
            const uint64_t d_q1 = smem_desc_sw128(smem_u32(smem + C::kQ1), 16, 1024);
            const uint64_t d_q2 = p.rerope ? smem_desc_sw128(smem_u32(smem + C::kQ2), 16, 1024) : d_q1;
            const uint64_t d_k0 = smem_desc_sw128(smem_u32(smem + C::kRing), 16, 1024);          // K tiles: K-major
            const uint64_t d_v0 = smem_desc_sw128(smem_u32(smem + C::kRing), kHalfBytes, 1024);  // V tiles: MN-major
            const int n_q2 = p.rerope ? work.n_far + (work.n_bd == 2 ? 1 : 0) : 0;               // items scored with q2
            bool ok = mbar_wait(&bar_q, 0, p.wait_limit);
            int slot = 0;
            uint32_t slot_par = 0;                 // phase of the ring slot about to be consumed
            int sbuf = 0, pbuf = 0;                // score buffer of the next S product / of the next P V product
            uint32_t p_par = 0;                    // phase of p_full[pbuf]
            auto next_slot = [&]() {
                if (++slot == NS) {
                    slot = 0;
                    slot_par ^= 1u;
                }
            };
            auto qk = [&](int it) {  // S(it) = Q K(it)^T into the next score buffer (free: its previous product was issued before)
                if (!ok) return;
                if (!mbar_wait(&kv_full[slot], slot_par, p.wait_limit)) {
                    ok = false;
                    return;
                }
                tc_fence_after();
                const uint64_t da = it < n_q2 ? d_q2 : d_q1;
                const uint64_t db = d_k0 + static_cast<uint64_t>((slot * C::kTile) >> 4);
                const uint32_t sdst = tmem + C::kColS + 128 * sbuf;
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        constexpr int kStep = 32 >> 4;
                        const uint64_t off = static_cast<uint64_t>((h * kHalfBytes) >> 4) + static_cast<uint64_t>(k4 * kStep);
                        if (h == 0 && k4 == 0) mma_ss_first(sdst, da + off, db + off, idesc_qk);
                        else mma_ss_acc(sdst, da + off, db + off, idesc_qk);
                    }
                tc_commit(&kv_empty[slot]);
                tc_commit(&s_full[sbuf]);
                next_slot();
                if (++sbuf == NB3) sbuf = 0;
            };
            auto pv = [&](int it) {  // O += P(it) V(it)
                if (!ok) return;
                if (!mbar_wait(&p_full[pbuf], p_par, p.wait_limit) || !mbar_wait(&kv_full[slot], slot_par, p.wait_limit)) {
                    ok = false;
                    return;
                }
                tc_fence_after();
                const uint64_t dv = d_v0 + static_cast<uint64_t>((slot * C::kTile) >> 4);
                const uint32_t odst = tmem + C::kColO, psrc = tmem + C::kColS + 128 * pbuf;
                if (it == 0) mma_ts_first(odst, psrc, dv, idesc_pv);
                else mma_ts_acc(odst, psrc, dv, idesc_pv);
#pragma unroll
                for (int kk = 1; kk < 8; ++kk)  // keys 16 kk ..: packed 16-bit P over the first 64 columns of the score buffer
                    mma_ts_acc(odst, psrc + 8 * kk, dv + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv);
                tc_commit(&kv_empty[slot]);
                tc_commit(&pv_done[pbuf]);
                next_slot();
                if (++pbuf == NB3) {
                    pbuf = 0;
                    p_par ^= 1u;
                }
            };
            for (int j = 0; j < NB3 && j < n; ++j) qk(j);
            for (int j = 0; j < n; ++j) {
                pv(j);
                if (j + NB3 < n) qk(j + NB3);
            }
            if (!ok) s_err = 1;
        }
    } else {
        // ================================================================== softmax
        constexpr unsigned kAll = 0xffffffffu;
        const int g = warp >> 2, lq = warp & 3;           // warpgroup (= score buffer) and lane quarter (32 query rows)
        const int row = lq * 32 + lane;                   // query row inside the tile (= TMEM lane)
        const uint32_t lane_off = static_cast<uint32_t>(lq * 32) << 16;
        const uint32_t sa = tmem + lane_off + C::kColS + 128 * g;
        const uint32_t o_addr = tmem + lane_off + C::kColO;
        float my_ref = -INFINITY, l_part = 0.f;           // l_part: sum over this thread's items, scaled to my_ref
        bool ok = true;
        // Counts of a far tile: lane l fetches those of columns l, 32 + l, 64 + l, 96 + l one of the
        // warp's items ahead; the warp keeps them in its own shared-memory row.
        const float *cnt_base = p.cnt + (static_cast<int64_t>(u) * p.NB + work.far_blk) * p.MK + lane;
        float *cw = &s_cw[warp][0];
        float cnt_reg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cnt_reg[i] = g < work.n_far ? __ldg(cnt_base + g * kBlock + 32 * i) : 0.f;
#pragma unroll 1
        for (int it = g; it < n; it += NB3) {
            const int par = (it / NB3) & 1;
            const int kind = work.kind(it);
            bool has_empty = false;                       // warp-uniform: some code of this far tile has no member
            if (kind == kFar) {
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; ++i) cw[32 * i + lane] = cnt_reg[i];
                has_empty = __any_sync(kAll, !(cnt_reg[0] > 0.f && cnt_reg[1] > 0.f && cnt_reg[2] > 0.f && cnt_reg[3] > 0.f));
                __syncwarp();
                if (it + NB3 < work.n_far) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) cnt_reg[i] = __ldg(cnt_base + (it + NB3) * kBlock + 32 * i);
                }
            }
            // valid key columns of this row: [lo, hi)
            int lo = 0, hi = kBlock;
            if (kind == kDiag) hi = row + 1;
            else if (kind == kBdA) hi = row;
            else if (kind == kBdB) lo = row;
            if (!__all_sync(kAll, mbar_wait(&s_full[g], par, p.wait_limit))) {
                ok = false;
                break;
            }
            tc_fence_after();
            // ---- row maximum of this item
            float mx = -INFINITY;
            if (kind == kFar && has_empty) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx = fmaxf(mx, t4_max_pass<3>(sa + 32 * c, 0, 0, cw + 32 * c));
            } else if (kind == kFar || kind == kFull) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx = fmaxf(mx, t4_max_pass<0>(sa + 32 * c, 0, 0));
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx = fmaxf(mx, t4_max_pass<1>(sa + 32 * c, lo - 32 * c, hi - 32 * c));
            }
            const float m_tile = mx * p.scale_log2;
            // ---- the reference left by the previous item; raise it only when this item is far above it
            if (it > 0 && !__all_sync(kAll, mbar_wait(&refbar[(g + NB3 - 1) % NB3][lq], ((it - 1) / NB3) & 1, p.wait_limit))) {
                ok = false;
                break;
            }
            const float ref = s_ref[row];
            float m_use = ref;
            if (m_tile > ref + kT4Lazy || ref == -INFINITY) m_use = fmaxf(ref, m_tile);
            if (m_use != ref) s_ref[row] = m_use;
            __syncwarp();
            if (lane == 0) mbar_arrive(&refbar[g][lq]);   // the warp's 32 stores are ordered before it
            const float m_safe = (m_use == -INFINITY) ? 0.f : m_use;
            // a row without any valid key so far has an all-zero O row: nothing to rescale
            const bool rescale = (m_use != ref) && (ref != -INFINITY);
            if (__any_sync(kAll, rescale)) {
                // O may be touched once the product of the previous item has finished (it >= 1 here)
                if (!__all_sync(kAll, mbar_wait(&pv_done[(it - 1) % NB3], ((it - 1) / NB3) & 1, p.wait_limit))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const float alpha = rescale ? ex2(ref - m_safe) : 1.f;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + 32 * c, r);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                    tmem_st32(o_addr + 32 * c, r);
                }
            }
            if (my_ref != m_use) {
                l_part *= ex2(my_ref - m_safe);           // my_ref = -inf: l_part is 0 and stays 0
                my_ref = m_use;
            }
            // ---- exponentials: chunk c reads columns [32c, 32c+32) and writes P over [16c, 16c+16), never ahead of a read
            float ls = 0.f;
            if (kind == kFar && has_empty) {
#pragma unroll
                for (int c = 0; c < 4; ++c) ls += t4_exp_pass<3, F16>(sa + 32 * c, sa + 16 * c, cw + 32 * c, 0, 0, p.scale_log2, -m_safe);
            } else if (kind == kFar) {
#pragma unroll
                for (int c = 0; c < 4; ++c) ls += t4_exp_pass<2, F16>(sa + 32 * c, sa + 16 * c, cw + 32 * c, 0, 0, p.scale_log2, -m_safe);
            } else if (kind == kFull) {
#pragma unroll
                for (int c = 0; c < 4; ++c) ls += t4_exp_pass<0, F16>(sa + 32 * c, sa + 16 * c, cw, 0, 0, p.scale_log2, -m_safe);
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) ls += t4_exp_pass<1, F16>(sa + 32 * c, sa + 16 * c, cw, lo - 32 * c, hi - 32 * c, p.scale_log2, -m_safe);
            }
            l_part += ls;
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[g]);
        }
        // ---- epilogue: merge the three partial denominators, O / l once the last product has finished
        s_lend[g][row] = l_part;
        s_mend[g][row] = my_ref;
        __syncwarp();
        if (lane == 0) mbar_arrive(&endbar);
        if (ok && !__all_sync(kAll, mbar_wait(&endbar, 0, p.wait_limit))) ok = false;
        if (ok && !__all_sync(kAll, mbar_wait(&pv_done[(n - 1) % NB3], ((n - 1) / NB3) & 1, p.wait_limit))) ok = false;
        tc_fence_after();
        if (!ok) s_err = 1;
        if (ok && g < 2) {
            const float ref = s_ref[row];
            float den = 0.f;
#pragma unroll
            for (int i = 0; i < NB3; ++i) {
                const float li = s_lend[i][row];
                if (li > 0.f) den += li * ex2(s_mend[i][row] - ref);
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
            const int64_t grow = static_cast<int64_t>(m) * kBlock + row;
            uint32_t r[C::kOq];
#pragma unroll
            for (int c = 0; c < C::kOq / 32; ++c) tmem_ld32(o_addr + g * C::kOq + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
            tc_wait_ld();
            // The thread holds kOq columns of its own row; stored from here, every instruction of the warp would touch 32
            // different rows.  So the warp's 32 x (2 kOq)-byte block goes through the tile ring (free: the last product has
            // completed, and with it every read of the ring) and is written out with eight lanes per row - whole 128-byte
            // lines.  Rows padded by 16 bytes: the 16-byte accesses of eight lanes fall into different banks.
            constexpr int kRowB = C::kOq * 2, kPitch = kRowB + 16;          // bytes per row of the warp's block
            uint8_t *stg = smem + C::kRing + warp * (32 * kPitch);
#pragma unroll
            for (int j = 0; j < C::kOq / 8; ++j) {
                uint4 w;
                w.x = pack16<F16>(__uint_as_float(r[8 * j]) * inv, __uint_as_float(r[8 * j + 1]) * inv);
                w.y = pack16<F16>(__uint_as_float(r[8 * j + 2]) * inv, __uint_as_float(r[8 * j + 3]) * inv);
                w.z = pack16<F16>(__uint_as_float(r[8 * j + 4]) * inv, __uint_as_float(r[8 * j + 5]) * inv);
                w.w = pack16<F16>(__uint_as_float(r[8 * j + 6]) * inv, __uint_as_float(r[8 * j + 7]) * inv);
                *reinterpret_cast<uint4 *>(stg + lane * kPitch + 16 * j) = w;
            }
            __syncwarp();
            constexpr int kLanesPerRow = kRowB / 16, kRowsPerIt = 32 / kLanesPerRow;
            const int sub = lane / kLanesPerRow, ch = lane % kLanesPerRow;
            uint16_t *obase = p.out + b * p.o_sb + hq * p.o_sh + g * C::kOq + 8 * ch;
#pragma unroll
            for (int it = 0; it < 32 / kRowsPerIt; ++it) {
                const int rr = it * kRowsPerIt + sub;                           // row inside the warp's block
                const int64_t gr = static_cast<int64_t>(m) * kBlock + lq * 32 + rr;
                const uint4 w = *reinterpret_cast<const uint4 *>(stg + rr * kPitch + 16 * ch);
                if (gr < p.L) *reinterpret_cast<uint4 *>(obase + gr * p.o_sl) = w;
            }
            if (grow < p.L) {
                if (g == 0 && p.lse2) p.lse2[static_cast<int64_t>(bh) * p.L + grow] = ref + log2f(den);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (s_err && tid == 0) {
        if (p.status) atomicExch(p.status, VQ_WORD_TIMEOUT);
        // a bounded wait expired: give tile loads still in flight time to land before leaving
#pragma unroll 1
        for (int w = 0; w < (1 << 14); ++w) __nanosleep(256);
    }
    __syncthreads();
    if (warp == C::kWarpTma) {
        __syncwarp();
        tmem_dealloc(tmem, C::kCols);
    }
}

template <int D, bool F16>
static int launch_tc4(const VqPrefillArgs *a, cudaStream_t stream)
{
    using C = T4Cfg<D>;
    TcMaps m;
    TcParams p;
    const int st = tc_setup<D>(a, m, p);
    if (st != VQ_OK) return st;
    auto kern = prefill_tc4_kernel<D, F16>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal) != cudaSuccess) return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>(p.ntiles * (p.Hq / p.Hkv)), static_cast<unsigned>(a->q1.shape[0] * p.Hkv));
    kern<<<grid, C::kThreads, C::kTotal, stream>>>(m.q1, m.q2, m.k1, m.k3, m.v, m.cb, m.vs, p);
    return launch_status();
}

int launch_prefill_tensor4(const VqPrefillArgs *a, cudaStream_t stream)
{
    const int D = static_cast<int>(a->q1.shape[3]);
    // 16-byte aligned rows for the output stores and the tensor maps
    if (a->out.stride[2] % 8 || a->out.stride[1] % 8 || a->out.stride[0] % 8) return VQ_EINVAL_STRIDE;
    if (a->q1.dtype == VQ_F16) return D == 64 ? launch_tc4<64, true>(a, stream) : launch_tc4<128, true>(a, stream);
    return D == 64 ? launch_tc4<64, false>(a, stream) : launch_tc4<128, false>(a, stream);
}

}  // namespace vq
