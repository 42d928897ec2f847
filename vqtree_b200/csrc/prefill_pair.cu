// Fused VQ-attention prefill on the sm_100a tensor cores: TWO adjacent 128-row query tiles of one
// (batch, query head) per CTA, so that the key / value / codebook tiles both of them need cross from
// L2 to shared memory once and feed two tensor-core products each.
//
// Every query tile keeps its own work list (far codebook tiles, boundary block, interior blocks,
// causal diagonal - see TcWork) and its own online softmax (this replaces the reference's two
// kernels and their log-sum-exp merge, ops/triton_fused_vq_attn.py:202-250).  The two lists are
// merged into steps by a key (far tile index < boundary block through the un-rotated keys < block
// number of a rotated-key item): items with equal keys form one step and share the codebook tile
// (far) or the key AND value tile (rotated keys of one block); see pair_walk.  Tensor memory holds
// one S/P buffer and one O accumulator per query tile (4 x 128 columns).  Roles:
//   warps 0-7 / 8-15  softmax of query tile A / B, two threads per query row: both read all 128 scores of
//               the row and find the same maximum (no exchange), meet at a barrier of the tile's eight
//               warps (P overwrites scores), then each exponentiates its own 64 columns into packed
//               bf16 over the first 32 of them; O is rescaled only when the maximum grew by more than
//               2^8; the two partial denominators of a row are merged at the end through the tile's
//               (by then free) Q buffer.  While one tile's threads exponentiate, the tensor pipe works
//               for the other tile.
//   warp 16     one thread issues every tcgen05.mma in the order PV_A(prev) QK_A(next) PV_B(prev)
//               QK_B(next): S = Q K^T with both operands in shared memory, O += P V with P from
//               tensor memory and V MN-major in shared memory;
//   warp 17     one thread issues the TMA tile loads into a ring of five 32 KB slots in the order of first
//               use; a shared tile is released by its second user.  Each query tile has ONE Q buffer:
//               it first holds the queries rotated to the constant far position (far tiles, boundary
//               block through the un-rotated keys), then is reloaded with the position-rotated queries.
// Measured on the 32K workload this kernel is slower than the one-tile kernel (1.52 vs 1.35 ms): with a
// single score buffer per tile the chain scores -> softmax -> product is exposed (per step of two
// items per tile: 2000 cycles waiting for scores, 650 maximum, 200 barrier, 2000 exponentials), and the
// two tiles exponentiate at the same time on one special-function unit.  It is kept selectable.
// Hand-offs are mbarriers (tcgen05.commit arrives for the MMA side); every wait is bounded and a
// failed wait raises the status word; all roles meet at one final barrier and TMEM is freed.
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr float kPairLazy = 8.f;    // log2 units: P stays below 2^8

template <int D>
struct PairCfg {
    static constexpr int kWarps = 16;                          // softmax warps: 8 per query tile, two threads per query row
    static constexpr int kWarpMma = kWarps, kWarpTma = kWarps + 1;
    static constexpr int kThreads = (kWarps + 2) * 32;
    static constexpr int NH = D / 64;
    static constexpr int kTile = NH * kHalfBytes;             // 128 x D bf16
    static constexpr int kSlots = D == 128 ? 5 : 8;            // ring of K / V tiles
    static constexpr int kQ = 0, kRing = 2 * kTile;            // Q_A Q_B, then the ring
    static constexpr int kTotal = kRing + kSlots * kTile + 1024;  // + slack for 1024-byte alignment
    static constexpr uint32_t kColS = 0, kColO = 256, kCols = 512;  // S_A S_B O_A O_B
};

constexpr int kKeyBdA = 1 << 20, kKeyLocal = 2 << 20;

// Merge key of an item: equal keys of the two query tiles mean "same step".
__device__ __forceinline__ int pair_key(const TcWork &w, int i)
{
    const int kind = w.kind(i);
    return kind == kFar ? i : (kind == kBdA ? kKeyBdA : kKeyLocal + w.block(i));
}

// Walks the merged work of the two query tiles in the order the tensor pipe executes it and calls
// f(op, X, item, load, release) for every product: op 0 = scores of `item` of tile X, 1 = its P V
// product; `load`: the operand tile (K for op 0, V for op 1) enters the ring here (first use);
// `release`: this is its last use.  Within a step, tile X first gets the P V product of its previous
// item (its S/P buffer is single), then the scores of the new one.  f returns false to stop.
template <class F>
__device__ __forceinline__ void pair_walk(const TcWork &wa, const TcWork &wb, int na, int nb, F &&f)
{
    int it[2] = {0, 0}, pend[2] = {-1, -1};
    const int n[2] = {na, nb};
    bool pend_sh[2] = {false, false}, sh_loaded = false;
    auto product = [&](int X) {  // P V of the pending item of tile X
        bool load = true, release = true;
        if (pend_sh[X]) {
            load = !sh_loaded;
            release = sh_loaded;
            sh_loaded = !sh_loaded;
        }
        const int i = pend[X];
        pend[X] = -1;
        return f(1, X, i, load, release);
    };
#pragma unroll 1
    while (it[0] < n[0] || it[1] < n[1]) {
        const int ka = it[0] < n[0] ? pair_key(wa, it[0]) : 0x7fffffff;
        const int kb = it[1] < n[1] ? pair_key(wb, it[1]) : 0x7fffffff;
        const bool act[2] = {ka <= kb, kb <= ka};
        const bool both = ka == kb;
        const bool share_k = both && ka != kKeyBdA, share_v = both && ka >= kKeyLocal;
#pragma unroll
        for (int X = 0; X < 2; ++X) {
            if (!act[X]) continue;
            if (pend[X] >= 0 && !product(X)) return;
            if (!f(0, X, it[X], !(share_k && X == 1), !(share_k && X == 0))) return;
            pend[X] = it[X]++;
            pend_sh[X] = share_v;
        }
    }
#pragma unroll
    for (int X = 0; X < 2; ++X)
        if (pend[X] >= 0 && !product(X)) return;
}

template <int MODE>
__device__ __forceinline__ void pair_mask2(float &x0, float &x1, int c0, int lo, int hi)
{
    if (MODE == 1) {
        x0 = (c0 >= lo && c0 < hi) ? x0 : -INFINITY;
        x1 = (c0 + 1 >= lo && c0 + 1 < hi) ? x1 : -INFINITY;
    }
}

// maximum of 32 score columns of the thread's row; MODE 1: columns [lo, hi) valid (relative to the chunk)
template <int MODE>
__device__ __forceinline__ float pair_max_pass(uint32_t s_addr, int lo, int hi)
{
    uint32_t r[32];
    tmem_ld32(s_addr, r);
    tc_wait_ld();
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float a0 = __uint_as_float(r[2 * j]), a1 = __uint_as_float(r[2 * j + 1]);
        pair_mask2<MODE>(a0, a1, 2 * j, lo, hi);
        mx[j & 3] = fmax3(mx[j & 3], a0, a1);
    }
    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// P = exp2(S * scale - m) for 32 columns, packed bf16 written to 16 columns at p_addr; returns the sum
// of the 32 values (MODE 2, far tile: weighted by the member counts cw[0..32), read from global memory
// with the same address in every lane; a far tile needs no mask - a code without members has a zero
// value-sum row and weight 0, it can only raise the reference maximum).
template <int MODE>
__device__ __forceinline__ float pair_exp_pass(uint32_t s_addr, uint32_t p_addr, const float4 *cw, int lo, int hi,
                                               float scale_log2, float neg_m)
{
    uint32_t r[32], pk[16];
    tmem_ld32(s_addr, r);
    tc_wait_ld();
    float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
        float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
        if (MODE == 2) w = __ldg(cw + (j >> 1));
        float x0 = __uint_as_float(r[2 * j]), x1 = __uint_as_float(r[2 * j + 1]);
        float x2 = __uint_as_float(r[2 * j + 2]), x3 = __uint_as_float(r[2 * j + 3]);
        float t0, t1, t2, t3;
        pair_mask2<MODE>(x0, x1, 2 * j, lo, hi);
        pair_mask2<MODE>(x2, x3, 2 * j + 2, lo, hi);
        ffma2(t0, t1, x0, x1, scale_log2, scale_log2, neg_m, neg_m);
        ffma2(t2, t3, x2, x3, scale_log2, scale_log2, neg_m, neg_m);
        const float p0 = ex2(t0), p1 = ex2(t1), p2 = ex2(t2), p3 = ex2(t3);
        if (MODE == 2) {
            ffma2(ls[0], ls[1], p0, p1, w.x, w.y, ls[0], ls[1]);
            ffma2(ls[2], ls[3], p2, p3, w.z, w.w, ls[2], ls[3]);
        } else {
            fadd2(ls[0], ls[1], ls[0], ls[1], p0, p1);
            fadd2(ls[2], ls[3], ls[2], ls[3], p2, p3);
        }
        pk[j] = pack_bf16(p0, p1);
        pk[j + 1] = pack_bf16(p2, p3);
    }
    tmem_st16(p_addr, pk);
    return (ls[0] + ls[1]) + (ls[2] + ls[3]);
}

template <int D>
__global__ void __launch_bounds__(PairCfg<D>::kThreads, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                    const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k3,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_cb,
                    const __grid_constant__ CUtensorMap tm_vs, TcParams p)
{
    using C = PairCfg<D>;
    constexpr int NH = C::NH, NS = C::kSlots;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bar_q[2], q_free[2], kv_full[NS], kv_empty[NS], s_full[2], rd_done[2], p_full[2], pv_done[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int npairs = (p.ntiles + 1) >> 1;
    const int pr = npairs - 1 - static_cast<int>(blockIdx.x);   // heavy pairs first
    const int bh = blockIdx.y;
    const int b = bh / p.Hq, hq = bh % p.Hq;
    const int hk = hq / (p.Hq / p.Hkv);
    const int u = b * p.Hkv + hk;
    const int m0 = 2 * pr, m1 = 2 * pr + 1;
    const TcWork wa(p, m0), wb(p, m1);
    const int na = wa.n_items, nb = m1 < p.ntiles ? wb.n_items : 0;
    // The Q buffer of a tile first holds the queries rotated to the constant far position (used by the
    // far tiles and the boundary block through the un-rotated keys, which come first in the work list),
    // then is reloaded with the queries rotated to their own positions.
    auto uses_q2 = [&](const TcWork &w, int it) {
        const int kind = w.kind(it);
        return p.rerope && (kind == kFar || kind == kBdA);
    };
    const bool q2_first[2] = {na > 0 && uses_q2(wa, 0), nb > 0 && uses_q2(wb, 0)};

    if (tid == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_q[i], 1);
            mbar_init(&q_free[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 8);  // one arrival per softmax warp of the tile
            mbar_init(&rd_done[i], 8);
            mbar_init(&pv_done[i], 1);
        }
        fence_mbar_init();
        s_err = 0;
    }
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
            for (int X = 0; X < 2; ++X) {
                if (X == 1 && nb == 0) break;
                mbar_expect_tx(&bar_q[X], C::kTile);
#pragma unroll
                for (int h = 0; h < NH; ++h)
                    tma_load_4d(smem + C::kQ + X * C::kTile + h * kHalfBytes, q2_first[X] ? &tm_q2 : &tm_q1, &bar_q[X], 64 * h,
                                (m0 + X) * kBlock, hq, b);
            }
            bool swapped[2] = {false, false};
            int q = 0;  // tiles loaded so far
            bool ok = true;
            pair_walk(wa, wb, na, nb, [&](int op, int X, int it, bool load, bool) {
                const TcWork &w = X ? wb : wa;
                if (op == 0 && q2_first[X] && !swapped[X] && !uses_q2(w, it)) {
                    // the last product with the far-position queries has been issued: reload the buffer when it finished
                    if (!mbar_wait(&q_free[X], 0)) {
                        ok = false;
                        return false;
                    }
                    mbar_expect_tx(&bar_q[X], C::kTile);
#pragma unroll
                    for (int h = 0; h < NH; ++h)
                        tma_load_4d(smem + C::kQ + X * C::kTile + h * kHalfBytes, &tm_q1, &bar_q[X], 64 * h, (m0 + X) * kBlock, hq, b);
                    swapped[X] = true;
                }
                if (!load) return true;
                const int slot = q % NS;
                if (q >= NS && !mbar_wait(&kv_empty[slot], ((q / NS) - 1) & 1)) {
                    ok = false;
                    return false;
                }
                const int kind = w.kind(it), blk = w.block(it);
                uint8_t *dst = smem + C::kRing + slot * C::kTile;
                mbar_expect_tx(&kv_full[slot], C::kTile);
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    if (kind == kFar) {
                        if (op) tma_load_3d(dst + h * kHalfBytes, &tm_vs, &kv_full[slot], 64 * h, blk * kBlock, u * p.NB + w.far_blk);
                        else tma_load_3d(dst + h * kHalfBytes, &tm_cb, &kv_full[slot], 64 * h, blk * kBlock, hk);
                    } else {
                        const CUtensorMap *tm = op ? &tm_v : (kind == kBdA ? &tm_k3 : &tm_k1);
                        tma_load_4d(dst + h * kHalfBytes, tm, &kv_full[slot], 64 * h, blk * kBlock, hk, b);
                    }
                }
                ++q;
                return true;
            });
            if (!ok) s_err = 1;
        }
    } else if (warp == C::kWarpMma) {
        // ================================================================== MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(128, D, 0, 1);
            // operand descriptors differ only in their 16-byte-granular start address
            const uint64_t d_q0 = smem_desc_sw128(smem_u32(smem + C::kQ), 16, 1024);
            const uint64_t d_k0 = smem_desc_sw128(smem_u32(smem + C::kRing), 16, 1024);          // K tiles: K-major
            const uint64_t d_v0 = smem_desc_sw128(smem_u32(smem + C::kRing), kHalfBytes, 1024);  // V tiles: MN-major
            int q = 0, k_slot = 0, v_slot = 0;  // tiles taken from the ring; slots of the shared K / V tile in use
            bool ok = true;
            int q_phase[2] = {0, 0};  // Q loads of each tile waited for so far
            pair_walk(wa, wb, na, nb, [&](int op, int X, int it, bool load, bool release) {
                int slot;
                if (op == 1 && !mbar_wait(&p_full[X], it & 1)) {
                    ok = false;
                    return false;
                }
                const TcWork &w = X ? wb : wa;
                if (op == 0) {
                    const int need = (q2_first[X] && !uses_q2(w, it)) ? 2 : 1;  // Q loads that must have landed
                    while (q_phase[X] < need) {
                        if (!mbar_wait(&bar_q[X], q_phase[X] & 1)) {
                            ok = false;
                            return false;
                        }
                        ++q_phase[X];
                    }
                }
                if (load) {
                    slot = q % NS;
                    if (!mbar_wait(&kv_full[slot], (q / NS) & 1)) {
                        ok = false;
                        return false;
                    }
                    ++q;
                    if (op) v_slot = slot;
                    else k_slot = slot;
                } else {
                    slot = op ? v_slot : k_slot;
                }
                tc_fence_after();
                if (op == 0) {
                    const uint64_t da = d_q0 + static_cast<uint64_t>((X * C::kTile) >> 4);
                    const uint64_t db = d_k0 + static_cast<uint64_t>((slot * C::kTile) >> 4);
                    const uint32_t sdst = tmem + C::kColS + 128 * X;
#pragma unroll
                    for (int h = 0; h < NH; ++h)
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4) {
                            const uint64_t off = static_cast<uint64_t>((h * kHalfBytes + k4 * 32) >> 4);
                            mma_ss(sdst, da + off, db + off, idesc_qk, (h | k4) ? 1u : 0u);
                        }
                    if (release) tc_commit(&kv_empty[slot]);
                    tc_commit(&s_full[X]);
                    if (q2_first[X] && uses_q2(w, it) && !uses_q2(w, it + 1)) tc_commit(&q_free[X]);
                } else {
                    const uint64_t dv = d_v0 + static_cast<uint64_t>((slot * C::kTile) >> 4);
                    const uint32_t odst = tmem + C::kColO + 128 * X, psrc = tmem + C::kColS + 128 * X;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)  // keys 16 kk ..: packed bf16, keys 0-63 over columns 0-31, keys 64-127 over columns 64-95
                        mma_ts(odst, psrc + 64 * (kk >> 2) + 8 * (kk & 3), dv + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv, (it | kk) ? 1u : 0u);
                    if (release) tc_commit(&kv_empty[slot]);
                    tc_commit(&pv_done[X]);
                }
                return true;
            });
            if (!ok) s_err = 1;
        }
    } else {
        // ================================================================== softmax
        constexpr unsigned kAll = 0xffffffffu;
        const int X = warp >> 3, half = (warp >> 2) & 1, lq = warp & 3;  // query tile, column half (64 keys), lane quarter (32 rows)
        const int row = lq * 32 + lane;                   // query row inside the tile (= TMEM lane)
        const uint32_t lane_off = static_cast<uint32_t>(lq * 32) << 16;
        const uint32_t sa = tmem + lane_off + C::kColS + 128 * X;
        const uint32_t sh = sa + 64 * half;               // this thread's half of the score columns; its P goes over the first 32 of them
        const uint32_t o_addr = tmem + lane_off + C::kColO + 128 * X + (D / 2) * half;  // and its half of the O columns
        const TcWork &w = X ? wb : wa;
        const int n = X ? nb : na;
        const int m = m0 + X;
        float row_m = -INFINITY, l_run = 0.f;             // reference maximum (log2 units); denominator over this thread's columns
        bool ok = true;
        const float4 *cnt4 = reinterpret_cast<const float4 *>(p.cnt + (static_cast<int64_t>(u) * p.NB + w.far_blk) * p.MK) + 16 * half;
        // all 8 warps of the tile: everybody has finished reading S (use number `use`)
        auto tile_sync = [&](int use) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&rd_done[X]);
            return __all_sync(kAll, mbar_wait(&rd_done[X], use & 1));
        };
#pragma unroll 1
        for (int it = 0; it < n; ++it) {
            const int kind = w.kind(it);
            // valid key columns of this row: [lo, hi)
            int lo = 0, hi = kBlock;
            if (kind == kDiag) hi = row + 1;
            else if (kind == kBdA) hi = row;
            else if (kind == kBdB) lo = row;
            if (!__all_sync(kAll, mbar_wait(&s_full[X], it & 1))) {
                ok = false;
                break;
            }
            tc_fence_after();
            // ---- row maximum of this item: both threads of a row read all 128 scores and find the same value
            float mx = -INFINITY;
            if (kind == kFar || kind == kFull) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx = fmaxf(mx, pair_max_pass<0>(sa + 32 * c, 0, 0));
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx = fmaxf(mx, pair_max_pass<1>(sa + 32 * c, lo - 32 * c, hi - 32 * c));
            }
            tc_fence_before();
            if (!tile_sync(it)) {  // P of one thread overwrites scores the other one has just read
                ok = false;
                break;
            }
            tc_fence_after();
            const float m_tile = mx * p.scale_log2;
            // lazy rescaling: keep the old reference maximum unless the new one is far above it
            float m_use = row_m;
            if (m_tile > row_m + kPairLazy || row_m == -INFINITY) m_use = fmaxf(row_m, m_tile);
            const float m_safe = (m_use == -INFINITY) ? 0.f : m_use;
            // a row without any valid key so far has an all-zero O row: nothing to rescale
            const bool rescale = (m_use != row_m) && (row_m != -INFINITY);
            const float alpha = rescale ? ex2(row_m - m_safe) : 1.f;
            if (__any_sync(kAll, rescale)) {
                // O may be touched once the product of the previous item has finished (it >= 1 here)
                if (!__all_sync(kAll, mbar_wait(&pv_done[X], (it - 1) & 1))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D / 64; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + 32 * c, r);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                    tmem_st32(o_addr + 32 * c, r);
                }
            }
            row_m = m_use;
            // ---- exponentials of this thread's 64 columns: chunk c reads [32c, 32c+32) and writes P over [16c, 16c+16)
            const int lo_h = lo - 64 * half, hi_h = hi - 64 * half;
            float ls = 0.f;
            if (kind == kFar) {
                const float4 *cw = cnt4 + it * (kBlock / 4);
#pragma unroll
                for (int c = 0; c < 2; ++c) ls += pair_exp_pass<2>(sh + 32 * c, sh + 16 * c, cw + 8 * c, 0, 0, p.scale_log2, -m_safe);
            } else if (kind == kFull) {
#pragma unroll
                for (int c = 0; c < 2; ++c) ls += pair_exp_pass<0>(sh + 32 * c, sh + 16 * c, cnt4, 0, 0, p.scale_log2, -m_safe);
            } else {
#pragma unroll
                for (int c = 0; c < 2; ++c) ls += pair_exp_pass<1>(sh + 32 * c, sh + 16 * c, cnt4, lo_h - 32 * c, hi_h - 32 * c, p.scale_log2, -m_safe);
            }
            l_run = l_run * alpha + ls;
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[X]);
        }
        // ---- epilogue: O / l once the last product has finished
        if (n > 0) {
            if (ok && !__all_sync(kAll, mbar_wait(&pv_done[X], (n - 1) & 1))) ok = false;
            tc_fence_after();
            // the tile's Q buffer is free now: the two threads of a row exchange their partial denominators through it
            float *xch = reinterpret_cast<float *>(smem + C::kQ + X * C::kTile);
            xch[half * kBlock + row] = l_run;
            if (ok && !tile_sync(n)) ok = false;
            if (ok) {
                const float den = l_run + xch[(half ^ 1) * kBlock + row];
                const float inv = den > 0.f ? 1.f / den : 0.f;
                const int64_t grow = static_cast<int64_t>(m) * kBlock + row;
                __nv_bfloat16 *o = p.out + b * p.o_sb + hq * p.o_sh + grow * p.o_sl + (D / 2) * half;
#pragma unroll
                for (int c = 0; c < D / 64; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + 32 * c, r);
                    tc_wait_ld();
                    if (grow < p.L) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 v4;
                            v4.x = pack_bf16(__uint_as_float(r[8 * j]) * inv, __uint_as_float(r[8 * j + 1]) * inv);
                            v4.y = pack_bf16(__uint_as_float(r[8 * j + 2]) * inv, __uint_as_float(r[8 * j + 3]) * inv);
                            v4.z = pack_bf16(__uint_as_float(r[8 * j + 4]) * inv, __uint_as_float(r[8 * j + 5]) * inv);
                            v4.w = pack_bf16(__uint_as_float(r[8 * j + 6]) * inv, __uint_as_float(r[8 * j + 7]) * inv);
                            *reinterpret_cast<uint4 *>(o + 32 * c + 8 * j) = v4;
                        }
                    }
                }
                if (half == 0 && grow < p.L && p.lse2) p.lse2[static_cast<int64_t>(bh) * p.L + grow] = row_m + log2f(den);
            }
        }
        if (!ok) s_err = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (s_err && tid == 0) {
        if (p.status) atomicExch(p.status, 1);
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

template <int D>
static int launch_pair(const VqPrefillArgs *a, cudaStream_t stream)
{
    using C = PairCfg<D>;
    TcMaps m;
    TcParams p;
    const int st = tc_setup<D>(a, m, p);
    if (st != VQ_OK) return st;
    auto kern = prefill_pair_kernel<D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal) != cudaSuccess) return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>((p.ntiles + 1) / 2), static_cast<unsigned>(a->q1.shape[0] * a->q1.shape[1]));
    kern<<<grid, C::kThreads, C::kTotal, stream>>>(m.q1, m.q2, m.k1, m.k3, m.v, m.cb, m.vs, p);
    return launch_status();
}

int launch_prefill_pair(const VqPrefillArgs *a, cudaStream_t stream)
{
    const int D = static_cast<int>(a->q1.shape[3]);
    // 16-byte aligned rows for the output stores and the tensor maps
    if (a->out.stride[2] % 8 || a->out.stride[1] % 8 || a->out.stride[0] % 8) return VQ_EINVAL_STRIDE;
    return D == 64 ? launch_pair<64>(a, stream) : launch_pair<128>(a, stream);
}

}  // namespace vq
