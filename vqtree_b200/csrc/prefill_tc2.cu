// Fused VQ-attention prefill on the sm_100a tensor cores, warp-specialised and pipelined.
//
// One CTA owns one 128-row query tile of one (batch, query head).  Its work items (far codebook
// tiles, boundary block, interior blocks, causal diagonal - see TcWork) are dealt alternately to
// two independent softmax streams, each with its own S/P buffer and O accumulator in tensor
// memory and its own running (max, denominator); the streams are merged once at the end (this is
// the single online softmax that replaces the reference's two kernels and its log-sum-exp merge,
// ops/triton_fused_vq_attn.py:202-250).  Roles:
//   warps 0-7 / 8-15 softmax of stream 0 / 1: TWO threads per query row (64 key columns each) read
//                    S with tcgen05.ld, mask, agree on the row maximum through shared memory,
//                    exponentiate, write P (packed bf16) over S, rescale their half of O only when
//                    the maximum grew by more than 2^8 (lazy rescaling), and do the epilogue;
//   warp 16          one thread issues every tcgen05.mma: S = Q K^T (operands in shared memory),
//                    O += P V (P from tensor memory, V MN-major in shared memory);
//   warp 17          one thread issues the TMA tile loads into a ring of 32 KB slots, in the order
//                    the tensor pipe consumes them (K0 K1 V0 K2 V1 K3 ...).
// While stream 0 runs its softmax the tensor pipe works for stream 1 and vice versa.
// Hand-offs are mbarriers (tcgen05.commit arrives for the MMA side); every wait is bounded and a
// failed wait raises the status word; all roles meet at one final barrier and TMEM is freed.
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr int kT2Threads = 576;   // 16 softmax warps + MMA warp + TMA warp
constexpr int kWarpMma = 16, kWarpTma = 17;
constexpr float kLazyThreshold = 8.f;  // log2 units: P stays below 2^8, exact in fp32, fine in bf16

template <int D>
struct T2Cfg {
    static constexpr int NH = D / 64;
    static constexpr int kTile = NH * kHalfBytes;             // 128 x D bf16
    static constexpr int kSlots = 4;                           // ring of K / V tiles
    static constexpr int kQ1 = 0, kQ2 = kTile, kRing = 2 * kTile;
    static constexpr int kTotal = kRing + kSlots * kTile + 1024;  // + slack for 1024-byte alignment
    // TMEM columns: S0 [0,128) S1 [128,256) (P aliases the first 64 columns of its S), O0, O1
    static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 256 + D;
    static constexpr uint32_t kCols = 512;
};

// Softmax of one work item for one HALF row: this thread owns 64 of the 128 key columns of its
// query row, its partner (same lane, warp + 4) the other 64.  MODE 0: no mask; 1: columns [lo,hi)
// valid (lo/hi relative to this half); 2: far tile - column c valid iff cw[c] > 0, denominator
// weighted by cw[c] (cw already offset to this half).
//   s_addr  this warp's lanes at this half's first S column      p_addr  where its 32 packed P columns go (= s_addr)
//   o_addr  this warp's lanes at this half's first O column (it rescales D/2 columns of O)
//   xch     shared float[2] of this row: partial maxima of the two halves; pub/pub_val: optional
//           extra shared word published before the barrier (the next far tile's count)
// P (32 packed columns per half) is written over the half's own S columns only, so the two
// threads of a row never touch each other's columns; S is read twice (maximum, then exponentials).
template <int D, int MODE>
__device__ __forceinline__ void softmax_half(uint32_t s_addr, uint32_t p_addr, uint32_t o_addr, bool rescale_o,
                                             const float *__restrict__ cw, int lo, int hi, float scale_log2, float &row_m,
                                             float &row_l, float *xch, int hf, int bar_id, float *pub, float pub_val)
{
    // MODE 2 masks by adding nb[c] (0 where the code has members, -inf where it has none)
    const float *nb = cw + 2 * kBlock;
    auto masked2 = [&](float &x0, float &x1, int c0) {
        if (MODE == 2) fadd2(x0, x1, x0, x1, nb[c0], nb[c0 + 1]);
        if (MODE == 1) {
            x0 = (c0 >= lo && c0 < hi) ? x0 : -INFINITY;
            x1 = (c0 + 1 >= lo && c0 + 1 < hi) ? x1 : -INFINITY;
        }
    };
    // pass 1: partial row maximum over this half's 64 columns
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    {
        uint32_t r0[32], r1[32];
        tmem_ld32(s_addr, r0);
        tmem_ld32(s_addr + 32, r1);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float a0 = __uint_as_float(r0[2 * j]), a1 = __uint_as_float(r0[2 * j + 1]);
            float b0 = __uint_as_float(r1[2 * j]), b1 = __uint_as_float(r1[2 * j + 1]);
            masked2(a0, a1, 2 * j);
            masked2(b0, b1, 32 + 2 * j);
            mx4[j & 1] = fmax3(mx4[j & 1], a0, a1);
            mx4[2 + (j & 1)] = fmax3(mx4[2 + (j & 1)], b0, b1);
        }
    }
    xch[hf] = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    if (pub != nullptr) {
        pub[0] = pub_val;
        pub[2 * kBlock] = pub_val > 0.f ? 0.f : -INFINITY;
    }
    asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
    const float mx = fmaxf(xch[0], xch[1]);
    // lazy rescaling: keep the old reference maximum unless the new one is far above it
    const float m_tile = mx * scale_log2;
    float m_use = row_m;
    if (m_tile > row_m + kLazyThreshold || row_m == -INFINITY) m_use = fmaxf(row_m, m_tile);
    const float m_safe = (m_use == -INFINITY) ? 0.f : m_use;
    const float alpha = (m_use == row_m) ? 1.f : ex2(row_m - m_safe);  // row_m = -inf -> 0
    if (rescale_o && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O of this stream is idle here: its last product finished before S was handed over
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
    // pass 2: P = exp2(S*scale - m) as packed bf16 over the first 32 of this half's own 64 columns.
    // Chunk c reads columns [32c, 32c+32) and writes [16c, 16c+16): never ahead of what has been read,
    // and never inside the partner's columns.  Two elements per packed fp32x2 instruction.
    float ls4[4] = {0.f, 0.f, 0.f, 0.f};
    const float neg_m = -m_safe;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint32_t r[32], pk[16];
        tmem_ld32(s_addr + 32 * c, r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int c0 = 32 * c + 2 * j;
            float x0 = __uint_as_float(r[2 * j]), x1 = __uint_as_float(r[2 * j + 1]);
            float t0, t1;
            if (MODE == 2) {
                float b0, b1;
                fadd2(b0, b1, nb[c0], nb[c0 + 1], neg_m, neg_m);
                ffma2(t0, t1, x0, x1, scale_log2, scale_log2, b0, b1);
            } else {
                masked2(x0, x1, c0);
                ffma2(t0, t1, x0, x1, scale_log2, scale_log2, neg_m, neg_m);
            }
            const float p0 = ex2(t0), p1 = ex2(t1);
            if (MODE == 2) ffma2(ls4[2 * (j & 1)], ls4[2 * (j & 1) + 1], p0, p1, cw[c0], cw[c0 + 1], ls4[2 * (j & 1)], ls4[2 * (j & 1) + 1]);
            else fadd2(ls4[2 * (j & 1)], ls4[2 * (j & 1) + 1], ls4[2 * (j & 1)], ls4[2 * (j & 1) + 1], p0, p1);
            pk[j] = pack_bf16(p0, p1);
        }
        tmem_st16(p_addr + 16 * c, pk);
    }
    row_l = row_l * alpha + (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
    row_m = m_use;
}

template <int D>
__global__ void __launch_bounds__(kT2Threads, 1)
prefill_tc2_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                   const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k3,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_cb,
                   const __grid_constant__ CUtensorMap tm_vs, TcParams p)
{
    using C = T2Cfg<D>;
    constexpr int NH = C::NH, NS = C::kSlots;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bar_q, kv_full[NS], kv_empty[NS], s_full[2], p_full[2], o_done[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;
    // counts of a far tile and their mask bias (0 / -inf): [stream][item parity][count | unused | bias | unused][code]
    __shared__ __align__(16) float s_cnt[2][2][4][kBlock];
    __shared__ float s_xch[2][kBlock][2];                // [stream][row][half]: partial row maxima of an item
    __shared__ float s_m[2][kBlock], s_l[2][2][kBlock];  // final (max, partial denominators) per stream / half

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m = p.ntiles - 1 - static_cast<int>(blockIdx.x);  // heavy tiles first
    const int bh = blockIdx.y;
    const int b = bh / p.Hq, hq = bh % p.Hq;
    const int hk = hq / (p.Hq / p.Hkv);
    const int u = b * p.Hkv + hk;
    const TcWork work(p, m);
    const int n = work.n_items;

    if (tid == 0) {
        mbar_init(&bar_q, 1);
        for (int i = 0; i < NS; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 256);
            mbar_init(&o_done[i], 1);
        }
        fence_mbar_init();
        s_err = 0;
    }
    if (warp == kWarpTma) {
        __syncwarp();
        tmem_alloc(&s_tmem, C::kCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp == kWarpTma) {
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
            int q = 0;  // position in the consumption sequence K0 K1 V0 K2 V1 ...
            auto load = [&](int it, bool is_v) {
                if (!ok) return;
                const int slot = q % NS;
                if (q >= NS && !mbar_wait(&kv_empty[slot], ((q / NS) - 1) & 1)) {
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
                ++q;
            };
            load(0, false);
            if (n > 1) load(1, false);
            for (int j = 0; j < n; ++j) {
                load(j, true);
                if (j + 2 < n) load(j + 2, false);
            }
            if (!ok) s_err = 1;
        }
    } else if (warp == kWarpMma) {
        // ================================================================== MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(128, D, 0, 1);
            // operand descriptors differ only in their 16-byte-granular start address: the bases are built
            // once, every MMA adds a compile-time offset (the issuing thread is a serial resource)
            const uint64_t d_q1 = smem_desc_sw128(smem_u32(smem + C::kQ1), 16, 1024);
            const uint64_t d_q2 = p.rerope ? smem_desc_sw128(smem_u32(smem + C::kQ2), 16, 1024) : d_q1;
            const uint64_t d_k0 = smem_desc_sw128(smem_u32(smem + C::kRing), 16, 1024);          // K tiles: K-major
            const uint64_t d_v0 = smem_desc_sw128(smem_u32(smem + C::kRing), kHalfBytes, 1024);  // V tiles: MN-major
            bool ok = mbar_wait(&bar_q, 0);
            int q = 0;
            auto qk = [&](int it) {
                if (!ok) return;
                const int slot = q % NS, s = it & 1;
                if (!mbar_wait(&kv_full[slot], (q / NS) & 1)) {
                    ok = false;
                    return;
                }
                tc_fence_after();
                const int kind = work.kind(it);
                const uint64_t da = (kind == kFar || kind == kBdA) ? d_q2 : d_q1;
                const uint64_t db = d_k0 + static_cast<uint64_t>((slot * C::kTile) >> 4);
                const uint32_t sdst = tmem + (s ? C::kColS1 : C::kColS0);
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const uint64_t off = static_cast<uint64_t>((h * kHalfBytes + k4 * 32) >> 4);
                        mma_ss(sdst, da + off, db + off, idesc_qk, (h | k4) ? 1u : 0u);
                    }
                tc_commit(&kv_empty[slot]);  // K tile free once these MMAs have read it
                tc_commit(&s_full[s]);       // S ready for the softmax warps of stream s
                ++q;
            };
            auto pv = [&](int it) {
                if (!ok) return;
                const int slot = q % NS, s = it & 1;
                if (!mbar_wait(&p_full[s], (it >> 1) & 1) || !mbar_wait(&kv_full[slot], (q / NS) & 1)) {
                    ok = false;
                    return;
                }
                tc_fence_after();
                const uint64_t dv = d_v0 + static_cast<uint64_t>((slot * C::kTile) >> 4);
                const uint32_t odst = tmem + (s ? C::kColO1 : C::kColO0);
                const uint32_t psrc = tmem + (s ? C::kColS1 : C::kColS0);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    mma_ts(odst, psrc + (kk < 4 ? 8 * kk : 64 + 8 * (kk - 4)),  // keys 0-63 at columns 0.., keys 64-127 at columns 64..
                           dv + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv, ((it >> 1) | kk) ? 1u : 0u);
                tc_commit(&kv_empty[slot]);
                if (it + 2 >= n) tc_commit(&o_done[s]);  // last product of this stream
                ++q;
            };
            qk(0);
            if (n > 1) qk(1);
            for (int j = 0; j < n; ++j) {
                pv(j);
                if (j + 2 < n) qk(j + 2);
            }
            if (!ok) s_err = 1;
        }
    } else {
        // ================================================================== softmax streams
        const int s = warp >> 3;                       // stream 0 / 1
        const int hf = (warp >> 2) & 1;                // which 64 key columns of the row
        const int row = (warp & 3) * 32 + lane;        // query row inside the tile (= TMEM lane)
        const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t col_s = s ? C::kColS1 : C::kColS0, col_o = s ? C::kColO1 : C::kColO0;
        const uint32_t s_addr = tmem + lane_off + col_s + 64 * hf, p_addr = s_addr;  // P of a half goes over that half's own S columns
        const uint32_t o_addr = tmem + lane_off + col_o + hf * (D / 2);
        const int bar_id = 2 + s;
        float row_m = -INFINITY, row_l = 0.f;          // row_m: the maximum P is currently scaled by
        bool ok = true;
        // Counts of far tiles (items 0..n_far-1) reach the stream through shared memory: the hf == 0
        // thread of row r fetches count r of the tile two items ahead and publishes it before the
        // item's barrier; the first tile's counts are published up front.
        const float *cnt_base = p.cnt + (static_cast<int64_t>(u) * p.NB + work.far_blk) * p.MK;
        if (s < work.n_far) {
            if (hf == 0) {
                const float c0v = __ldg(cnt_base + s * kBlock + row);
                s_cnt[s][0][0][row] = c0v;
                s_cnt[s][0][2][row] = c0v > 0.f ? 0.f : -INFINITY;
            }
            asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
        }
        for (int it = s; it < n && ok; it += 2) {
            const int kind = work.kind(it);
            const int par = (it >> 1) & 1;
            float cnt_next = 0.f;
            float *pub = nullptr;
            if (hf == 0 && it + 2 < work.n_far) {
                cnt_next = __ldg(cnt_base + (it + 2) * kBlock + row);
                pub = &s_cnt[s][par ^ 1][0][row];
            }
            if (!mbar_wait(&s_full[s], par)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const float *cw = &s_cnt[s][par][0][64 * hf];
            // valid key columns of this row, relative to this half: [lo, hi)
            int lo = 0, hi = 64;
            if (kind == kDiag) hi = row + 1 - 64 * hf;
            else if (kind == kBdA) hi = row - 64 * hf;
            else if (kind == kBdB) lo = row - 64 * hf;
            float *xch = &s_xch[s][row][0];
            if (kind == kFar) softmax_half<D, 2>(s_addr, p_addr, o_addr, it >= 2, cw, lo, hi, p.scale_log2, row_m, row_l, xch, hf, bar_id, pub, cnt_next);
            else if (kind == kFull) softmax_half<D, 0>(s_addr, p_addr, o_addr, it >= 2, cw, lo, hi, p.scale_log2, row_m, row_l, xch, hf, bar_id, pub, cnt_next);
            else softmax_half<D, 1>(s_addr, p_addr, o_addr, it >= 2, cw, lo, hi, p.scale_log2, row_m, row_l, xch, hf, bar_id, pub, cnt_next);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(&p_full[s]);
        }
        // ---- epilogue: merge the two streams ----
        const int my_items = (n - s + 1) / 2;
        if (ok && my_items > 0 && !mbar_wait(&o_done[s], 0)) ok = false;
        tc_fence_after();
        if (hf == 0) s_m[s][row] = row_m;
        s_l[s][hf][row] = (ok && my_items > 0) ? row_l : 0.f;
        if (!ok) s_err = 1;
        asm volatile("bar.sync 1, 512;" ::: "memory");   // the 512 softmax threads
        tc_fence_after();
        if (!s_err) {
            const float m0 = s_m[0][row], l0 = s_l[0][0][row] + s_l[0][1][row];
            const float m1 = s_m[1][row], l1 = s_l[1][0][row] + s_l[1][1][row];
            const float mm = fmaxf(l0 > 0.f ? m0 : -INFINITY, l1 > 0.f ? m1 : -INFINITY);
            const float e0 = l0 > 0.f ? ex2(m0 - mm) : 0.f, e1 = l1 > 0.f ? ex2(m1 - mm) : 0.f;
            const float den = l0 * e0 + l1 * e1;
            const float f0 = e0 / den, f1 = e1 / den;
            const int64_t grow = static_cast<int64_t>(m) * kBlock + row;
            __nv_bfloat16 *o = p.out + b * p.o_sb + hq * p.o_sh + grow * p.o_sl;
            // thread (stream s, half hf) writes the column quarter [(2s+hf)*D/4, +D/4) of its row
            constexpr int QC = D / 4;
            const int col = (2 * s + hf) * QC;
            uint32_t r0[QC], r1[QC];
            __syncwarp();
            if constexpr (QC == 32) {
                tmem_ld32(tmem + lane_off + C::kColO0 + col, r0);
                tmem_ld32(tmem + lane_off + C::kColO1 + col, r1);
            } else {
                tmem_ld16(tmem + lane_off + C::kColO0 + col, r0);
                tmem_ld16(tmem + lane_off + C::kColO1 + col, r1);
            }
            tc_wait_ld();
            if (grow < p.L) {
#pragma unroll
                for (int j = 0; j < QC / 8; ++j) {
                    float x[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float a0 = l0 > 0.f ? __uint_as_float(r0[8 * j + e]) * f0 : 0.f;
                        const float a1 = l1 > 0.f ? __uint_as_float(r1[8 * j + e]) * f1 : 0.f;
                        x[e] = a0 + a1;
                    }
                    uint4 w;
                    w.x = pack_bf16(x[0], x[1]);
                    w.y = pack_bf16(x[2], x[3]);
                    w.z = pack_bf16(x[4], x[5]);
                    w.w = pack_bf16(x[6], x[7]);
                    *reinterpret_cast<uint4 *>(o + col + 8 * j) = w;
                }
            }
            if (s == 0 && hf == 0 && p.lse2 && grow < p.L) p.lse2[static_cast<int64_t>(bh) * p.L + grow] = mm + log2f(den);
        }
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
    if (warp == kWarpTma) {
        __syncwarp();
        tmem_dealloc(tmem, C::kCols);
    }
}

template <int D>
static int launch_tc2(const VqPrefillArgs *a, cudaStream_t stream)
{
    using C = T2Cfg<D>;
    TcMaps m;
    TcParams p;
    const int st = tc_setup<D>(a, m, p);
    if (st != VQ_OK) return st;
    auto kern = prefill_tc2_kernel<D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal) != cudaSuccess) return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>(p.ntiles), static_cast<unsigned>(a->q1.shape[0] * a->q1.shape[1]));
    kern<<<grid, kT2Threads, C::kTotal, stream>>>(m.q1, m.q2, m.k1, m.k3, m.v, m.cb, m.vs, p);
    return launch_status();
}

int launch_prefill_tensor(const VqPrefillArgs *a, cudaStream_t stream)
{
    const int D = static_cast<int>(a->q1.shape[3]);
    // 16-byte aligned rows for the output stores and the tensor maps
    if (a->out.stride[2] % 8 || a->out.stride[1] % 8 || a->out.stride[0] % 8) return VQ_EINVAL_STRIDE;
    return D == 64 ? launch_tc2<64>(a, stream) : launch_tc2<128>(a, stream);
}

}  // namespace vq
