// Decode (seqlen_q == 1) for bf16 caches with dense rows: a persistent, bandwidth-bound stream.
//
// All the rows of the problem - for every (batch, kv head, query-head group): the window rows and
// the far pseudo-key rows - are cut into 64-row tiles and the global tile list is split EVENLY over
// a fixed number of CTAs (two per SM), whatever the number of units: a CTA's range may start and
// end in the middle of a unit.  Inside a CTA
//   warp 8  (one lane) is the producer: for every tile it issues bulk async copies
//           (cp.async.bulk, completion on an mbarrier) of the key-like rows, the value rows, the 64
//           counts of a far tile and - on the first tile of a unit segment - the query rows, into a
//           2-stage shared-memory ring (two CTAs per SM: four tiles in flight per SM), also
//           across unit boundaries, so the HBM stream never drains;
//   warps 0..7 are consumers: a lane group (D/8 lanes) owns one row per step, reads 16-byte slices
//           from shared memory, reduces the dot product with shuffles and folds the row into its
//           running softmax state (an fp32 codebook row, twice as wide, is scored by D/4 lanes in
//           two sub-steps).  When the unit changes they merge lane groups -> warps -> one partial
//           (max, denominator, numerator) per head, written to the workspace; the last CTA to
//           contribute to a unit (atomic ticket) merges its partials into the output row.
// Every mbarrier wait is bounded; a failed wait raises the status word and the CTA leaves.
#include "decode_common.cuh"
#include "tc_ptx.cuh"

namespace vq {

using namespace ptx;

#ifndef VQ_BULK_ROWS
#define VQ_BULK_ROWS 64
#endif
#ifndef VQ_BULK_STAGES
#define VQ_BULK_STAGES 2
#endif
#ifndef VQ_BULK_CTAS_PER_SM
#define VQ_BULK_CTAS_PER_SM 2
#endif
constexpr int kBulkRows = VQ_BULK_ROWS;     // rows per tile
constexpr int kBulkThreads = kDecThreads + 32;

__device__ __forceinline__ void bulk_copy(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void consumer_barrier()  // the 256 consumer threads only
{
    asm volatile("bar.sync 1, 256;" ::: "memory");
}

template <typename TC, int D, int GH>
struct BulkStage {
    static constexpr int kKeyBytes = kBulkRows * D * static_cast<int>(sizeof(TC) > 2 ? sizeof(TC) : 2);  // widest key-like row
    static constexpr int kValBytes = kBulkRows * D * 2;
    static constexpr int kCntBytes = kBulkRows * 4;
    static constexpr int kQBytes = 2 * GH * D * 2;     // q1 rows then q2 rows of the head group, bf16
    static constexpr int kOffVal = kKeyBytes, kOffCnt = kKeyBytes + kValBytes, kOffQ = kOffCnt + kCntBytes;
    static constexpr int kBytes = kOffQ + kQBytes;
    static constexpr int kStages = VQ_BULK_STAGES;                    // two CTAs per SM stay resident (<= ~100 KB each)
};

struct BulkParams {
    DecodeParams d;
    int tiles_w, tiles_f;   // tiles per unit
    int units;              // (batch*kv-head) * head groups
    int num_ctas;
    float *partial;         // [(num_ctas + units)][GH][D+2]
    int *ticket;            // [units]
    int32_t *status;
    long long wait_limit;  // cycles a device-side wait may last before the kernel gives up
};

__device__ __forceinline__ void ld_slice_bf16(const uint8_t *p, float (&x)[8])
{
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    Slice<__nv_bfloat16>::unpack(raw, x);
}

// index of the CTA whose tile range [c*T/NC, (c+1)*T/NC) holds global tile x
__device__ __forceinline__ int owner_of(int64_t x, int64_t T, int NC)
{
    return static_cast<int>(((x + 1) * NC - 1) / T);
}

template <typename TC, int D, int GH>
__global__ void __launch_bounds__(kBulkThreads, VQ_BULK_CTAS_PER_SM) decode_bulk_kernel(BulkParams bp)
{
    using ST = BulkStage<TC, D, GH>;
    const DecodeParams &p = bp.d;
    constexpr int NW = kDecThreads / 32;
    constexpr int LPR = D / 8, GPW = 32 / LPR, NG = NW * GPW;   // bf16 rows
    constexpr bool kCb32 = sizeof(TC) == 4;
    constexpr int kBulkStages = ST::kStages;
    extern __shared__ __align__(128) uint8_t ring[];              // kBulkStages * ST::kBytes
    __shared__ __align__(8) uint64_t full[kBulkStages], empty[kBulkStages];
    __shared__ __align__(16) float s_red[NW * GH * (D + 2)];
    __shared__ int s_last, s_err;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int HG = p.G / GH;
    const int TU = bp.tiles_w + bp.tiles_f;
    const int64_t T = static_cast<int64_t>(bp.units) * TU;
    const int NC = bp.num_ctas, c = blockIdx.x;
    const int64_t g0 = static_cast<int64_t>(c) * T / NC, g1 = static_cast<int64_t>(c + 1) * T / NC;
    // (unit, tile) of the first tile; the loops step them (a 64-bit division per tile would cost more than the tile's arithmetic)
    const int ue_first = static_cast<int>(g0 / TU), tt_first = static_cast<int>(g0 % TU);

    if (tid == 0) {
        for (int s = 0; s < kBulkStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NW);
        }
        fence_mbar_init();
        s_err = 0;
    }
    __syncthreads();

    if (warp == NW) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            bool ok = true;
            int ue = ue_first, tt = tt_first - 1;
            for (int64_t g = g0; g < g1; ++g) {
                const int t = static_cast<int>(g - g0), sidx = t % kBulkStages;
                if (++tt == TU) {
                    tt = 0;
                    ++ue;
                }
                if (t >= kBulkStages && !mbar_wait(&empty[sidx], ((t / kBulkStages) - 1) & 1, bp.wait_limit)) {
                    ok = false;
                    break;
                }
                const int u = ue / HG, hg = ue % HG;
                const int b = u / p.Hkv, hk = u % p.Hkv;
                uint8_t *dst = ring + sidx * ST::kBytes;
                uint32_t bytes = 0;
                const bool seg_start = (g == g0) || (tt == 0);
                if (seg_start) bytes += ST::kQBytes;
                if (tt < bp.tiles_w) {
                    const int r0 = tt * kBulkRows, r1 = min(r0 + kBulkRows, p.n_valid);
                    const int rb = min(max(p.n_bd, r0), r1);  // rows [r0,rb) from k3, [rb,r1) from k1
                    bytes += static_cast<uint32_t>((r1 - r0) * D * 2 * 2);
                    mbar_expect_tx(&full[sidx], bytes);
                    const __nv_bfloat16 *k1w = static_cast<const __nv_bfloat16 *>(p.k1w) + b * p.k_sb + hk * p.k_sh;
                    const __nv_bfloat16 *k3w = static_cast<const __nv_bfloat16 *>(p.k3w) + b * p.k3_sb + hk * p.k3_sh;
                    const __nv_bfloat16 *vw = static_cast<const __nv_bfloat16 *>(p.vw) + b * p.v_sb + hk * p.v_sh;
                    if (rb > r0) bulk_copy(dst, k3w + static_cast<int64_t>(r0) * D, (rb - r0) * D * 2, &full[sidx]);
                    if (r1 > rb) bulk_copy(dst + (rb - r0) * D * 2, k1w + static_cast<int64_t>(rb) * D, (r1 - rb) * D * 2, &full[sidx]);
                    bulk_copy(dst + ST::kOffVal, vw + static_cast<int64_t>(r0) * D, (r1 - r0) * D * 2, &full[sidx]);
                } else {
                    const int r0 = (tt - bp.tiles_w) * kBulkRows, r1 = min(r0 + kBulkRows, p.MK);
                    const uint32_t kb = static_cast<uint32_t>((r1 - r0) * D * sizeof(TC));
                    bytes += kb + (r1 - r0) * D * 2 + (r1 - r0) * 4;
                    mbar_expect_tx(&full[sidx], bytes);
                    const TC *cbk = static_cast<const TC *>(p.codebook) + static_cast<int64_t>(hk) * p.MK * D;
                    const __nv_bfloat16 *vs = static_cast<const __nv_bfloat16 *>(p.vsum) + static_cast<int64_t>(u) * p.MK * D;
                    const float *cn = p.cnt + static_cast<int64_t>(u) * p.MK;
                    bulk_copy(dst, cbk + static_cast<int64_t>(r0) * D, kb, &full[sidx]);
                    bulk_copy(dst + ST::kOffVal, vs + static_cast<int64_t>(r0) * D, (r1 - r0) * D * 2, &full[sidx]);
                    bulk_copy(dst + ST::kOffCnt, cn + r0, (r1 - r0) * 4, &full[sidx]);
                }
                if (seg_start) {
                    const int hq0 = hk * p.G + hg * GH;
                    bulk_copy(dst + ST::kOffQ, static_cast<const __nv_bfloat16 *>(p.q1) + b * p.q_sb + hq0 * p.q_sh, GH * D * 2, &full[sidx]);
                    bulk_copy(dst + ST::kOffQ + GH * D * 2, static_cast<const __nv_bfloat16 *>(p.q2) + b * p.q2_sb + hq0 * p.q2_sh,
                              GH * D * 2, &full[sidx]);
                }
            }
            if (!ok) s_err = 1;
        }
    } else {
        // ------------------------------------------------------------------ consumers
        const int vg = lane / LPR, sub = lane % LPR, gidx = warp * GPW + vg;
        DecState<GH, 8> st;
        st.init();
        float q1r[GH][8], q2r[GH][8];
        float qc[GH][4];  // fp32-codebook rows: this lane's 4 columns of q2 (D/4 lanes per row)
        bool ok = true;
        int cur_ue = -1;

        // write this CTA's partial of unit `ue` and let the last contributor merge the unit
        auto flush = [&](int ue) {
#pragma unroll
            for (int off = LPR; off < 32; off <<= 1) st.merge_xor(off);
            if (lane < LPR) {
#pragma unroll
                for (int g = 0; g < GH; ++g) {
                    float *dst = s_red + (warp * GH + g) * (D + 2);
#pragma unroll
                    for (int e = 0; e < 8; ++e) dst[lane * 8 + e] = st.acc[g][e];
                    if (lane == 0) {
                        dst[D] = st.m[g];
                        dst[D + 1] = st.l[g];
                    }
                }
            }
            consumer_barrier();
            const int first_c = owner_of(static_cast<int64_t>(ue) * TU, T, NC);
            const int last_c = owner_of(static_cast<int64_t>(ue + 1) * TU - 1, T, NC);
            if (first_c == last_c) {
                // the whole unit was processed by this CTA: merge the warps and write the output row directly
                const int u = ue / HG, hg = ue % HG;
                const int b = u / p.Hkv, hk = u % p.Hkv;
                const int hq0 = hk * p.G + hg * GH;
                for (int i = tid; i < GH * D; i += kDecThreads) {
                    const int g = i / D, d = i % D;
                    float M = -INFINITY;
#pragma unroll
                    for (int w = 0; w < NW; ++w) M = fmaxf(M, s_red[(w * GH + g) * (D + 2) + D]);
                    float num = 0.f, den = 0.f;
#pragma unroll
                    for (int w = 0; w < NW; ++w) {
                        const float mw = s_red[(w * GH + g) * (D + 2) + D];
                        const float a = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
                        num += a * s_red[(w * GH + g) * (D + 2) + d];
                        den += a * s_red[(w * GH + g) * (D + 2) + D + 1];
                    }
                    static_cast<__nv_bfloat16 *>(p.out)[b * p.o_sb + (hq0 + g) * p.o_sh + d] = __float2bfloat16_rn(num / den);
                }
                consumer_barrier();  // s_red is reused by the next segment
                return;
            }
            float *part = bp.partial + static_cast<int64_t>(c + ue) * GH * (D + 2);
            for (int i = tid; i < GH * (D + 1); i += kDecThreads) {
                const int g = i / (D + 1), d = i % (D + 1);
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < NW; ++w) M = fmaxf(M, s_red[(w * GH + g) * (D + 2) + D]);
                float x = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    const float mw = s_red[(w * GH + g) * (D + 2) + D];
                    const float a = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
                    x += a * s_red[(w * GH + g) * (D + 2) + (d < D ? d : D + 1)];
                }
                if (d < D) part[g * (D + 2) + d] = x;
                else {
                    part[g * (D + 2) + D] = M;
                    part[g * (D + 2) + D + 1] = x;
                }
            }
            __threadfence();
            consumer_barrier();
            if (tid == 0) {
                const int tk = atomicAdd(bp.ticket + ue, 1);
                s_last = (tk == last_c - first_c);
            }
            consumer_barrier();
            if (s_last) {
                __threadfence();
                const int u = ue / HG, hg = ue % HG;
                const int b = u / p.Hkv, hk = u % p.Hkv;
                const int hq0 = hk * p.G + hg * GH;
                for (int i = tid; i < GH * D; i += kDecThreads) {
                    const int g = i / D, d = i % D;
                    float M = -INFINITY;
                    for (int cc = first_c; cc <= last_c; ++cc)
                        M = fmaxf(M, __ldcg(bp.partial + (static_cast<int64_t>(cc + ue) * GH + g) * (D + 2) + D));
                    float num = 0.f, den = 0.f;
                    for (int cc = first_c; cc <= last_c; ++cc) {
                        const float *pg = bp.partial + (static_cast<int64_t>(cc + ue) * GH + g) * (D + 2);
                        const float ms = __ldcg(pg + D);
                        const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
                        num += w * __ldcg(pg + d);
                        den += w * __ldcg(pg + D + 1);
                    }
                    static_cast<__nv_bfloat16 *>(p.out)[b * p.o_sb + (hq0 + g) * p.o_sh + d] = __float2bfloat16_rn(num / den);
                }
                if (tid == 0) bp.ticket[ue] = 0;  // ready for the next call on this stream
            }
            consumer_barrier();  // s_red and s_last are reused by the next segment
        };

        int ue = ue_first, tt = tt_first - 1;
        for (int64_t g = g0; g < g1; ++g) {
            const int t = static_cast<int>(g - g0), sidx = t % kBulkStages;
            if (++tt == TU) {
                tt = 0;
                ++ue;
            }
            if (ue != cur_ue) {
                if (cur_ue >= 0) flush(cur_ue);
                st.init();
            }
            if (!mbar_wait(&full[sidx], (t / kBulkStages) & 1, bp.wait_limit)) {
                ok = false;
                break;
            }
            const uint8_t *src = ring + sidx * ST::kBytes;
            if (ue != cur_ue) {
                cur_ue = ue;
                const __nv_bfloat16 *qs = reinterpret_cast<const __nv_bfloat16 *>(src + ST::kOffQ);
#pragma unroll
                for (int gq = 0; gq < GH; ++gq) {
                    ld_slice_bf16(reinterpret_cast<const uint8_t *>(qs + gq * D + sub * 8), q1r[gq]);
                    ld_slice_bf16(reinterpret_cast<const uint8_t *>(qs + (GH + gq) * D + sub * 8), q2r[gq]);
                    if constexpr (kCb32) {
                        const int csub_q = lane % (D / 4);
#pragma unroll
                        for (int e = 0; e < 4; ++e) qc[gq][e] = __bfloat162float(qs[(GH + gq) * D + csub_q * 4 + e]);
                    }
                }
            }
            constexpr int RPG = kBulkRows / NG;  // rows of a tile owned by one lane group
            float sc[GH][RPG], wt[RPG], vx[RPG][8];
            if (tt < bp.tiles_w || !kCb32) {
                // bf16 key-like rows (window keys, or a bf16 codebook): D/8 lanes per row
                const bool is_far = tt >= bp.tiles_w;
                const int r0 = (is_far ? tt - bp.tiles_w : tt) * kBulkRows;
                const int r1 = min(r0 + kBulkRows, is_far ? p.MK : p.n_valid);
                const float *cw = reinterpret_cast<const float *>(src + ST::kOffCnt);
                const bool all_q2 = is_far || r1 <= p.n_bd, all_q1 = !is_far && r0 >= p.n_bd;
#pragma unroll
                for (int j = 0; j < RPG; ++j) {
                    const int lr = j * NG + gidx, r = r0 + lr;
                    const bool valid = r < r1;
                    float kx[8];
                    wt[j] = 0.f;
                    if (valid) {
                        ld_slice_bf16(src + lr * D * 2 + sub * 16, kx);
                        ld_slice_bf16(src + ST::kOffVal + lr * D * 2 + sub * 16, vx[j]);
                        wt[j] = is_far ? cw[lr] : 1.f;
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) kx[e] = vx[j][e] = 0.f;
                    }
                    // q2 scores the far rows and the window rows below n_bd; whole tiles are usually one kind
                    if (all_q2 || (!all_q1 && r < p.n_bd)) {
#pragma unroll
                        for (int gq = 0; gq < GH; ++gq) {
                            float a = 0.f;
#pragma unroll
                            for (int e = 0; e < 8; ++e) a = fmaf(q2r[gq][e], kx[e], a);
                            sc[gq][j] = a;
                        }
                    } else {
#pragma unroll
                        for (int gq = 0; gq < GH; ++gq) {
                            float a = 0.f;
#pragma unroll
                            for (int e = 0; e < 8; ++e) a = fmaf(q1r[gq][e], kx[e], a);
                            sc[gq][j] = a;
                        }
                    }
                }
#pragma unroll
                for (int off = LPR / 2; off >= 1; off >>= 1)
#pragma unroll
                    for (int gq = 0; gq < GH; ++gq)
#pragma unroll
                        for (int j = 0; j < RPG; ++j) sc[gq][j] += __shfl_xor_sync(0xffffffffu, sc[gq][j], off);
            } else {
                // fp32 codebook rows: D/4 lanes per row, two sub-steps cover the warp's GPW rows of a step
                constexpr int LPRC = D / 4, GPWC = 32 / LPRC, SUB = GPW / GPWC;
                const int cg = lane / LPRC, csub = lane % LPRC;
                const int r0 = (tt - bp.tiles_w) * kBulkRows, r1 = min(r0 + kBulkRows, p.MK);
                const float *cw = reinterpret_cast<const float *>(src + ST::kOffCnt);
                float part[GH][RPG][SUB];
#pragma unroll
                for (int j = 0; j < RPG; ++j) {
                    const int base = j * NG + warp * GPW;      // first of this warp's GPW rows in step j
                    const int lr = base + vg;
                    const bool valid = r0 + lr < r1;
                    wt[j] = 0.f;
                    if (valid) {
                        ld_slice_bf16(src + ST::kOffVal + lr * D * 2 + sub * 16, vx[j]);
                        wt[j] = cw[lr];
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) vx[j][e] = 0.f;
                    }
#pragma unroll
                    for (int ss = 0; ss < SUB; ++ss) {
                        const int lrc = base + ss * GPWC + cg;
                        float4 c4 = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (r0 + lrc < r1) c4 = *reinterpret_cast<const float4 *>(src + lrc * D * 4 + csub * 16);
#pragma unroll
                        for (int gq = 0; gq < GH; ++gq)
                            part[gq][j][ss] = fmaf(qc[gq][0], c4.x, fmaf(qc[gq][1], c4.y, fmaf(qc[gq][2], c4.z, qc[gq][3] * c4.w)));
                    }
                }
#pragma unroll
                for (int off = LPRC / 2; off >= 1; off >>= 1)
#pragma unroll
                    for (int gq = 0; gq < GH; ++gq)
#pragma unroll
                        for (int j = 0; j < RPG; ++j)
#pragma unroll
                            for (int ss = 0; ss < SUB; ++ss)
                                part[gq][j][ss] += __shfl_xor_sync(0xffffffffu, part[gq][j][ss], off);
                // the score of value group vg was formed in sub-step vg / GPWC by codebook group vg % GPWC
#pragma unroll
                for (int gq = 0; gq < GH; ++gq)
#pragma unroll
                    for (int j = 0; j < RPG; ++j) {
                        float mine = 0.f;
#pragma unroll
                        for (int ss = 0; ss < SUB; ++ss) {
                            const float got = __shfl_sync(0xffffffffu, part[gq][j][ss], (vg % GPWC) * LPRC);
                            if (ss == vg / GPWC) mine = got;
                        }
                        sc[gq][j] = mine;
                    }
            }
            // one softmax update per tile for this lane group
#pragma unroll
            for (int gq = 0; gq < GH; ++gq) {
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < RPG; ++j) {
                    sc[gq][j] = wt[j] > 0.f ? sc[gq][j] * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, sc[gq][j]);
                }
                const float mn = fmaxf(st.m[gq], mx);
                if (mn != -INFINITY) {
                    const float alpha = ex2(st.m[gq] - mn);
                    float l = st.l[gq] * alpha;
#pragma unroll
                    for (int e = 0; e < 8; ++e) st.acc[gq][e] *= alpha;
#pragma unroll
                    for (int j = 0; j < RPG; ++j) {
                        const float pj = ex2(sc[gq][j] - mn);
                        l = fmaf(pj, wt[j], l);
#pragma unroll
                        for (int e = 0; e < 8; ++e) st.acc[gq][e] = fmaf(pj, vx[j][e], st.acc[gq][e]);
                    }
                    st.l[gq] = l;
                    st.m[gq] = mn;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[sidx]);
        }
        if (ok && cur_ue >= 0) flush(cur_ue);
        if (!ok) s_err = 1;
    }
    __syncthreads();
    if (s_err) {
        if (tid == 0 && bp.status) atomicExch(bp.status, VQ_WORD_TIMEOUT);
        // copies still in flight must land before the shared memory is released
        if (tid == 0)
#pragma unroll 1
            for (int w = 0; w < (1 << 14); ++w) __nanosleep(256);
        __syncthreads();
    }
}

static int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

template <typename TC, int D, int GH>
static int launch_bulk_t(BulkParams &bp, cudaStream_t s)
{
    auto kern = decode_bulk_kernel<TC, D, GH>;
    const int smem = BulkStage<TC, D, GH>::kStages * BulkStage<TC, D, GH>::kBytes;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return VQ_ELAUNCH;
    kern<<<bp.num_ctas, kBulkThreads, smem, s>>>(bp);
    return launch_status();
}

size_t decode_bulk_workspace_bytes(int64_t units_times_groups, int64_t heads_per_group, int64_t D)
{
    const size_t tickets = (static_cast<size_t>(units_times_groups) * sizeof(int) + 255) / 256 * 256;
    const size_t slots = 4096 + static_cast<size_t>(units_times_groups);  // (CTAs <= 4096) + units
    return tickets + slots * heads_per_group * (D + 2) * sizeof(float);
}

// bf16 activations, dense rows (row stride == D) for the window buffers and q; codebook fp32 or bf16.
int launch_decode_bulk(const DecodeParams &p, int64_t units, int D, int GH, bool cb32, void *workspace, size_t workspace_bytes,
                       int32_t *status, cudaStream_t s)
{
    BulkParams bp{};
    bp.d = p;
    bp.tiles_w = (p.n_valid + kBulkRows - 1) / kBulkRows;
    bp.tiles_f = p.use_far ? (p.MK + kBulkRows - 1) / kBulkRows : 0;
    const int HG = p.G / GH;
    bp.units = static_cast<int>(units * HG);
    const int64_t T = static_cast<int64_t>(bp.units) * (bp.tiles_w + bp.tiles_f);
    int64_t nc = VQ_BULK_CTAS_PER_SM * static_cast<int64_t>(sm_count());
    if (nc > 4096) nc = 4096;
    if (nc > T) nc = T;
    bp.num_ctas = static_cast<int>(nc);
    if (workspace_bytes < decode_bulk_workspace_bytes(bp.units, GH, D)) return VQ_EWORKSPACE;
    const size_t tickets = (static_cast<size_t>(bp.units) * sizeof(int) + 255) / 256 * 256;
    bp.ticket = static_cast<int *>(workspace);
    bp.partial = reinterpret_cast<float *>(static_cast<char *>(workspace) + tickets);
    bp.status = status;
    bp.wait_limit = wait_limit_cycles();
#define VQ_BULK_G(TC, DD)                                            \
    do {                                                             \
        if (GH == 4) return launch_bulk_t<TC, DD, 4>(bp, s);         \
        if (GH == 2) return launch_bulk_t<TC, DD, 2>(bp, s);         \
        return launch_bulk_t<TC, DD, 1>(bp, s);                      \
    } while (0)
    if (cb32) {
        if (D == 64) VQ_BULK_G(float, 64);
        VQ_BULK_G(float, 128);
    }
    if (D == 64) VQ_BULK_G(__nv_bfloat16, 64);
    VQ_BULK_G(__nv_bfloat16, 128);
#undef VQ_BULK_G
}

}  // namespace vq
