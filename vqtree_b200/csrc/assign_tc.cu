// Key -> code assignment with the score matrix on the tensor cores, still bit-exact.
//
// Replaces ops/mini_vq.py:4-18 of the reference (and its greedy-residual extension to M codebooks)
// for bf16 keys.  The defining arithmetic is unchanged: the code of a key in codebook m is the first
// arg-max over c of the fp32 fused-multiply-add chain  sum_d r_m[d] * C_m[c][d] (+ bias),
// r_0 = k, r_{m+1} = r_m - C_m[code] (fp32 subtraction).  What changes is how the arg-max is found:
//   1. APPROXIMATE scores of a 128-key tile against all K codewords come from tcgen05.mma.  The
//      fp32 codebook is split into two bf16 terms, C = Ch + Cl + eC with |eC| <= 2^-18 |C|.  The
//      residual is carried as two bf16 terms as well, rho_m = Rh + Rl (rho_0 = k exactly, Rl = 0);
//      after the code of codebook m is known, t = (Rh + Rl) - C_m[code] in fp32 is re-split.  The
//      tensor cores form  s~ = Rh.Ch + Rl.Ch + Rh.Cl  with fp32 accumulation.
//   2. Error of s~ against the defining chain, in units of |r| |C| (|r|: the norm of the residual,
//      bounded from the residual itself, which the thread has in hand when it re-splits it; a priori
//      |r| <= |k| + sum of the largest codeword norms of the codebooks before m):
//      split of C and dropped Rl.Cl: 2 * 2^-18;
//      re-splits of the residual: m * (2^-18 + 3 * 2^-24);  the fp32 chain itself: D * 2^-24 <= 2^-17;
//      tensor-core accumulation of 3 D (codebook 0: 2 D) exact products, each addition truncated to fp32:
//      3 D * 2^-23 <= 12 * 2^-18;  index tag in the low five mantissa bits (see tag_score): 2^-18.
//      Sum for D = 128: 13 units of 2^-18 for codebook 0, 17 + 1.05 m for codebook m; the kernel uses
//      eps_m = (4 + D/64 + (2 or 3) D/32 + 1.1 m) 2^-18, one unit above that.
//      A key whose best approximate score leads the runner-up by more than thr = 2 eps |r| max|C_m|
//      has a unique arg-max: that code is final.
//   3. The other keys (a few per cent for random data) are settled exactly on the spot: every
//      (key, candidate code within thr of the best) pair of a warp gets a lane, which runs the
//      defining fp32 chain from global memory; first maximum wins.
// One CTA owns NS key tiles of 128 keys ("streams", NS = 2 when K <= 256): per stream four warps
// with one key per thread scan the scores in tensor memory; one warp issues the MMAs of the
// streams in turn, so the scan of one stream overlaps the MMAs of the other; one warp issues the
// TMA loads of the codebook terms (16 KB units, 6-slot ring).  Every wait is bounded.
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr int kAtMinChunk = 128;   // codewords per MMA chunk: 128, or 256 (one N = 256 instruction) when K allows
constexpr int kAtMaxM = 8;
constexpr int kAtMaxK = 512;
constexpr int kAtPairCap = 32;     // (key, candidate) pairs re-scored per pass of a warp
constexpr int kAtLanesPerPair = 8;  // ... eight lanes per pair when there are at most four

// ------------------------------------------------------------------------------------------------
// fp32 codebook -> bf16 hi / lo terms [Hkv, M*K, D] and the largest row norm of every codebook.
__global__ void __launch_bounds__(256)
split_codebook_kernel(const float *__restrict__ cb, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo,
                      float *__restrict__ cmax, int K, int D)
{
    __shared__ float s_max[8];
    const int hm = blockIdx.x;  // h * M + m
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float wmax = 0.f;
    for (int c = warp; c < K; c += 8) {
        const int64_t row = static_cast<int64_t>(hm) * K + c;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float x = cb[row * D + d];
            const __nv_bfloat16 h = __float2bfloat16_rn(x);
            const __nv_bfloat16 l = __float2bfloat16_rn(x - __bfloat162float(h));
            hi[row * D + d] = h;
            lo[row * D + d] = l;
            ss = fmaf(x, x, ss);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        wmax = fmaxf(wmax, sqrtf(ss));
    }
    if (lane == 0) s_max[warp] = wmax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.f;
        for (int w = 0; w < 8; ++w) m = fmaxf(m, s_max[w]);
        cmax[hm] = m * 1.0001f;  // sqrt / summation rounding
    }
}

struct AtParams {
    const __nv_bfloat16 *k;
    int64_t k_sb, k_sh, k_sl;
    const float *cb;     // [Hkv, M, K, D]
    const float *bias;   // nullptr or [Hkv, M, K]
    const float *cmax;   // [Hkv, M]
    void *codes;
    int code_dtype;
    int64_t c_sb, c_sh, c_sl;
    int Hkv, M, K, ntiles;
    int64_t L;
    int32_t *status;
    long long wait_limit;  // cycles a device-side wait may last before the kernel gives up
};

template <int D, int NS, int CH>
struct AtCfg {
    static constexpr int NH = D / 64;
    static constexpr int kATile = NH * kHalfBytes;     // 128 keys x D bf16 (one term of the residual)
    static constexpr int kUnit = CH * 64 * 2;          // CH codewords x 64 columns of one term: one ring slot
    static constexpr int kSlots = 96 * 1024 / kUnit;   // 96 KB of ring
    static constexpr int kB = NS * 2 * kATile;         // per stream: Rh then Rl
    static constexpr int kTotal = kB + kSlots * kUnit + 1024;
    static constexpr int kRegion = NS == 2 ? 256 : 512;  // score columns of a stream in tensor memory
    static constexpr int kMaxChunks = kRegion / CH;
    static constexpr int kGroupsPerChunk = CH / 32;
    static constexpr int kMaxGroups = kRegion / 32;
    static constexpr int kWarpMma = 4 * NS, kWarpTma = 4 * NS + 1;
    static constexpr int kThreads = (4 * NS + 2) * 32;
};

// Largest (hi) and second largest (lo) of 32 values: pairs, then merges of (hi, lo) pairs.
__device__ __forceinline__ void top2_32(const float (&v)[32], float &hi, float &lo)
{
    float h[16], l[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        h[i] = fmaxf(v[2 * i], v[2 * i + 1]);
        l[i] = fminf(v[2 * i], v[2 * i + 1]);
    }
#pragma unroll
    for (int n = 8; n >= 1; n >>= 1)
#pragma unroll
        for (int i = 0; i < n; ++i) {
            const float a = h[2 * i], b = h[2 * i + 1];
            l[i] = fmax3(fminf(a, b), l[2 * i], l[2 * i + 1]);
            h[i] = fmaxf(a, b);
        }
    hi = h[0];
    lo = l[0];
}

// A score with its low five mantissa bits replaced by 31 - i (i: index inside a group of 32 codes):
// the maximum of such values carries the index of a maximal element; the values move by < 2^-18 |v|.
__device__ __forceinline__ float tag_score(float v, int i)
{
    return __uint_as_float((__float_as_uint(v) & 0xffffffe0u) | static_cast<uint32_t>(31 - i));
}

// 32 score columns of this thread's key as floats (+ bias of their codes)
__device__ __forceinline__ void load_scores(uint32_t taddr, const float *bm, int c0, float (&v)[32])
{
    uint32_t r[32];
    tmem_ld32(taddr, r);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = __uint_as_float(r[i]);
        if (bm) v[i] += __ldg(bm + c0 + i);
    }
}

template <int D, int NS, int CH>
__global__ void __launch_bounds__(AtCfg<D, NS, CH>::kThreads, 1)
assign_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_hi,
                 const __grid_constant__ CUtensorMap tm_lo, AtParams p)
{
    using C = AtCfg<D, NS, CH>;
    constexpr int NH = C::NH, SL = C::kSlots;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bar_k[NS], bar_q[NS], bar_c[NS][C::kMaxChunks], b_full[SL], b_free[SL];
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;
    __shared__ uint16_t s_pairs[4 * NS][kAtPairCap];  // per scan warp: (owner lane << 9) | candidate code

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int u = blockIdx.y, b = u / p.Hkv, h = u % p.Hkv;
    const int M = p.M, K = p.K, MK = M * K;
    const int chunks = K / CH;
    const int tile0 = static_cast<int>(blockIdx.x) * NS;
    const int n_act = min(NS, p.ntiles - tile0);       // streams with a tile

    if (tid == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&bar_k[i], 1);
            mbar_init(&bar_q[i], 128);
            for (int c = 0; c < C::kMaxChunks; ++c) mbar_init(&bar_c[i][c], 1);
        }
        for (int i = 0; i < SL; ++i) {
            mbar_init(&b_full[i], 1);
            mbar_init(&b_free[i], 1);
        }
        fence_mbar_init();
        s_err = 0;
    }
    if (warp == C::kWarpMma) {
        __syncwarp();
        tmem_alloc(&s_tmem, 512u);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp == C::kWarpTma) {
        // ============================================================ TMA producer
        if (lane == 0) {
            prefetch_tmap(&tm_k); prefetch_tmap(&tm_hi); prefetch_tmap(&tm_lo);
            for (int s = 0; s < n_act; ++s) {
                mbar_expect_tx(&bar_k[s], C::kATile);
#pragma unroll
                for (int hh = 0; hh < NH; ++hh)
                    tma_load_4d(smem + s * 2 * C::kATile + hh * kHalfBytes, &tm_k, &bar_k[s], 64 * hh, (tile0 + s) * kBlock, h, b);
            }
            // Units in the order the MMA warp consumes them: jobs (codebook m, stream s) with s fastest;
            // inside a job, per chunk: hi term columns 0-63, 64-127 (D = 128), then the lo term likewise.
            // (nested counters instead of divisions of a flat index: this thread's instructions are serial)
            bool ok = true;
            int g = 0;
            for (int m = 0; m < M && ok; ++m)
                for (int s = 0; s < n_act && ok; ++s)
                    for (int ch = 0; ch < chunks && ok; ++ch)
#pragma unroll
                        for (int rem = 0; rem < 2 * NH; ++rem, ++g) {
                            const int slot = g % SL, is_lo = rem / NH, hh = rem % NH;
                            if (g >= SL && !mbar_wait(&b_free[slot], ((g / SL) - 1) & 1, p.wait_limit)) {
                                ok = false;
                                break;
                            }
                            const int row = h * MK + m * K + ch * CH;  // row in [Hkv*M*K, D]
                            mbar_expect_tx(&b_full[slot], C::kUnit);
                            tma_load_3d(smem + C::kB + slot * C::kUnit, is_lo ? &tm_lo : &tm_hi, &b_full[slot], 64 * hh, row, 0);
                        }
            if (!ok) s_err = 1;
        }
    } else if (warp == C::kWarpMma) {
        // ============================================================ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(128, CH, 0, 0, 0);
            // descriptors differ only in their 16-byte-granular start address: build the bases once
            const uint64_t d_a0 = smem_desc_sw128(smem_u32(smem), 16, 1024);
            const uint64_t d_b0 = smem_desc_sw128(smem_u32(smem + C::kB), 16, 1024);
            bool ok = true;
            int g = 0;
            for (int m = 0; m < M && ok; ++m)
                for (int s = 0; s < n_act && ok; ++s) {
                    // the residual terms of (s, m): the key tile itself for m = 0, else written by the scan threads
                    if (!(m == 0 ? mbar_wait(&bar_k[s], 0, p.wait_limit) : mbar_wait(&bar_q[s], (m - 1) & 1, p.wait_limit))) {
                        ok = false;
                        break;
                    }
                    for (int ch = 0; ch < chunks && ok; ++ch) {
                        const uint32_t dcol = tmem + s * C::kRegion + ch * CH;
#pragma unroll
                        for (int rem = 0; rem < 2 * NH; ++rem, ++g) {
                            const int slot = g % SL, is_lo = rem / NH, hh = rem % NH;
                            if (!mbar_wait(&b_full[slot], (g / SL) & 1, p.wait_limit)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            const uint64_t d_b = d_b0 + static_cast<uint64_t>((slot * C::kUnit) >> 4);
                            const uint64_t d_rh = d_a0 + static_cast<uint64_t>((s * 2 * C::kATile + hh * kHalfBytes) >> 4);
                            const uint64_t d_rl = d_rh + static_cast<uint64_t>(C::kATile >> 4);
#pragma unroll
                            for (int k4 = 0; k4 < 4; ++k4)
                                mma_ss(dcol, d_rh + static_cast<uint64_t>((k4 * 32) >> 4), d_b + static_cast<uint64_t>((k4 * 32) >> 4), idesc,
                                       (rem | k4) ? 1u : 0u);
                            if (!is_lo && m > 0) {
#pragma unroll
                                for (int k4 = 0; k4 < 4; ++k4)
                                    mma_ss(dcol, d_rl + static_cast<uint64_t>((k4 * 32) >> 4), d_b + static_cast<uint64_t>((k4 * 32) >> 4), idesc, 1u);
                            }
                            tc_commit(&b_free[slot]);
                            if (rem == 2 * NH - 1) tc_commit(&bar_c[s][ch]);  // this chunk's score columns are complete
                        }
                    }
                }
            if (!ok) s_err = 1;
        }
    } else if ((warp >> 2) < n_act) {
        // ============================================================ scan warps: one key per thread
        // Loops are kept rolled on purpose: the warps of the two streams run different phases of this
        // code at the same time, and it has to stay inside the instruction cache.
        constexpr unsigned kAll = 0xffffffffu;
        const int s = warp >> 2, wq = warp & 3;
        const int row = wq * 32 + lane;
        const int64_t j0 = static_cast<int64_t>(tile0 + s) * kBlock;
        const int64_t j = j0 + row;
        const bool valid = j < p.L;
        const uint32_t tbase = tmem + (static_cast<uint32_t>(wq * 32) << 16) + s * C::kRegion;
        const __nv_bfloat16 *kbase = p.k + b * p.k_sb + h * p.k_sh;
        const __nv_bfloat16 *krow = kbase + (valid ? j : 0) * p.k_sl;
        const float *cbh = p.cb + static_cast<int64_t>(h) * MK * D;
        uint8_t *a_rh = smem + s * 2 * C::kATile, *a_rl = a_rh + C::kATile;
        const int groups = K / 32;
        float rbound;  // |k| + sum of the largest codeword norms so far: a priori bound of the residual's norm
        float rnow;    // bound of the current residual's norm from the residual itself (tighter)
        {
            float ss = 0.f;
#pragma unroll 4
            for (int d = 0; d < D; d += 8) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(krow + d);
                const __nv_bfloat162 *hp = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float x = __low2float(hp[i]), y = __high2float(hp[i]);
                    ss = fmaf(x, x, fmaf(y, y, ss));
                }
            }
            rbound = sqrtf(ss) * 1.0001f;
            rnow = rbound;
        }
        bool ok = true;
        int prev[kAtMaxM];
#pragma unroll
        for (int mm = 0; mm < kAtMaxM; ++mm) prev[mm] = 0;
        for (int m = 0; m < M && ok; ++m) {
            const float cm = p.cmax[h * M + m];
            // eps of this codebook in units of 2^-18: the terms listed at the top of the file plus one unit of slack
            const float eps_m = (4.f + D / 64 + (m > 0 ? 3 : 2) * (D / 32) + 1.1f * m) * 3.814697265625e-6f;
            const float thr0 = 2.f * eps_m * rnow * cm + 1e-30f;
            const float *bm = p.bias ? p.bias + (static_cast<int64_t>(h) * M + m) * K : nullptr;
            // ---- scan, chunk by chunk as the tensor pipe finishes them: best and runner-up of the tagged
            // scores (the tag of the best gives its index inside its group of 32).  gbits marks the groups
            // whose maximum was within the threshold of the running best: a superset of the groups that
            // can hold a candidate at the end.
            float best = -INFINITY, second = -INFINITY;
            int bgrp = 0;
            uint32_t gbits = 0;
#pragma unroll 1
            for (int g = 0; g < groups && ok; ++g) {
                if (g % C::kGroupsPerChunk == 0) {
                    ok = __all_sync(kAll, mbar_wait(&bar_c[s][g / C::kGroupsPerChunk], m & 1, p.wait_limit));
                    tc_fence_after();
                    if (!ok) break;
                }
                float v[32];
                load_scores(tbase + 32 * g, bm, 32 * g, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = tag_score(v[i], i);
                float hi, lo;
                top2_32(v, hi, lo);
                second = fmax3(second, fminf(best, hi), lo);
                bgrp = hi > best ? g : bgrp;
                best = fmaxf(best, hi);
                // with a bias the fp32 additions s + bias round by up to 2^-24 |s + bias| each
                const float thr_g = bm ? thr0 + fabsf(best) * 4.76837158203125e-7f : thr0;
                gbits |= (hi >= best - thr_g ? 1u : 0u) << g;
            }
            if (!ok) break;
            int code = bgrp * 32 + 31 - static_cast<int>(__float_as_uint(best) & 31u);  // first group holding the maximum
            const float thr = bm ? thr0 + fabsf(best) * 4.76837158203125e-7f : thr0;
            const bool flagged = valid && !(best - second > thr);
            if (__ballot_sync(kAll, flagged)) {
                // ---- exact settlement of the warp's doubtful keys: every (key, candidate code) pair gets a
                // lane; pairs are collected in a list and re-scored whenever it is full, and at the end
                const float cut = best - thr;
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                uint16_t *list = s_pairs[warp];
                int n = 0;  // pairs in the list (same in all lanes)
#pragma unroll 1
                for (int g = 0; g <= groups; ++g) {
                    const bool flush = g == groups;
                    uint32_t bits = 0;  // this thread's candidates inside group g
                    if (!flush) {
                        const bool cg = flagged && ((gbits >> g) & 1u);
                        if (!__ballot_sync(kAll, cg)) continue;
                        float v[32];
                        load_scores(tbase + 32 * g, bm, 32 * g, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (v[i] >= cut) bits |= 1u << i;
                        bits = cg ? bits : 0u;
                    }
                    for (;;) {
                        const int cnt = __popc(bits);
                        int incl = cnt;
#pragma unroll
                        for (int off = 1; off < 32; off <<= 1) {
                            const int t = __shfl_up_sync(kAll, incl, off);
                            if (lane >= off) incl += t;
                        }
                        const int total = __shfl_sync(kAll, incl, 31);
                        if (total == 0 && !(flush && n > 0)) break;
                        int q = n + incl - cnt;
                        while (bits != 0 && q < kAtPairCap) {
                            const int bit = __ffs(bits) - 1;
                            list[q++] = static_cast<uint16_t>((lane << 9) | (g * 32 + bit));
                            bits &= bits - 1;
                        }
                        n = min(kAtPairCap, n + total);
                        if (n < kAtPairCap && !flush) break;  // room left: collect from the next group first
                        __syncwarp();
                        // A few pairs (the usual case): eight lanes per pair, each loads one eighth of the rows (all
                        // loads in flight at once) and the FMA chain walks from lane to lane in d order.  Many pairs:
                        // one lane per pair.
                        const bool few = n <= 32 / kAtLanesPerPair;
                        const int slot = few ? lane / kAtLanesPerPair : lane;   // pair of this lane
                        const bool act = slot < n;
                        int owner = lane, c = 0;
                        if (act) {
                            const int e = list[slot];
                            owner = e >> 9;
                            c = e & 511;
                        }
                        int pv[kAtMaxM];
#pragma unroll
                        for (int mm = 0; mm < kAtMaxM; ++mm) pv[mm] = (mm < m) ? __shfl_sync(kAll, prev[mm], owner) : 0;
                        float sc = -INFINITY;
                        // the defining chain: r_m = ((k - C_0[c_0]) - C_1[c_1]) - ..., one FMA chain over d
                        const __nv_bfloat16 *ks = kbase + (j0 + wq * 32 + owner) * p.k_sl;
                        const float *cc = cbh + (static_cast<int64_t>(m) * K + c) * D;
                        auto residual4 = [&](int d) {
                            const uint2 raw = *reinterpret_cast<const uint2 *>(ks + d);
                            const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x);
                            const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
                            float4 r4 = make_float4(__low2float(lo2), __high2float(lo2), __low2float(hi2), __high2float(hi2));
#pragma unroll
                            for (int mm = 0; mm < kAtMaxM; ++mm)
                                if (mm < m) {
                                    const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cbh + (static_cast<int64_t>(mm) * K + pv[mm]) * D + d));
                                    r4.x = __fsub_rn(r4.x, c4.x);
                                    r4.y = __fsub_rn(r4.y, c4.y);
                                    r4.z = __fsub_rn(r4.z, c4.z);
                                    r4.w = __fsub_rn(r4.w, c4.w);
                                }
                            return r4;
                        };
                        if (few) {
                            constexpr int SEG = D / kAtLanesPerPair, STEPS = SEG / 4;  // columns / float4 steps of a lane
                            const int q = lane % kAtLanesPerPair;
                            float4 r4[STEPS], c4[STEPS];
                            if (act) {
#pragma unroll
                                for (int st = 0; st < STEPS; ++st) {
                                    r4[st] = residual4(SEG * q + 4 * st);
                                    c4[st] = __ldg(reinterpret_cast<const float4 *>(cc + SEG * q + 4 * st));
                                }
                            } else {
#pragma unroll
                                for (int st = 0; st < STEPS; ++st) r4[st] = c4[st] = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                            float acc = 0.f;
#pragma unroll 1
                            for (int seg = 0; seg < kAtLanesPerPair; ++seg) {
                                if (q == seg) {
#pragma unroll
                                    for (int st = 0; st < STEPS; ++st) {
                                        acc = __fmaf_rn(r4[st].x, c4[st].x, acc);
                                        acc = __fmaf_rn(r4[st].y, c4[st].y, acc);
                                        acc = __fmaf_rn(r4[st].z, c4[st].z, acc);
                                        acc = __fmaf_rn(r4[st].w, c4[st].w, acc);
                                    }
                                }
                                acc = __shfl_sync(kAll, acc, (lane & ~(kAtLanesPerPair - 1)) | seg);
                            }
                            if (act) sc = bm ? __fadd_rn(acc, __ldg(bm + c)) : acc;
                        } else if (act) {
                            float acc = 0.f;
#pragma unroll 8
                            for (int d = 0; d < D; d += 4) {
                                const float4 r4 = residual4(d);
                                const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cc + d));
                                acc = __fmaf_rn(r4.x, c4.x, acc);
                                acc = __fmaf_rn(r4.y, c4.y, acc);
                                acc = __fmaf_rn(r4.z, c4.z, acc);
                                acc = __fmaf_rn(r4.w, c4.w, acc);
                            }
                            sc = bm ? __fadd_rn(acc, __ldg(bm + c)) : acc;
                        }
                        __syncwarp();
                        const int stride = few ? kAtLanesPerPair : 1;
#pragma unroll 1
                        for (int t = 0; t < n; ++t) {
                            const int ot = __shfl_sync(kAll, owner, t * stride), ct = __shfl_sync(kAll, c, t * stride);
                            const float st = __shfl_sync(kAll, sc, t * stride);
                            if (lane == ot && (st > bv || (st == bv && ct < bi))) {
                                bv = st;
                                bi = ct;
                            }
                        }
                        n = 0;
                    }
                }
                if (flagged && bi != 0x7fffffff) code = bi;
            }
#pragma unroll
            for (int mm = 0; mm < kAtMaxM; ++mm)
                if (mm == m) prev[mm] = code;
            if (valid) store_code(p.codes, p.code_dtype, b * p.c_sb + h * p.c_sh + j * p.c_sl + m, code);
            rbound += cm;
            if (m + 1 < M) {
                // ---- residual -= C_m[code], re-split into bf16 hi / lo in the 128B-swizzled operand layout.
                // Every thread updates its own key's row, 8 columns (one 16-byte chunk of each term) at a time.
                const float *crow = cbh + (static_cast<int64_t>(m) * K + code) * D;
                const uint32_t rbase = row * 128;
                float ss = 0.f;  // squared norm of the new residual
#pragma unroll 16
                for (int ck = 0; ck < D / 8; ++ck) {
                    const float4 ca = __ldg(reinterpret_cast<const float4 *>(crow + 8 * ck));
                    const float4 cb4 = __ldg(reinterpret_cast<const float4 *>(crow + 8 * ck + 4));
                    const uint32_t off = (ck >> 3) * kHalfBytes + rbase + (((ck & 7) ^ (row & 7)) << 4);
                    uint4 *ph = reinterpret_cast<uint4 *>(a_rh + off);
                    uint4 *pl = reinterpret_cast<uint4 *>(a_rl + off);
                    const uint4 vh = *ph;
                    const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&vh);
                    float x[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        x[2 * e] = __low2float(h2[e]);
                        x[2 * e + 1] = __high2float(h2[e]);
                    }
                    if (m > 0) {
                        const uint4 vl = *pl;
                        const __nv_bfloat162 *l2 = reinterpret_cast<const __nv_bfloat162 *>(&vl);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            x[2 * e] += __low2float(l2[e]);
                            x[2 * e + 1] += __high2float(l2[e]);
                        }
                    }
                    x[0] -= ca.x; x[1] -= ca.y; x[2] -= ca.z; x[3] -= ca.w;
                    x[4] -= cb4.x; x[5] -= cb4.y; x[6] -= cb4.z; x[7] -= cb4.w;
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
                    uint32_t wh[4], wl[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat16 h0 = __float2bfloat16_rn(x[2 * e]), h1 = __float2bfloat16_rn(x[2 * e + 1]);
                        __nv_bfloat162 hv = __halves2bfloat162(h0, h1);
                        wh[e] = *reinterpret_cast<uint32_t *>(&hv);
                        wl[e] = pack_bf16(x[2 * e] - __bfloat162float(h0), x[2 * e + 1] - __bfloat162float(h1));
                    }
                    *ph = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                    *pl = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                }
                // The operand of the next scores is this residual (norm sqrt(ss) up to rounding); the exact chain's
                // residual differs from it by at most (m + 1) (2^-18 + 3 * 2^-24) times the a priori bound.
                rnow = sqrtf(ss) * 1.001f + static_cast<float>(m + 1) * 7.7e-6f * rbound;
                fence_proxy_async_smem();
                tc_fence_before();
                mbar_arrive(&bar_q[s]);
            }
        }
        if (!ok) s_err = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (s_err && tid == 0) {
        if (p.status) atomicExch(p.status, VQ_WORD_TIMEOUT);
#pragma unroll 1
        for (int w = 0; w < (1 << 14); ++w) __nanosleep(256);  // let tile loads in flight land
    }
    __syncthreads();
    if (warp == C::kWarpMma) {
        __syncwarp();
        tmem_dealloc(tmem, 512u);
    }
}

template <int D, int NS, int CH>
static int launch_assign_tc(const VqTensorDesc *k, const VqTensorDesc *cb, const VqTensorDesc *bias, VqTensorDesc *codes,
                            void *workspace, int32_t *status, cudaStream_t stream)
{
    using C = AtCfg<D, NS, CH>;
    const int64_t B = k->shape[0], Hkv = k->shape[1], L = k->shape[2];
    const int64_t M = cb->shape[1], K = cb->shape[2], MK = M * K;
    __nv_bfloat16 *hi = static_cast<__nv_bfloat16 *>(workspace);
    __nv_bfloat16 *lo = hi + Hkv * MK * D;
    float *cmax = reinterpret_cast<float *>(lo + Hkv * MK * D);
    split_codebook_kernel<<<static_cast<unsigned>(Hkv * M), 256, 0, stream>>>(static_cast<const float *>(cb->ptr), hi, lo, cmax,
                                                                              static_cast<int>(K), D);
    if (launch_status() != VQ_OK) return VQ_ELAUNCH;
    CUtensorMap mk, mhi, mlo;
    const uint64_t cd[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(Hkv * MK), 1};
    const uint64_t cs[3] = {1, static_cast<uint64_t>(D), static_cast<uint64_t>(Hkv * MK * D)};
    if (!map_bhld(&mk, *k) || !make_map(&mhi, hi, 3, cd, cs, CH) || !make_map(&mlo, lo, 3, cd, cs, CH)) return VQ_ELAUNCH;
    AtParams p{};
    p.k = static_cast<const __nv_bfloat16 *>(k->ptr);
    p.k_sb = k->stride[0]; p.k_sh = k->stride[1]; p.k_sl = k->stride[2];
    p.cb = static_cast<const float *>(cb->ptr);
    p.bias = bias ? static_cast<const float *>(bias->ptr) : nullptr;
    p.cmax = cmax;
    p.codes = codes->ptr; p.code_dtype = codes->dtype;
    p.c_sb = codes->stride[0]; p.c_sh = codes->stride[1]; p.c_sl = codes->stride[2];
    p.Hkv = static_cast<int>(Hkv); p.M = static_cast<int>(M); p.K = static_cast<int>(K);
    p.L = L;
    p.ntiles = static_cast<int>((L + kBlock - 1) / kBlock);
    p.status = status;
    p.wait_limit = wait_limit_cycles();
    auto kern = assign_tc_kernel<D, NS, CH>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal) != cudaSuccess) return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>((p.ntiles + NS - 1) / NS), static_cast<unsigned>(B * Hkv));
    kern<<<grid, C::kThreads, C::kTotal, stream>>>(mk, mhi, mlo, p);
    return launch_status();
}

}  // namespace vq

extern "C" size_t vqattn_assign_workspace_bytes(int64_t B, int64_t Hkv, int64_t L, int64_t M, int64_t K, int64_t D)
{
    (void)B;
    (void)L;
    const size_t split = static_cast<size_t>(Hkv) * M * K * D * 2 * 2;                           // bf16 hi / lo codebooks
    const size_t norms = (static_cast<size_t>(Hkv) * M * sizeof(float) + 255) / 256 * 256;        // max row norm per codebook
    return split + norms + 256;
}

extern "C" int vqattn_assign_codes_ws(const VqTensorDesc *k, const VqTensorDesc *codebooks, const VqTensorDesc *bias,
                                      VqTensorDesc *codes, void *workspace, size_t workspace_bytes, int32_t *status_word,
                                      void *stream)
{
    using namespace vq;
    if (k == nullptr || codebooks == nullptr || codes == nullptr) return VQ_EINVAL_ARG;
    if (bias != nullptr && bias->ptr == nullptr) bias = nullptr;
    const bool shapes_ok = k->ndim == 4 && codebooks->ndim == 4;
    const int64_t D = shapes_ok ? k->shape[3] : 0, M = shapes_ok ? codebooks->shape[1] : 0, K = shapes_ok ? codebooks->shape[2] : 0;
    const bool tensor_path = shapes_ok && k->dtype == VQ_BF16 && (D == 64 || D == 128) && M >= 1 && M <= kAtMaxM &&
                             K % kAtMinChunk == 0 && K <= kAtMaxK && k->stride[0] % 8 == 0 && k->stride[1] % 8 == 0 &&
                             k->stride[2] % 8 == 0 && k->shape[2] < (int64_t(1) << 31);
    if (!tensor_path) return vqattn_assign_codes(k, codebooks, bias, codes, stream);
    // same argument checks as the exact kernel's entry point
    int st;
    if ((st = check_basic(k, 4)) != VQ_OK) return st;
    if ((st = check_basic(codebooks, 4)) != VQ_OK) return st;
    if ((st = check_basic(codes, 4)) != VQ_OK) return st;
    if (bias != nullptr && (st = check_basic(bias, 3)) != VQ_OK) return st;
    const VqTensorDesc *all[] = {k, codebooks, bias, codes};
    if ((st = check_device(all, 4)) != VQ_OK) return st;
    if (codebooks->dtype != VQ_F32 || !is_code_dtype(codes->dtype) || (bias && bias->dtype != VQ_F32)) return VQ_EINVAL_DTYPE;
    const int64_t B = k->shape[0], Hkv = k->shape[1], L = k->shape[2];
    if (codebooks->shape[0] != Hkv || codebooks->shape[3] != D) return VQ_EINVAL_SHAPE;
    if (codes->shape[0] != B || codes->shape[1] != Hkv || codes->shape[2] != L || codes->shape[3] != M) return VQ_EINVAL_SHAPE;
    if (bias && (bias->shape[0] != Hkv || bias->shape[1] != M || bias->shape[2] != K)) return VQ_EINVAL_SHAPE;
    if (!is_dense(*codebooks) || (bias && !is_dense(*bias))) return VQ_EINVAL_STRIDE;
    if (codes->dtype == VQ_U8 && K > 256) return VQ_EINVAL_DTYPE;
    if (reinterpret_cast<uintptr_t>(k->ptr) % 16 || reinterpret_cast<uintptr_t>(codebooks->ptr) % 16) return VQ_EINVAL_STRIDE;
    if (B * Hkv > 65535) return VQ_EUNSUPPORTED;
    if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256 ||
        workspace_bytes < vqattn_assign_workspace_bytes(B, Hkv, L, M, K, D))
        return VQ_EWORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // two key tiles per CTA share the 512 score columns of tensor memory when a codebook fits 256 of them;
    // N = 256 instructions when K is a multiple of 256
    if (K == 128)
        return D == 64 ? launch_assign_tc<64, 2, 128>(k, codebooks, bias, codes, workspace, status_word, s)
                       : launch_assign_tc<128, 2, 128>(k, codebooks, bias, codes, workspace, status_word, s);
    if (K == 256)
        return D == 64 ? launch_assign_tc<64, 2, 256>(k, codebooks, bias, codes, workspace, status_word, s)
                       : launch_assign_tc<128, 2, 256>(k, codebooks, bias, codes, workspace, status_word, s);
    if (K == 512)
        return D == 64 ? launch_assign_tc<64, 1, 256>(k, codebooks, bias, codes, workspace, status_word, s)
                       : launch_assign_tc<128, 1, 256>(k, codebooks, bias, codes, workspace, status_word, s);
    return D == 64 ? launch_assign_tc<64, 1, 128>(k, codebooks, bias, codes, workspace, status_word, s)   // K = 384
                   : launch_assign_tc<128, 1, 128>(k, codebooks, bias, codes, workspace, status_word, s);
}
