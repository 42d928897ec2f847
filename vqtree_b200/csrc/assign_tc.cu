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
//   3. The other keys (well under one per cent of the (key, codebook) pairs for random data) keep the
//      approximate winner for the time being.  Their candidates - the codes whose approximate score is
//      within thr of the best; the exact arg-max is among them - are written to a record (up to four codes;
//      more, as for an all-zero key, means "all of them"), the records of a key are chained, and the key
//      goes on a work list.  A second, small kernel (assign_repair_kernel) walks the list: it follows the
//      key through the codebooks with the defining fp32 arithmetic, runs the defining chain for the
//      candidates of every doubtful codebook (first maximum wins), and - in the rare case that this changes
//      a code - recomputes every later codebook of that key over all its codewords, since its residual
//      changed.  The scan kernel never waits for any of this.
//      When a codebook is larger than the 256 score columns a stream owns in tensor memory (K = 512, 1024), its
//      chunks pass through that region in rounds and the scores of a chunk are gone once the next one lands.  The
//      candidates are then tracked during the scan: best, runner-up (each with its group of 32 codes) and the third
//      largest of all group maxima and group runners-up.  If the third lies below the cut and no group's runner-up
//      ever came within thr of the running best (the 30 unranked scores of a group are at most its runner-up, and
//      the cut only rises with the running best), the best and the runner-up are the only candidates; otherwise,
//      and always with a bias (thr then moves with the best score), the record says "all of them".
// One CTA owns NS key tiles of 128 keys ("streams", NS = 2 except for K = 384): per stream eight warps,
// two threads per key, each ranking half of the key's scores in tensor memory and updating half of
// its residual row (the arithmetic between the MMAs is a chain of dependent instructions and loads
// from L2: it needs the warps to hide its latency); one warp issues the MMAs of the streams in turn,
// so the scan of one stream overlaps the MMAs of the other; one warp issues the TMA loads of the
// codebook terms (16 KB units, 5-slot ring).  Every wait is bounded.
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr int kAtMinChunk = 128;   // codewords per MMA chunk: 128, or 256 (one N = 256 instruction) when K allows
constexpr int kAtMaxM = 8;
constexpr int kAtMaxK = 1024;   // 32 groups of 32 codes: one bit each in a thread's group mask
constexpr int kAtRepairWarps = 4;  // warps per CTA of the repair kernel (one doubtful key per warp at a time)

// ------------------------------------------------------------------------------------------------
// fp32 codebook -> bf16 hi / lo terms [Hkv, M*K, D], the squared norm of every row and the largest row
// norm of every codebook (grid.x: codebook, grid.y: slices of kSplitRows rows; cmax zeroed by the launcher, the
// slices meet in it through an atomic maximum on the bits of their non-negative norms).
constexpr int kSplitRows = 64;
__global__ void __launch_bounds__(256)
split_codebook_kernel(const float *__restrict__ cb, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo,
                      float *__restrict__ cmax, float *__restrict__ cn2, unsigned int *__restrict__ work_count, int K, int D)
{
    __shared__ float s_max[8];
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < 2) work_count[threadIdx.x] = 0u;   // the scan kernel that follows fills the lists
    const int hm = blockIdx.x;  // h * M + m
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float wmax = 0.f;
    const int c_end = min(K, (static_cast<int>(blockIdx.y) + 1) * kSplitRows);
    for (int c = static_cast<int>(blockIdx.y) * kSplitRows + warp; c < c_end; c += 8) {
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
        if (lane == 0) cn2[row] = ss;
        wmax = fmaxf(wmax, sqrtf(ss));
    }
    if (lane == 0) s_max[warp] = wmax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.f;
        for (int w = 0; w < 8; ++w) m = fmaxf(m, s_max[w]);
        atomicMax(reinterpret_cast<unsigned int *>(cmax + hm), __float_as_uint(m * 1.0001f));  // sqrt / summation rounding
    }
}

struct AtParams {
    const __nv_bfloat16 *k;
    int64_t k_sb, k_sh, k_sl;
    const float *cb;     // [Hkv, M, K, D]
    const float *bias;   // nullptr or [Hkv, M, K]
    const float *cmax;   // [Hkv, M]
    const float *cn2;    // [Hkv, M*K] squared row norms
    void *codes;
    int code_dtype;
    int64_t c_sb, c_sh, c_sl;
    int Hkv, M, K, ntiles;
    int64_t L;
    int32_t *status;
    long long wait_limit;  // cycles a device-side wait may last before the kernel gives up
    uint4 *work;                // doubtful keys: {key index lo, hi, last record, doubtful codebooks | brute-force codebooks << 8}
    uint4 *pool;                // candidate records: {previous record of the key, m | n << 8, codes 0-1, codes 2-3}
    unsigned int *counters;     // [0] entries in `work`, [1] records in `pool` (zeroed by split_codebook_kernel)
    unsigned int pool_cap;
};

template <int D, int NS, int CH>
struct AtCfg {
    static constexpr int NH = D / 64;
    static constexpr int kATile = NH * kHalfBytes;     // 128 keys x D bf16 (one term of the residual)
    static constexpr int kUnit = CH * 64 * 2;          // CH codewords x 64 columns of one term: one ring slot
    static constexpr int kSlots = 80 * 1024 / kUnit;   // 80 KB of ring
    static constexpr int kB = NS * 2 * kATile;         // per stream: Rh then Rl
    static constexpr int kTotal = kB + kSlots * kUnit + 1024;
    static constexpr int kRegion = NS == 2 ? 256 : 512;  // score columns of a stream in tensor memory
    static constexpr int kMaxChunks = kRegion / CH;
    static constexpr int kGroupsPerChunk = CH / 32;
    static constexpr int kMaxGroups = kRegion / 32;
    static constexpr int kScanWarps = 8;               // per stream: two threads per key
    static constexpr int kWarpMma = kScanWarps * NS, kWarpTma = kScanWarps * NS + 1;
    static constexpr int kThreads = (kScanWarps * NS + 2) * 32;
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

// WRAP: a codebook has more chunks than the stream's score region holds and goes through it in rounds.
template <int D, int NS, int CH, bool WRAP>
__global__ void __launch_bounds__(AtCfg<D, NS, CH>::kThreads, 1)
assign_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_hi,
                 const __grid_constant__ CUtensorMap tm_lo, AtParams p)
{
    using C = AtCfg<D, NS, CH>;
    constexpr int NH = C::NH, SL = C::kSlots;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bar_k[NS], bar_q[NS], bar_c[NS][C::kMaxChunks], c_free[NS][C::kMaxChunks], b_full[SL], b_free[SL];
    __shared__ __align__(8) uint64_t x_half[NS][4], x_done[NS][4];   // hand-offs between the two warps of a lane quarter
    __shared__ __align__(16) float4 s_x[NS][kBlock];                  // per key: what its two threads tell each other
    __shared__ __align__(16) float4 s_y[NS][kBlock];                  // ... the rest of it (third best, runner-up's group, flag)
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int u = blockIdx.y, b = u / p.Hkv, h = u % p.Hkv;
    const int M = p.M, K = p.K, MK = M * K;
    const int chunks = K / CH;
    // A codebook with more chunks than the stream's score region holds (K = 1024: four chunks of 256 columns in a region of
    // 512) goes through the region in rounds: chunk ch lands in slot ch mod kMaxChunks once the scan threads have
    // released the chunk that was there; `rounds` uses of every slot per codebook.
    constexpr bool wrap = WRAP;                        // (the launcher picks WRAP = chunks > kMaxChunks)
    const int rounds = wrap ? chunks / C::kMaxChunks : 1;
    const int tile0 = static_cast<int>(blockIdx.x) * NS;
    const int n_act = min(NS, p.ntiles - tile0);       // streams with a tile

    if (tid == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&bar_k[i], 1);
            mbar_init(&bar_q[i], 32 * C::kScanWarps);
            for (int qd = 0; qd < 4; ++qd) {
                mbar_init(&x_half[i][qd], 1);
                mbar_init(&x_done[i][qd], 1);
            }
            for (int c = 0; c < C::kMaxChunks; ++c) {
                mbar_init(&bar_c[i][c], 1);
                mbar_init(&c_free[i][c], C::kScanWarps);
            }
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
            // Units in the order the MMA warp consumes them: per codebook m the chunks in turn, each chunk for the
            // streams in turn (so that the scan of one stream's chunk runs under the other stream's MMAs); per
            // (chunk, stream): hi term columns 0-63, 64-127 (D = 128), then the lo term likewise.
            // (nested counters instead of divisions of a flat index: this thread's instructions are serial)
            bool ok = true;
            int g = 0;
            for (int m = 0; m < M && ok; ++m)
                for (int ch = 0; ch < chunks && ok; ++ch)
                    for (int s = 0; s < n_act && ok; ++s)
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
                for (int ch = 0; ch < chunks && ok; ++ch)
                    for (int s = 0; s < n_act && ok; ++s) {
                        // the residual terms of (s, m): the key tile itself for m = 0, else written by the scan threads
                        if (ch == 0 && !(m == 0 ? mbar_wait(&bar_k[s], 0, p.wait_limit) : mbar_wait(&bar_q[s], (m - 1) & 1, p.wait_limit))) {
                            ok = false;
                            break;
                        }
                        const int cs = wrap ? ch % C::kMaxChunks : ch, use = m * rounds + (wrap ? ch / C::kMaxChunks : 0);
                        if (wrap && use >= 1 && !mbar_wait(&c_free[s][cs], (use - 1) & 1, p.wait_limit)) {   // the slot's previous chunk has been scanned
                            ok = false;
                            break;
                        }
                        if (ch == 0 || wrap) tc_fence_after();
                        const uint32_t dcol = tmem + s * C::kRegion + cs * CH;
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
                            if (rem == 2 * NH - 1) tc_commit(&bar_c[s][cs]);  // this chunk's score columns are complete
                        }
                    }
            if (!ok) s_err = 1;
        }
    } else if (warp / C::kScanWarps < n_act) {
        // ============================================================ scan warps: two threads per key
        // Thread (hf, row) ranks the groups [hf * groups / 2, (hf + 1) * groups / 2) of its key's scores and
        // updates half hf of its residual row; the two meet through shared memory once per codebook.
        constexpr unsigned kAll = 0xffffffffu;
        const int s = warp / C::kScanWarps, hf = (warp >> 2) & 1, wq = warp & 3;
        const int row = wq * 32 + lane;
        const int64_t j0 = static_cast<int64_t>(tile0 + s) * kBlock;
        const int64_t j = j0 + row;
        const bool valid = j < p.L;
        const uint32_t tbase = tmem + (static_cast<uint32_t>(wq * 32) << 16) + s * C::kRegion;
        const float *cbh = p.cb + static_cast<int64_t>(h) * MK * D;
        uint8_t *a_rh = smem + s * 2 * C::kATile, *a_rl = a_rh + C::kATile;
        const int groups = K / 32, g_lo = hf * (groups / 2), g_hi = g_lo + groups / 2;
        float4 *xch = &s_x[s][row];
        float rbound;  // |k| + sum of the largest codeword norms so far: a priori bound of the residual's norm
        float rnow;    // bound of the current residual's norm (tighter): see the residual update below
        bool ok = __all_sync(kAll, mbar_wait(&bar_k[s], 0, p.wait_limit));
        {
            // |k| from the key tile the TMA load put into shared memory (this thread's row, 16-byte chunks in the
            // 128-byte swizzle: eight consecutive rows read eight different chunks, so the reads do not collide)
            float ss = 0.f;
#pragma unroll 4
            for (int ck = 0; ck < D / 8; ++ck) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(a_rh + (ck >> 3) * kHalfBytes + row * 128 + (((ck & 7) ^ (row & 7)) << 4));
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
        uint32_t doubt = 0;   // bit m: the lead of codebook m's best score did not prove its arg-max (bit 8 + m: no record)
        uint32_t last_rec = 0xffffffffu;   // the key's most recent candidate record
        for (int m = 0; m < M && ok; ++m) {
            const float cm = p.cmax[h * M + m];
            // eps of this codebook in units of 2^-18: the terms listed at the top of the file plus one unit of slack
            const float eps_m = (4.f + D / 64 + (m > 0 ? 3 : 2) * (D / 32) + 1.1f * m) * 3.814697265625e-6f;
            const float thr0 = 2.f * eps_m * rnow * cm + 1e-30f;
            const float *bm = p.bias ? p.bias + (static_cast<int64_t>(h) * M + m) * K : nullptr;
            // ---- scan of this thread's groups, chunk by chunk as the tensor pipe finishes them: best and runner-up
            // of the tagged scores (the tag of the best gives its index inside its group of 32)
            float best = -INFINITY, second = -INFINITY;
            int bgrp = g_lo;
            uint32_t gbits = 0;   // groups whose maximum came within the threshold of the running best: a superset of
                                  // the groups that can hold a candidate at the end
            // The candidates of a key that turns out doubtful are tracked on the way: the group of the runner-up, the third
            // largest of all group maxima and group runners-up, and whether the runner-up of any group came within the
            // threshold of the running best (the other 30 scores of such a group are unknown here and may hold further
            // candidates).  A doubtful key whose third lies below the cut needs no second look at its scores - which WRAP
            // could not take anyway: the scores of earlier chunks are gone by then.
            float third = -INFINITY;
            int sgrp = g_lo;
            bool amb = bm != nullptr;   // with a bias the threshold moves with the best score: no short list then
            auto rank_group = [&](int g, uint32_t col) {   // group g of the codebook, its 32 score columns at `col` of the stream's region
                float v[32];
                load_scores(tbase + col, bm, 32 * g, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = tag_score(v[i], i);
                float hi, lo;
                top2_32(v, hi, lo);
                // hi, then lo (<= hi) into the sorted triple (best, second, third); a tie with the best goes to the
                // earlier group, which holds the lower codes
                if (hi > best) {
                    third = second; second = best; sgrp = bgrp; best = hi; bgrp = g;
                } else if (hi > second) {
                    third = second; second = hi; sgrp = g;
                } else {
                    third = fmaxf(third, hi);
                }
                if (lo > second) {
                    third = second; second = lo; sgrp = g;
                } else {
                    third = fmaxf(third, lo);
                }
                amb |= lo >= best - thr0;
                if constexpr (!wrap) {
                    // for the keys that do need a second look: the groups whose maximum came within the threshold
                    // (with a bias the fp32 additions s + bias round by up to 2^-24 |s + bias| each)
                    const float thr_g = bm ? thr0 + fabsf(best) * 4.76837158203125e-7f : thr0;
                    gbits |= (hi >= best - thr_g ? 1u : 0u) << g;
                }
            };
            if constexpr (!wrap) {
#pragma unroll 1
                for (int g = g_lo; g < g_hi && ok; ++g) {
                    if (g == g_lo || g % C::kGroupsPerChunk == 0) {
                        ok = __all_sync(kAll, mbar_wait(&bar_c[s][g / C::kGroupsPerChunk], m & 1, p.wait_limit));
                        tc_fence_after();
                        if (!ok) break;
                    }
                    rank_group(g, 32 * g);
                }
            } else {
                // rounds through the region: of every chunk this thread ranks half hf of the groups, then releases the slot
                constexpr int GPC = C::kGroupsPerChunk;
                bgrp = sgrp = hf * (GPC / 2);
#pragma unroll 1
                for (int ch = 0; ch < chunks && ok; ++ch) {
                    const int cs = ch % C::kMaxChunks, use = m * rounds + ch / C::kMaxChunks;
                    ok = __all_sync(kAll, mbar_wait(&bar_c[s][cs], use & 1, p.wait_limit));
                    tc_fence_after();
                    if (!ok) break;
#pragma unroll 1
                    for (int i = hf * (GPC / 2); i < (hf + 1) * (GPC / 2); ++i) rank_group(ch * GPC + i, cs * CH + 32 * i);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&c_free[s][cs]);
                }
            }
            if (!ok) break;
            // ---- the two halves meet: the upper half hands its result over, the lower half merges (a tie between
            // the halves goes to the lower one, which holds the lower codes) and hands the result back
            int code;
            if (hf == 1) {
                *xch = make_float4(best, second, __int_as_float(bgrp), __uint_as_float(gbits));
                s_y[s][row] = make_float4(third, __int_as_float(sgrp), amb ? 1.f : 0.f, 0.f);
                __syncwarp();
                if (lane == 0) mbar_arrive(&x_half[s][wq]);
                ok = __all_sync(kAll, mbar_wait(&x_done[s][wq], m & 1, p.wait_limit));
                if (!ok) break;
                const float4 r = *xch;
                best = r.x;
                code = __float_as_int(r.y);
            } else {
                ok = __all_sync(kAll, mbar_wait(&x_half[s][wq], m & 1, p.wait_limit));
                if (!ok) break;
                const float4 o = *xch;
                {
                    // the other half's sorted triple into this one (its best with its group, its runner-up with its group, its third)
                    const float4 oy = s_y[s][row];
                    const int obg = __float_as_int(o.z), osg = __float_as_int(oy.y);
                    amb |= oy.z != 0.f;
                    if (o.x > best || (o.x == best && obg < bgrp)) {   // equal tagged scores: the lower group holds the lower code
                        third = second; second = best; sgrp = bgrp; best = o.x; bgrp = obg;
                    } else if (o.x > second) {
                        third = second; second = o.x; sgrp = obg;
                    } else {
                        third = fmaxf(third, o.x);
                    }
                    if (o.y > second) {
                        third = second; second = o.y; sgrp = osg;
                    } else {
                        third = fmaxf(third, o.y);
                    }
                    third = fmaxf(third, oy.x);
                }
                code = bgrp * 32 + 31 - static_cast<int>(__float_as_uint(best) & 31u);  // first group holding the maximum
                *xch = make_float4(best, __int_as_float(code), 0.f, 0.f);
                __syncwarp();
                if (lane == 0) mbar_arrive(&x_done[s][wq]);
                // with a bias the fp32 additions s + bias round by up to 2^-24 |s + bias| each
                const float thr = bm ? thr0 + fabsf(best) * 4.76837158203125e-7f : thr0;
                const bool dflag = valid && !(best - second > thr);
                if (__ballot_sync(kAll, dflag)) {
                    // ---- some key of this warp is doubtful: its candidates (scores within thr of the best) go into a
                    // record for the repair kernel; carry on with the approximate winner.  The best and the runner-up are
                    // the only candidates when the third largest tracked score is below the cut and no group's runner-up
                    // came near the best.  The other doubtful keys take a second look at their scores (tensor-memory
                    // loads are warp-wide, so the warp re-reads the union of those keys' marked groups) - or, with WRAP,
                    // name every code a candidate (the repair kernel then scores the whole codebook).
                    const float cut = best - thr;
                    const bool quick = dflag && !amb && third < cut;
                    const bool slow = dflag && !quick;
                    int n = 0;
                    uint32_t c01 = 0, c23 = 0;
                    if (quick) {
                        n = 2;
                        c01 = static_cast<uint32_t>(code) |
                              (static_cast<uint32_t>(sgrp * 32 + 31 - static_cast<int>(__float_as_uint(second) & 31u)) << 16);
                    }
                    if (wrap && slow) n = 255;
                    const uint32_t gb = (!wrap && slow) ? (gbits | __float_as_uint(o.w)) : 0u;
                    const uint32_t un = __reduce_or_sync(kAll, gb);
#pragma unroll 1
                    for (int g = 0; g < groups && !wrap; ++g) {
                        if (!((un >> g) & 1u)) continue;
                        if (!__all_sync(kAll, mbar_wait(&bar_c[s][g / C::kGroupsPerChunk], m & 1, p.wait_limit))) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        float v[32];
                        load_scores(tbase + 32 * g, bm, 32 * g, v);
                        if ((gb >> g) & 1u) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (v[i] >= cut) {
                                    const uint32_t c = static_cast<uint32_t>(g * 32 + i);
                                    if (n < 2) c01 |= c << (16 * n);
                                    else if (n < 4) c23 |= c << (16 * (n - 2));
                                    ++n;
                                }
                        }
                    }
                    if (!ok) break;
                    if (dflag) {
                        const unsigned int at = atomicAdd(p.counters + 1, 1u);
                        if (at < p.pool_cap) {
                            p.pool[at] = make_uint4(last_rec, static_cast<uint32_t>(m) | (static_cast<uint32_t>(n > 4 ? 255 : n) << 8), c01, c23);
                            last_rec = at;
                            doubt |= 1u << m;
                        } else {
                            doubt |= 0x100u << m;   // no room for the record: the repair kernel scores every code of this codebook
                        }
                    }
                }
                if (valid) store_code(p.codes, p.code_dtype, b * p.c_sb + h * p.c_sh + j * p.c_sl + m, code);
            }
            rbound += cm;
            if (m + 1 < M) {
                // ---- residual -= C_m[code] (fp32), re-split into bf16 hi / lo in the 128B-swizzled operand layout
                {
                    // The warp walks 16 of its quarter's 32 keys (the partner warp the other 16); D/4 lanes share a key, lane l
                    // of them owns its columns 4l .. 4l+3.  One load instruction then covers whole codebook rows - full
                    // 128-byte lines - where a thread fetching its own key's half row touched 32 different lines per
                    // instruction; eight loads are in flight at a time.
                    constexpr int LPR = D / 4, KPI = 32 / LPR, NIT = 16 / KPI;   // lanes per row, keys per instruction, instructions
                    constexpr int NB = NIT < 8 ? NIT : 8;                       // loads in flight (registers)
                    const int sub = lane / LPR, l = lane % LPR;
                    const uint32_t lane_off = (l >> 4) * kHalfBytes + 8 * (l & 1);   // the 64-column half and the 8 bytes inside a 16-byte chunk
                    const int chunk = (l & 15) >> 1;
#pragma unroll 1
                    for (int i0 = 0; i0 < NIT; i0 += NB) {
                        float4 crow4[NB];
#pragma unroll
                        for (int i = 0; i < NB; ++i) {
                            const int ck = __shfl_sync(kAll, code, 16 * hf + (i0 + i) * KPI + sub);
                            crow4[i] = __ldg(reinterpret_cast<const float4 *>(cbh + (static_cast<int64_t>(m) * K + ck) * D) + l);
                        }
#pragma unroll
                        for (int i = 0; i < NB; ++i) {
                            const int r = wq * 32 + 16 * hf + (i0 + i) * KPI + sub;
                            const uint32_t off = lane_off + r * 128 + ((chunk ^ (r & 7)) << 4);
                            uint2 *ph = reinterpret_cast<uint2 *>(a_rh + off);
                            uint2 *pl = reinterpret_cast<uint2 *>(a_rl + off);
                            const uint2 vh = *ph;
                            float x[4] = {__uint_as_float(vh.x << 16), __uint_as_float(vh.x & 0xffff0000u), __uint_as_float(vh.y << 16),
                                          __uint_as_float(vh.y & 0xffff0000u)};
                            if (m > 0) {
                                const uint2 vl = *pl;
                                x[0] += __uint_as_float(vl.x << 16); x[1] += __uint_as_float(vl.x & 0xffff0000u);
                                x[2] += __uint_as_float(vl.y << 16); x[3] += __uint_as_float(vl.y & 0xffff0000u);
                            }
                            x[0] -= crow4[i].x; x[1] -= crow4[i].y; x[2] -= crow4[i].z; x[3] -= crow4[i].w;
                            uint32_t wh[2], wl[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const __nv_bfloat16 h0 = __float2bfloat16_rn(x[2 * e]), h1 = __float2bfloat16_rn(x[2 * e + 1]);
                                __nv_bfloat162 hv = __halves2bfloat162(h0, h1);
                                wh[e] = *reinterpret_cast<uint32_t *>(&hv);
                                wl[e] = pack_bf16(x[2 * e] - __bfloat162float(h0), x[2 * e + 1] - __bfloat162float(h1));
                            }
                            *ph = make_uint2(wh[0], wh[1]);
                            *pl = make_uint2(wl[0], wl[1]);
                        }
                    }
                }
                // Norm of the new residual rho' = rho - C[code] without another pass over it:
                //   |rho'|^2 = |rho|^2 - 2 rho.C + |C|^2,   rho.C >= s - eps |rho| max|C|
                // where s is the tensor-core score the code was chosen with (within eps |rho| max|C| of rho.C; the
                // bias taken out again), |rho| <= rnow, and |C|^2 comes from the table the split kernel wrote.  The
                // stored terms round rho' (the factor 1.001 covers that and the table's rounding); the exact chain's
                // residual differs from it by at most (m + 1) (2^-18 + 3 * 2^-24) times the a priori bound.
                float s_code = best;
                if (bm) s_code -= __ldg(bm + code);
                const float c2 = __ldg(p.cn2 + static_cast<int64_t>(h) * MK + m * K + code);
                const float slack = 2.f * eps_m * rnow * cm + (bm ? fabsf(best) * 4.76837158203125e-7f : 0.f);
                const float ss = fmaxf(rnow * rnow - 2.f * (s_code - slack) + c2, 0.f);
                rnow = sqrtf(ss) * 1.001f + static_cast<float>(m + 1) * 7.7e-6f * rbound;
                fence_proxy_async_smem();
                tc_fence_before();
                mbar_arrive(&bar_q[s]);
            }
        }
        if (doubt != 0 && ok) {
            const unsigned int at = atomicAdd(p.counters, 1u);   // at most one entry per key: the list holds every key if need be
            const unsigned long long lin = static_cast<unsigned long long>(static_cast<int64_t>(u) * p.L + j);
            p.work[at] = make_uint4(static_cast<uint32_t>(lin), static_cast<uint32_t>(lin >> 32), last_rec, doubt);
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


// ------------------------------------------------------------------------------------------------
// Exact settlement of the doubtful keys.  One warp per list entry: it follows the key through the
// codebooks with the defining arithmetic - residual r_0 = k, r_{m+1} = r_m - C_m[code_m] (fp32
// subtraction) - and settles every doubtful codebook: each score is ONE fused-multiply-add chain over
// d = 0..D-1 starting from +0 (+ bias), ties go to the lowest code.  With a candidate record, one lane
// per candidate runs the chain; without one (too many candidates, no room for the record, or a code of
// an earlier codebook has changed and with it the residual) lane l scores the codes l, l + 32, ... of
// the whole codebook.  The residual is broadcast from shared memory.
template <int D>
__global__ void __launch_bounds__(kAtRepairWarps * 32)
assign_repair_kernel(AtParams p)
{
    __shared__ __align__(16) float s_r[kAtRepairWarps][D];
    __shared__ uint4 s_rec[kAtRepairWarps][kAtMaxM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned int count = p.counters[0];
    const int M = p.M, K = p.K;
    float *r = s_r[warp];
    constexpr int PER = D / 32;   // residual elements a lane keeps up to date
    for (unsigned int e = blockIdx.x * kAtRepairWarps + warp; e < count; e += gridDim.x * kAtRepairWarps) {
        const uint4 ent = p.work[e];
        const uint32_t doubt = ent.w & 0xffu, brute = (ent.w >> 8) & 0xffu;
        const int64_t lin = static_cast<int64_t>((static_cast<unsigned long long>(ent.y) << 32) | ent.x);
        const int64_t u = lin / p.L, j = lin % p.L;
        const int b = static_cast<int>(u / p.Hkv), h = static_cast<int>(u % p.Hkv);
        const __nv_bfloat16 *krow = p.k + b * p.k_sb + h * p.k_sh + j * p.k_sl;
        const float *cbh = p.cb + static_cast<int64_t>(h) * M * K * D;
        __syncwarp();
        // the key's records, newest first, into a table indexed by codebook
        if (lane == 0) {
            uint32_t at = ent.z;
            for (int guard = 0; guard < kAtMaxM && at != 0xffffffffu && at < p.pool_cap; ++guard) {
                const uint4 rec = p.pool[at];
                s_rec[warp][rec.y & 0xffu & (kAtMaxM - 1)] = rec;
                at = rec.x;
            }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) r[lane + 32 * i] = __bfloat162float(krow[lane + 32 * i]);
        __syncwarp();
        const int64_t cbase = b * p.c_sb + h * p.c_sh + j * p.c_sl;
        bool changed = false;
        for (int m = 0; m < M; ++m) {
            int code = load_code(p.codes, p.code_dtype, cbase + m);
            const bool dm = (doubt >> m) & 1u;
            const uint4 rec = dm ? s_rec[warp][m] : make_uint4(0, 0, 0, 0);
            const int ncand = static_cast<int>((rec.y >> 8) & 0xffu);
            const bool all = changed || ((brute >> m) & 1u) || (dm && (ncand > 4 || ncand == 0));
            if (all || dm) {
                const float *cm = cbh + static_cast<int64_t>(m) * K * D;
                const float *bm = p.bias ? p.bias + (static_cast<int64_t>(h) * M + m) * K : nullptr;
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                if (all) {
                    for (int c0 = 0; c0 < K; c0 += 128) {       // four codes per lane at a time: four independent chains
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
                        const float *row[4];
#pragma unroll
                        for (int t = 0; t < 4; ++t) row[t] = cm + static_cast<int64_t>(min(c0 + lane + 32 * t, K - 1)) * D;
#pragma unroll 4
                        for (int d = 0; d < D; d += 4) {
                            const float4 r4 = *reinterpret_cast<const float4 *>(r + d);
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const float4 c4 = __ldg(reinterpret_cast<const float4 *>(row[t] + d));
                                acc[t] = __fmaf_rn(r4.x, c4.x, acc[t]);
                                acc[t] = __fmaf_rn(r4.y, c4.y, acc[t]);
                                acc[t] = __fmaf_rn(r4.z, c4.z, acc[t]);
                                acc[t] = __fmaf_rn(r4.w, c4.w, acc[t]);
                            }
                        }
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const int c = c0 + lane + 32 * t;
                            if (c < K) {
                                const float sc = bm ? __fadd_rn(acc[t], __ldg(bm + c)) : acc[t];
                                if (sc > bv) {      // codes come in increasing order: the first maximum stays
                                    bv = sc;
                                    bi = c;
                                }
                            }
                        }
                    }
                } else if (lane < ncand) {
                    const int c = static_cast<int>(((lane < 2 ? rec.z : rec.w) >> (16 * (lane & 1))) & 0xffffu);
                    if (c < K) {
                        const float *crow = cm + static_cast<int64_t>(c) * D;
                        float acc = 0.f;
#pragma unroll 8
                        for (int d = 0; d < D; d += 4) {
                            const float4 r4 = *reinterpret_cast<const float4 *>(r + d);
                            const float4 c4 = __ldg(reinterpret_cast<const float4 *>(crow + d));
                            acc = __fmaf_rn(r4.x, c4.x, acc);
                            acc = __fmaf_rn(r4.y, c4.y, acc);
                            acc = __fmaf_rn(r4.z, c4.z, acc);
                            acc = __fmaf_rn(r4.w, c4.w, acc);
                        }
                        bv = bm ? __fadd_rn(acc, __ldg(bm + c)) : acc;
                        bi = c;
                    }
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
                    if (ov > bv || (ov == bv && oi < bi)) {
                        bv = ov;
                        bi = oi;
                    }
                }
                if (bi != code && bi != 0x7fffffff) {
                    changed = true;
                    code = bi;
                    if (lane == 0) store_code(p.codes, p.code_dtype, cbase + m, code);
                }
            }
            if (m + 1 < M) {
                const float *crow = cbh + (static_cast<int64_t>(m) * K + code) * D;
                __syncwarp();
#pragma unroll
                for (int i = 0; i < PER; ++i) r[lane + 32 * i] = __fsub_rn(r[lane + 32 * i], __ldg(crow + lane + 32 * i));
                __syncwarp();
            }
        }
    }
}

template <int D, int NS, int CH, bool WRAP = false>
static int launch_assign_tc(const VqTensorDesc *k, const VqTensorDesc *cb, const VqTensorDesc *bias, VqTensorDesc *codes,
                            void *workspace, int32_t *status, cudaStream_t stream)
{
    using C = AtCfg<D, NS, CH>;
    const int64_t B = k->shape[0], Hkv = k->shape[1], L = k->shape[2];
    const int64_t M = cb->shape[1], K = cb->shape[2], MK = M * K;
    __nv_bfloat16 *hi = static_cast<__nv_bfloat16 *>(workspace);
    __nv_bfloat16 *lo = hi + Hkv * MK * D;
    float *cmax = reinterpret_cast<float *>(lo + Hkv * MK * D);
    float *cn2 = cmax + (Hkv * M + 63) / 64 * 64;
    unsigned int *counters = reinterpret_cast<unsigned int *>(cn2 + (Hkv * MK + 63) / 64 * 64);
    uint4 *work = reinterpret_cast<uint4 *>(counters + 64);
    uint4 *pool = work + B * Hkv * L;
    if (cudaMemsetAsync(cmax, 0, sizeof(float) * static_cast<size_t>(Hkv * M), stream) != cudaSuccess) return VQ_ELAUNCH;
    split_codebook_kernel<<<dim3(static_cast<unsigned>(Hkv * M), static_cast<unsigned>((K + kSplitRows - 1) / kSplitRows)), 256, 0, stream>>>(
        static_cast<const float *>(cb->ptr), hi, lo, cmax, cn2, counters, static_cast<int>(K), D);
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
    p.cn2 = cn2;
    p.work = work;
    p.pool = pool;
    p.counters = counters;
    p.pool_cap = static_cast<unsigned int>(B * Hkv * L < 0xfffffff0ll ? B * Hkv * L : 0xfffffff0ll);
    p.codes = codes->ptr; p.code_dtype = codes->dtype;
    p.c_sb = codes->stride[0]; p.c_sh = codes->stride[1]; p.c_sl = codes->stride[2];
    p.Hkv = static_cast<int>(Hkv); p.M = static_cast<int>(M); p.K = static_cast<int>(K);
    p.L = L;
    p.ntiles = static_cast<int>((L + kBlock - 1) / kBlock);
    p.status = status;
    p.wait_limit = wait_limit_cycles();
    static_assert(!WRAP || CH == AtCfg<D, NS, CH>::kRegion, "rounds of one chunk per use of the region");
    if (WRAP != (K / CH > C::kMaxChunks)) return VQ_EUNSUPPORTED;
    auto kern = assign_tc_kernel<D, NS, CH, WRAP>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal) != cudaSuccess) return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>((p.ntiles + NS - 1) / NS), static_cast<unsigned>(B * Hkv));
    kern<<<grid, C::kThreads, C::kTotal, stream>>>(mk, mhi, mlo, p);
    if (launch_status() != VQ_OK) return VQ_ELAUNCH;
    // the doubtful keys, exactly; the list length is only known on the device: a fixed grid walks it
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return VQ_EDEVICE;
    assign_repair_kernel<D><<<static_cast<unsigned>(sms * 8), kAtRepairWarps * 32, 0, stream>>>(p);
    return launch_status();
}

}  // namespace vq

extern "C" size_t vqattn_assign_workspace_bytes(int64_t B, int64_t Hkv, int64_t L, int64_t M, int64_t K, int64_t D)
{
    const size_t split = static_cast<size_t>(Hkv) * M * K * D * 2 * 2;                           // bf16 hi / lo codebooks
    const size_t norms = (static_cast<size_t>(Hkv) * M * sizeof(float) + 255) / 256 * 256;        // max row norm per codebook
    const size_t rows = (static_cast<size_t>(Hkv) * M * K * sizeof(float) + 255) / 256 * 256;    // squared norm of every row
    const size_t list = 256 + 2 * static_cast<size_t>(B) * Hkv * L * 16;   // counters; doubtful keys and candidate records, 16 bytes each, one per key at most
    return split + norms + rows + list + 256;
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
                             K % kAtMinChunk == 0 && (K <= 512 || K == kAtMaxK) && k->stride[0] % 8 == 0 && k->stride[1] % 8 == 0 &&
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
    // K = 512 and K = 1024: two streams, the codebook's 256-column chunks in rounds through each stream's region (the
    // candidates of a doubtful key are tracked during the scan, the earlier chunks being gone by the end)
    if (K == 512)
        return D == 64 ? launch_assign_tc<64, 2, 256, true>(k, codebooks, bias, codes, workspace, status_word, s)
                       : launch_assign_tc<128, 2, 256, true>(k, codebooks, bias, codes, workspace, status_word, s);
    if (K == 1024)
        return D == 64 ? launch_assign_tc<64, 2, 256, true>(k, codebooks, bias, codes, workspace, status_word, s)
                       : launch_assign_tc<128, 2, 256, true>(k, codebooks, bias, codes, workspace, status_word, s);
    return D == 64 ? launch_assign_tc<64, 1, 128>(k, codebooks, bias, codes, workspace, status_word, s)   // K = 384
                   : launch_assign_tc<128, 1, 128>(k, codebooks, bias, codes, workspace, status_word, s);
}
