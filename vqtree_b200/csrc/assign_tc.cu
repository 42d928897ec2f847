// Key -> code assignment with the score matrix on the tensor cores, still bit-exact.
//
// Replaces ops/mini_vq.py:4-18 of the reference (and its greedy-residual extension to M codebooks)
// for bf16 keys.  The defining arithmetic is unchanged: the code of a key in codebook m is the first
// arg-max over c of the fp32 fused-multiply-add chain  sum_d r_m[d] * C_m[c][d] (+ bias),
// r_{m+1} = r_m - C_m[code].  What changes is how the arg-max is found:
//   1. APPROXIMATE scores of a 128-key tile against all K codewords come from tcgen05.mma.  The
//      fp32 codebook is split into two bf16 terms (C ~ Chi + Clo, error <= 2^-16 |C|), a bf16 key is
//      exact, and for m > 0 the part already quantised, q_m = sum_{m'<m} C_m'[code], is kept as two
//      bf16 terms too and subtracted with negated MMAs:  s~ = k.Chi + k.Clo - qh.Chi - ql.Chi - qh.Clo.
//   2. Every approximate score is within eps = 2^-15 (|k| + sum_m' max|C_m'|) max|C_m| of the exact
//      chain (split error 2^-18, dropped ql.Clo 2^-18, fp32 accumulation < 2^-17 on each side).  A key whose best approximate score leads the runner-up by more than 2 eps has a
//      unique arg-max: that code is final.
//   3. The other keys (about 1 % for random data) are settled exactly on the spot: their candidates
//      (all codes within 2 eps of the best) are re-scored by the warp with the defining fp32 chain,
//      first maximum wins.
// One CTA = 128 keys of one (batch, kv head); warps 0-3 own one key each per thread, warp 4 issues
// TMA loads (hi / lo terms of 128-codeword chunks through a 3-slot ring) and the MMAs.  Every wait is bounded.
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr int kAtChunk = 128;      // codewords per MMA chunk (one N = 128 instruction)
constexpr int kAtThreads = 160;    // 4 scan warps + 1 control warp
constexpr int kAtMaxM = 8;
constexpr int kAtMaxK = 512;
constexpr float kAtEps = 3.0517578125e-5f;  // 2^-15

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
    int Hkv, M, K;
    int64_t L;
    int32_t *status;
};

template <int D>
struct AtCfg {
    static constexpr int NH = D / 64;
    static constexpr int kATile = NH * kHalfBytes;               // 128 keys x D bf16
    static constexpr int kBHalf = kAtChunk * 64 * 2;              // 128 codewords x 64 bf16
    static constexpr int kUnit = NH * kBHalf;                     // one term (hi or lo) of a chunk = one ring slot
    static constexpr int kSlots = 3;
    static constexpr int kAk = 0, kAqh = kATile, kAql = 2 * kATile, kB = 3 * kATile;
    static constexpr int kTotal = kB + kSlots * kUnit + 1024;
};

// The defining score: one fp32 FMA chain over d of the residual r (shared memory, fp32) against
// codeword row cc (global, fp32).
template <int D>
__device__ __forceinline__ float exact_chain(const float *__restrict__ r, const float *__restrict__ cc)
{
    float acc = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; d += 4) {
        const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cc + d));
        const float4 r4 = *reinterpret_cast<const float4 *>(r + d);
        acc = __fmaf_rn(r4.x, c4.x, acc);
        acc = __fmaf_rn(r4.y, c4.y, acc);
        acc = __fmaf_rn(r4.z, c4.z, acc);
        acc = __fmaf_rn(r4.w, c4.w, acc);
    }
    return acc;
}

template <int D>
__global__ void __launch_bounds__(kAtThreads, 1)
assign_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_hi,
                 const __grid_constant__ CUtensorMap tm_lo, AtParams p)
{
    using C = AtCfg<D>;
    constexpr int NH = C::NH;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bar_k, b_full[3], b_free[3], bar_c[kAtMaxK / kAtChunk], bar_q;
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;
    __shared__ __align__(16) float s_res[4][D];  // per scan warp: exact fp32 residual of the key being re-scored

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int u = blockIdx.y, b = u / p.Hkv, h = u % p.Hkv;
    const int64_t j0 = static_cast<int64_t>(blockIdx.x) * kBlock;
    const int M = p.M, K = p.K, MK = M * K;
    const int chunks = K / kAtChunk;
    const uint32_t tmem_cols = 512u;
    // K <= 256: the score columns of consecutive codebooks alternate between two 256-column regions, so
    // the key term of codebook m may be issued while the scan threads still read codebook m - 1
    const bool two_regions = K <= 256;

    if (tid == 0) {
        mbar_init(&bar_k, 1);
        for (int i = 0; i < 3; ++i) {
            mbar_init(&b_full[i], 1);
            mbar_init(&b_free[i], 1);
        }
        for (int i = 0; i < kAtMaxK / kAtChunk; ++i) mbar_init(&bar_c[i], 1);
        mbar_init(&bar_q, 128);
        fence_mbar_init();
        s_err = 0;
    }
    if (warp == 4) {
        __syncwarp();
        tmem_alloc(&s_tmem, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp == 4) {
        // ============================================================ control: TMA loads + MMA issue
        if (lane == 0) {
            bool ok = true;
            mbar_expect_tx(&bar_k, C::kATile);
#pragma unroll
            for (int hh = 0; hh < NH; ++hh)
                tma_load_4d(smem + C::kAk + hh * kHalfBytes, &tm_k, &bar_k, 64 * hh, static_cast<int>(j0), h, b);
            // The codebook streams through a 3-slot ring in UNITS: unit 2c is the hi term of chunk c
            // (128 codewords), unit 2c+1 its lo term, chunks numbered through all M codebooks.
            const int total = 2 * M * chunks;
            auto issue_load = [&](int g) {
                const int slot = g % C::kSlots;
                if (g >= C::kSlots && !mbar_wait(&b_free[slot], ((g / C::kSlots) - 1) & 1)) {
                    ok = false;
                    return;
                }
                const int c = g >> 1;
                const int row = h * MK + (c / chunks) * K + (c % chunks) * kAtChunk;  // row in [Hkv*M*K, D]
                uint8_t *dst = smem + C::kB + slot * C::kUnit;
                mbar_expect_tx(&b_full[slot], C::kUnit);
#pragma unroll
                for (int hh = 0; hh < NH; ++hh) tma_load_3d(dst + hh * C::kBHalf, (g & 1) ? &tm_lo : &tm_hi, &b_full[slot], 64 * hh, row, 0);
            };
            constexpr uint32_t id_pos = idesc_bf16(128, kAtChunk, 0, 0, 0), id_neg = idesc_bf16(128, kAtChunk, 0, 0, 1);
            // descriptors differ only in their 16-byte-granular start address: build the bases once
            const uint64_t d_k = smem_desc_sw128(smem_u32(smem + C::kAk), 16, 1024);
            const uint64_t d_qh = smem_desc_sw128(smem_u32(smem + C::kAqh), 16, 1024);
            const uint64_t d_ql = smem_desc_sw128(smem_u32(smem + C::kAql), 16, 1024);
            const uint64_t d_b0 = smem_desc_sw128(smem_u32(smem + C::kB), 16, 1024);
            issue_load(0);
            if (total > 1) issue_load(1);
            if (!mbar_wait(&bar_k, 0)) ok = false;
            for (int g = 0; g < total && ok; ++g) {
                const int c = g >> 1, m = c / chunks, ch = c % chunks, slot = g % C::kSlots;
                const bool is_lo = g & 1;
                if (g + 2 < total) issue_load(g + 2);
                if (!ok || !mbar_wait(&b_full[slot], (g / C::kSlots) & 1)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint64_t d_b = d_b0 + static_cast<uint64_t>((slot * C::kUnit) >> 4);
                const uint32_t dcol = tmem + (two_regions ? (m & 1) * 256 : 0) + ch * kAtChunk;
                uint32_t acc = is_lo ? 1u : 0u;
                if (m > 0 && !two_regions && ch == 0 && !is_lo && !mbar_wait(&bar_q, (m - 1) & 1)) {
                    ok = false;  // one region only: it is free once the scan of codebook m - 1 is over
                    break;
                }
                auto term = [&](uint64_t a_desc, uint32_t idesc) {
#pragma unroll
                    for (int hh = 0; hh < NH; ++hh)
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4) {
                            mma_ss(dcol, a_desc + static_cast<uint64_t>((hh * kHalfBytes + k4 * 32) >> 4),
                                   d_b + static_cast<uint64_t>((hh * C::kBHalf + k4 * 32) >> 4), idesc, acc);
                            acc = 1;
                        }
                };
                term(d_k, id_pos);  // the key term needs nothing from the previous codebook's scan
                if (m > 0) {
                    // the q terms of codebook m exist once every scan thread has folded in its code of m - 1
                    if (two_regions && ch == 0 && !is_lo && !mbar_wait(&bar_q, (m - 1) & 1)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    term(d_qh, id_neg);
                    if (!is_lo) term(d_ql, id_neg);
                }
                tc_commit(&b_free[slot]);
                if (is_lo) tc_commit(&bar_c[ch]);  // this chunk's 128 score columns are complete
            }
            if (!ok) s_err = 1;
        }
    } else {
        // ============================================================ scan warps: one key per thread
        const int row = tid;
        const int64_t j = j0 + row;
        const bool valid = j < p.L;
        const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
        const __nv_bfloat16 *krow = p.k + b * p.k_sb + h * p.k_sh + (valid ? j : 0) * p.k_sl;
        const float *cbh = p.cb + static_cast<int64_t>(h) * MK * D;
        float knorm = 0.f;
        {
            float ss = 0.f;
#pragma unroll
            for (int d = 0; d < D; d += 8) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(krow + d);
                const __nv_bfloat162 *hp = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float x = __low2float(hp[i]), y = __high2float(hp[i]);
                    ss = fmaf(x, x, fmaf(y, y, ss));
                }
            }
            knorm = sqrtf(ss) * 1.0001f;
        }
        float qbound = 0.f;
        bool ok = true;
        int prev[kAtMaxM];
#pragma unroll
        for (int mm = 0; mm < kAtMaxM; ++mm) prev[mm] = 0;
        for (int m = 0; m < M && ok; ++m) {
            const float cm = p.cmax[h * M + m];
            const float thr = 2.f * kAtEps * (knorm + qbound) * cm + 1e-30f;
            const float *bm = p.bias ? p.bias + (static_cast<int64_t>(h) * M + m) * K : nullptr;
            const uint32_t region = two_regions ? (m & 1) * 256 : 0;
            // ---- scan, chunk by chunk as the tensor pipe finishes them: best (first maximum) and runner-up
            float best = -INFINITY, second = -INFINITY;
            int bidx = 0;
            for (int ch = 0; ch < chunks && ok; ++ch) {
                if (!mbar_wait(&bar_c[ch], m & 1)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (int q4 = 0; q4 < kAtChunk / 32; ++q4) {
                    uint32_t r[32];
                    tmem_ld32(tmem + lane_off + region + ch * kAtChunk + 32 * q4, r);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int c = ch * kAtChunk + 32 * q4 + i;
                        float v = __uint_as_float(r[i]);
                        if (bm) v += __ldg(bm + c);
                        const bool gt = v > best;
                        second = gt ? best : fmaxf(second, v);
                        bidx = gt ? c : bidx;
                        best = gt ? v : best;
                    }
                }
            }
            if (!ok) break;
            int code = bidx;
            const bool flagged = valid && !(best - second > thr);
            unsigned fl = __ballot_sync(0xffffffffu, flagged);
            if (fl) {
                // candidate bit-mask of this thread's own row: codes within thr of the best
                uint32_t mask[kAtMaxK / 32];
#pragma unroll
                for (int w = 0; w < kAtMaxK / 32; ++w) {
                    mask[w] = 0;
                    if (w * 32 < K) {
                        uint32_t r[32];
                        tmem_ld32(tmem + lane_off + region + w * 32, r);
                        tc_wait_ld();
                        uint32_t bits = 0;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float v = __uint_as_float(r[i]);
                            if (bm) v += __ldg(bm + w * 32 + i);
                            if (v >= best - thr) bits |= 1u << i;
                        }
                        mask[w] = bits;
                    }
                }
                while (fl) {
                    const int src = __ffs(fl) - 1;
                    fl &= fl - 1;
                    const int64_t js = __shfl_sync(0xffffffffu, j, src);
                    int pv[kAtMaxM];
#pragma unroll
                    for (int mm = 0; mm < kAtMaxM; ++mm) pv[mm] = __shfl_sync(0xffffffffu, prev[mm], src);
                    const __nv_bfloat16 *ks = p.k + b * p.k_sb + h * p.k_sh + js * p.k_sl;
                    // the warp forms the exact residual r_m = ((k - C_0[c_0]) - C_1[c_1]) - ... (4 columns per lane)
                    __syncwarp();
                    if (lane * 4 < D) {
                        const uint2 raw = *reinterpret_cast<const uint2 *>(ks + lane * 4);
                        const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x);
                        const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
                        float4 r4 = make_float4(__low2float(lo2), __high2float(lo2), __low2float(hi2), __high2float(hi2));
#pragma unroll
                        for (int mm = 0; mm < kAtMaxM; ++mm)
                            if (mm < m) {
                                const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cbh + (static_cast<int64_t>(mm) * K + pv[mm]) * D + lane * 4));
                                r4.x = __fsub_rn(r4.x, c4.x);
                                r4.y = __fsub_rn(r4.y, c4.y);
                                r4.z = __fsub_rn(r4.z, c4.z);
                                r4.w = __fsub_rn(r4.w, c4.w);
                            }
                        *reinterpret_cast<float4 *>(&s_res[warp][lane * 4]) = r4;
                    }
                    __syncwarp();
                    float bv = -INFINITY;
                    int bi = 0x7fffffff;
#pragma unroll
                    for (int w = 0; w < kAtMaxK / 32; ++w) {
                        const uint32_t word = __shfl_sync(0xffffffffu, mask[w], src);
                        if ((word >> lane) & 1u) {
                            const int c = w * 32 + lane;
                            float s = exact_chain<D>(&s_res[warp][0], cbh + (static_cast<int64_t>(m) * K + c) * D);
                            if (bm) s = __fadd_rn(s, __ldg(bm + c));
                            if (s > bv || (s == bv && c < bi)) {
                                bv = s;
                                bi = c;
                            }
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
                    if (lane == src && bi != 0x7fffffff) code = bi;
                }
            }
#pragma unroll
            for (int mm = 0; mm < kAtMaxM; ++mm)
                if (mm == m) prev[mm] = code;
            if (valid) store_code(p.codes, p.code_dtype, b * p.c_sb + h * p.c_sh + j * p.c_sl + m, code);
            qbound += cm;
            if (m + 1 < M) {
                // ---- q += C_m[code], re-split into bf16 hi / lo, written in the 128B-swizzled operand layout.
                // The warp walks its 32 rows together: lane l owns columns 4l..4l+3 of every row, so the
                // codeword rows are read with coalesced 16-byte loads.
                {
                    const int col = (lane * 4) % D, hh = col >> 6, ch8 = (col & 63) >> 3, sub8 = (col & 7) * 2;
#pragma unroll 8
                    for (int rr = 0; rr < 32; ++rr) {
                        const int r_row = warp * 32 + rr;
                        const int r_code = __shfl_sync(0xffffffffu, code, rr);
                        if (lane * 4 >= D) continue;  // D = 64: half of the lanes have no column
                        const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cbh + (static_cast<int64_t>(m) * K + r_code) * D + col));
                        const uint32_t off = hh * kHalfBytes + r_row * 128 + ((ch8 ^ (r_row & 7)) << 4) + sub8;
                        uint2 *ph = reinterpret_cast<uint2 *>(smem + C::kAqh + off);
                        uint2 *pl = reinterpret_cast<uint2 *>(smem + C::kAql + off);
                        float q[4] = {0.f, 0.f, 0.f, 0.f};
                        if (m > 0) {
                            const uint2 vh = *ph, vl = *pl;
                            const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&vh);
                            const __nv_bfloat162 *l2 = reinterpret_cast<const __nv_bfloat162 *>(&vl);
                            q[0] = __low2float(h2[0]) + __low2float(l2[0]);
                            q[1] = __high2float(h2[0]) + __high2float(l2[0]);
                            q[2] = __low2float(h2[1]) + __low2float(l2[1]);
                            q[3] = __high2float(h2[1]) + __high2float(l2[1]);
                        }
                        q[0] += c4.x; q[1] += c4.y; q[2] += c4.z; q[3] += c4.w;
                        uint32_t wh[2], wl[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const __nv_bfloat16 h0 = __float2bfloat16_rn(q[2 * e]), h1 = __float2bfloat16_rn(q[2 * e + 1]);
                            __nv_bfloat162 hv = __halves2bfloat162(h0, h1);
                            wh[e] = *reinterpret_cast<uint32_t *>(&hv);
                            wl[e] = pack_bf16(q[2 * e] - __bfloat162float(h0), q[2 * e + 1] - __bfloat162float(h1));
                        }
                        *ph = make_uint2(wh[0], wh[1]);
                        *pl = make_uint2(wl[0], wl[1]);
                    }
                }
                fence_proxy_async_smem();
                tc_fence_before();
                mbar_arrive(&bar_q);
            }
        }
        if (!ok) s_err = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (s_err && tid == 0) {
        if (p.status) atomicExch(p.status, 3);
        for (int w = 0; w < (1 << 14); ++w) __nanosleep(256);  // let tile loads in flight land
    }
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tmem_dealloc(tmem, tmem_cols);
    }
}

template <int D>
static int launch_assign_tc(const VqTensorDesc *k, const VqTensorDesc *cb, const VqTensorDesc *bias, VqTensorDesc *codes,
                            void *workspace, int32_t *status, cudaStream_t stream)
{
    using C = AtCfg<D>;
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
    if (!map_bhld(&mk, *k) || !make_map(&mhi, hi, 3, cd, cs) || !make_map(&mlo, lo, 3, cd, cs)) return VQ_ELAUNCH;
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
    p.status = status;
    auto kern = assign_tc_kernel<D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal) != cudaSuccess) return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>((L + kBlock - 1) / kBlock), static_cast<unsigned>(B * Hkv));
    kern<<<grid, kAtThreads, C::kTotal, stream>>>(mk, mhi, mlo, p);
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
                             K % kAtChunk == 0 && K <= kAtMaxK && k->stride[0] % 8 == 0 && k->stride[1] % 8 == 0 &&
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
    return D == 64 ? launch_assign_tc<64>(k, codebooks, bias, codes, workspace, status_word, s)
                   : launch_assign_tc<128>(k, codebooks, bias, codes, workspace, status_word, s);
}
