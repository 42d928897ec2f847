// Fused VQ-attention prefill on the sm_100a tensor cores (bf16 operands, fp32 accumulation).
//
// One CTA owns one 128-row query tile of one (batch, query head) and walks a list of 128-wide
// work items with ONE online softmax (this replaces the far kernel, the local ReRoPE kernel and the
// log-sum-exp merge of the reference: ops/triton_fused_vq_attn.py:88-251,
// ops/triton_fused_local_attn_rerope.py:121-226):
//   FAR    q2 . codebook tile       value = vsum tile of the block   weights cnt   (:38-68)
//   BD_A   q2 . k3 (boundary block) keys older than the window      (rerope mode)  (:68-75)
//   BD_B   q1 . k1 (boundary block) keys inside the window
//   FULL   q1 . k1 interior block, no mask
//   DIAG   q1 . k1 diagonal block, causal mask                                        (:76-78)
// Per item: TMA loads the K-like and V-like tiles (128B-swizzled) into a 2-stage ring,
// tcgen05.mma forms S = Q K^T in tensor memory, the four warps read their rows of S with
// tcgen05.ld (one thread = one query row), apply mask / max / exp2, write P back to tensor memory
// as packed bf16, rescale the accumulator O when the row maximum moved, and a second tcgen05.mma
// (A = P from tensor memory, B = V tile, MN-major) adds P V into O.
#include "prefill_tc_common.cuh"

namespace vq {

using namespace ptx;

constexpr int kTcThreads = 128;

// TMEM column map: S fp32 [0,128), P bf16x2 [128,192), O fp32 [kColO, kColO+D)
constexpr uint32_t kColS = 0, kColP = 128;
template <int D> struct TcTmem {
    static constexpr uint32_t kColO = D == 128 ? 256 : 192;
    static constexpr uint32_t kCols = D == 128 ? 512 : 256;  // power of two >= kColO + D
};

template <int D>
struct TcSmem {
    static constexpr int NH = D / 64;
    static constexpr int kTile = NH * kHalfBytes;       // bytes of one 128 x D bf16 tile
    static constexpr int kQ1 = 0, kQ2 = kTile;
    static constexpr int kStage0 = 2 * kTile;           // per stage: K tile then V tile
    static constexpr int kStageBytes = 2 * kTile;
    static constexpr int kTotal = kStage0 + 2 * kStageBytes + 1024;  // + slack for 1024-byte alignment
};

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                  const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k3,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_cb,
                  const __grid_constant__ CUtensorMap tm_vs, TcParams p)
{
    using SM = TcSmem<D>;
    constexpr int NH = SM::NH;
    constexpr uint32_t kColO = TcTmem<D>::kColO, kTmemCols = TcTmem<D>::kCols;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bar_q, bar_kv[2], bar_s, bar_o;
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;
    __shared__ __align__(16) float s_cnt[2][kBlock];

    const int tid = threadIdx.x, warp = tid >> 5;
    const int m = p.ntiles - 1 - static_cast<int>(blockIdx.x);  // heavy tiles first
    const int bh = blockIdx.y;
    const int b = bh / p.Hq, hq = bh % p.Hq;
    const int hk = hq / (p.Hq / p.Hkv);
    const int u = b * p.Hkv + hk;

    const TcWork work(p, m);
    const int n_items = work.n_items, far_blk = work.far_blk;
    auto item_kind = [&](int it) -> int { return work.kind(it); };
    auto item_block = [&](int it) -> int { return work.block(it); };

    if (tid == 0) {
        mbar_init(&bar_q, 1);
        mbar_init(&bar_kv[0], 1);
        mbar_init(&bar_kv[1], 1);
        mbar_init(&bar_s, 1);
        mbar_init(&bar_o, 1);
        fence_mbar_init();
        s_err = 0;
        prefetch_tmap(&tm_q1); prefetch_tmap(&tm_q2); prefetch_tmap(&tm_k1); prefetch_tmap(&tm_k3);
        prefetch_tmap(&tm_v); prefetch_tmap(&tm_cb); prefetch_tmap(&tm_vs);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(&s_tmem, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    // producer: issue the loads of item `it` into stage `st`
    auto issue_item = [&](int it, int st) {
        const int kind = item_kind(it), blk = item_block(it);
        uint8_t *kdst = smem + SM::kStage0 + st * SM::kStageBytes;
        uint8_t *vdst = kdst + SM::kTile;
        mbar_expect_tx(&bar_kv[st], 2 * SM::kTile);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            if (kind == kFar) {
                tma_load_3d(kdst + h * kHalfBytes, &tm_cb, &bar_kv[st], 64 * h, blk * kBlock, hk);
                tma_load_3d(vdst + h * kHalfBytes, &tm_vs, &bar_kv[st], 64 * h, blk * kBlock, u * p.NB + far_blk);
            } else {
                tma_load_4d(kdst + h * kHalfBytes, kind == kBdA ? &tm_k3 : &tm_k1, &bar_kv[st], 64 * h, blk * kBlock, hk, b);
                tma_load_4d(vdst + h * kHalfBytes, &tm_v, &bar_kv[st], 64 * h, blk * kBlock, hk, b);
            }
        }
    };

    if (tid == 0) {
        mbar_expect_tx(&bar_q, (p.rerope ? 2 : 1) * SM::kTile);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            tma_load_4d(smem + SM::kQ1 + h * kHalfBytes, &tm_q1, &bar_q, 64 * h, m * kBlock, hq, b);
            if (p.rerope) tma_load_4d(smem + SM::kQ2 + h * kHalfBytes, &tm_q2, &bar_q, 64 * h, m * kBlock, hq, b);
        }
        issue_item(0, 0);
    }

    const uint32_t q1_addr = smem_u32(smem + SM::kQ1);
    const uint32_t q2_addr = p.rerope ? smem_u32(smem + SM::kQ2) : q1_addr;
    constexpr uint32_t idesc_qk = idesc_bf16(128, 128, 0, 0);
    constexpr uint32_t idesc_pv = idesc_bf16(128, D, 0, 1);
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;  // this warp's TMEM lanes

    float row_m = -INFINITY, row_l = 0.f;
    bool ok = true;
    if (!mbar_wait(&bar_q, 0)) ok = false;

    for (int it = 0; it < n_items; ++it) {
        const int st = it & 1;
        const int kind = item_kind(it), blk = item_block(it);
        const uint32_t kv_parity = (it >> 1) & 1, it_parity = it & 1;
        // prefetch the next item: its stage was last read by the PV product of item it-1, already complete
        if (tid == 0 && it + 1 < n_items) issue_item(it + 1, st ^ 1);
        if (kind == kFar)
            s_cnt[st][tid] = p.cnt[(static_cast<int64_t>(u) * p.NB + far_blk) * p.MK + blk * kBlock + tid];

        // ---- S = Q K^T ----
        if (tid == 0) {
            if (!mbar_wait(&bar_kv[st], kv_parity)) ok = false;
            tc_fence_after();
            const uint32_t qa = (kind == kFar || kind == kBdA) ? q2_addr : q1_addr;
            const uint32_t ka = smem_u32(smem + SM::kStage0 + st * SM::kStageBytes);
#pragma unroll
            for (int h = 0; h < NH; ++h)
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    const uint64_t ad = smem_desc_sw128(qa + h * kHalfBytes + k4 * 32, 16, 1024);
                    const uint64_t bd = smem_desc_sw128(ka + h * kHalfBytes + k4 * 32, 16, 1024);
                    mma_ss(tmem + kColS, ad, bd, idesc_qk, (h | k4) ? 1u : 0u);
                }
            tc_commit(&bar_s);
        }
        __syncthreads();  // s_cnt visible; also orders the producer's error flag
        if (!mbar_wait(&bar_s, it_parity)) ok = false;
        tc_fence_after();

        // ---- softmax on this thread's row ----
        float s[kBlock];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_off + kColS + 32 * c, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) s[32 * c + j] = __uint_as_float(r[j]);
        }
        // column window of valid keys for this row: [lo, hi)
        int lo = 0, hi = kBlock;
        if (kind == kDiag) hi = tid + 1;
        else if (kind == kBdA) hi = tid;
        else if (kind == kBdB) lo = tid;
        float mx = -INFINITY;
        if (kind == kFar) {
#pragma unroll
            for (int c = 0; c < kBlock; ++c) {
                if (!(s_cnt[st][c] > 0.f)) s[c] = -INFINITY;
                mx = fmaxf(mx, s[c]);
            }
        } else if (kind == kFull) {
#pragma unroll
            for (int c = 0; c < kBlock; ++c) mx = fmaxf(mx, s[c]);
        } else {
#pragma unroll
            for (int c = 0; c < kBlock; ++c) {
                if (c < lo || c >= hi) s[c] = -INFINITY;
                mx = fmaxf(mx, s[c]);
            }
        }
        const float m_new = fmaxf(row_m, mx * p.scale_log2);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = ex2(row_m - m_safe);  // row_m = -inf -> 0
        float lsum = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float p0 = ex2(fmaf(s[32 * c + 2 * j], p.scale_log2, -m_safe));
                const float p1 = ex2(fmaf(s[32 * c + 2 * j + 1], p.scale_log2, -m_safe));
                if (kind == kFar) {
                    lsum = fmaf(p0, s_cnt[st][32 * c + 2 * j], lsum);
                    lsum = fmaf(p1, s_cnt[st][32 * c + 2 * j + 1], lsum);
                } else {
                    lsum += p0 + p1;
                }
                pk[j] = pack_bf16(p0, p1);
            }
            tmem_st16(tmem + lane_off + kColP + 16 * c, pk);
        }
        row_l = row_l * alpha + lsum;
        row_m = m_new;
        // ---- rescale O where the maximum moved (O is idle: the previous P V product has completed) ----
        if (it > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_off + kColO + 32 * c, r);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                tmem_st32(tmem + lane_off + kColO + 32 * c, r);
            }
        }
        tc_wait_st();
        tc_fence_before();
        __syncthreads();

        // ---- O += P V ----
        if (tid == 0) {
            tc_fence_after();
            const uint32_t va = smem_u32(smem + SM::kStage0 + st * SM::kStageBytes + SM::kTile);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint64_t bd = smem_desc_sw128(va + kk * 2048, kHalfBytes, 1024);
                mma_ts(tmem + kColO, tmem + kColP + 8 * kk, bd, idesc_pv, (it | kk) ? 1u : 0u);
            }
            tc_commit(&bar_o);
        }
        if (!mbar_wait(&bar_o, it_parity)) ok = false;
        tc_fence_after();
        if (!ok) s_err = 1;
        __syncthreads();
        if (s_err) break;
    }

    // ---- epilogue: out = O / l ----
    if (!s_err) {
        const int64_t row = static_cast<int64_t>(m) * kBlock + tid;
        const float inv = 1.f / row_l;
        __nv_bfloat16 *o = p.out + b * p.o_sb + hq * p.o_sh + row * p.o_sl;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            __syncwarp();
            tmem_ld32(tmem + lane_off + kColO + 32 * c, r);
            tc_wait_ld();
            if (row < p.L) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 w;
                    w.x = pack_bf16(__uint_as_float(r[8 * j + 0]) * inv, __uint_as_float(r[8 * j + 1]) * inv);
                    w.y = pack_bf16(__uint_as_float(r[8 * j + 2]) * inv, __uint_as_float(r[8 * j + 3]) * inv);
                    w.z = pack_bf16(__uint_as_float(r[8 * j + 4]) * inv, __uint_as_float(r[8 * j + 5]) * inv);
                    w.w = pack_bf16(__uint_as_float(r[8 * j + 6]) * inv, __uint_as_float(r[8 * j + 7]) * inv);
                    *reinterpret_cast<uint4 *>(o + 32 * c + 8 * j) = w;
                }
            }
        }
        if (p.lse2 && row < p.L) p.lse2[static_cast<int64_t>(bh) * p.L + row] = row_m + log2f(row_l);
    } else if (tid == 0) {
        if (p.status) atomicExch(p.status, 1);
        // a bounded wait expired: give the tile loads still in flight time to land before the
        // shared memory is handed back (a few milliseconds, then leave regardless)
#pragma unroll 1
        for (int w = 0; w < (1 << 14); ++w) __nanosleep(256);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem, kTmemCols);
    }
}

template <int D>
static int launch_tc(const VqPrefillArgs *a, cudaStream_t stream)
{
    using SM = TcSmem<D>;
    TcMaps m;
    TcParams p;
    const int st = tc_setup<D>(a, m, p);
    if (st != VQ_OK) return st;
    auto kern = prefill_tc_kernel<D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal) != cudaSuccess) return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>(p.ntiles), static_cast<unsigned>(a->q1.shape[0] * a->q1.shape[1]));
    kern<<<grid, kTcThreads, SM::kTotal, stream>>>(m.q1, m.q2, m.k1, m.k3, m.v, m.cb, m.vs, p);
    return launch_status();
}

// The serial form: one warpgroup does MMA issue, softmax and rescaling in turn (kept as a second
// implementation of the same arithmetic; the pipelined kernel is the default).
int launch_prefill_tensor_serial(const VqPrefillArgs *a, cudaStream_t stream)
{
    const int D = static_cast<int>(a->q1.shape[3]);
    if (a->out.stride[2] % 8 || a->out.stride[1] % 8 || a->out.stride[0] % 8) return VQ_EINVAL_STRIDE;
    return D == 64 ? launch_tc<64>(a, stream) : launch_tc<128>(a, stream);
}

}  // namespace vq
