// Fused VQ-attention prefill, fp32 arithmetic on the regular cores (any activation dtype).
//
// This is the full-precision form of the fused kernel: it serves fp32 inputs (whose tolerance a
// 16-bit tensor-core product cannot meet) and is the on-device cross-check of the tensor-core
// kernel.  One warp owns one query row and runs ONE online softmax over, in this order,
//   the far pseudo-keys   (q2 . codebook[r], weight cnt[r], value vsum[r])   ops/triton_fused_vq_attn.py:38-68
//   the boundary keys     (q2 . k3)            ops/triton_fused_local_attn_rerope.py:68-75
//   the window keys       (q1 . k1, causal)    ops/triton_fused_local_attn_rerope.py:45-49,76-78
// 32 keys per step: each lane scores one key (full dot product), the warp agrees on the new
// maximum, then the lanes switch to owning D/32 output columns for the value update.
#include "vq_common.cuh"

namespace vq {

constexpr int kSimtWarps = 4;

template <typename T, int D> struct RowDot;
template <int D> struct RowDot<float, D> {
    static __device__ __forceinline__ float dot(const float *__restrict__ q, const float *__restrict__ k)
    {
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < D; d += 4) {
            const float4 kv = *reinterpret_cast<const float4 *>(k + d);
            const float4 qv = *reinterpret_cast<const float4 *>(q + d);
            s = fmaf(qv.x, kv.x, s);
            s = fmaf(qv.y, kv.y, s);
            s = fmaf(qv.z, kv.z, s);
            s = fmaf(qv.w, kv.w, s);
        }
        return s;
    }
};
template <int D> struct RowDot<__nv_bfloat16, D> {
    static __device__ __forceinline__ float dot(const float *__restrict__ q, const __nv_bfloat16 *__restrict__ k)
    {
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < D; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(k + d);
            const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
            const float4 qa = *reinterpret_cast<const float4 *>(q + d);
            const float4 qb = *reinterpret_cast<const float4 *>(q + d + 4);
            s = fmaf(qa.x, __low2float(h[0]), s);
            s = fmaf(qa.y, __high2float(h[0]), s);
            s = fmaf(qa.z, __low2float(h[1]), s);
            s = fmaf(qa.w, __high2float(h[1]), s);
            s = fmaf(qb.x, __low2float(h[2]), s);
            s = fmaf(qb.y, __high2float(h[2]), s);
            s = fmaf(qb.z, __low2float(h[3]), s);
            s = fmaf(qb.w, __high2float(h[3]), s);
        }
        return s;
    }
};

template <int D> struct RowDot<__half, D> {
    static __device__ __forceinline__ float dot(const float *__restrict__ q, const __half *__restrict__ k)
    {
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < D; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(k + d);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 kk = Pair16<__half>::unpack(w[i]);
                s = fmaf(q[d + 2 * i], kk.x, s);
                s = fmaf(q[d + 2 * i + 1], kk.y, s);
            }
        }
        return s;
    }
};

struct SimtPrefillParams {
    const void *q1, *q2, *k1, *k3, *v, *codebook, *vsum;
    const float *cnt;
    void *out;
    float *lse2;
    int64_t q_sb, q_sh, q_sl;      // q1/q2/out strides (elements)
    int64_t q2_sb, q2_sh, q2_sl;
    int64_t o_sb, o_sh, o_sl;
    int64_t k_sb, k_sh, k_sl;      // k1
    int64_t k3_sb, k3_sh, k3_sl;
    int64_t v_sb, v_sh, v_sl;
    int Hq, Hkv, MK, NB;
    int64_t L, window;
    float scale_log2;
};

template <typename T, int D>
struct OnlineRow {
    float m, l;
    float acc[D / 32];
    int lane;

    __device__ __forceinline__ void init(int ln)
    {
        m = -INFINITY;
        l = 0.f;
        lane = ln;
#pragma unroll
        for (int t = 0; t < D / 32; ++t) acc[t] = 0.f;
    }

    // rows [0,n) of K (row stride ks) scored against q (shared memory, fp32); values from V (row stride vs);
    // w: per-row weights (far counts) or nullptr.
    __device__ __forceinline__ void segment(const float *q, const T *K, int64_t ks, const T *V, int64_t vs, int64_t n,
                                            const float *w, float scale_log2)
    {
        for (int64_t base = 0; base < n; base += 32) {
            const int64_t r = base + lane;
            float s = -INFINITY, wt = 1.f;
            if (r < n) {
                if (w) wt = w[r];
                if (wt > 0.f) s = scale_log2 * RowDot<T, D>::dot(q, K + r * ks);
            }
            float cmax = s;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, off));
            if (cmax == -INFINITY) continue;  // nothing to attend to in this step (warp-uniform)
            const float m_new = fmaxf(m, cmax);
            const float alpha = exp2f(m - m_new);  // m = -inf -> 0
            const float p = exp2f(s - m_new);      // s = -inf -> 0
            float psum = p * wt;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
            l = l * alpha + psum;
            m = m_new;
#pragma unroll
            for (int t = 0; t < D / 32; ++t) acc[t] *= alpha;
            const int cnt_rows = static_cast<int>(n - base < 32 ? n - base : 32);
            for (int jj = 0; jj < cnt_rows; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                if (pj == 0.f) continue;
                const T *vr = V + (base + jj) * vs;
#pragma unroll
                for (int t = 0; t < D / 32; ++t) acc[t] = fmaf(pj, to_f32(vr[lane + 32 * t]), acc[t]);
            }
        }
    }
};

template <typename T, int D>
__global__ void __launch_bounds__(kSimtWarps * 32) prefill_simt_kernel(SimtPrefillParams p)
{
    __shared__ __align__(16) float s_q[kSimtWarps][2][D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * kSimtWarps + warp;
    const int bh = blockIdx.y;
    const int b = bh / p.Hq, hq = bh % p.Hq;
    const int hk = hq / (p.Hq / p.Hkv);
    const int64_t u = static_cast<int64_t>(b) * p.Hkv + hk;
    if (i >= p.L) return;  // whole warp leaves together

    const T *q1 = static_cast<const T *>(p.q1) + b * p.q_sb + hq * p.q_sh + i * p.q_sl;
    const T *q2 = static_cast<const T *>(p.q2) + b * p.q2_sb + hq * p.q2_sh + i * p.q2_sl;
    for (int d = lane; d < D; d += 32) {
        s_q[warp][0][d] = to_f32(q1[d]);
        s_q[warp][1][d] = to_f32(q2[d]);
    }
    __syncwarp();

    const int64_t W = p.window;
    const int64_t lb = i - W > 0 ? i - W : 0;
    const int64_t bd = i - W > 0 ? ((i - W) / kBlock) * kBlock : 0;

    OnlineRow<T, D> st;
    st.init(lane);

    const T *k1 = static_cast<const T *>(p.k1) + b * p.k_sb + hk * p.k_sh;
    const T *k3 = static_cast<const T *>(p.k3) + b * p.k3_sb + hk * p.k3_sh;
    const T *v = static_cast<const T *>(p.v) + b * p.v_sb + hk * p.v_sh;

    if (bd > 0 && p.MK > 0) {
        const int64_t blk = bd / kBlock - 1;
        const T *cbk = static_cast<const T *>(p.codebook) + static_cast<int64_t>(hk) * p.MK * D;
        const T *vs = static_cast<const T *>(p.vsum) + (u * p.NB + blk) * p.MK * D;
        const float *cn = p.cnt + (u * p.NB + blk) * p.MK;
        st.segment(s_q[warp][1], cbk, D, vs, D, p.MK, cn, p.scale_log2);
    }
    if (lb > bd) st.segment(s_q[warp][1], k3 + bd * p.k3_sl, p.k3_sl, v + bd * p.v_sl, p.v_sl, lb - bd, nullptr, p.scale_log2);
    st.segment(s_q[warp][0], k1 + lb * p.k_sl, p.k_sl, v + lb * p.v_sl, p.v_sl, i - lb + 1, nullptr, p.scale_log2);

    T *o = static_cast<T *>(p.out) + b * p.o_sb + hq * p.o_sh + i * p.o_sl;
    const float inv = 1.f / st.l;
#pragma unroll
    for (int t = 0; t < D / 32; ++t) o[lane + 32 * t] = from_f32<T>(st.acc[t] * inv);
    if (p.lse2 && lane == 0) p.lse2[static_cast<int64_t>(bh) * p.L + i] = st.m + log2f(st.l);
}

int launch_prefill_simt(const VqPrefillArgs *a, cudaStream_t stream)
{
    SimtPrefillParams p{};
    p.q1 = a->q1.ptr; p.q2 = a->q2.ptr; p.k1 = a->k1.ptr; p.k3 = a->k3.ptr; p.v = a->v.ptr;
    p.codebook = a->codebook.ptr; p.vsum = a->vsum.ptr; p.cnt = static_cast<const float *>(a->cnt.ptr);
    p.out = a->out.ptr; p.lse2 = static_cast<float *>(a->lse2.ptr);
    p.q_sb = a->q1.stride[0]; p.q_sh = a->q1.stride[1]; p.q_sl = a->q1.stride[2];
    p.q2_sb = a->q2.stride[0]; p.q2_sh = a->q2.stride[1]; p.q2_sl = a->q2.stride[2];
    p.o_sb = a->out.stride[0]; p.o_sh = a->out.stride[1]; p.o_sl = a->out.stride[2];
    p.k_sb = a->k1.stride[0]; p.k_sh = a->k1.stride[1]; p.k_sl = a->k1.stride[2];
    p.k3_sb = a->k3.stride[0]; p.k3_sh = a->k3.stride[1]; p.k3_sl = a->k3.stride[2];
    p.v_sb = a->v.stride[0]; p.v_sh = a->v.stride[1]; p.v_sl = a->v.stride[2];
    p.Hq = static_cast<int>(a->q1.shape[1]); p.Hkv = static_cast<int>(a->k1.shape[1]);
    p.L = a->q1.shape[2];
    p.MK = a->codebook.ptr ? static_cast<int>(a->codebook.shape[1]) : 0;
    p.NB = a->cnt.ptr ? static_cast<int>(a->cnt.shape[2]) : 0;
    p.window = a->window;
    const int D = static_cast<int>(a->q1.shape[3]);
    const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(D));
    p.scale_log2 = scale * 1.4426950408889634f;
    const int64_t B = a->q1.shape[0];
    dim3 grid(static_cast<unsigned>((p.L + kSimtWarps - 1) / kSimtWarps), static_cast<unsigned>(B * p.Hq));
    if (a->q1.dtype == VQ_F32) {
        if (D == 64) prefill_simt_kernel<float, 64><<<grid, kSimtWarps * 32, 0, stream>>>(p);
        else prefill_simt_kernel<float, 128><<<grid, kSimtWarps * 32, 0, stream>>>(p);
    } else if (a->q1.dtype == VQ_F16) {
        if (D == 64) prefill_simt_kernel<__half, 64><<<grid, kSimtWarps * 32, 0, stream>>>(p);
        else prefill_simt_kernel<__half, 128><<<grid, kSimtWarps * 32, 0, stream>>>(p);
    } else {
        if (D == 64) prefill_simt_kernel<__nv_bfloat16, 64><<<grid, kSimtWarps * 32, 0, stream>>>(p);
        else prefill_simt_kernel<__nv_bfloat16, 128><<<grid, kSimtWarps * 32, 0, stream>>>(p);
    }
    return launch_status();
}

}  // namespace vq
