// Shared pieces of the decode kernels: 16-byte row slices, kernel parameters, the running softmax
// state of a lane group and the CTA epilogue (merge lane groups -> warps -> splits).
#pragma once

#include "vq_common.cuh"

namespace vq {

constexpr int kDecThreads = 256;   // consumer threads (8 warps)
constexpr int kDecMaxSplits = 16;

template <typename TR> struct Slice;  // 16-byte slice of a row as floats
template <> struct Slice<float> {
    static constexpr int E = 4;
    static __device__ __forceinline__ void ld(const float *p, float (&x)[4])
    {
        const float4 v = __ldcs(reinterpret_cast<const float4 *>(p));
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
    static __device__ __forceinline__ void ld_cached(const float *p, float (&x)[4])
    {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
};
template <> struct Slice<__nv_bfloat16> {
    static constexpr int E = 8;
    static __device__ __forceinline__ void unpack(const uint4 &raw, float (&x)[8])
    {
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __low2float(h[i]);
            x[2 * i + 1] = __high2float(h[i]);
        }
    }
    static __device__ __forceinline__ void ld(const __nv_bfloat16 *p, float (&x)[8])
    {
        unpack(__ldcs(reinterpret_cast<const uint4 *>(p)), x);
    }
    static __device__ __forceinline__ void ld_cached(const __nv_bfloat16 *p, float (&x)[8])
    {
        unpack(__ldg(reinterpret_cast<const uint4 *>(p)), x);
    }
};

template <> struct Slice<__half> {
    static constexpr int E = 8;
    static __device__ __forceinline__ void unpack(const uint4 &raw, float (&x)[8])
    {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = Pair16<__half>::unpack(w[i]);
            x[2 * i] = t.x;
            x[2 * i + 1] = t.y;
        }
    }
    static __device__ __forceinline__ void ld(const __half *p, float (&x)[8]) { unpack(__ldcs(reinterpret_cast<const uint4 *>(p)), x); }
    static __device__ __forceinline__ void ld_cached(const __half *p, float (&x)[8]) { unpack(__ldg(reinterpret_cast<const uint4 *>(p)), x); }
};

struct DecodeParams {
    const void *q1, *q2, *k1w, *k3w, *vw, *codebook, *vsum;
    const float *cnt;
    void *out;
    float *partial;   // [units][G][splits][D + 2]
    int *ticket;      // [units * head_groups]
    int64_t q_sb, q_sh, q2_sb, q2_sh, o_sb, o_sh;
    int64_t k_sb, k_sh, k_sl, k3_sb, k3_sh, k3_sl, v_sb, v_sh, v_sl;
    int Hq, Hkv, G, MK, n_valid, n_bd, use_far, splits, rows_w, rows_f;
    float scale_log2;
};

// Running softmax state of one lane group: GH heads, E output columns per lane.
template <int GH, int E>
struct DecState {
    float m[GH], l[GH], acc[GH][E];
    __device__ __forceinline__ void init()
    {
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
        }
    }
    // one row: score s (already scaled, -inf = masked), denominator weight w, value slice x
    __device__ __forceinline__ void update(int g, float s, float w, const float (&x)[E])
    {
        const float mn = fmaxf(m[g], s);
        if (mn == -INFINITY) return;
        const float alpha = exp2f(m[g] - mn);
        const float pp = exp2f(s - mn);
        l[g] = fmaf(l[g], alpha, pp * w);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[g][e] = fmaf(acc[g][e], alpha, pp * x[e]);
        m[g] = mn;
    }
    // merge the state held by another lane (xor distance `off`)
    __device__ __forceinline__ void merge_xor(int off)
    {
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            const float om = __shfl_xor_sync(0xffffffffu, m[g], off);
            const float ol = __shfl_xor_sync(0xffffffffu, l[g], off);
            const float mn = fmaxf(m[g], om);
            const float a = (mn == -INFINITY) ? 0.f : exp2f(m[g] - mn);
            const float b = (mn == -INFINITY) ? 0.f : exp2f(om - mn);
            l[g] = l[g] * a + ol * b;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const float oa = __shfl_xor_sync(0xffffffffu, acc[g][e], off);
                acc[g][e] = acc[g][e] * a + oa * b;
            }
            m[g] = mn;
        }
    }
};


// CTA epilogue shared by the decode kernels.  Warps [0, NW) hold a DecState each (already merged
// across their lane groups: lanes [0, LPR) own the D columns); other warps only take part in the
// barriers.  Writes the CTA's partial (numerator, max, denominator) to the workspace, takes a ticket,
// and the last CTA of the unit merges all splits into the output row and re-arms the ticket.
template <typename T, int D, int GH, int NW, int E>
__device__ __forceinline__ void decode_finish(const DecodeParams &p, DecState<GH, E> &st, float *s_red /*[NW*GH*(D+2)]*/,
                                              int *s_last, int split, int hg, int u, int b, int hq0)
{
    constexpr int LPR = D / E;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nthreads = blockDim.x;
    if (warp < NW && lane < LPR) {
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            float *dst = s_red + (warp * GH + g) * (D + 2);
#pragma unroll
            for (int e = 0; e < E; ++e) dst[lane * E + e] = st.acc[g][e];
            if (lane == 0) {
                dst[D] = st.m[g];
                dst[D + 1] = st.l[g];
            }
        }
    }
    __syncthreads();
    // partial[(u*G + head)][split][D+2]
    float *part = p.partial + ((static_cast<int64_t>(u) * p.G + hg * GH) * p.splits) * (D + 2);
    for (int i = tid; i < GH * (D + 1); i += nthreads) {
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
        float *dst = part + (static_cast<int64_t>(g) * p.splits + split) * (D + 2);
        if (d < D) dst[d] = x;
        else {
            dst[D] = M;
            dst[D + 1] = x;
        }
    }
    __threadfence();
    __syncthreads();
    int *ticket = p.ticket + u * gridDim.y + hg;
    if (tid == 0) {
        const int t = atomicAdd(ticket, 1);
        *s_last = (t == p.splits - 1);
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    for (int i = tid; i < GH * D; i += nthreads) {
        const int g = i / D, d = i % D;
        const float *pg = part + static_cast<int64_t>(g) * p.splits * (D + 2);
        float M = -INFINITY;
        for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(pg + s * (D + 2) + D));
        float num = 0.f, den = 0.f;
        for (int s = 0; s < p.splits; ++s) {
            const float ms = __ldcg(pg + s * (D + 2) + D);
            const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
            num += w * __ldcg(pg + s * (D + 2) + d);
            den += w * __ldcg(pg + s * (D + 2) + D + 1);
        }
        static_cast<T *>(p.out)[b * p.o_sb + (hq0 + g) * p.o_sh + d] = from_f32<T>(num / den);
    }
    if (tid == 0) *ticket = 0;  // ready for the next call on this stream
}

}  // namespace vq
