// Single-query (seqlen_q == 1) VQ-attention decode: a bandwidth-bound stream over the exact window
// (bf16/f32 keys and values), the per-code value sums and counts, and the codebook.
//
// The reference has no working decode for its VQ cache (ops/attn_vq.py:128-165); the semantics are
// those of prefill row n-1 (ops/attn_vq.py:311-332): window rows scored q1.k1 (the first n_bd of
// them q2.k3), far pseudo-keys scored q2.codebook[r] with weight cnt[r] and value vsum[r].
//
// Work split: grid = (splits, head groups, batch*kv-head).  A CTA owns a contiguous share of the
// window rows and of the far rows of one (batch, kv head) and up to GH query heads of its group:
//   pass 1  every row is read once with 16-byte loads by a group of lanes (one row per group),
//           the dot products are reduced with shuffles, scores land in shared memory;
//   pass 2  block max, p = exp2(s - max), denominator (far rows weighted by cnt);
//   pass 3  value rows streamed the same way, fp32 accumulators in registers, reduced across
//           lane groups by shuffles and across warps in shared memory.
// Partial (max, denominator, numerator) triples go to a workspace; the last CTA of a unit to
// finish (atomic ticket) merges them and writes the output row, then re-arms the ticket.
#include "vq_common.cuh"

namespace vq {

constexpr int kDecThreads = 256;
constexpr int kDecMaxSplits = 16;
constexpr int kDecUnroll = 4;

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

// Scores rows [r0, r1) of `base` against GH query vectors held in shared memory (fp32, [GH][D]).
// s_out[g * sstride + (r - r0)] receives scale_log2 * q_g . row, or -inf where wts[r] <= 0.
template <typename TR, int D, int GH, bool kCached>
__device__ __forceinline__ void score_rows(const TR *__restrict__ base, int64_t row_stride, int r0, int r1,
                                           const float *__restrict__ qs, float *__restrict__ s_out, int sstride,
                                           float scale_log2, const float *__restrict__ wts)
{
    constexpr int E = Slice<TR>::E;
    constexpr int LPR = D / E;  // lanes per row
    constexpr int GROUPS = kDecThreads / LPR;
    const int gid = threadIdx.x / LPR, sub = threadIdx.x % LPR;
    float q[GH][E];
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
        for (int e = 0; e < E; ++e) q[g][e] = qs[g * D + sub * E + e];
    for (int rb = r0; rb < r1; rb += GROUPS * kDecUnroll) {
        float x[kDecUnroll][E];
        bool ok[kDecUnroll];
#pragma unroll
        for (int uu = 0; uu < kDecUnroll; ++uu) {
            const int r = rb + uu * GROUPS + gid;
            ok[uu] = r < r1;
            if (ok[uu]) {
                if (kCached) Slice<TR>::ld_cached(base + static_cast<int64_t>(r) * row_stride + sub * E, x[uu]);
                else Slice<TR>::ld(base + static_cast<int64_t>(r) * row_stride + sub * E, x[uu]);
            } else {
#pragma unroll
                for (int e = 0; e < E; ++e) x[uu][e] = 0.f;
            }
        }
#pragma unroll
        for (int uu = 0; uu < kDecUnroll; ++uu) {
            const int r = rb + uu * GROUPS + gid;
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < E; ++e) s = fmaf(q[g][e], x[uu][e], s);
#pragma unroll
                for (int off = LPR / 2; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                if (sub == 0 && ok[uu]) {
                    float val = s * scale_log2;
                    if (wts != nullptr && wts[r] <= 0.f) val = -INFINITY;
                    s_out[g * sstride + (r - r0)] = val;
                }
            }
        }
    }
}

// acc[g][e] += sum over rows [r0,r1) of p[g*sstride + (r-r0)] * row[r][sub*E + e]
template <typename TR, int D, int GH>
__device__ __forceinline__ void accum_rows(const TR *__restrict__ base, int64_t row_stride, int r0, int r1,
                                           const float *__restrict__ p, int sstride, float (&acc)[GH][Slice<TR>::E])
{
    constexpr int E = Slice<TR>::E;
    constexpr int LPR = D / E;
    constexpr int GROUPS = kDecThreads / LPR;
    const int gid = threadIdx.x / LPR, sub = threadIdx.x % LPR;
    for (int rb = r0; rb < r1; rb += GROUPS * kDecUnroll) {
        float x[kDecUnroll][E];
        bool ok[kDecUnroll];
#pragma unroll
        for (int uu = 0; uu < kDecUnroll; ++uu) {
            const int r = rb + uu * GROUPS + gid;
            ok[uu] = r < r1;
            if (ok[uu]) Slice<TR>::ld(base + static_cast<int64_t>(r) * row_stride + sub * E, x[uu]);
        }
#pragma unroll
        for (int uu = 0; uu < kDecUnroll; ++uu) {
            if (!ok[uu]) continue;
            const int r = rb + uu * GROUPS + gid;
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                const float pv = p[g * sstride + (r - r0)];
#pragma unroll
                for (int e = 0; e < E; ++e) acc[g][e] = fmaf(pv, x[uu][e], acc[g][e]);
            }
        }
    }
}

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

template <typename T, typename TC, int D, int GH>
__global__ void __launch_bounds__(kDecThreads) decode_kernel(DecodeParams p)
{
    constexpr int E = Slice<T>::E;
    constexpr int LPR = D / E;
    extern __shared__ __align__(16) float dsm[];
    // layout: q [2][GH][D] | scores [GH][rows_w + rows_f] | red [8][GH][D] | stats
    float *s_q = dsm;
    const int nrows = p.rows_w + p.rows_f;
    float *s_sc = s_q + 2 * GH * D;
    float *s_red = s_sc + GH * nrows;
    __shared__ float s_stat[kDecThreads / 32][GH];
    __shared__ float s_m[GH], s_l[GH];
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, hg = blockIdx.y, u = blockIdx.z;
    const int b = u / p.Hkv, hk = u % p.Hkv;
    const int hq0 = hk * p.G + hg * GH;

    for (int i = tid; i < GH * D; i += kDecThreads) {
        const int g = i / D, d = i % D;
        s_q[i] = to_f32(static_cast<const T *>(p.q1)[b * p.q_sb + (hq0 + g) * p.q_sh + d]);
        s_q[GH * D + i] = to_f32(static_cast<const T *>(p.q2)[b * p.q2_sb + (hq0 + g) * p.q2_sh + d]);
    }
    __syncthreads();

    // this CTA's share of the rows
    const int w0 = min(split * p.rows_w, p.n_valid), w1 = min(w0 + p.rows_w, p.n_valid);
    const int f0 = p.use_far ? min(split * p.rows_f, p.MK) : 0, f1 = p.use_far ? min(f0 + p.rows_f, p.MK) : 0;
    const int nw = w1 - w0, nf = f1 - f0;

    const T *k1w = static_cast<const T *>(p.k1w) + b * p.k_sb + hk * p.k_sh;
    const T *k3w = static_cast<const T *>(p.k3w) + b * p.k3_sb + hk * p.k3_sh;
    const T *vw = static_cast<const T *>(p.vw) + b * p.v_sb + hk * p.v_sh;
    const TC *cbk = static_cast<const TC *>(p.codebook) + static_cast<int64_t>(hk) * p.MK * D;
    const T *vs = static_cast<const T *>(p.vsum) + static_cast<int64_t>(u) * p.MK * D;
    const float *cn = p.cnt + static_cast<int64_t>(u) * p.MK;

    // ---- pass 1: scores ----
    {
        const int wb = min(max(p.n_bd, w0), w1);  // rows [w0,wb) use q2.k3, [wb,w1) use q1.k1
        if (wb > w0)
            score_rows<T, D, GH, false>(k3w, p.k3_sl, w0, wb, s_q + GH * D, s_sc, nrows, p.scale_log2, nullptr);
        if (w1 > wb)
            score_rows<T, D, GH, false>(k1w, p.k_sl, wb, w1, s_q, s_sc + (wb - w0), nrows, p.scale_log2, nullptr);
        if (nf > 0)
            score_rows<TC, D, GH, true>(cbk, D, f0, f1, s_q + GH * D, s_sc + nw, nrows, p.scale_log2, cn);
    }
    __syncthreads();

    // ---- pass 2: max, exponentials, denominator ----
    float mx[GH];
#pragma unroll
    for (int g = 0; g < GH; ++g) {
        float m = -INFINITY;
        for (int i = tid; i < nw + nf; i += kDecThreads) m = fmaxf(m, s_sc[g * nrows + i]);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        if (lane == 0) s_stat[warp][g] = m;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GH; ++g) {
        float m = s_stat[0][g];
#pragma unroll
        for (int w = 1; w < kDecThreads / 32; ++w) m = fmaxf(m, s_stat[w][g]);
        mx[g] = m;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GH; ++g) {
        float l = 0.f;
        for (int i = tid; i < nw + nf; i += kDecThreads) {
            const float s = s_sc[g * nrows + i];
            const float e = (mx[g] == -INFINITY) ? 0.f : exp2f(s - mx[g]);
            s_sc[g * nrows + i] = e;
            l += (i >= nw) ? e * cn[f0 + (i - nw)] : e;
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        if (lane == 0) s_stat[warp][g] = l;
    }
    __syncthreads();
    if (tid < GH) {
        float l = 0.f;
        for (int w = 0; w < kDecThreads / 32; ++w) l += s_stat[w][tid];
        s_l[tid] = l;
    }
#pragma unroll
    for (int g = 0; g < GH; ++g)
        if (tid == g) s_m[g] = mx[g];

    // ---- pass 3: values ----
    float acc[GH][E];
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
        for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
    if (nw > 0) accum_rows<T, D, GH>(vw, p.v_sl, w0, w1, s_sc, nrows, acc);
    if (nf > 0) accum_rows<T, D, GH>(vs, D, f0, f1, s_sc + nw, nrows, acc);
    // reduce over the lane groups of a warp, then over warps
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
        for (int e = 0; e < E; ++e) {
            float x = acc[g][e];
#pragma unroll
            for (int off = 16; off >= LPR; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
            acc[g][e] = x;
        }
    if (lane < LPR) {
#pragma unroll
        for (int g = 0; g < GH; ++g)
#pragma unroll
            for (int e = 0; e < E; ++e) s_red[(warp * GH + g) * D + lane * E + e] = acc[g][e];
    }
    __syncthreads();
    // partial[(u*G + head)][split][D+2]
    float *part = p.partial + ((static_cast<int64_t>(u) * p.G + hg * GH) * p.splits) * (D + 2);
    for (int i = tid; i < GH * D; i += kDecThreads) {
        const int g = i / D, d = i % D;
        float x = 0.f;
#pragma unroll
        for (int w = 0; w < kDecThreads / 32; ++w) x += s_red[(w * GH + g) * D + d];
        part[(static_cast<int64_t>(g) * p.splits + split) * (D + 2) + d] = x;
    }
    if (tid < GH) {
        part[(static_cast<int64_t>(tid) * p.splits + split) * (D + 2) + D] = s_m[tid];
        part[(static_cast<int64_t>(tid) * p.splits + split) * (D + 2) + D + 1] = s_l[tid];
    }
    __threadfence();
    __syncthreads();
    int *ticket = p.ticket + u * gridDim.y + hg;
    if (tid == 0) {
        const int t = atomicAdd(ticket, 1);
        s_last = (t == p.splits - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // merge the splits
    for (int i = tid; i < GH * D; i += kDecThreads) {
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

static int pick_splits(int64_t units, int n_valid, int MK)
{
    // aim for roughly 4 CTAs per SM (148 SMs) without making a split smaller than 128 rows
    int64_t s = (592 + units - 1) / units;
    int64_t cap = (static_cast<int64_t>(n_valid) + MK + 255) / 256;
    if (s > cap) s = cap;
    if (s > kDecMaxSplits) s = kDecMaxSplits;
    if (s < 1) s = 1;
    return static_cast<int>(s);
}

}  // namespace vq

extern "C" size_t vqattn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t D)
{
    (void)Hkv;
    const size_t tickets = (static_cast<size_t>(B) * Hq * sizeof(int) + 255) / 256 * 256;
    return tickets + static_cast<size_t>(B) * Hq * vq::kDecMaxSplits * (D + 2) * sizeof(float);
}

extern "C" int vqattn_decode(const VqDecodeArgs *a, void *stream)
{
    using namespace vq;
    if (a == nullptr) return VQ_EINVAL_ARG;
    int st;
    const VqTensorDesc *t3[] = {&a->q1, &a->q2, &a->out};
    for (auto t : t3)
        if ((st = check_basic(t, 3)) != VQ_OK) return st;
    const VqTensorDesc *t4[] = {&a->k1_win, &a->k3_win, &a->v_win};
    for (auto t : t4)
        if ((st = check_basic(t, 4)) != VQ_OK) return st;
    const bool far = a->use_far != 0;
    if (far) {
        if ((st = check_basic(&a->codebook, 3)) != VQ_OK) return st;
        if ((st = check_basic(&a->cnt, 3)) != VQ_OK) return st;
        if ((st = check_basic(&a->vsum, 4)) != VQ_OK) return st;
    }
    const VqTensorDesc *all[] = {&a->q1, &a->q2, &a->out, &a->k1_win, &a->k3_win, &a->v_win,
                                 far ? &a->codebook : nullptr, far ? &a->cnt : nullptr, far ? &a->vsum : nullptr};
    if ((st = check_device(all, 9)) != VQ_OK) return st;
    const int dt = a->q1.dtype;
    if (!is_act_dtype(dt)) return VQ_EINVAL_DTYPE;
    if (a->q2.dtype != dt || a->out.dtype != dt || a->k1_win.dtype != dt || a->k3_win.dtype != dt || a->v_win.dtype != dt)
        return VQ_EINVAL_DTYPE;
    if (far && (a->vsum.dtype != dt || a->cnt.dtype != VQ_F32 || (a->codebook.dtype != dt && a->codebook.dtype != VQ_F32)))
        return VQ_EINVAL_DTYPE;
    const int64_t B = a->q1.shape[0], Hq = a->q1.shape[1], D = a->q1.shape[2];
    const int64_t Hkv = a->k1_win.shape[1], Nwin = a->k1_win.shape[2];
    if (Hkv <= 0 || Hq % Hkv != 0) return VQ_EINVAL_SHAPE;
    for (auto t : t3)
        if (t->shape[0] != B || t->shape[1] != Hq || t->shape[2] != D) return VQ_EINVAL_SHAPE;
    for (auto t : t4)
        if (t->shape[0] != B || t->shape[1] != Hkv || t->shape[2] != Nwin || t->shape[3] != D) return VQ_EINVAL_SHAPE;
    if (a->n_valid < 0 || a->n_valid > Nwin || a->n_bd < 0 || a->n_bd > a->n_valid) return VQ_EINVAL_ARG;
    int64_t MK = 0;
    if (far) {
        MK = a->codebook.shape[1];
        if (a->codebook.shape[0] != Hkv || a->codebook.shape[2] != D) return VQ_EINVAL_SHAPE;
        if (a->cnt.shape[0] != B || a->cnt.shape[1] != Hkv || a->cnt.shape[2] != MK) return VQ_EINVAL_SHAPE;
        if (a->vsum.shape[0] != B || a->vsum.shape[1] != Hkv || a->vsum.shape[2] != MK || a->vsum.shape[3] != D)
            return VQ_EINVAL_SHAPE;
        if (!is_dense(a->codebook) || !is_dense(a->cnt) || !is_dense(a->vsum)) return VQ_EINVAL_STRIDE;
    }
    if (a->n_valid == 0 && !far) return VQ_EINVAL_ARG;
    if (D != 64 && D != 128) return VQ_EUNSUPPORTED;
    const int64_t row_align = dt == VQ_F32 ? 4 : 8;
    for (auto t : t4) {
        if (t->stride[0] % row_align || t->stride[1] % row_align || t->stride[2] % row_align) return VQ_EINVAL_STRIDE;
        if (reinterpret_cast<uintptr_t>(t->ptr) % 16) return VQ_EINVAL_STRIDE;
    }
    if (far && (reinterpret_cast<uintptr_t>(a->codebook.ptr) % 16 || reinterpret_cast<uintptr_t>(a->vsum.ptr) % 16))
        return VQ_EINVAL_STRIDE;
    if (B * Hkv > 65535 || a->n_valid > (1 << 24) || MK > (1 << 24)) return VQ_EUNSUPPORTED;
    if (a->workspace == nullptr || a->workspace_bytes < vqattn_decode_workspace_bytes(B, Hq, Hkv, D)) return VQ_EWORKSPACE;

    const int G = static_cast<int>(Hq / Hkv);
    int GH = 1;
    if (G % 4 == 0) GH = 4;
    else if (G % 2 == 0) GH = 2;
    DecodeParams p{};
    p.q1 = a->q1.ptr; p.q2 = a->q2.ptr; p.k1w = a->k1_win.ptr; p.k3w = a->k3_win.ptr; p.vw = a->v_win.ptr;
    p.codebook = a->codebook.ptr; p.vsum = a->vsum.ptr; p.cnt = static_cast<const float *>(a->cnt.ptr);
    p.out = a->out.ptr;
    const size_t tickets = (static_cast<size_t>(B) * Hq * sizeof(int) + 255) / 256 * 256;
    p.ticket = static_cast<int *>(a->workspace);
    p.partial = reinterpret_cast<float *>(static_cast<char *>(a->workspace) + tickets);
    p.q_sb = a->q1.stride[0]; p.q_sh = a->q1.stride[1];
    p.q2_sb = a->q2.stride[0]; p.q2_sh = a->q2.stride[1];
    p.o_sb = a->out.stride[0]; p.o_sh = a->out.stride[1];
    p.k_sb = a->k1_win.stride[0]; p.k_sh = a->k1_win.stride[1]; p.k_sl = a->k1_win.stride[2];
    p.k3_sb = a->k3_win.stride[0]; p.k3_sh = a->k3_win.stride[1]; p.k3_sl = a->k3_win.stride[2];
    p.v_sb = a->v_win.stride[0]; p.v_sh = a->v_win.stride[1]; p.v_sl = a->v_win.stride[2];
    p.Hq = static_cast<int>(Hq); p.Hkv = static_cast<int>(Hkv); p.G = G; p.MK = static_cast<int>(MK);
    p.n_valid = static_cast<int>(a->n_valid); p.n_bd = static_cast<int>(a->n_bd); p.use_far = far ? 1 : 0;
    p.splits = pick_splits(B * Hkv, p.n_valid, p.MK);
    p.rows_w = (p.n_valid + p.splits - 1) / p.splits;
    p.rows_f = far ? (p.MK + p.splits - 1) / p.splits : 0;
    const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(D));
    p.scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = sizeof(float) * (static_cast<size_t>(2 * GH * D) + static_cast<size_t>(GH) * (p.rows_w + p.rows_f) +
                                         static_cast<size_t>(kDecThreads / 32) * GH * D);
    if (smem > 200 * 1024) return VQ_EUNSUPPORTED;
    dim3 grid(static_cast<unsigned>(p.splits), static_cast<unsigned>(G / GH), static_cast<unsigned>(B * Hkv));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool cb32 = far ? a->codebook.dtype == VQ_F32 : dt == VQ_F32;

#define VQ_DEC(T, TC, DD, GG)                                                                                   \
    do {                                                                                                         \
        auto kern = decode_kernel<T, TC, DD, GG>;                                                                \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=  \
            cudaSuccess)                                                                                         \
            return VQ_ELAUNCH;                                                                                   \
        kern<<<grid, kDecThreads, smem, s>>>(p);                                                                 \
        return launch_status();                                                                                  \
    } while (0)
#define VQ_DEC_G(T, TC, DD)                     \
    do {                                        \
        if (GH == 4) VQ_DEC(T, TC, DD, 4);      \
        else if (GH == 2) VQ_DEC(T, TC, DD, 2); \
        else VQ_DEC(T, TC, DD, 1);              \
    } while (0)
    if (dt == VQ_F32) {
        if (D == 64) VQ_DEC_G(float, float, 64);
        else VQ_DEC_G(float, float, 128);
    } else if (cb32) {
        if (D == 64) VQ_DEC_G(__nv_bfloat16, float, 64);
        else VQ_DEC_G(__nv_bfloat16, float, 128);
    } else {
        if (D == 64) VQ_DEC_G(__nv_bfloat16, __nv_bfloat16, 64);
        else VQ_DEC_G(__nv_bfloat16, __nv_bfloat16, 128);
    }
#undef VQ_DEC_G
#undef VQ_DEC
    return VQ_ELAUNCH;
}
