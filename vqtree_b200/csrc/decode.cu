// Single-query (seqlen_q == 1) VQ-attention decode: a bandwidth-bound stream over the exact window
// (bf16/f32 keys and values), the per-code value sums and counts, and the codebook.
//
// The reference has no working decode for its VQ cache (ops/attn_vq.py:128-165); the semantics are
// those of prefill row n-1 (ops/attn_vq.py:311-332): window rows scored q1.k1 (the first n_bd of
// them q2.k3), far pseudo-keys scored q2.codebook[r] with weight cnt[r] and value vsum[r].
//
// Work split: grid = (splits, head groups, batch*kv-head).  A CTA owns a contiguous share of the
// window rows and of the far rows of one (batch, kv head) and up to GH query heads of its group:
// and streams them once: a group of lanes (D*sizeof/16 of them) owns one row per step, loads its
// 16-byte slice of the key row and of the value row together (several rows in flight per lane),
// reduces the dot product with shuffles and folds the row into its own running softmax state
// (max, denominator, D/lanes output columns).  No block-wide barrier sits between loads.
// The lane groups of a warp, then the warps (shared memory), then the splits (workspace; the last
// CTA of a unit to finish takes an atomic ticket, merges and re-arms it) are merged at the end.
#include <mutex>

#include "decode_common.cuh"

namespace vq {

// decode_tc.cu: tensor-core kernel (bf16, D = 128, bf16 codebook, dense rows, <= 16 query heads per kv head)
bool decode_tc_eligible(const VqDecodeArgs *a);
int launch_decode_tc(const VqDecodeArgs *a, const DecodeParams &p, cudaStream_t s);

int launch_decode_bulk(const DecodeParams &p, int64_t units, int D, int GH, bool cb32, void *workspace, size_t workspace_bytes,
                       int32_t *status, cudaStream_t s);
size_t decode_bulk_workspace_bytes(int64_t units_times_groups, int64_t heads_per_group, int64_t D);

// Window rows [r0,r1): key row and value row have the same type, one row per lane group per step.
template <typename T, int D, int GH, int U>
__device__ __forceinline__ void stream_rows(DecState<GH, Slice<T>::E> &st, const T *__restrict__ K, int64_t ks,
                                            const T *__restrict__ V, int64_t vs, int r0, int r1,
                                            const float *__restrict__ qs, float scale_log2, const float *__restrict__ wts)
{
    constexpr int E = Slice<T>::E, LPR = D / E, GPW = 32 / LPR, NG = (kDecThreads / 32) * GPW;
    const int lane = threadIdx.x & 31, gidx = (threadIdx.x >> 5) * GPW + lane / LPR, sub = lane % LPR;
    float q[GH][E];
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
        for (int e = 0; e < E; ++e) q[g][e] = qs[g * D + sub * E + e];
    const int iters = (r1 - r0 + NG * U - 1) / (NG * U);
    for (int it = 0; it < iters; ++it) {
        float kx[U][E], vx[U][E];
        bool ok[U];
#pragma unroll
        for (int uu = 0; uu < U; ++uu) {
            const int r = r0 + (it * U + uu) * NG + gidx;
            ok[uu] = r < r1;
            if (ok[uu]) {
                Slice<T>::ld(K + static_cast<int64_t>(r) * ks + sub * E, kx[uu]);
                Slice<T>::ld(V + static_cast<int64_t>(r) * vs + sub * E, vx[uu]);
            } else {
#pragma unroll
                for (int e = 0; e < E; ++e) kx[uu][e] = vx[uu][e] = 0.f;
            }
        }
#pragma unroll
        for (int uu = 0; uu < U; ++uu) {
            const int r = r0 + (it * U + uu) * NG + gidx;
            float w = 1.f;
            if (wts != nullptr && ok[uu]) w = wts[r];
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < E; ++e) s = fmaf(q[g][e], kx[uu][e], s);
#pragma unroll
                for (int off = LPR / 2; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                s = (ok[uu] && w > 0.f) ? s * scale_log2 : -INFINITY;
                st.update(g, s, w, vx[uu]);
            }
        }
    }
}

// Far rows [r0,r1) with an fp32 codebook (512-byte rows for D = 128) and bf16 value sums: a step
// covers GPW rows of the warp; their scores are formed by groups of D/4 lanes in GPW/GPWC sub-steps.
template <typename TV, int D, int GH, int U>
__device__ __forceinline__ void stream_far_f32cb(DecState<GH, 8> &st, const float *__restrict__ C,
                                                 const TV *__restrict__ V, int r0, int r1,
                                                 const float *__restrict__ qs, float scale_log2, const float *__restrict__ wts)
{
    constexpr int LPR = D / 8, GPW = 32 / LPR;     // value-row lane groups
    constexpr int LPRC = D / 4, GPWC = 32 / LPRC;  // codebook-row lane groups
    constexpr int SUB = GPW / GPWC;                // = 2
    constexpr int NW = kDecThreads / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int vg = lane / LPR, sub = lane % LPR, cg = lane / LPRC, csub = lane % LPRC;
    float q[GH][4];
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) q[g][e] = qs[g * D + csub * 4 + e];
    const int rows_per_step = NW * GPW;
    const int iters = (r1 - r0 + rows_per_step * U - 1) / (rows_per_step * U);
    for (int it = 0; it < iters; ++it) {
        float cx[U][SUB][4], vx[U][8];
#pragma unroll
        for (int uu = 0; uu < U; ++uu) {
            const int base = r0 + ((it * U + uu) * NW + warp) * GPW;  // first of this warp's GPW rows
#pragma unroll
            for (int ss = 0; ss < SUB; ++ss) {
                const int r = base + ss * GPWC + cg;
                if (r < r1) Slice<float>::ld_cached(C + static_cast<int64_t>(r) * D + csub * 4, cx[uu][ss]);
                else cx[uu][ss][0] = cx[uu][ss][1] = cx[uu][ss][2] = cx[uu][ss][3] = 0.f;
            }
            const int rv = base + vg;
            if (rv < r1) Slice<TV>::ld(V + static_cast<int64_t>(rv) * D + sub * 8, vx[uu]);
            else {
#pragma unroll
                for (int e = 0; e < 8; ++e) vx[uu][e] = 0.f;
            }
        }
#pragma unroll
        for (int uu = 0; uu < U; ++uu) {
            const int base = r0 + ((it * U + uu) * NW + warp) * GPW;
            const int rv = base + vg;
            const bool ok = rv < r1;
            const float w = ok ? wts[rv] : 0.f;
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                float mine = 0.f;
#pragma unroll
                for (int ss = 0; ss < SUB; ++ss) {
                    float s = 0.f;
#pragma unroll
                    for (int e = 0; e < 4; ++e) s = fmaf(q[g][e], cx[uu][ss][e], s);
#pragma unroll
                    for (int off = LPRC / 2; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                    // the score of value group vg was formed in sub-step vg / GPWC by codebook group vg % GPWC
                    const float got = __shfl_sync(0xffffffffu, s, (vg % GPWC) * LPRC);
                    if (ss == vg / GPWC) mine = got;
                }
                const float s = (ok && w > 0.f) ? mine * scale_log2 : -INFINITY;
                st.update(g, s, w, vx[uu]);
            }
        }
    }
}

template <typename T, typename TC, int D, int GH>
__global__ void __launch_bounds__(kDecThreads) decode_kernel(DecodeParams p)
{
    constexpr int E = Slice<T>::E;
    constexpr int LPR = D / E;
    constexpr int NW = kDecThreads / 32;
    constexpr int U = GH >= 4 ? 2 : 4;
    __shared__ __align__(16) float s_q[2 * GH * D];
    __shared__ __align__(16) float s_red[NW * GH * (D + 2)];
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

    const T *k1w = static_cast<const T *>(p.k1w) + b * p.k_sb + hk * p.k_sh;
    const T *k3w = static_cast<const T *>(p.k3w) + b * p.k3_sb + hk * p.k3_sh;
    const T *vw = static_cast<const T *>(p.vw) + b * p.v_sb + hk * p.v_sh;
    const TC *cbk = static_cast<const TC *>(p.codebook) + static_cast<int64_t>(hk) * p.MK * D;
    const T *vs = static_cast<const T *>(p.vsum) + static_cast<int64_t>(u) * p.MK * D;
    const float *cn = p.cnt + static_cast<int64_t>(u) * p.MK;

    DecState<GH, E> st;
    st.init();
    const int wb = min(max(p.n_bd, w0), w1);  // rows [w0,wb) use q2.k3, [wb,w1) use q1.k1
    if (wb > w0) stream_rows<T, D, GH, U>(st, k3w, p.k3_sl, vw, p.v_sl, w0, wb, s_q + GH * D, p.scale_log2, nullptr);
    if (w1 > wb) stream_rows<T, D, GH, U>(st, k1w, p.k_sl, vw, p.v_sl, wb, w1, s_q, p.scale_log2, nullptr);
    if (f1 > f0) {
        if constexpr (sizeof(TC) == sizeof(T))
            stream_rows<T, D, GH, U>(st, reinterpret_cast<const T *>(cbk), D, vs, D, f0, f1, s_q + GH * D, p.scale_log2, cn);
        else if constexpr (sizeof(T) == 2)
            stream_far_f32cb<T, D, GH, U>(st, reinterpret_cast<const float *>(cbk), vs, f0, f1, s_q + GH * D, p.scale_log2, cn);
    }
    // merge the lane groups of a warp, then the warps
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) st.merge_xor(off);
    decode_finish<T, D, GH, NW, E>(p, st, s_red, &s_last, split, hg, u, b, hq0);
}

#ifndef VQ_DECODE_TARGET_CTAS
#define VQ_DECODE_TARGET_CTAS 2048
#endif

static int pick_splits(int64_t ctas_per_split, int n_valid, int MK)
{
    // enough CTAs for several waves over 148 SMs, but at least ~256 rows per CTA
    int64_t s = (VQ_DECODE_TARGET_CTAS + ctas_per_split - 1) / ctas_per_split;
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
    const size_t split_kernel = tickets + static_cast<size_t>(B) * Hq * vq::kDecMaxSplits * (D + 2) * sizeof(float);
    const size_t stream_kernel = vq::decode_bulk_workspace_bytes(B * Hq, 4, D);
    return split_kernel > stream_kernel ? split_kernel : stream_kernel;
}

// Argument checks shared by vqattn_decode and vqattn_decode_static (everything but the workspace).
static int decode_validate(const VqDecodeArgs *a)
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
    return VQ_OK;
}

extern "C" int vqattn_decode(const VqDecodeArgs *a, void *stream)
{
    using namespace vq;
    int st = decode_validate(a);
    if (st != VQ_OK) return st;
    const bool far = a->use_far != 0;
    const int dt = a->q1.dtype;
    const int64_t B = a->q1.shape[0], Hq = a->q1.shape[1], D = a->q1.shape[2];
    const int64_t Hkv = a->k1_win.shape[1];
    const int64_t MK = far ? a->codebook.shape[1] : 0;
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
    p.splits = pick_splits(B * Hkv * (G / GH), p.n_valid, p.MK);
    // rows per split, rounded to whole 32-row tiles (keeps every tile copy 16-byte aligned)
    p.rows_w = ((p.n_valid + p.splits - 1) / p.splits + 31) / 32 * 32;
    p.rows_f = far ? ((p.MK + p.splits - 1) / p.splits + 31) / 32 * 32 : 0;
    const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(D));
    p.scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(static_cast<unsigned>(p.splits), static_cast<unsigned>(G / GH), static_cast<unsigned>(B * Hkv));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool cb32 = far ? a->codebook.dtype == VQ_F32 : dt == VQ_F32;
    // bf16 caches with dense rows take the bulk-copy kernel; anything else the register-streaming one
    const bool dense_rows = a->k1_win.stride[2] == D && a->k3_win.stride[2] == D && a->v_win.stride[2] == D &&
                            a->q1.stride[1] == D && a->q2.stride[1] == D && a->q1.stride[0] % 8 == 0 && a->q2.stride[0] % 8 == 0 &&
                            reinterpret_cast<uintptr_t>(a->q1.ptr) % 16 == 0 && reinterpret_cast<uintptr_t>(a->q2.ptr) % 16 == 0;
    if (dt == VQ_BF16 && dense_rows && decode_tc_eligible(a)) {
        const int r = launch_decode_tc(a, p, s);
        if (r != VQ_EWORKSPACE) return r;  // too small a workspace for it: the SIMT kernel below
    }
    if (dt == VQ_BF16 && dense_rows)
        return launch_decode_bulk(p, B * Hkv, static_cast<int>(D), GH, far && cb32, a->workspace, a->workspace_bytes,
                                  a->status_word, s);

#define VQ_DEC(T, TC, DD, GG)                                                                                   \
    do {                                                                                                         \
        decode_kernel<T, TC, DD, GG><<<grid, kDecThreads, 0, s>>>(p);                                            \
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
    } else if (dt == VQ_F16 && cb32) {
        if (D == 64) VQ_DEC_G(__half, float, 64);
        else VQ_DEC_G(__half, float, 128);
    } else if (dt == VQ_F16) {
        if (D == 64) VQ_DEC_G(__half, __half, 64);
        else VQ_DEC_G(__half, __half, 128);
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

// ---------------------------------------------------------------------------------------------
// Decode without a caller-provided workspace.
//
// Some hosts cannot hand this library a workspace buffer: an inference server that gives every free
// byte of HBM to its KV-cache pool at start-up, or a runtime whose plugin contract forbids device
// allocation once serving has begun, has nowhere to take the split/merge scratch of the decode kernel
// from.  For them the scratch lives in the library image itself: one fixed array per GPU that loads
// the library, held until the process exits.
#define VQATTN_DECODE_STATIC_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_decode_static_scratch[VQATTN_DECODE_STATIC_BYTES];

extern "C" size_t vqattn_decode_static_capacity(void) { return VQATTN_DECODE_STATIC_BYTES; }

extern "C" int vqattn_decode_static(const VqDecodeArgs *a, void *stream)
{
    using namespace vq;
    // every argument check comes first: a rejected call must not touch the shared array, which a
    // previous call's kernel may still be using
    const int vst = decode_validate(a);
    if (vst != VQ_OK) return vst;
    const int64_t B = a->q1.shape[0], Hq = a->q1.shape[1], D = a->q1.shape[2], Hkv = a->k1_win.shape[1];
    // the built-in scratch has a fixed size: larger problems must use vqattn_decode with their own workspace
    if (vqattn_decode_workspace_bytes(B, Hq, Hkv, D) > VQATTN_DECODE_STATIC_BYTES) return VQ_EWORKSPACE;

    // In host code the array's name is only a handle; the device address is looked up once per
    // device, with that device current, and cached.
    static std::mutex mu;
    static void *dev_ptr[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return VQ_EDEVICE;
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev_ptr[dev] == nullptr) {
            void *ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_decode_static_scratch) != cudaSuccess || ptr == nullptr) return VQ_ELAUNCH;
            dev_ptr[dev] = ptr;
        }
        scratch = dev_ptr[dev];
    }
    // The array keeps whatever the last call left.  The merge tickets at its start must be zero when
    // a launch begins (a call that was cut short could have left some raised), so clear them here.
    const size_t tickets = (static_cast<size_t>(B) * Hq * sizeof(int) + 255) / 256 * 256;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(scratch, 0, tickets, s) != cudaSuccess) return VQ_ELAUNCH;
    VqDecodeArgs b = *a;
    b.workspace = scratch;
    b.workspace_bytes = VQATTN_DECODE_STATIC_BYTES;
    return vqattn_decode(&b, stream);
}

// One generated token: rotate-and-append, then attention, on one stream (see vqattn.h).
extern "C" int vqattn_decode_step(const VqDecodeStepArgs *a, void *stream)
{
    if (a == nullptr) return VQ_EINVAL_ARG;
    // validate the attention's arguments before the append writes anything into the caches
    const int vst = decode_validate(&a->decode);
    if (vst != VQ_OK) return vst;
    VqTensorDesc q1 = a->q1, q2 = a->q2, k1w = a->decode.k1_win, k3w = a->decode.k3_win, vw = a->decode.v_win;
    const int st = vqattn_decode_append(&a->q, &a->k, &a->v, a->positions, a->pos, a->cos_tab, a->sin_tab, a->n_pos, a->const_pos,
                                        &q1, &q2, &k1w, &k3w, &vw, a->row, a->decode.status_word, stream);
    if (st != VQ_OK) return st;
    return vqattn_decode(&a->decode, stream);
}
