// Rotary position embedding of a [B,H,L,D] tensor in the HF Llama half-split convention
// (ops/attn_vq.py:55-64,296-299: x*cos + rotate_half(x)*sin with rotate_half(x) = cat(-x2, x1)),
// to each row's own position and / or to one constant position (the ReRoPE query of
// ops/attn_vq.py:402-407), both from one read of x.  HBM-bound: one thread moves 16 bytes of the
// first half of a row and the matching 16 bytes of the second half; cos / sin come from fp32 tables
// [n_pos, D/2] that stay in L2 (every head reads the same rows).  Products and the sum are rounded
// separately (no fused multiply-add), which is what the element-wise PyTorch expression computes.
#include "vq_common.cuh"

namespace vq {

template <typename T> struct RopeVec;
template <> struct RopeVec<float> {
    static constexpr int kN = 4;
    __device__ static void load(const float *p, float (&f)[4])
    {
        const float4 v = *reinterpret_cast<const float4 *>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    __device__ static void store(float *p, const float (&f)[4]) { *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct RopeVec<__nv_bfloat16> {
    static constexpr int kN = 8;
    __device__ static void load(const __nv_bfloat16 *p, float (&f)[8])
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static void store(__nv_bfloat16 *p, const float (&f)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <> struct RopeVec<__half> {
    static constexpr int kN = 8;
    __device__ static void load(const __half *p, float (&f)[8])
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = Pair16<__half>::unpack(w[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
    __device__ static void store(__half *p, const float (&f)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = Pair16<__half>::pack(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// out = x * cos + rotate_half(x) * sin for the kN elements at d (first half) and d + D/2 (second half)
template <int N>
__device__ __forceinline__ void rope_rotate(const float (&x1)[N], const float (&x2)[N], const float *c, const float *s, float (&o1)[N], float (&o2)[N])
{
    // the table rows start on 16-byte boundaries (D/2 and d are multiples of four floats): 128-bit loads
    static_assert(N % 4 == 0, "vector width");
#pragma unroll
    for (int i4 = 0; i4 < N / 4; ++i4) {
        const float4 c4 = __ldg(reinterpret_cast<const float4 *>(c) + i4), s4 = __ldg(reinterpret_cast<const float4 *>(s) + i4);
        const float cv[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 4 * i4 + e;
            o1[i] = __fadd_rn(__fmul_rn(x1[i], cv[e]), __fmul_rn(-x2[i], sv[e]));
            o2[i] = __fadd_rn(__fmul_rn(x2[i], cv[e]), __fmul_rn(x1[i], sv[e]));
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T *__restrict__ x, int64_t x_sb, int64_t x_sh, int64_t x_sl,
                                                   const int64_t *__restrict__ positions, const float *__restrict__ cos_tab,
                                                   const float *__restrict__ sin_tab, int64_t n_pos, int64_t const_pos,
                                                   T *__restrict__ out_pos, int64_t p_sb, int64_t p_sh, int64_t p_sl,
                                                   T *__restrict__ out_const, int64_t c_sb, int64_t c_sh, int64_t c_sl, int H,
                                                   int64_t L, int D, int64_t rows, int *__restrict__ status)
{
    constexpr int N = RopeVec<T>::kN;
    const int half = D / 2, tpr = half / N;          // threads per row
    const int64_t total = rows * tpr;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / tpr;
        const int d = static_cast<int>(i % tpr) * N;
        // rows in the order they lie in memory: heads vary fastest when the tensor is a [B,H,L,D] view of [B,L,H,D]
        // storage (consecutive work items then touch consecutive addresses instead of 256 bytes in every H*D)
        int64_t l, b;
        int h;
        if (x_sh < x_sl) {
            h = static_cast<int>(r % H);
            l = (r / H) % L;
            b = r / (static_cast<int64_t>(H) * L);
        } else {
            l = r % L;
            h = static_cast<int>((r / L) % H);
            b = r / (static_cast<int64_t>(H) * L);
        }
        float x1[N], x2[N], o1[N], o2[N];
        const T *xp = x + b * x_sb + h * x_sh + l * x_sl + d;
        RopeVec<T>::load(xp, x1);
        RopeVec<T>::load(xp + half, x2);
        if (out_pos != nullptr) {
            int64_t pos = positions ? positions[b * L + l] : l;
            if (pos < 0 || pos >= n_pos) {               // outside the tables: report, rotate to the nearest row
                if (status) atomicExch(status, VQ_WORD_BAD_POSITION);
                pos = pos < 0 ? 0 : n_pos - 1;
            }
            rope_rotate<N>(x1, x2, cos_tab + pos * half + d, sin_tab + pos * half + d, o1, o2);
            T *op = out_pos + b * p_sb + h * p_sh + l * p_sl + d;
            RopeVec<T>::store(op, o1);
            RopeVec<T>::store(op + half, o2);
        }
        if (out_const != nullptr) {
            rope_rotate<N>(x1, x2, cos_tab + const_pos * half + d, sin_tab + const_pos * half + d, o1, o2);
            T *op = out_const + b * c_sb + h * c_sh + l * c_sl + d;
            RopeVec<T>::store(op, o1);
            RopeVec<T>::store(op + half, o2);
        }
    }
}


// ---------------------------------------------------------------------------------------------
// Several tensors in one launch: each job reads rows of one [B,H,L,D] tensor and writes up to three
// results - the rows rotated to their own positions, rotated to the constant position, and copied
// unchanged.  Used for "q and k of a prefill in one pass" and for the per-token step of a decode
// (q -> q1, q2; k -> rotated key and raw key into the window cache; v -> the window cache).
constexpr int kRopeMaxJobs = 3;
struct RopeJob {
    const void *x;
    void *out_pos, *out_const, *out_copy;
    int64_t x_sb, x_sh, x_sl, p_sb, p_sh, p_sl, c_sb, c_sh, c_sl, y_sb, y_sh, y_sl;
    int64_t first;   // index of the job's first (row, vector) work item in the launch
    int H;
};
struct RopeMultiParams {
    RopeJob job[kRopeMaxJobs];
    int njobs;
    int64_t total;   // work items of all jobs
    const int64_t *positions;  // [B, L] or nullptr (position = pos0 + l)
    int64_t pos0;
    const float *cos_tab, *sin_tab;
    int64_t n_pos, const_pos, L;
    int D;
    int32_t *status;
};

template <typename T>
__global__ void __launch_bounds__(256) rope_multi_kernel(const RopeMultiParams p)
{
    constexpr int N = RopeVec<T>::kN;
    const int half = p.D / 2, tpr = half / N;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < p.total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int j = 0;
#pragma unroll
        for (int t = 1; t < kRopeMaxJobs; ++t)
            if (t < p.njobs && i >= p.job[t].first) j = t;
        const RopeJob &jb = p.job[j];
        const int64_t w = i - jb.first;
        const int64_t r = w / tpr;
        const int d = static_cast<int>(w % tpr) * N;
        // rows in the order they lie in memory (see rope_kernel)
        int64_t l, b;
        int h;
        if (jb.x_sh < jb.x_sl) {
            h = static_cast<int>(r % jb.H);
            l = (r / jb.H) % p.L;
            b = r / (static_cast<int64_t>(jb.H) * p.L);
        } else {
            l = r % p.L;
            h = static_cast<int>((r / p.L) % jb.H);
            b = r / (static_cast<int64_t>(jb.H) * p.L);
        }
        float x1[N], x2[N], o1[N], o2[N];
        const T *xp = static_cast<const T *>(jb.x) + b * jb.x_sb + h * jb.x_sh + l * jb.x_sl + d;
        RopeVec<T>::load(xp, x1);
        RopeVec<T>::load(xp + half, x2);
        if (jb.out_copy != nullptr) {
            T *op = static_cast<T *>(jb.out_copy) + b * jb.y_sb + h * jb.y_sh + l * jb.y_sl + d;
            RopeVec<T>::store(op, x1);
            RopeVec<T>::store(op + half, x2);
        }
        if (jb.out_pos != nullptr) {
            int64_t pos = p.positions ? p.positions[b * p.L + l] : p.pos0 + l;
            if (pos < 0 || pos >= p.n_pos) {
                if (p.status) atomicExch(p.status, VQ_WORD_BAD_POSITION);
                pos = pos < 0 ? 0 : p.n_pos - 1;
            }
            rope_rotate<N>(x1, x2, p.cos_tab + pos * half + d, p.sin_tab + pos * half + d, o1, o2);
            T *op = static_cast<T *>(jb.out_pos) + b * jb.p_sb + h * jb.p_sh + l * jb.p_sl + d;
            RopeVec<T>::store(op, o1);
            RopeVec<T>::store(op + half, o2);
        }
        if (jb.out_const != nullptr) {
            rope_rotate<N>(x1, x2, p.cos_tab + p.const_pos * half + d, p.sin_tab + p.const_pos * half + d, o1, o2);
            T *op = static_cast<T *>(jb.out_const) + b * jb.c_sb + h * jb.c_sh + l * jb.c_sl + d;
            RopeVec<T>::store(op, o1);
            RopeVec<T>::store(op + half, o2);
        }
    }
}

// Adds one job; outputs may be NULL descriptors.  `row_of_out`: outputs that are [B,H,N,D] caches
// receive the job's L rows starting at that row.
static int rope_add_job(RopeMultiParams &p, const VqTensorDesc *x, const VqTensorDesc *out_pos, const VqTensorDesc *out_const,
                        const VqTensorDesc *out_copy, int64_t row_of_out, int vec)
{
    int st;
    if ((st = check_basic(x, 4)) != VQ_OK) return st;
    if (p.njobs >= kRopeMaxJobs) return VQ_EINVAL_ARG;
    RopeJob &jb = p.job[p.njobs];
    jb = RopeJob{};
    const int64_t B = x->shape[0], H = x->shape[1], L = x->shape[2], D = x->shape[3];
    if (L != p.L || D != p.D) return VQ_EINVAL_SHAPE;
    if (reinterpret_cast<uintptr_t>(x->ptr) % 16 || x->stride[0] % vec || x->stride[1] % vec || x->stride[2] % vec) return VQ_EINVAL_STRIDE;
    jb.x = x->ptr; jb.x_sb = x->stride[0]; jb.x_sh = x->stride[1]; jb.x_sl = x->stride[2];
    jb.H = static_cast<int>(H);
    const VqTensorDesc *outs[3] = {out_pos, out_const, out_copy};
    for (int i = 0; i < 3; ++i) {
        const VqTensorDesc *t = outs[i];
        if (t == nullptr || t->ptr == nullptr) continue;
        if ((st = check_basic(t, 4)) != VQ_OK) return st;
        if (t->dtype != x->dtype) return VQ_EINVAL_DTYPE;
        if (t->device != x->device) return VQ_EDEVICE;
        if (t->shape[0] != B || t->shape[1] != H || t->shape[3] != D || row_of_out < 0 || row_of_out + L > t->shape[2]) return VQ_EINVAL_SHAPE;
        if (reinterpret_cast<uintptr_t>(t->ptr) % 16 || t->stride[0] % vec || t->stride[1] % vec || t->stride[2] % vec) return VQ_EINVAL_STRIDE;
        char *base = static_cast<char *>(t->ptr) + row_of_out * t->stride[2] * (x->dtype == VQ_F32 ? 4 : 2);
        if (i == 0) { jb.out_pos = base; jb.p_sb = t->stride[0]; jb.p_sh = t->stride[1]; jb.p_sl = t->stride[2]; }
        if (i == 1) { jb.out_const = base; jb.c_sb = t->stride[0]; jb.c_sh = t->stride[1]; jb.c_sl = t->stride[2]; }
        if (i == 2) { jb.out_copy = base; jb.y_sb = t->stride[0]; jb.y_sh = t->stride[1]; jb.y_sl = t->stride[2]; }
    }
    jb.first = p.total;
    p.total += B * H * L * (D / 2 / vec);
    ++p.njobs;
    return VQ_OK;
}

static int rope_multi_launch(const RopeMultiParams &p, int dtype, cudaStream_t s)
{
    if (p.total == 0) return VQ_OK;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return VQ_EDEVICE;
    const int64_t want = (p.total + 255) / 256;
    const unsigned grid = static_cast<unsigned>(want < static_cast<int64_t>(sms) * 16 ? want : static_cast<int64_t>(sms) * 16);
    if (dtype == VQ_F32) rope_multi_kernel<float><<<grid, 256, 0, s>>>(p);
    else if (dtype == VQ_F16) rope_multi_kernel<__half><<<grid, 256, 0, s>>>(p);
    else rope_multi_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p);
    return launch_status();
}

}  // namespace vq

extern "C" int vqattn_rope(const VqTensorDesc *x, const int64_t *positions, const float *cos_tab, const float *sin_tab,
                           int64_t n_pos, int64_t const_pos, VqTensorDesc *out_pos, VqTensorDesc *out_const,
                           int32_t *status_word, void *stream)
{
    using namespace vq;
    int st;
    if (out_pos != nullptr && out_pos->ptr == nullptr) out_pos = nullptr;
    if (out_const != nullptr && out_const->ptr == nullptr) out_const = nullptr;
    if ((st = check_basic(x, 4)) != VQ_OK) return st;
    if (cos_tab == nullptr || sin_tab == nullptr || n_pos <= 0 || (out_pos == nullptr && out_const == nullptr)) return VQ_EINVAL_ARG;
    if (reinterpret_cast<uintptr_t>(cos_tab) % 16 || reinterpret_cast<uintptr_t>(sin_tab) % 16) return VQ_EINVAL_STRIDE;   // 128-bit table loads
    if (out_const != nullptr && (const_pos < 0 || const_pos >= n_pos)) return VQ_EINVAL_ARG;
    if (!is_act_dtype(x->dtype)) return VQ_EINVAL_DTYPE;
    const int64_t B = x->shape[0], H = x->shape[1], L = x->shape[2], D = x->shape[3];
    const int vec = x->dtype == VQ_F32 ? 4 : 8;
    if (D % (2 * vec) != 0) return VQ_EINVAL_SHAPE;
    const VqTensorDesc *ts[3] = {x, out_pos, out_const};
    if ((st = check_device(ts, 3)) != VQ_OK) return st;
    for (int i = 0; i < 3; ++i) {
        const VqTensorDesc *t = ts[i];
        if (t == nullptr) continue;
        if (i > 0) {
            if ((st = check_basic(t, 4)) != VQ_OK) return st;
            if (t->dtype != x->dtype) return VQ_EINVAL_DTYPE;
            if (t->shape[0] != B || t->shape[1] != H || t->shape[2] != L || t->shape[3] != D) return VQ_EINVAL_SHAPE;
        }
        // 16-byte vectors: aligned base and row strides
        if (reinterpret_cast<uintptr_t>(t->ptr) % 16 || t->stride[0] % vec || t->stride[1] % vec || t->stride[2] % vec) return VQ_EINVAL_STRIDE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t rows = B * H * L, total = rows * (D / 2 / vec);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return VQ_EDEVICE;
    const int64_t want = (total + 255) / 256;
    const unsigned grid = static_cast<unsigned>(want < static_cast<int64_t>(sms) * 16 ? want : static_cast<int64_t>(sms) * 16);
#define VQ_ROPE_LAUNCH(T)                                                                                                   \
    rope_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T *>(x->ptr), x->stride[0], x->stride[1], x->stride[2], positions,  \
                                        cos_tab, sin_tab, n_pos, const_pos, out_pos ? static_cast<T *>(out_pos->ptr) : nullptr, \
                                        out_pos ? out_pos->stride[0] : 0, out_pos ? out_pos->stride[1] : 0,                   \
                                        out_pos ? out_pos->stride[2] : 0, out_const ? static_cast<T *>(out_const->ptr) : nullptr, \
                                        out_const ? out_const->stride[0] : 0, out_const ? out_const->stride[1] : 0,           \
                                        out_const ? out_const->stride[2] : 0, static_cast<int>(H), L, static_cast<int>(D), rows, \
                                        status_word)
    if (x->dtype == VQ_F32) VQ_ROPE_LAUNCH(float);
    else if (x->dtype == VQ_F16) VQ_ROPE_LAUNCH(__half);
    else VQ_ROPE_LAUNCH(__nv_bfloat16);
#undef VQ_ROPE_LAUNCH
    return launch_status();
}

extern "C" int vqattn_rope_qk(const VqTensorDesc *q, const VqTensorDesc *k, const int64_t *positions, const float *cos_tab,
                              const float *sin_tab, int64_t n_pos, int64_t const_pos, VqTensorDesc *q1, VqTensorDesc *q2,
                              VqTensorDesc *k1, int32_t *status_word, void *stream)
{
    using namespace vq;
    if (q == nullptr || k == nullptr || q1 == nullptr || k1 == nullptr || cos_tab == nullptr || sin_tab == nullptr || n_pos <= 0)
        return VQ_EINVAL_ARG;
    if (reinterpret_cast<uintptr_t>(cos_tab) % 16 || reinterpret_cast<uintptr_t>(sin_tab) % 16) return VQ_EINVAL_STRIDE;   // 128-bit table loads
    const bool want_q2 = q2 != nullptr && q2->ptr != nullptr;
    if (want_q2 && (const_pos < 0 || const_pos >= n_pos)) return VQ_EINVAL_ARG;
    if (q->ndim != 4 || k->ndim != 4) return VQ_EINVAL_SHAPE;
    if (!is_act_dtype(q->dtype) || k->dtype != q->dtype) return VQ_EINVAL_DTYPE;
    if (q->shape[0] != k->shape[0]) return VQ_EINVAL_SHAPE;
    const int vec = q->dtype == VQ_F32 ? 4 : 8;
    if (q->shape[3] % (2 * vec) != 0) return VQ_EINVAL_SHAPE;
    const VqTensorDesc *ts[5] = {q, k, q1, want_q2 ? q2 : nullptr, k1};
    int st;
    if ((st = check_device(ts, 5)) != VQ_OK) return st;
    RopeMultiParams p{};
    p.L = q->shape[2]; p.D = static_cast<int>(q->shape[3]);
    p.positions = positions; p.pos0 = 0;
    p.cos_tab = cos_tab; p.sin_tab = sin_tab; p.n_pos = n_pos; p.const_pos = want_q2 ? const_pos : 0;
    p.status = status_word;
    if ((st = rope_add_job(p, q, q1, want_q2 ? q2 : nullptr, nullptr, 0, vec)) != VQ_OK) return st;
    if ((st = rope_add_job(p, k, k1, nullptr, nullptr, 0, vec)) != VQ_OK) return st;
    return rope_multi_launch(p, q->dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int vqattn_decode_append(const VqTensorDesc *q, const VqTensorDesc *k, const VqTensorDesc *v, const int64_t *positions,
                                    int64_t pos, const float *cos_tab, const float *sin_tab, int64_t n_pos, int64_t const_pos,
                                    VqTensorDesc *q1, VqTensorDesc *q2, VqTensorDesc *k1_win, VqTensorDesc *k3_win,
                                    VqTensorDesc *v_win, int64_t row, int32_t *status_word, void *stream)
{
    using namespace vq;
    if (q == nullptr || k == nullptr || v == nullptr || q1 == nullptr || q2 == nullptr || k1_win == nullptr || k3_win == nullptr ||
        v_win == nullptr || cos_tab == nullptr || sin_tab == nullptr || n_pos <= 0)
        return VQ_EINVAL_ARG;
    if (reinterpret_cast<uintptr_t>(cos_tab) % 16 || reinterpret_cast<uintptr_t>(sin_tab) % 16) return VQ_EINVAL_STRIDE;   // 128-bit table loads
    if (const_pos < 0 || const_pos >= n_pos) return VQ_EINVAL_ARG;
    if (q->ndim != 4 || k->ndim != 4 || v->ndim != 4 || q->shape[2] != 1) return VQ_EINVAL_SHAPE;
    if (!is_act_dtype(q->dtype) || k->dtype != q->dtype || v->dtype != q->dtype) return VQ_EINVAL_DTYPE;
    if (k->shape[0] != q->shape[0] || v->shape[0] != q->shape[0] || v->shape[1] != k->shape[1]) return VQ_EINVAL_SHAPE;
    const int vec = q->dtype == VQ_F32 ? 4 : 8;
    if (q->shape[3] % (2 * vec) != 0) return VQ_EINVAL_SHAPE;
    const VqTensorDesc *ts[8] = {q, k, v, q1, q2, k1_win, k3_win, v_win};
    int st;
    if ((st = check_device(ts, 8)) != VQ_OK) return st;
    RopeMultiParams p{};
    p.L = 1; p.D = static_cast<int>(q->shape[3]);
    p.positions = positions; p.pos0 = pos;
    p.cos_tab = cos_tab; p.sin_tab = sin_tab; p.n_pos = n_pos; p.const_pos = const_pos;
    p.status = status_word;
    if (positions == nullptr && (pos < 0 || pos >= n_pos)) return VQ_EINVAL_ARG;
    if ((st = rope_add_job(p, q, q1, q2, nullptr, 0, vec)) != VQ_OK) return st;
    if ((st = rope_add_job(p, k, k1_win, nullptr, k3_win, row, vec)) != VQ_OK) return st;
    if ((st = rope_add_job(p, v, nullptr, nullptr, v_win, row, vec)) != VQ_OK) return st;
    return rope_multi_launch(p, q->dtype, static_cast<cudaStream_t>(stream));
}
