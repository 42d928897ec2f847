// Key -> code assignment (exact fp32): replaces ops/mini_vq.py:4-18 of the reference.
//
// One CTA scores a tile of 64 keys of one (batch, kv head) against every codeword of every
// codebook.  Scores are a register-tiled fp32 product; each score is ONE fused-multiply-add
// chain over d = 0..D-1 starting from +0, which makes the result independent of the tiling and
// reproducible bit for bit by a scalar loop.  Ties go to the lowest code (torch.argmax order).
// For M > 1 the residual r -= C_m[code] is updated in shared memory between codebooks.
#include "vq_common.cuh"

namespace vq {

constexpr int kAssignKeys = 64;   // keys per CTA
constexpr int kAssignCodes = 64;  // codewords per shared-memory chunk
constexpr int kAssignThreads = 256;

template <typename T> struct Vec4Load;
template <> struct Vec4Load<float> {
    static __device__ __forceinline__ float4 ld(const float *p) { return *reinterpret_cast<const float4 *>(p); }
};
template <> struct Vec4Load<__nv_bfloat16> {
    static __device__ __forceinline__ float4 ld(const __nv_bfloat16 *p)
    {
        uint2 raw = *reinterpret_cast<const uint2 *>(p);
        __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&raw.x);
        __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
};

template <> struct Vec4Load<__half> {
    static __device__ __forceinline__ float4 ld(const __half *p)
    {
        uint2 raw = *reinterpret_cast<const uint2 *>(p);
        const float2 a = Pair16<__half>::unpack(raw.x), b = Pair16<__half>::unpack(raw.y);
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

template <typename T, int D>
__global__ void __launch_bounds__(kAssignThreads)
assign_codes_kernel(const T *__restrict__ k, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                    const float *__restrict__ cb,    // [Hkv, M, K, D] dense
                    const float *__restrict__ bias,  // nullptr or [Hkv, M, K] dense
                    void *__restrict__ codes, int code_dtype, int64_t c_sb, int64_t c_sh, int64_t c_sl,
                    int Hkv, int64_t L, int M, int K)
{
    extern __shared__ __align__(16) float smem[];
    float *rT = smem;                     // [D][64]  residual, transposed
    float *cT = smem + D * kAssignKeys;   // [D][64]  codeword chunk, transposed
    __shared__ int s_best[kAssignKeys];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int u = blockIdx.y;
    const int b = u / Hkv, h = u % Hkv;
    const int64_t key0 = static_cast<int64_t>(blockIdx.x) * kAssignKeys;

    // fill rT: lane -> key, each thread moves 4 consecutive d of its key per step
    {
        const int key = tid & 63;
        const int64_t j = key0 + key;
        const T *src = k + b * k_sb + h * k_sh + j * k_sl;
        for (int g = tid >> 6; g < D / 4; g += kAssignThreads / 64) {
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (j < L) x = Vec4Load<T>::ld(src + 4 * g);
            rT[(4 * g + 0) * kAssignKeys + key] = x.x;
            rT[(4 * g + 1) * kAssignKeys + key] = x.y;
            rT[(4 * g + 2) * kAssignKeys + key] = x.z;
            rT[(4 * g + 3) * kAssignKeys + key] = x.w;
        }
    }

    for (int m = 0; m < M; ++m) {
        const float *cbm = cb + (static_cast<int64_t>(h) * M + m) * K * D;
        const float *bm = bias ? bias + (static_cast<int64_t>(h) * M + m) * K : nullptr;
        float best[4];
        int besti[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            best[i] = -INFINITY;
            besti[i] = 0;
        }
        for (int c0 = 0; c0 < K; c0 += kAssignCodes) {
            __syncthreads();  // previous chunk consumed; rT writes (fill / residual update) visible
            {
                const int code = tid & 63;
                const float *src = cbm + static_cast<int64_t>(c0 + code) * D;
                for (int g = tid >> 6; g < D / 4; g += kAssignThreads / 64) {
                    float4 x = *reinterpret_cast<const float4 *>(src + 4 * g);
                    cT[(4 * g + 0) * kAssignCodes + code] = x.x;
                    cT[(4 * g + 1) * kAssignCodes + code] = x.y;
                    cT[(4 * g + 2) * kAssignCodes + code] = x.z;
                    cT[(4 * g + 3) * kAssignCodes + code] = x.w;
                }
            }
            __syncthreads();
            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 8
            for (int d = 0; d < D; ++d) {
                const float4 rv = *reinterpret_cast<const float4 *>(rT + d * kAssignKeys + 4 * ty);
                const float4 cv = *reinterpret_cast<const float4 *>(cT + d * kAssignCodes + 4 * tx);
                const float r[4] = {rv.x, rv.y, rv.z, rv.w};
                const float c[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(r[i], c[j], acc[i][j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int code = c0 + 4 * tx + j;
                const float bj = bm ? bm[code] : 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float s = acc[i][j];
                    if (bm) s = __fadd_rn(s, bj);
                    if (s > best[i]) {
                        best[i] = s;
                        besti[i] = code;
                    }
                }
            }
        }
        // reduce over the 16 threads that share these keys; ties to the lowest code
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float ov = __shfl_xor_sync(0xffffffffu, best[i], off);
                const int oi = __shfl_xor_sync(0xffffffffu, besti[i], off);
                if (ov > best[i] || (ov == best[i] && oi < besti[i])) {
                    best[i] = ov;
                    besti[i] = oi;
                }
            }
        }
        if (tx == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = 4 * ty + i;
                s_best[key] = besti[i];
                const int64_t j = key0 + key;
                if (j < L) store_code(codes, code_dtype, b * c_sb + h * c_sh + j * c_sl + m, besti[i]);
            }
        }
        if (m + 1 < M) {
            __syncthreads();
            const int key = tid & 63;
            const float *src = cbm + static_cast<int64_t>(s_best[key]) * D;
            for (int g = tid >> 6; g < D / 4; g += kAssignThreads / 64) {
                float4 x = *reinterpret_cast<const float4 *>(src + 4 * g);
                float *p0 = rT + (4 * g) * kAssignKeys + key;
                p0[0 * kAssignKeys] = __fsub_rn(p0[0 * kAssignKeys], x.x);
                p0[1 * kAssignKeys] = __fsub_rn(p0[1 * kAssignKeys], x.y);
                p0[2 * kAssignKeys] = __fsub_rn(p0[2 * kAssignKeys], x.z);
                p0[3 * kAssignKeys] = __fsub_rn(p0[3 * kAssignKeys], x.w);
            }
        }
    }
}

template <typename T, int D>
static int launch_assign(const VqTensorDesc *k, const VqTensorDesc *cb, const VqTensorDesc *bias, VqTensorDesc *codes,
                         cudaStream_t stream)
{
    const int B = static_cast<int>(k->shape[0]), Hkv = static_cast<int>(k->shape[1]);
    const int64_t L = k->shape[2];
    const int M = static_cast<int>(cb->shape[1]), K = static_cast<int>(cb->shape[2]);
    const size_t smem = sizeof(float) * D * (kAssignKeys + kAssignCodes);
    auto kern = assign_codes_kernel<T, D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return VQ_ELAUNCH;
    dim3 grid(static_cast<unsigned>((L + kAssignKeys - 1) / kAssignKeys), static_cast<unsigned>(B * Hkv));
    kern<<<grid, kAssignThreads, smem, stream>>>(
        static_cast<const T *>(k->ptr), k->stride[0], k->stride[1], k->stride[2], static_cast<const float *>(cb->ptr),
        bias ? static_cast<const float *>(bias->ptr) : nullptr, codes->ptr, codes->dtype, codes->stride[0],
        codes->stride[1], codes->stride[2], Hkv, L, M, K);
    return launch_status();
}

}  // namespace vq

extern "C" int vqattn_assign_codes(const VqTensorDesc *k, const VqTensorDesc *codebooks, const VqTensorDesc *bias,
                                   VqTensorDesc *codes, void *stream)
{
    using namespace vq;
    int st;
    if ((st = check_basic(k, 4)) != VQ_OK) return st;
    if ((st = check_basic(codebooks, 4)) != VQ_OK) return st;
    if ((st = check_basic(codes, 4)) != VQ_OK) return st;
    if (bias != nullptr && bias->ptr == nullptr) bias = nullptr;
    if (bias != nullptr && (st = check_basic(bias, 3)) != VQ_OK) return st;
    const VqTensorDesc *all[] = {k, codebooks, bias, codes};
    if ((st = check_device(all, 4)) != VQ_OK) return st;
    if (!is_act_dtype(k->dtype) || codebooks->dtype != VQ_F32 || !is_code_dtype(codes->dtype)) return VQ_EINVAL_DTYPE;
    if (bias && bias->dtype != VQ_F32) return VQ_EINVAL_DTYPE;
    const int64_t B = k->shape[0], Hkv = k->shape[1], L = k->shape[2], D = k->shape[3];
    const int64_t M = codebooks->shape[1], K = codebooks->shape[2];
    if (codebooks->shape[0] != Hkv || codebooks->shape[3] != D) return VQ_EINVAL_SHAPE;
    if (codes->shape[0] != B || codes->shape[1] != Hkv || codes->shape[2] != L || codes->shape[3] != M) return VQ_EINVAL_SHAPE;
    if (bias && (bias->shape[0] != Hkv || bias->shape[1] != M || bias->shape[2] != K)) return VQ_EINVAL_SHAPE;
    if (!is_dense(*codebooks) || (bias && !is_dense(*bias))) return VQ_EINVAL_STRIDE;
    if (D != 64 && D != 128) return VQ_EUNSUPPORTED;
    if (K % kAssignCodes != 0 || K > 65536) return VQ_EUNSUPPORTED;
    if (codes->dtype == VQ_U8 && K > 256) return VQ_EINVAL_DTYPE;
    // vector loads need 16-byte (f32) / 8-byte (bf16) aligned rows
    const int64_t align = k->dtype == VQ_F32 ? 4 : 4;
    if (k->stride[0] % align || k->stride[1] % align || k->stride[2] % align) return VQ_EINVAL_STRIDE;
    if (reinterpret_cast<uintptr_t>(k->ptr) % 16 != 0 || reinterpret_cast<uintptr_t>(codebooks->ptr) % 16 != 0)
        return VQ_EINVAL_STRIDE;
    if (B * Hkv > 65535) return VQ_EUNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (k->dtype == VQ_F32)
        return D == 64 ? launch_assign<float, 64>(k, codebooks, bias, codes, s)
                       : launch_assign<float, 128>(k, codebooks, bias, codes, s);
    if (k->dtype == VQ_F16)
        return D == 64 ? launch_assign<__half, 64>(k, codebooks, bias, codes, s)
                       : launch_assign<__half, 128>(k, codebooks, bias, codes, s);
    return D == 64 ? launch_assign<__nv_bfloat16, 64>(k, codebooks, bias, codes, s)
                   : launch_assign<__nv_bfloat16, 128>(k, codebooks, bias, codes, s);
}
