// Shared helpers for the vqattn kernels: descriptor checks, dtype conversion, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vqattn.h"

namespace vq {

constexpr int kBlock = VQATTN_BLOCK;

inline bool last_dim_contiguous(const VqTensorDesc &t) { return t.ndim >= 1 && (t.stride[t.ndim - 1] == 1 || t.shape[t.ndim - 1] == 1); }

// Checks ndim, non-null pointer and a unit innermost stride.
inline int check_basic(const VqTensorDesc *t, int ndim)
{
    if (t == nullptr || t->ptr == nullptr) return VQ_EINVAL_ARG;
    if (t->ndim != ndim) return VQ_EINVAL_SHAPE;
    for (int i = 0; i < ndim; ++i)
        if (t->shape[i] <= 0) return VQ_EINVAL_SHAPE;
    if (!last_dim_contiguous(*t)) return VQ_EINVAL_STRIDE;
    return VQ_OK;
}

// True when the view is fully dense row-major.
inline bool is_dense(const VqTensorDesc &t)
{
    int64_t expect = 1;
    for (int i = t.ndim - 1; i >= 0; --i) {
        if (t.shape[i] != 1 && t.stride[i] != expect) return false;
        expect *= t.shape[i];
    }
    return true;
}

inline int check_device(const VqTensorDesc *const *ts, int n)
{
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) return VQ_EDEVICE;
    for (int i = 0; i < n; ++i)
        if (ts[i] != nullptr && ts[i]->ptr != nullptr && ts[i]->device != cur) return VQ_EDEVICE;
    return VQ_OK;
}

// Cycles a device-side wait may last before a kernel gives up (set by vqattn_set_wait_limit_cycles).
long long wait_limit_cycles();

inline int launch_status()
{
    return cudaGetLastError() == cudaSuccess ? VQ_OK : VQ_ELAUNCH;
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Two packed 16-bit floats <-> two fp32 values, for either 16-bit activation type.
template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
    static __device__ __forceinline__ float2 unpack(uint32_t w) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&w)); }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi)
    {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};
template <> struct Pair16<__half> {
    static __device__ __forceinline__ float2 unpack(uint32_t w) { return __half22float2(*reinterpret_cast<__half2 *>(&w)); }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi)
    {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};

// Reads one code of any supported integer width.
__device__ __forceinline__ int load_code(const void *base, int dtype, int64_t idx)
{
    switch (dtype) {
    case VQ_U8: return static_cast<const uint8_t *>(base)[idx];
    case VQ_U16: return static_cast<const uint16_t *>(base)[idx];
    case VQ_I32: return static_cast<const int32_t *>(base)[idx];
    default: return static_cast<int>(static_cast<const int64_t *>(base)[idx]);
    }
}

__device__ __forceinline__ void store_code(void *base, int dtype, int64_t idx, int code)
{
    switch (dtype) {
    case VQ_U8: static_cast<uint8_t *>(base)[idx] = static_cast<uint8_t>(code); break;
    case VQ_U16: static_cast<uint16_t *>(base)[idx] = static_cast<uint16_t>(code); break;
    case VQ_I32: static_cast<int32_t *>(base)[idx] = code; break;
    default: static_cast<int64_t *>(base)[idx] = code; break;
    }
}

inline bool is_code_dtype(int dt) { return dt == VQ_U8 || dt == VQ_U16 || dt == VQ_I32 || dt == VQ_I64; }
inline bool is_act_dtype(int dt) { return dt == VQ_F32 || dt == VQ_BF16 || dt == VQ_F16; }
inline bool is_16bit(int dt) { return dt == VQ_BF16 || dt == VQ_F16; }

}  // namespace vq
