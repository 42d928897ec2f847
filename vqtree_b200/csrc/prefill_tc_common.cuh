// Shared by the tensor-core prefill kernels: parameters, the per-tile work list, tensor-map helpers.
#pragma once

#include <cuda.h>

#include "tc_ptx.cuh"
#include "vq_common.cuh"

namespace vq {

constexpr int kHalfBytes = kBlock * 64 * 2;  // one TMA box: 128 rows x 64 bf16 (128 B per row)

enum ItemKind : int { kFar = 0, kBdA = 1, kBdB = 2, kFull = 3, kDiag = 4 };

struct TcParams {
    int Hq, Hkv, NB, MK, rerope, ntiles;
    int64_t L;
    int wblocks;  // window / 128
    float scale_log2;
    const float *cnt;  // [B*Hkv, NB, MK]
    uint16_t *out;     // 16-bit activation dtype (bf16 or half)
    int64_t o_sb, o_sh, o_sl;
    float *lse2;
    int32_t *status;
    long long wait_limit;  // cycles a device-side wait may last before the kernel gives up
};

// Work list of query tile m: far codebook tiles, the boundary block (two masked passes in ReRoPE
// mode), interior blocks, the causal diagonal block.
struct TcWork {
    int kb0, far_blk, n_far, n_bd, first_full, n_full, n_items, rerope;
    __device__ __forceinline__ TcWork(const TcParams &p, int m)
    {
        rerope = p.rerope;
        kb0 = m - p.wblocks;                              // boundary block (exists when >= 0)
        const bool has_far = kb0 >= 1 && p.MK > 0;
        far_blk = kb0 - 1;
        n_far = has_far ? p.MK / kBlock : 0;
        n_bd = (kb0 >= 0) ? (p.rerope ? 2 : 1) : 0;
        first_full = kb0 >= 0 ? kb0 + 1 : 0;
        n_full = m - first_full;                          // interior blocks
        n_items = n_far + n_bd + n_full + 1;
    }
    __device__ __forceinline__ int kind(int it) const
    {
        if (it < n_far) return kFar;
        it -= n_far;
        if (it < n_bd) return rerope ? (it == 0 ? kBdA : kBdB) : kFull;
        it -= n_bd;
        return it < n_full ? kFull : kDiag;
    }
    __device__ __forceinline__ int block(int it) const  // far: codebook tile index; local: key block index
    {
        if (it < n_far) return it;
        it -= n_far;
        if (it < n_bd) return kb0;
        it -= n_bd;
        return first_full + it;
    }
};

// ------------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// bf16 tensor with up to 4 dims given innermost-first; box = 64 x box_rows (x 1 x 1), 128-byte swizzle.
inline bool make_map(CUtensorMap *out, const void *ptr, int rank, const uint64_t *dims, const uint64_t *strides_elems,
                     int box_rows = kBlock, bool f16 = false)
{
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t gdim[4], gstride[3];
    cuuint32_t box[4], estr[4];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        box[i] = i == 0 ? 64 : (i == 1 ? box_rows : 1);
        estr[i] = 1;
        if (i > 0) gstride[i - 1] = strides_elems[i] * 2;
    }
    return fn(out, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(ptr), gdim, gstride, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool map_bhld(CUtensorMap *out, const VqTensorDesc &t)
{
    const uint64_t dims[4] = {static_cast<uint64_t>(t.shape[3]), static_cast<uint64_t>(t.shape[2]),
                              static_cast<uint64_t>(t.shape[1]), static_cast<uint64_t>(t.shape[0])};
    const uint64_t str[4] = {1, static_cast<uint64_t>(t.stride[2]), static_cast<uint64_t>(t.stride[1]),
                             static_cast<uint64_t>(t.stride[0])};
    return make_map(out, t.ptr, 4, dims, str, kBlock, t.dtype == VQ_F16);
}

struct TcMaps {
    CUtensorMap q1, q2, k1, k3, v, cb, vs;
};

// Fills the seven tensor maps and the kernel parameters from the C-ABI arguments.
template <int D>
inline int tc_setup(const VqPrefillArgs *a, TcMaps &m, TcParams &p)
{
    const int64_t B = a->q1.shape[0], Hq = a->q1.shape[1], L = a->q1.shape[2], Hkv = a->k1.shape[1];
    const bool far = a->codebook.ptr != nullptr && a->cnt.ptr != nullptr;
    if (!map_bhld(&m.q1, a->q1) || !map_bhld(&m.q2, a->q2) || !map_bhld(&m.k1, a->k1) || !map_bhld(&m.k3, a->k3) ||
        !map_bhld(&m.v, a->v))
        return VQ_ELAUNCH;
    p = TcParams{};
    if (far) {
        const uint64_t MK = a->codebook.shape[1], NB = a->cnt.shape[2];
        const uint64_t cd[3] = {static_cast<uint64_t>(D), MK, static_cast<uint64_t>(Hkv)};
        const uint64_t cs[3] = {1, static_cast<uint64_t>(D), MK * D};
        const uint64_t vd[3] = {static_cast<uint64_t>(D), MK, static_cast<uint64_t>(B * Hkv) * NB};
        const bool f16 = a->q1.dtype == VQ_F16;
        if (!make_map(&m.cb, a->codebook.ptr, 3, cd, cs, kBlock, f16) || !make_map(&m.vs, a->vsum.ptr, 3, vd, cs, kBlock, f16))
            return VQ_ELAUNCH;
        p.MK = static_cast<int>(MK);
        p.NB = static_cast<int>(NB);
        p.cnt = static_cast<const float *>(a->cnt.ptr);
    } else {
        m.cb = m.k1;  // never dereferenced: the work list has no far items
        m.vs = m.v;
    }
    p.Hq = static_cast<int>(Hq); p.Hkv = static_cast<int>(Hkv);
    p.L = L;
    p.ntiles = static_cast<int>((L + kBlock - 1) / kBlock);
    p.wblocks = static_cast<int>(a->window / kBlock);
    p.rerope = (a->q2.ptr != a->q1.ptr || a->k3.ptr != a->k1.ptr) ? 1 : 0;
    const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf(static_cast<float>(D));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = static_cast<uint16_t *>(a->out.ptr);
    p.o_sb = a->out.stride[0]; p.o_sh = a->out.stride[1]; p.o_sl = a->out.stride[2];
    p.lse2 = static_cast<float *>(a->lse2.ptr);
    p.status = a->status_word;
    p.wait_limit = wait_limit_cycles();
    return VQ_OK;
}

}  // namespace vq
