// Per-block aggregates of the quantised keys: replaces the host preparation of the reference
// (ops/attn_vq.py:352-384,411-417: one-hot cumsum over [B,H,L,C], argsort, gather, prefix sums).
//
// For every 128-key block n the outputs describe the keys [0, 128(n+1)):
//   cnt[n][r]  = number of keys whose code in codebook m is c   (r = m*K + c)
//   vsum[n][r] = sum of their value rows, fp32, added in position order, stored in the output dtype.
// One CTA owns (batch*kv-head, codebook m, a part of <= 256 codes, a 32-column slice of D), keeps
// the running fp32 sums of its rows in shared memory, walks the blocks in order and writes a
// snapshot after each.  A row is always updated by the same thread in position order, so the
// sums are deterministic and equal a scalar left-to-right loop.
#include "vq_common.cuh"

namespace vq {

// aggregate_reg.cu: bf16 kernel with the running sums in registers
bool aggregates_reg_eligible(const VqTensorDesc *v, const VqTensorDesc *vsum, int K);
bool aggregates_sorted_eligible(const VqTensorDesc *v, const VqTensorDesc *vsum, int K);
size_t aggregates_sorted_workspace_bytes(int64_t B, int64_t Hkv, int64_t NB, int64_t M, int64_t K);
int launch_aggregates_sorted(const VqTensorDesc *codes, const VqTensorDesc *v, int K, VqTensorDesc *cnt, VqTensorDesc *vsum, void *workspace,
                             int32_t *status, cudaStream_t stream, float *state_cnt = nullptr, float *state_vsum = nullptr,
                             int64_t state_blocks = 0);
int launch_aggregates_reg(const VqTensorDesc *codes, const VqTensorDesc *v, int K, VqTensorDesc *cnt, VqTensorDesc *vsum,
                          cudaStream_t stream);

constexpr int kAggThreads = 256;
constexpr int kAggCols = 32;    // D-slice per CTA
constexpr int kAggRows = 256;   // code rows per CTA

template <typename T> __device__ __forceinline__ float4 ld4(const T *p);
template <> __device__ __forceinline__ float4 ld4<float>(const float *p) { return *reinterpret_cast<const float4 *>(p); }
template <> __device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16 *p)
{
    uint2 raw = *reinterpret_cast<const uint2 *>(p);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&raw.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <> __device__ __forceinline__ float4 ld4<__half>(const __half *p)
{
    uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = Pair16<__half>::unpack(raw.x), b = Pair16<__half>::unpack(raw.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void st4(T *p, float4 x);
template <> __device__ __forceinline__ void st4<__half>(__half *p, float4 x)
{
    uint2 raw;
    raw.x = Pair16<__half>::pack(x.x, x.y);
    raw.y = Pair16<__half>::pack(x.z, x.w);
    *reinterpret_cast<uint2 *>(p) = raw;
}
template <> __device__ __forceinline__ void st4<float>(float *p, float4 x) { *reinterpret_cast<float4 *>(p) = x; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16 *p, float4 x)
{
    __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y);
    __nv_bfloat162 b = __floats2bfloat162_rn(x.z, x.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t *>(&a);
    raw.y = *reinterpret_cast<uint32_t *>(&b);
    *reinterpret_cast<uint2 *>(p) = raw;
}

template <typename T> __device__ __forceinline__ void st8(T *p, float4 x, float4 y);
template <> __device__ __forceinline__ void st8<float>(float *p, float4 x, float4 y)
{
    *reinterpret_cast<float4 *>(p) = x;
    *reinterpret_cast<float4 *>(p + 4) = y;
}
template <> __device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16 *p, float4 x, float4 y)
{
    __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y), b = __floats2bfloat162_rn(x.z, x.w);
    __nv_bfloat162 c = __floats2bfloat162_rn(y.x, y.y), d = __floats2bfloat162_rn(y.z, y.w);
    uint4 raw;
    raw.x = *reinterpret_cast<uint32_t *>(&a);
    raw.y = *reinterpret_cast<uint32_t *>(&b);
    raw.z = *reinterpret_cast<uint32_t *>(&c);
    raw.w = *reinterpret_cast<uint32_t *>(&d);
    *reinterpret_cast<uint4 *>(p) = raw;
}

template <> __device__ __forceinline__ void st8<__half>(__half *p, float4 x, float4 y)
{
    uint4 raw;
    raw.x = Pair16<__half>::pack(x.x, x.y);
    raw.y = Pair16<__half>::pack(x.z, x.w);
    raw.z = Pair16<__half>::pack(y.x, y.y);
    raw.w = Pair16<__half>::pack(y.z, y.w);
    *reinterpret_cast<uint4 *>(p) = raw;
}

template <typename TV, typename TO>
__global__ void __launch_bounds__(kAggThreads, 4)
build_aggregates_kernel(const void *__restrict__ codes, int code_dtype, int64_t c_sb, int64_t c_sh, int64_t c_sl,
                        const TV *__restrict__ v, int64_t v_sb, int64_t v_sh, int64_t v_sl,
                        float *__restrict__ cnt,  // [B,Hkv,NB,MK] dense
                        TO *__restrict__ vsum,    // [B,Hkv,NB,MK,D] dense
                        int Hkv, int D, int M, int K, int NB, int parts, int rows_per_part)
{
    extern __shared__ __align__(16) float smem[];
    float *acc = smem;                               // [rows_per_part][32]
    float *vt = smem + rows_per_part * kAggCols;     // [128][32]
    __shared__ int s_code[kBlock];
    __shared__ int s_cnt[kAggRows];

    const int tid = threadIdx.x;
    const int slices = D / kAggCols;
    int bx = blockIdx.x;
    const int ds = bx % slices; bx /= slices;
    const int kp = bx % parts;  bx /= parts;
    const int m = bx % M;
    const int u = blockIdx.y;
    const int b = u / Hkv, h = u % Hkv;
    const int MK = M * K;
    const int row0 = kp * rows_per_part;  // first code of this part (within codebook m)

    for (int i = tid; i < rows_per_part * kAggCols; i += kAggThreads) acc[i] = 0.f;
    for (int i = tid; i < kAggRows; i += kAggThreads) s_cnt[i] = 0;

    const int col = tid & (kAggCols - 1);
    const int grp = tid / kAggCols;  // 8 groups; group g owns the code rows with (row & 7) == g
    constexpr int kVecPerThread = kBlock * (kAggCols / 4) / kAggThreads;  // 4

    // the next block's codes and value tile travel in registers while the current block is summed
    float4 nv[kVecPerThread];
    int ncode = -1;
    auto fetch = [&](int n) {
        const int64_t j0 = static_cast<int64_t>(n) * kBlock;
        if (tid < kBlock) ncode = load_code(codes, code_dtype, b * c_sb + h * c_sh + (j0 + tid) * c_sl + m);
#pragma unroll
        for (int t = 0; t < kVecPerThread; ++t) {
            const int i = tid + t * kAggThreads;
            const int r = i / (kAggCols / 4), c4 = i % (kAggCols / 4);
            nv[t] = ld4<TV>(v + b * v_sb + h * v_sh + (j0 + r) * v_sl + ds * kAggCols + 4 * c4);
        }
    };
    if (NB > 0) fetch(0);
    __syncthreads();

    for (int n = 0; n < NB; ++n) {
        if (tid < kBlock) {
            const int local = ncode - row0;
            const bool mine = local >= 0 && local < rows_per_part;
            s_code[tid] = mine ? local : -1;
            if (mine) atomicAdd(&s_cnt[local], 1);
        }
#pragma unroll
        for (int t = 0; t < kVecPerThread; ++t) {
            const int i = tid + t * kAggThreads;
            *reinterpret_cast<float4 *>(vt + (i / (kAggCols / 4)) * kAggCols + 4 * (i % (kAggCols / 4))) = nv[t];
        }
        __syncthreads();
        if (n + 1 < NB) fetch(n + 1);
        // warp `grp` owns the code rows with (row & 7) == grp: it picks its keys out of the block with
        // ballots and adds them in position order (lowest bit first), 32 columns wide
#pragma unroll
        for (int t = 0; t < kBlock / 32; ++t) {
            const int lc_t = s_code[32 * t + (tid & 31)];
            unsigned bal = __ballot_sync(0xffffffffu, lc_t >= 0 && (lc_t & 7) == grp);
            while (bal) {
                const int bit = __ffs(bal) - 1;
                bal &= bal - 1;
                const int lc = __shfl_sync(0xffffffffu, lc_t, bit);
                acc[lc * kAggCols + col] = __fadd_rn(acc[lc * kAggCols + col], vt[(32 * t + bit) * kAggCols + col]);
            }
        }
        __syncthreads();
        const int64_t out_row0 = (static_cast<int64_t>(u) * NB + n) * MK + m * K + row0;
        for (int i = tid; i < rows_per_part * (kAggCols / 8); i += kAggThreads) {
            const int r = i / (kAggCols / 8), c8 = i % (kAggCols / 8);
            const float4 x = *reinterpret_cast<const float4 *>(acc + r * kAggCols + 8 * c8);
            const float4 y = *reinterpret_cast<const float4 *>(acc + r * kAggCols + 8 * c8 + 4);
            st8<TO>(vsum + (out_row0 + r) * D + ds * kAggCols + 8 * c8, x, y);
        }
        if (ds == 0)
            for (int i = tid; i < rows_per_part; i += kAggThreads) cnt[out_row0 + i] = static_cast<float>(s_cnt[i]);
        // the next iteration rewrites s_code, vt and s_cnt right away: wait for this snapshot's readers
        __syncthreads();
    }
}

template <typename T>
__global__ void gather_aggregates_kernel(const T *__restrict__ v_vq, int64_t s_b, int64_t s_h, int64_t s_n,
                                         const void *__restrict__ vi, int vi_dtype, int64_t i_b, int64_t i_h, int64_t i_n,
                                         const float *__restrict__ cnt, T *__restrict__ vsum, int H, int NB, int C, int D,
                                         int64_t rows_in)
{
    // one warp per output row
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x & 31;
    const int u = blockIdx.y;
    if (row >= static_cast<int64_t>(NB) * C) return;
    const int n = static_cast<int>(row / C), c = static_cast<int>(row % C);
    const int b = u / H, h = u % H;
    const int64_t at = b * i_b + h * i_h + n * i_n + c;
    const int64_t src = vi_dtype == VQ_I64 ? static_cast<const int64_t *>(vi)[at] : static_cast<const int32_t *>(vi)[at];
    T *dst = vsum + ((static_cast<int64_t>(u) * NB + n) * C + c) * D;
    const bool ok = src >= 0 && src < rows_in && (cnt == nullptr || cnt[(static_cast<int64_t>(u) * NB + n) * C + c] > 0.f);
    const T *s = v_vq + b * s_b + h * s_h + (ok ? src : 0) * s_n;
    for (int d = lane; d < D; d += 32) dst[d] = ok ? s[d] : from_f32<T>(0.f);
}

// Cache advance: one CTA owns kAdvRows code rows of one codebook of one (batch, kv head); it keeps their
// fp32 sums in shared memory, walks the new keys in position order and adds the value rows of the keys
// whose code falls into its rows - the same left-to-right fp32 sum per row as build_aggregates.
// A code outside [0, K) would address another row (or memory outside the buffers): such a key is
// skipped and the status word is raised instead.
constexpr int kAdvRows = 16;
constexpr int kAdvThreads = 128;

template <typename TV, typename TS>
__global__ void __launch_bounds__(kAdvThreads)
cache_advance_kernel(const void *__restrict__ codes, int code_dtype, int64_t c_sb, int64_t c_sh, int64_t c_sl,
                     const TV *__restrict__ v, int64_t v_sb, int64_t v_sh, int64_t v_sl, float *__restrict__ cnt,
                     float *__restrict__ vsum, TS *__restrict__ shadow, int Hkv, int D, int M, int K, int n_new,
                     int32_t *__restrict__ status)
{
    extern __shared__ float s_acc[];  // [kAdvRows][D]
    __shared__ int s_rel[kAdvThreads];
    __shared__ float s_cnt[kAdvRows];
    const int tid = threadIdx.x;
    const int parts = (K + kAdvRows - 1) / kAdvRows;
    const int m = static_cast<int>(blockIdx.x) / parts, r0 = (static_cast<int>(blockIdx.x) % parts) * kAdvRows;
    const int nrows = min(kAdvRows, K - r0);
    const int u = blockIdx.y;
    const int b = u / Hkv, h = u % Hkv;
    const int64_t row0 = static_cast<int64_t>(u) * M * K + static_cast<int64_t>(m) * K + r0;
    for (int i = tid; i < nrows * D; i += kAdvThreads) s_acc[i] = vsum[row0 * D + i];
    if (tid < kAdvRows) s_cnt[tid] = tid < nrows ? cnt[row0 + tid] : 0.f;
    __syncthreads();
    const TV *vb = v + b * v_sb + h * v_sh;
    for (int j0 = 0; j0 < n_new; j0 += kAdvThreads) {
        int rel = -1;
        if (j0 + tid < n_new) {
            const int code = load_code(codes, code_dtype, b * c_sb + h * c_sh + (j0 + tid) * c_sl + m);
            if (static_cast<unsigned>(code) >= static_cast<unsigned>(K)) {
                if (status) atomicExch(status, VQ_WORD_BAD_CODE);
            } else {
                rel = code - r0;
            }
        }
        s_rel[tid] = rel;
        __syncthreads();
        const int nk = min(kAdvThreads, n_new - j0);
        for (int jj = 0; jj < nk; ++jj) {
            const int rr = s_rel[jj];
            if (static_cast<unsigned>(rr) < static_cast<unsigned>(nrows)) {
                const TV *vr = vb + static_cast<int64_t>(j0 + jj) * v_sl;
                for (int d = tid; d < D; d += kAdvThreads) s_acc[rr * D + d] = __fadd_rn(s_acc[rr * D + d], to_f32(vr[d]));
                if (tid == 0) s_cnt[rr] += 1.f;
            }
        }
        __syncthreads();
    }
    for (int i = tid; i < nrows * D; i += kAdvThreads) {
        vsum[row0 * D + i] = s_acc[i];
        if (shadow) shadow[row0 * D + i] = from_f32<TS>(s_acc[i]);
    }
    if (tid < nrows) cnt[row0 + tid] = s_cnt[tid];
}

}  // namespace vq

namespace vq {
static int build_aggregates_impl(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt, VqTensorDesc *vsum,
                                 void *workspace, size_t workspace_bytes, int32_t *status_word, void *stream,
                                 VqTensorDesc *state_cnt = nullptr, VqTensorDesc *state_vsum = nullptr, int64_t state_blocks = 0);
}

extern "C" int vqattn_build_aggregates(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt,
                                       VqTensorDesc *vsum, void *stream)
{
    return vq::build_aggregates_impl(codes, v, K, cnt, vsum, nullptr, 0, nullptr, stream);
}

extern "C" size_t vqattn_aggregates_workspace_bytes(int64_t B, int64_t Hkv, int64_t NB, int64_t M, int64_t K)
{
    if (B <= 0 || Hkv <= 0 || NB <= 0 || M <= 0 || K <= 0) return 0;
    return vq::aggregates_sorted_workspace_bytes(B, Hkv, NB, M, K);
}

extern "C" int vqattn_build_aggregates_ws(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt,
                                          VqTensorDesc *vsum, void *workspace, size_t workspace_bytes, int32_t *status_word,
                                          void *stream)
{
    return vq::build_aggregates_impl(codes, v, K, cnt, vsum, workspace, workspace_bytes, status_word, stream);
}

extern "C" int vqattn_build_aggregates_state(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt,
                                             VqTensorDesc *vsum, VqTensorDesc *state_cnt, VqTensorDesc *state_vsum, int64_t state_blocks,
                                             void *workspace, size_t workspace_bytes, int32_t *status_word, void *stream)
{
    if (state_cnt == nullptr || state_vsum == nullptr) return VQ_EINVAL_ARG;
    return vq::build_aggregates_impl(codes, v, K, cnt, vsum, workspace, workspace_bytes, status_word, stream, state_cnt, state_vsum,
                                     state_blocks);
}

static int vq::build_aggregates_impl(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt, VqTensorDesc *vsum,
                                     void *workspace, size_t workspace_bytes, int32_t *status_word, void *stream,
                                     VqTensorDesc *state_cnt, VqTensorDesc *state_vsum, int64_t state_blocks)
{
    using namespace vq;
    int st;
    if ((st = check_basic(codes, 4)) != VQ_OK) return st;
    if ((st = check_basic(v, 4)) != VQ_OK) return st;
    if ((st = check_basic(cnt, 4)) != VQ_OK) return st;
    if ((st = check_basic(vsum, 5)) != VQ_OK) return st;
    const VqTensorDesc *all[] = {codes, v, cnt, vsum};
    if ((st = check_device(all, 4)) != VQ_OK) return st;
    if (!is_code_dtype(codes->dtype) || !is_act_dtype(v->dtype) || cnt->dtype != VQ_F32 || !is_act_dtype(vsum->dtype))
        return VQ_EINVAL_DTYPE;
    const int64_t B = codes->shape[0], Hkv = codes->shape[1], L = codes->shape[2], M = codes->shape[3];
    const int64_t D = v->shape[3], NB = cnt->shape[2], MK = cnt->shape[3];
    if (K <= 0 || MK != M * K) return VQ_EINVAL_SHAPE;
    if (v->shape[0] != B || v->shape[1] != Hkv || v->shape[2] != L) return VQ_EINVAL_SHAPE;
    if (cnt->shape[0] != B || cnt->shape[1] != Hkv) return VQ_EINVAL_SHAPE;
    if (vsum->shape[0] != B || vsum->shape[1] != Hkv || vsum->shape[2] != NB || vsum->shape[3] != MK || vsum->shape[4] != D)
        return VQ_EINVAL_SHAPE;
    if (NB * kBlock > L) return VQ_EINVAL_SHAPE;
    if (!is_dense(*cnt) || !is_dense(*vsum)) return VQ_EINVAL_STRIDE;
    if (D % kAggCols != 0 || D > 256) return VQ_EUNSUPPORTED;
    if (v->stride[0] % 4 || v->stride[1] % 4 || v->stride[2] % 4 || reinterpret_cast<uintptr_t>(v->ptr) % 16) return VQ_EINVAL_STRIDE;
    if (reinterpret_cast<uintptr_t>(vsum->ptr) % 16) return VQ_EINVAL_STRIDE;
    if (B * Hkv > 65535) return VQ_EUNSUPPORTED;
    if (state_cnt != nullptr) {
        // the state after state_blocks blocks: fp32, dense, on the same device; at least as many blocks as snapshots
        if ((st = check_basic(state_cnt, 3)) != VQ_OK) return st;
        if ((st = check_basic(state_vsum, 4)) != VQ_OK) return st;
        const VqTensorDesc *sd[] = {codes, state_cnt, state_vsum};
        if ((st = check_device(sd, 3)) != VQ_OK) return st;
        if (state_cnt->dtype != VQ_F32 || state_vsum->dtype != VQ_F32) return VQ_EINVAL_DTYPE;
        if (state_blocks < NB || state_blocks < 1 || state_blocks * kBlock > L) return VQ_EINVAL_SHAPE;
        if (state_cnt->shape[0] != B || state_cnt->shape[1] != Hkv || state_cnt->shape[2] != MK) return VQ_EINVAL_SHAPE;
        if (state_vsum->shape[0] != B || state_vsum->shape[1] != Hkv || state_vsum->shape[2] != MK || state_vsum->shape[3] != D)
            return VQ_EINVAL_SHAPE;
        if (!is_dense(*state_cnt) || !is_dense(*state_vsum) || reinterpret_cast<uintptr_t>(state_vsum->ptr) % 16) return VQ_EINVAL_STRIDE;
        if (NB > 0 && workspace != nullptr && aggregates_sorted_eligible(v, vsum, K) &&
            workspace_bytes >= aggregates_sorted_workspace_bytes(B, Hkv, state_blocks, M, K))
            return launch_aggregates_sorted(codes, v, K, cnt, vsum, workspace, status_word, static_cast<cudaStream_t>(stream),
                                            static_cast<float *>(state_cnt->ptr), static_cast<float *>(state_vsum->ptr), state_blocks);
        // other inputs: the snapshots as without a state, then the state by the cache-advance kernel from zero
        if ((st = build_aggregates_impl(codes, v, K, cnt, vsum, workspace, workspace_bytes, status_word, stream)) != VQ_OK) return st;
        cudaStream_t cs = static_cast<cudaStream_t>(stream);
        if (cudaMemsetAsync(state_cnt->ptr, 0, sizeof(float) * static_cast<size_t>(B * Hkv * MK), cs) != cudaSuccess ||
            cudaMemsetAsync(state_vsum->ptr, 0, sizeof(float) * static_cast<size_t>(B * Hkv * MK * D), cs) != cudaSuccess)
            return VQ_ELAUNCH;
        VqTensorDesc c2 = *codes, v2 = *v;
        c2.shape[2] = v2.shape[2] = state_blocks * kBlock;
        return vqattn_cache_advance(&c2, &v2, K, state_cnt, state_vsum, nullptr, status_word, stream);
    }
    if (NB > 0 && workspace != nullptr && aggregates_sorted_eligible(v, vsum, K) &&
        workspace_bytes >= aggregates_sorted_workspace_bytes(B, Hkv, NB, M, K))
        return launch_aggregates_sorted(codes, v, K, cnt, vsum, workspace, status_word, static_cast<cudaStream_t>(stream));
    if (NB > 0 && aggregates_reg_eligible(v, vsum, K))
        return launch_aggregates_reg(codes, v, K, cnt, vsum, static_cast<cudaStream_t>(stream));
    int rows = static_cast<int>(K < kAggRows ? K : kAggRows);
    if (K % rows != 0) return VQ_EUNSUPPORTED;
    const int parts = static_cast<int>(K / rows);
    const size_t smem = sizeof(float) * (static_cast<size_t>(rows) * kAggCols + kBlock * kAggCols);
    dim3 grid(static_cast<unsigned>(M * parts * (D / kAggCols)), static_cast<unsigned>(B * Hkv));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define VQ_LAUNCH_AGG(TV, TO)                                                                                          \
    do {                                                                                                               \
        auto kern = build_aggregates_kernel<TV, TO>;                                                                   \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=        \
            cudaSuccess)                                                                                               \
            return VQ_ELAUNCH;                                                                                         \
        kern<<<grid, kAggThreads, smem, s>>>(codes->ptr, codes->dtype, codes->stride[0], codes->stride[1],            \
                                             codes->stride[2], static_cast<const TV *>(v->ptr), v->stride[0],         \
                                             v->stride[1], v->stride[2], static_cast<float *>(cnt->ptr),              \
                                             static_cast<TO *>(vsum->ptr), static_cast<int>(Hkv), static_cast<int>(D), \
                                             static_cast<int>(M), static_cast<int>(K), static_cast<int>(NB), parts, rows); \
    } while (0)
    if (v->dtype == VQ_F32 && vsum->dtype == VQ_F32) VQ_LAUNCH_AGG(float, float);
    else if (v->dtype == VQ_F16 && vsum->dtype == VQ_F16) VQ_LAUNCH_AGG(__half, __half);
    else if (v->dtype == VQ_F16 && vsum->dtype == VQ_F32) VQ_LAUNCH_AGG(__half, float);
    else if (v->dtype == VQ_F16 || vsum->dtype == VQ_F16) return VQ_EINVAL_DTYPE;
    else if (v->dtype == VQ_F32) VQ_LAUNCH_AGG(float, __nv_bfloat16);
    else if (vsum->dtype == VQ_F32) VQ_LAUNCH_AGG(__nv_bfloat16, float);
    else VQ_LAUNCH_AGG(__nv_bfloat16, __nv_bfloat16);
#undef VQ_LAUNCH_AGG
    return launch_status();
}

extern "C" int vqattn_gather_aggregates(const VqTensorDesc *v_vq, const VqTensorDesc *vi, const VqTensorDesc *cnt,
                                        VqTensorDesc *vsum, void *stream)
{
    using namespace vq;
    int st;
    if (cnt != nullptr && cnt->ptr == nullptr) cnt = nullptr;
    if ((st = check_basic(v_vq, 4)) != VQ_OK) return st;
    if ((st = check_basic(vi, 4)) != VQ_OK) return st;
    if ((st = check_basic(vsum, 5)) != VQ_OK) return st;
    const VqTensorDesc *all[] = {v_vq, vi, vsum};
    if ((st = check_device(all, 3)) != VQ_OK) return st;
    if (!is_act_dtype(v_vq->dtype) || vsum->dtype != v_vq->dtype) return VQ_EINVAL_DTYPE;
    if (vi->dtype != VQ_I32 && vi->dtype != VQ_I64) return VQ_EINVAL_DTYPE;
    const int64_t B = v_vq->shape[0], H = v_vq->shape[1], D = v_vq->shape[3];
    const int64_t NB = vsum->shape[2], C = vsum->shape[3];
    if (vi->shape[0] != B || vi->shape[1] != H || vi->shape[2] < NB || vi->shape[3] != C) return VQ_EINVAL_SHAPE;
    if (vsum->shape[0] != B || vsum->shape[1] != H || vsum->shape[4] != D) return VQ_EINVAL_SHAPE;
    if (!is_dense(*vsum)) return VQ_EINVAL_STRIDE;
    if (cnt != nullptr) {
        if ((st = check_basic(cnt, 4)) != VQ_OK) return st;
        if (cnt->dtype != VQ_F32) return VQ_EINVAL_DTYPE;
        if (cnt->shape[0] != B || cnt->shape[1] != H || cnt->shape[2] != NB || cnt->shape[3] != C) return VQ_EINVAL_SHAPE;
        if (!is_dense(*cnt) || cnt->device != vsum->device) return VQ_EINVAL_STRIDE;
    }
    const float *cntp = cnt ? static_cast<const float *>(cnt->ptr) : nullptr;
    if (B * H > 65535) return VQ_EUNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int warps = 8;
    dim3 grid(static_cast<unsigned>((NB * C + warps - 1) / warps), static_cast<unsigned>(B * H));
    if (v_vq->dtype == VQ_F32)
        gather_aggregates_kernel<float><<<grid, warps * 32, 0, s>>>(
            static_cast<const float *>(v_vq->ptr), v_vq->stride[0], v_vq->stride[1], v_vq->stride[2], vi->ptr, vi->dtype,
            vi->stride[0], vi->stride[1], vi->stride[2], cntp, static_cast<float *>(vsum->ptr), static_cast<int>(H),
            static_cast<int>(NB), static_cast<int>(C), static_cast<int>(D), v_vq->shape[2]);
    else if (v_vq->dtype == VQ_F16)
        gather_aggregates_kernel<__half><<<grid, warps * 32, 0, s>>>(
            static_cast<const __half *>(v_vq->ptr), v_vq->stride[0], v_vq->stride[1], v_vq->stride[2], vi->ptr,
            vi->dtype, vi->stride[0], vi->stride[1], vi->stride[2], cntp, static_cast<__half *>(vsum->ptr),
            static_cast<int>(H), static_cast<int>(NB), static_cast<int>(C), static_cast<int>(D), v_vq->shape[2]);
    else
        gather_aggregates_kernel<__nv_bfloat16><<<grid, warps * 32, 0, s>>>(
            static_cast<const __nv_bfloat16 *>(v_vq->ptr), v_vq->stride[0], v_vq->stride[1], v_vq->stride[2], vi->ptr,
            vi->dtype, vi->stride[0], vi->stride[1], vi->stride[2], cntp, static_cast<__nv_bfloat16 *>(vsum->ptr),
            static_cast<int>(H), static_cast<int>(NB), static_cast<int>(C), static_cast<int>(D), v_vq->shape[2]);
    return launch_status();
}

extern "C" int vqattn_cache_advance(const VqTensorDesc *codes, const VqTensorDesc *v_new, int32_t K, VqTensorDesc *cnt,
                                    VqTensorDesc *vsum_f32, VqTensorDesc *vsum_act, int32_t *status_word, void *stream)
{
    using namespace vq;
    int st;
    if ((st = check_basic(codes, 4)) != VQ_OK) return st;
    if ((st = check_basic(v_new, 4)) != VQ_OK) return st;
    if ((st = check_basic(cnt, 3)) != VQ_OK) return st;
    if ((st = check_basic(vsum_f32, 4)) != VQ_OK) return st;
    if (vsum_act != nullptr && vsum_act->ptr == nullptr) vsum_act = nullptr;
    if (vsum_act && (st = check_basic(vsum_act, 4)) != VQ_OK) return st;
    const VqTensorDesc *all[] = {codes, v_new, cnt, vsum_f32, vsum_act};
    if ((st = check_device(all, 5)) != VQ_OK) return st;
    if (!is_code_dtype(codes->dtype) || !is_act_dtype(v_new->dtype) || cnt->dtype != VQ_F32 || vsum_f32->dtype != VQ_F32)
        return VQ_EINVAL_DTYPE;
    // the shadow copy is in the 16-bit activation dtype of the values (bf16 when the values are fp32)
    if (vsum_act && vsum_act->dtype != (v_new->dtype == VQ_F16 ? VQ_F16 : VQ_BF16)) return VQ_EINVAL_DTYPE;
    const int64_t B = codes->shape[0], Hkv = codes->shape[1], n_new = codes->shape[2], M = codes->shape[3];
    const int64_t D = v_new->shape[3], MK = cnt->shape[2];
    if (K <= 0 || MK != M * K) return VQ_EINVAL_SHAPE;
    if (v_new->shape[0] != B || v_new->shape[1] != Hkv || v_new->shape[2] != n_new) return VQ_EINVAL_SHAPE;
    if (cnt->shape[0] != B || cnt->shape[1] != Hkv) return VQ_EINVAL_SHAPE;
    if (vsum_f32->shape[0] != B || vsum_f32->shape[1] != Hkv || vsum_f32->shape[2] != MK || vsum_f32->shape[3] != D)
        return VQ_EINVAL_SHAPE;
    if (vsum_act && (vsum_act->shape[0] != B || vsum_act->shape[1] != Hkv || vsum_act->shape[2] != MK || vsum_act->shape[3] != D))
        return VQ_EINVAL_SHAPE;
    if (!is_dense(*cnt) || !is_dense(*vsum_f32) || (vsum_act && !is_dense(*vsum_act))) return VQ_EINVAL_STRIDE;
    if (D > 512 || B * Hkv > 65535) return VQ_EUNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t parts = (K + kAdvRows - 1) / kAdvRows;
    if (M * parts > 0x7fffffff) return VQ_EUNSUPPORTED;
    dim3 grid(static_cast<unsigned>(M * parts), static_cast<unsigned>(B * Hkv));
    const size_t smem = sizeof(float) * kAdvRows * static_cast<size_t>(D);
    void *shadow = vsum_act ? vsum_act->ptr : nullptr;
#define VQ_ADVANCE(TV, TS)                                                                                              \
    cache_advance_kernel<TV, TS><<<grid, kAdvThreads, smem, s>>>(                                                              \
        codes->ptr, codes->dtype, codes->stride[0], codes->stride[1], codes->stride[2], static_cast<const TV *>(v_new->ptr), \
        v_new->stride[0], v_new->stride[1], v_new->stride[2], static_cast<float *>(cnt->ptr),                           \
        static_cast<float *>(vsum_f32->ptr), static_cast<TS *>(shadow), static_cast<int>(Hkv), static_cast<int>(D),     \
        static_cast<int>(M), static_cast<int>(K), static_cast<int>(n_new), status_word)
    if (v_new->dtype == VQ_F32) VQ_ADVANCE(float, __nv_bfloat16);
    else if (v_new->dtype == VQ_F16) VQ_ADVANCE(__half, __half);
    else VQ_ADVANCE(__nv_bfloat16, __nv_bfloat16);
#undef VQ_ADVANCE
    return launch_status();
}
