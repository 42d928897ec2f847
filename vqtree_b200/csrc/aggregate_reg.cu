// Per-block aggregates with the running sums in registers: bf16 values -> bf16 snapshots.
//
// Same outputs as build_aggregates_kernel (aggregate.cu; replaces ops/attn_vq.py:352-384,411-417 of
// the reference): after every 128-key block n, cnt[n][r] and vsum[n][r] of all keys [0, 128(n+1)),
// every row summed in fp32 in position order, rounded to bf16 when written.
//
// A WARP owns eight consecutive code rows of one codebook of one (batch, kv head): 8 x D fp32 sums,
// D / 32 columns per lane, live in its registers for the whole sequence.  Per block it finds the keys
// of its rows with ballots over the block's 128 codes (loaded two blocks ahead; the value rows are
// copied into a small per-warp staging area one block ahead), adds their value rows in position order, and writes its 8 x D snapshot with coalesced 8-byte stores (a row is 256
// contiguous bytes).  Warps never synchronise with each other: there is no barrier, so the other warps of the SM hide a warp's load latency and the kernel runs at the
// speed the snapshot stores drain.
#include "vq_common.cuh"

namespace vq {

constexpr int kArWarps = 4;   // warps per CTA (independent of each other)
constexpr int kArRows = 8;    // code rows per warp
constexpr int kArSlots = 8;   // value rows staged per warp and block

__device__ __forceinline__ uint32_t ar_pack(float lo, float hi)
{
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&p);
}

template <int D>
__global__ void __launch_bounds__(kArWarps * 32, 7)
build_aggregates_reg_kernel(const void *__restrict__ codes, int code_dtype, int64_t c_sb, int64_t c_sh, int64_t c_sl,
                            const __nv_bfloat16 *__restrict__ v, int64_t v_sb, int64_t v_sh, int64_t v_sl,
                            float *__restrict__ cnt,           // [B,Hkv,NB,MK] dense
                            __nv_bfloat16 *__restrict__ vsum,  // [B,Hkv,NB,MK,D] dense
                            int Hkv, int M, int K, int NB)
{
    constexpr int CPL = D / 32;  // columns per lane: 4 (D = 128) or 2 (D = 64)
    constexpr unsigned kAll = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int MK = M * K;
    const int base = (static_cast<int>(blockIdx.x) * kArWarps + (threadIdx.x >> 5)) * kArRows;  // first row, in [0, MK)
    if (base >= MK) return;
    const int m = base / K, row0 = base % K;  // K is a multiple of 8: the eight rows lie in one codebook
    const int u = blockIdx.y, b = u / Hkv, h = u % Hkv;
    const int64_t cbase = b * c_sb + h * c_sh + m;
    const __nv_bfloat16 *vbase = v + b * v_sb + h * v_sh + CPL * lane;

    float acc[kArRows][CPL];
#pragma unroll
    for (int r = 0; r < kArRows; ++r)
#pragma unroll
        for (int c = 0; c < CPL; ++c) acc[r][c] = 0.f;
    float my_cnt = 0.f;  // lane r < 8: number of keys of row r so far

    // codes of keys lane, 32 + lane, 64 + lane, 96 + lane of a block
    auto load_codes = [&](int n, int (&raw)[4]) {
#pragma unroll
        for (int t = 0; t < 4; ++t)
            raw[t] = load_code(codes, code_dtype, cbase + (static_cast<int64_t>(n) * kBlock + 32 * t + lane) * c_sl);
    };
    auto unpack = [&](const uint2 raw, float (&x)[CPL]) {
        const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x);
        x[0] = __low2float(p0);
        x[1] = __high2float(p0);
        if constexpr (CPL == 4) {
            const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
            x[2] = __low2float(p1);
            x[3] = __high2float(p1);
        }
    };
    auto add_row = [&](int r, const uint2 raw) {
        float x[CPL];
        unpack(raw, x);
        // r is the same in all lanes: one taken branch instead of eight predicated copies of the adds
#define VQ_AR_ADD(rr)                                                                  \
    case rr:                                                                           \
        _Pragma("unroll") for (int c = 0; c < CPL; ++c) acc[rr][c] = __fadd_rn(acc[rr][c], x[c]); \
        break;
        switch (r) {
            VQ_AR_ADD(0) VQ_AR_ADD(1) VQ_AR_ADD(2) VQ_AR_ADD(3) VQ_AR_ADD(4) VQ_AR_ADD(5) VQ_AR_ADD(6) VQ_AR_ADD(7)
        default: break;
        }
#undef VQ_AR_ADD
        if (lane == r) my_cnt += 1.f;
    };
    // Value rows travel through a per-warp staging area in shared memory: the rows of a block's first
    // kArSlots keys are copied there asynchronously one block ahead (cp.async holds no register; every
    // lane copies and later reads only its own CPL columns), together with the code row of each.
    __shared__ __align__(16) uint8_t s_stage[kArWarps][2][kArSlots][D * 2];
    __shared__ int s_row[kArWarps][2][kArSlots];
    uint8_t *stage = &s_stage[threadIdx.x >> 5][0][0][0] + CPL * 2 * lane;
    int *rows = &s_row[threadIdx.x >> 5][0][0];
    auto copy_row = [&](const __nv_bfloat16 *src, int buf, int slot) {
        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(stage + (buf * kArSlots + slot) * (D * 2)));
        if constexpr (CPL == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
        else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
    };
    // Stage the keys of block n whose codes (c) fall into this warp's rows; returns how many were staged,
    // rest[] keeps the keys beyond the slots (bit k of rest[t]: key 32 t + k).
    auto stage_block = [&](int n, const int (&c)[4], int buf, uint32_t (&rest)[4]) {
        const __nv_bfloat16 *vb = vbase + static_cast<int64_t>(n) * kBlock * v_sl;
        int slot = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int lc = c[t] - row0;
            uint32_t w = __ballot_sync(kAll, static_cast<unsigned>(lc) < static_cast<unsigned>(kArRows));
            while (w != 0 && slot < kArSlots) {
                const int bit = __ffs(w) - 1;
                w &= w - 1;
                const int r = __shfl_sync(kAll, lc, bit);
                copy_row(vb + static_cast<int64_t>(32 * t + bit) * v_sl, buf, slot);
                if (lane == 0) rows[buf * kArSlots + slot] = r;
                ++slot;
            }
            rest[t] = w;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        return slot;
    };
    auto read_row = [&](int buf, int slot) {
        const uint8_t *sp = stage + (buf * kArSlots + slot) * (D * 2);
        uint2 raw = make_uint2(0u, 0u);
        if constexpr (CPL == 4) raw = *reinterpret_cast<const uint2 *>(sp);
        else raw.x = *reinterpret_cast<const uint32_t *>(sp);
        return raw;
    };

    // Software pipeline over the blocks: codes are loaded two blocks ahead, value rows one block ahead.
    int c_nxt[4] = {0, 0, 0, 0}, c_nn[4] = {0, 0, 0, 0};
    uint32_t rest[4] = {0, 0, 0, 0};  // keys of the current block beyond the staged ones
    int staged = 0;                    // staged keys of the current block
    if (NB > 0) {
        int c0[4];
        load_codes(0, c0);
        if (NB > 1) load_codes(1, c_nxt);
        staged = stage_block(0, c0, 0, rest);
    }
    for (int n = 0; n < NB; ++n) {
        const int buf = n & 1;
        if (n + 2 < NB) load_codes(n + 2, c_nn);
        uint32_t rest_n[4] = {0, 0, 0, 0};
        int staged_n = 0;
        if (n + 1 < NB) staged_n = stage_block(n + 1, c_nxt, buf ^ 1, rest_n);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this block's rows have landed
        __syncwarp();                                          // ... and lane 0's row numbers are visible
        // ---- this block's keys, in position order
#pragma unroll 1
        for (int slot = 0; slot < staged; ++slot) add_row(rows[buf * kArSlots + slot], read_row(buf, slot));
        if ((rest[0] | rest[1] | rest[2] | rest[3]) != 0) {
            // More keys than staging slots (skewed codes): staged into the same slots in chunks and waited
            // for at once; their code rows are read again from global memory.
            const __nv_bfloat16 *vb = vbase + static_cast<int64_t>(n) * kBlock * v_sl;
#pragma unroll 1
            for (int t = 0; t < 4; ++t) {
                uint32_t w = rest[t];
                while (w != 0) {
                    __syncwarp();
                    int cnt = 0;
                    uint32_t w2 = w;
                    while (w2 != 0 && cnt < kArSlots) {
                        const int bit = __ffs(w2) - 1;
                        w2 &= w2 - 1;
                        copy_row(vb + static_cast<int64_t>(32 * t + bit) * v_sl, buf, cnt);
                        ++cnt;
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    for (int i = 0; i < cnt; ++i) {
                        const int bit = __ffs(w) - 1;
                        w &= w - 1;
                        const int64_t j = static_cast<int64_t>(n) * kBlock + 32 * t + bit;
                        add_row(load_code(codes, code_dtype, cbase + j * c_sl) - row0, read_row(buf, i));
                    }
                }
            }
        }
        // ---- snapshot of the eight rows
        const int64_t out_row0 = (static_cast<int64_t>(u) * NB + n) * MK + base;
        __nv_bfloat16 *dst = vsum + out_row0 * D + CPL * lane;
#pragma unroll
        for (int r = 0; r < kArRows; ++r) {
            if constexpr (CPL == 4)
                __stcs(reinterpret_cast<uint2 *>(dst + r * D), make_uint2(ar_pack(acc[r][0], acc[r][1]), ar_pack(acc[r][2], acc[r][3])));
            else
                __stcs(reinterpret_cast<uint32_t *>(dst + r * D), ar_pack(acc[r][0], acc[r][1]));
        }
        if (lane < kArRows) __stcs(cnt + out_row0 + lane, my_cnt);
        // ---- rotate the pipeline
        staged = staged_n;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            rest[t] = rest_n[t];
            c_nxt[t] = c_nn[t];
        }
    }
}

int launch_aggregates_reg(const VqTensorDesc *codes, const VqTensorDesc *v, int K, VqTensorDesc *cnt, VqTensorDesc *vsum,
                          cudaStream_t stream)
{
    const int64_t B = codes->shape[0], Hkv = codes->shape[1], M = codes->shape[3];
    const int64_t D = v->shape[3], NB = cnt->shape[2];
    if (v->stride[0] % 4 || v->stride[1] % 4 || v->stride[2] % 4 || reinterpret_cast<uintptr_t>(v->ptr) % 8) return VQ_EINVAL_STRIDE;
    const int64_t warps = M * K / kArRows;
    dim3 grid(static_cast<unsigned>((warps + kArWarps - 1) / kArWarps), static_cast<unsigned>(B * Hkv));
    if (D == 64)
        build_aggregates_reg_kernel<64><<<grid, kArWarps * 32, 0, stream>>>(
            codes->ptr, codes->dtype, codes->stride[0], codes->stride[1], codes->stride[2], static_cast<const __nv_bfloat16 *>(v->ptr),
            v->stride[0], v->stride[1], v->stride[2], static_cast<float *>(cnt->ptr), static_cast<__nv_bfloat16 *>(vsum->ptr),
            static_cast<int>(Hkv), static_cast<int>(M), K, static_cast<int>(NB));
    else
        build_aggregates_reg_kernel<128><<<grid, kArWarps * 32, 0, stream>>>(
            codes->ptr, codes->dtype, codes->stride[0], codes->stride[1], codes->stride[2], static_cast<const __nv_bfloat16 *>(v->ptr),
            v->stride[0], v->stride[1], v->stride[2], static_cast<float *>(cnt->ptr), static_cast<__nv_bfloat16 *>(vsum->ptr),
            static_cast<int>(Hkv), static_cast<int>(M), K, static_cast<int>(NB));
    return launch_status();
}

// The register kernel covers bf16 values and snapshots, D = 64 or 128, K a multiple of 8.
bool aggregates_reg_eligible(const VqTensorDesc *v, const VqTensorDesc *vsum, int K)
{
    const int64_t D = v->shape[3];
    return v->dtype == VQ_BF16 && vsum->dtype == VQ_BF16 && (D == 64 || D == 128) && K % kArRows == 0;
}

}  // namespace vq
