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
#pragma unroll
        for (int rr = 0; rr < kArRows; ++rr)
            if (r == rr) {
#pragma unroll
                for (int c = 0; c < CPL; ++c) acc[rr][c] = __fadd_rn(acc[rr][c], x[c]);
            }
        if (lane == r) my_cnt += 1.f;
    };
    // this warp's keys in a block with codes c[]: bit k of (lo, hi) set when key k's code is one of its rows
    auto my_keys = [&](const int (&c)[4], uint64_t &lo, uint64_t &hi) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) w[t] = __ballot_sync(kAll, static_cast<unsigned>(c[t] - row0) < static_cast<unsigned>(kArRows));
        lo = w[0] | (static_cast<uint64_t>(w[1]) << 32);
        hi = w[2] | (static_cast<uint64_t>(w[3]) << 32);
    };
    auto pop = [&](uint64_t &lo, uint64_t &hi) {  // lowest key of a non-empty mask
        int key;
        if (lo != 0) {
            key = __ffsll(static_cast<long long>(lo)) - 1;
            lo &= lo - 1;
        } else {
            key = 64 + __ffsll(static_cast<long long>(hi)) - 1;
            hi &= hi - 1;
        }
        return key;
    };
    // Value rows travel through a per-warp staging area in shared memory: the rows of a block's first
    // kArSlots keys are copied there asynchronously one block ahead (cp.async holds no register; every
    // lane copies and later reads only its own CPL columns, so no synchronisation is needed).
    __shared__ __align__(16) uint8_t s_stage[kArWarps][2][kArSlots][D * 2];
    uint8_t *stage = &s_stage[threadIdx.x >> 5][0][0][0] + CPL * 2 * lane;
    auto stage_rows = [&](int n, int buf, uint64_t lo, uint64_t hi) {
#pragma unroll 1
        for (int slot = 0; slot < kArSlots && (lo | hi) != 0; ++slot) {
            const int key = pop(lo, hi);
            const __nv_bfloat16 *src = vbase + (static_cast<int64_t>(n) * kBlock + key) * v_sl;
            const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(stage + (buf * kArSlots + slot) * (D * 2)));
            if constexpr (CPL == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
            else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // Software pipeline over the blocks: codes are loaded two blocks ahead, value rows one block ahead.
    int c_nxt[4] = {0, 0, 0, 0}, c_nn[4] = {0, 0, 0, 0};
    uint64_t lo = 0, hi = 0;       // keys of the current block
    uint32_t p01 = 0, p23 = 0;     // its codes, 16 bits each: key k in lane k & 31, field k >> 5
    if (NB > 0) {
        int c0[4];
        load_codes(0, c0);
        if (NB > 1) load_codes(1, c_nxt);
        my_keys(c0, lo, hi);
        stage_rows(0, 0, lo, hi);
        p01 = (c0[0] & 0xffff) | (c0[1] << 16);
        p23 = (c0[2] & 0xffff) | (c0[3] << 16);
    }
    for (int n = 0; n < NB; ++n) {
        const int buf = n & 1;
        if (n + 2 < NB) load_codes(n + 2, c_nn);
        uint64_t nlo = 0, nhi = 0;
        if (n + 1 < NB) my_keys(c_nxt, nlo, nhi);
        stage_rows(n + 1, buf ^ 1, nlo, nhi);
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this block's rows have landed
        // ---- this block's keys, in position order
        int slot = 0;
        while ((lo | hi) != 0) {
            if (slot == kArSlots) {
                // More keys than staging slots (skewed codes): every lane has read its columns of the
                // slots, so the next keys of this block are staged into them and waited for at once.
                uint64_t tlo = lo, thi = hi;
#pragma unroll 1
                for (int s2 = 0; s2 < kArSlots && (tlo | thi) != 0; ++s2) {
                    const int key = pop(tlo, thi);
                    const __nv_bfloat16 *src = vbase + (static_cast<int64_t>(n) * kBlock + key) * v_sl;
                    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(stage + (buf * kArSlots + s2) * (D * 2)));
                    if constexpr (CPL == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
                    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                slot = 0;
            }
            const int key = pop(lo, hi);
            const uint32_t c01 = __shfl_sync(kAll, p01, key & 31), c23 = __shfl_sync(kAll, p23, key & 31);
            const int r = static_cast<int>(((key & 64 ? c23 : c01) >> (key & 32 ? 16 : 0)) & 0xffffu) - row0;
            const uint8_t *sp = stage + (buf * kArSlots + slot) * (D * 2);
            uint2 raw = make_uint2(0u, 0u);
            if constexpr (CPL == 4) raw = *reinterpret_cast<const uint2 *>(sp);
            else raw.x = *reinterpret_cast<const uint32_t *>(sp);
            add_row(r, raw);
            ++slot;
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
        lo = nlo;
        hi = nhi;
        p01 = (c_nxt[0] & 0xffff) | (c_nxt[1] << 16);
        p23 = (c_nxt[2] & 0xffff) | (c_nxt[3] << 16);
#pragma unroll
        for (int t = 0; t < 4; ++t) c_nxt[t] = c_nn[t];
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
