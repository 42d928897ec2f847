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

bool aggregates_reg_eligible(const VqTensorDesc *v, const VqTensorDesc *vsum, int K);

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

// ------------------------------------------------------------------------------------------------
// The same sums with the keys of every block sorted by code first (caller workspace).
//
// In the kernel above every warp scans all 128 codes of a block to find the keys of its eight rows: 128 warps per
// (batch, kv head) repeat the same scan.  With a workspace, sort_block_codes_kernel sorts the keys of every
// (unit, block, codebook) by code once (stable: keys of one code stay in position order) and leaves a record
//   entries[128] u8   key index inside the block, in sorted order
//   start[K + 1] u8   start[c] = number of keys with a code below c
// and a warp of build_aggregates_sorted_kernel reads nine bytes of `start` and the entries between them - no scan,
// no ballots - and adds row by row (the rows of one code are contiguous, so there is no dispatch on the row either).
// The sums are formed in the same order as above: bit-identical results.
constexpr int kSortWarps = 4;

__host__ __device__ inline int64_t sorted_record_bytes(int64_t K) { return (kBlock + K + 1 + 15) / 16 * 16; }

__global__ void __launch_bounds__(kSortWarps * 32)
sort_block_codes_kernel(const void *__restrict__ codes, int code_dtype, int64_t c_sb, int64_t c_sh, int64_t c_sl, uint8_t *__restrict__ ws,
                        int Hkv, int M, int K, int NB, int32_t *__restrict__ status)
{
    constexpr unsigned kAll = 0xffffffffu;
    extern __shared__ int s_sort[];   // per warp: cnt[K + 1], start[K + 1]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int idx = blockIdx.x * kSortWarps + w;
    if (idx >= NB * M) return;
    const int n = idx / M, m = idx % M;
    const int u = blockIdx.y, b = u / Hkv, h = u % Hkv;
    uint8_t *rec = ws + ((static_cast<int64_t>(u) * NB + n) * M + m) * sorted_record_bytes(K);
    int *cnt = s_sort + w * 2 * (K + 1), *st = cnt + (K + 1);
    for (int i = lane; i <= K; i += 32) cnt[i] = 0;
    __syncwarp();
    int c[4];
    const int64_t cbase = b * c_sb + h * c_sh + m;
    bool bad = false;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        c[t] = load_code(codes, code_dtype, cbase + (static_cast<int64_t>(n) * kBlock + 32 * t + lane) * c_sl);
        if (c[t] < 0 || c[t] >= K) {   // a code outside [0, K): the key is left out (it sorts behind every row) and reported
            bad = true;
            c[t] = K;
        }
        atomicAdd(&cnt[c[t]], 1);
    }
    if (bad && status != nullptr) atomicExch(status, VQ_WORD_BAD_CODE);
    __syncwarp();
    // exclusive scan over the K + 1 counters: a run of per consecutive counters per lane, then across the lanes
    const int per = (K + 1 + 31) / 32;
    int sum = 0;
    for (int i = 0; i < per; ++i) {
        const int j = lane * per + i;
        if (j <= K) sum += cnt[j];
    }
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(kAll, incl, d);
        if (lane >= d) incl += t;
    }
    int run = incl - sum;
    for (int i = 0; i < per; ++i) {
        const int j = lane * per + i;
        if (j <= K) {
            st[j] = run;
            rec[kBlock + j] = static_cast<uint8_t>(run);
            run += cnt[j];
        }
    }
    __syncwarp();
    for (int i = lane; i <= K; i += 32) cnt[i] = 0;
    __syncwarp();
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const unsigned mask = __match_any_sync(kAll, c[t]);
        const int rank = __popc(mask & ((1u << lane) - 1u));
        const int pos = st[c[t]] + cnt[c[t]] + rank;
        if (pos < kBlock) rec[pos] = static_cast<uint8_t>(32 * t + lane);
        __syncwarp();
        if (rank == 0) cnt[c[t]] += __popc(mask);
        __syncwarp();
    }
}

template <int D, bool kState>
__global__ void __launch_bounds__(kArWarps * 32, 7)
build_aggregates_sorted_kernel(const uint8_t *__restrict__ ws, const __nv_bfloat16 *__restrict__ v, int64_t v_sb, int64_t v_sh, int v_row_bytes,
                               float *__restrict__ cnt,           // [B,Hkv,NB,MK] dense
                               __nv_bfloat16 *__restrict__ vsum,  // [B,Hkv,NB,MK,D] dense
                               float *__restrict__ state_cnt,     // nullptr or [B,Hkv,MK]: counts after NBT blocks
                               float *__restrict__ state_vsum,    // nullptr or [B,Hkv,MK,D]: fp32 sums after NBT blocks
                               int Hkv, int M, int K, int NB, int NBT_arg)
{
    // The warp walks NBT >= NB blocks (the workspace holds NBT records per unit and codebook), writes a snapshot after
    // each of the first NB and, if asked, its fp32 running sums at the end: the state a decode phase starts from.
    // (kState = false: NBT = NB and no state - the loop below then has no test on the block index.)
    const int NBT = kState ? NBT_arg : NB;
    constexpr int CPL = D / 32;  // columns per lane: 4 (D = 128) or 2 (D = 64)
    constexpr unsigned kAll = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int MK = M * K;
    const int base = (static_cast<int>(blockIdx.x) * kArWarps + (threadIdx.x >> 5)) * kArRows;  // first row, in [0, MK)
    if (base >= MK) return;
    const int m = base / K, row0 = base % K;
    const int u = blockIdx.y, b = u / Hkv, h = u % Hkv;
    const int rec_bytes = static_cast<int>(sorted_record_bytes(K));
    // running pointers (no multiplications in the loop): this block's value rows, its record, its outputs
    const uint8_t *vblk = reinterpret_cast<const uint8_t *>(v + b * v_sb + h * v_sh + CPL * lane);
    const uint8_t *rec = ws + (static_cast<int64_t>(u) * NBT * M + m) * rec_bytes;
    const int rec_step = M * rec_bytes, v_step = kBlock * v_row_bytes;
    __nv_bfloat16 *dst = vsum + (static_cast<int64_t>(u) * NB * MK + base) * D + CPL * lane;
    float *cdst = cnt + static_cast<int64_t>(u) * NB * MK + base + lane;

    float acc[kArRows][CPL];
#pragma unroll
    for (int r = 0; r < kArRows; ++r)
#pragma unroll
        for (int c = 0; c < CPL; ++c) acc[r][c] = 0.f;
    float my_cnt = 0.f;  // lane r < 8: number of keys of row r so far

    __shared__ __align__(16) uint8_t s_stage[kArWarps][2][kArSlots][D * 2];
    const uint32_t stage = static_cast<uint32_t>(__cvta_generic_to_shared(&s_stage[threadIdx.x >> 5][0][0][0])) + CPL * 2 * lane;
    auto copy_row = [&](const uint8_t *src, int buf, int slot) {
        const uint32_t d = stage + (buf * kArSlots + slot) * (D * 2);
        if constexpr (CPL == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src) : "memory");
        else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
    };
    auto add_slot = [&](float (&a)[CPL], int buf, int slot) {
        const uint32_t sp = stage + (buf * kArSlots + slot) * (D * 2);
        uint32_t x0, x1 = 0;
        if constexpr (CPL == 4) asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(x0), "=r"(x1) : "r"(sp));
        else asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x0) : "r"(sp));
        a[0] = __fadd_rn(a[0], __uint_as_float(x0 << 16));
        a[1] = __fadd_rn(a[1], __uint_as_float(x0 & 0xffff0000u));
        if constexpr (CPL == 4) {
            a[2] = __fadd_rn(a[2], __uint_as_float(x1 << 16));
            a[3] = __fadd_rn(a[3], __uint_as_float(x1 & 0xffff0000u));
        }
    };
    // lane r <= 8: start[row0 + r] of a block's record (the other lanes repeat the last one)
    auto load_start = [&](const uint8_t *rc) { return static_cast<int>(__ldg(rc + kBlock + row0 + (lane < kArRows ? lane : kArRows))); };
    // lane i: key index of entry first + i of the warp's rows
    auto load_entry = [&](const uint8_t *rc, int first) { return static_cast<int>(__ldg(rc + ((first + lane) & (kBlock - 1)))); };
    // copies the value rows of the first min(count, slots) entries into the staging buffer
    auto stage_entries = [&](const uint8_t *vb, int e, int count, int buf) {
        const int ns = count < kArSlots ? count : kArSlots;
        for (int i = 0; i < ns; ++i) copy_row(vb + __shfl_sync(kAll, e, i) * v_row_bytes, buf, i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // Software pipeline over the blocks: starts two blocks ahead, entries and value rows one block ahead.
    int st_cur = 0, st_nxt = 0, st_nn = 0, e_cur = 0, e_nxt = 0;
    if (NBT > 0) {
        st_cur = load_start(rec);
        if (NBT > 1) st_nxt = load_start(rec + rec_step);
        const int s0 = __shfl_sync(kAll, st_cur, 0);
        e_cur = load_entry(rec, s0);
        stage_entries(vblk, e_cur, __shfl_sync(kAll, st_cur, kArRows) - s0, 0);
    }
    for (int n = 0; n < NBT; ++n) {
        const int buf = n & 1;
        if (n + 2 < NBT) st_nn = load_start(rec + 2 * rec_step);
        if (n + 1 < NBT) {
            const int s0n = __shfl_sync(kAll, st_nxt, 0);
            e_nxt = load_entry(rec + rec_step, s0n);
            stage_entries(vblk + v_step, e_nxt, __shfl_sync(kAll, st_nxt, kArRows) - s0n, buf ^ 1);
        } else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this block's rows have landed
        __syncwarp();
        // ---- this block's keys: row by row, position order within a row
        const int s0 = __shfl_sync(kAll, st_cur, 0);
        const int count = __shfl_sync(kAll, st_cur, kArRows) - s0;
        my_cnt += static_cast<float>(__shfl_down_sync(kAll, st_cur, 1) - st_cur);   // lanes 0..7: keys of their row in this block
        if (count <= kArSlots) {
            int slot = 0;
#pragma unroll
            for (int r = 0; r < kArRows; ++r) {
                const int end = __shfl_sync(kAll, st_cur, r + 1) - s0;
                for (; slot < end; ++slot) add_slot(acc[r], buf, slot);
            }
        } else {
            // more keys than staging slots (skewed codes): chunks of the sorted entries, staged and waited for at once
            int first = 0, e = e_cur;
#pragma unroll 1
            while (true) {
                const int ns = count - first < kArSlots ? count - first : kArSlots;
                int slot = 0;
#pragma unroll
                for (int r = 0; r < kArRows; ++r) {
                    int end = __shfl_sync(kAll, st_cur, r + 1) - s0 - first;
                    end = end < ns ? end : ns;
                    for (; slot < end; ++slot) add_slot(acc[r], buf, slot);
                }
                first += kArSlots;
                if (first >= count) break;
                __syncwarp();
                e = load_entry(rec, s0 + first);
                const int nn = count - first < kArSlots ? count - first : kArSlots;
                for (int i = 0; i < nn; ++i) copy_row(vblk + __shfl_sync(kAll, e, i) * v_row_bytes, buf, i);
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncwarp();
            }
        }
        // ---- snapshot of the eight rows
        if (!kState || n < NB) {
#pragma unroll
            for (int r = 0; r < kArRows; ++r) {
                if constexpr (CPL == 4)
                    __stcs(reinterpret_cast<uint2 *>(dst + r * D), make_uint2(ar_pack(acc[r][0], acc[r][1]), ar_pack(acc[r][2], acc[r][3])));
                else
                    __stcs(reinterpret_cast<uint32_t *>(dst + r * D), ar_pack(acc[r][0], acc[r][1]));
            }
            if (lane < kArRows) __stcs(cdst, my_cnt);
        }
        // ---- next block
        st_cur = st_nxt;
        st_nxt = st_nn;
        e_cur = e_nxt;
        rec += rec_step;
        vblk += v_step;
        dst += static_cast<int64_t>(MK) * D;
        cdst += MK;
    }
    if (kState && state_vsum != nullptr) {
        float *sd = state_vsum + (static_cast<int64_t>(u) * MK + base) * D + CPL * lane;
#pragma unroll
        for (int r = 0; r < kArRows; ++r) {
            if constexpr (CPL == 4) *reinterpret_cast<float4 *>(sd + r * D) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
            else *reinterpret_cast<float2 *>(sd + r * D) = make_float2(acc[r][0], acc[r][1]);
        }
        if (lane < kArRows) state_cnt[static_cast<int64_t>(u) * MK + base + lane] = my_cnt;
    }
}

size_t aggregates_sorted_workspace_bytes(int64_t B, int64_t Hkv, int64_t NB, int64_t M, int64_t K)
{
    return static_cast<size_t>(B * Hkv * NB * M * sorted_record_bytes(K));
}

// bf16 values and snapshots, D = 64 or 128, K a multiple of 8 and at most 2^15 (shared memory of the sort), rows of v
// less than 16 MB apart (32-bit offsets inside a block)
bool aggregates_sorted_eligible(const VqTensorDesc *v, const VqTensorDesc *vsum, int K)
{
    return aggregates_reg_eligible(v, vsum, K) && K <= 4096 && v->stride[2] * 2 * kBlock < (int64_t(1) << 31);
}

// state_blocks > 0: the walk covers state_blocks >= NB blocks (records for as many in the workspace) and leaves the fp32 counts
// and sums after the last one in state_cnt / state_vsum.
int launch_aggregates_sorted(const VqTensorDesc *codes, const VqTensorDesc *v, int K, VqTensorDesc *cnt, VqTensorDesc *vsum, void *workspace,
                             int32_t *status, cudaStream_t stream, float *state_cnt, float *state_vsum, int64_t state_blocks)
{
    const int64_t B = codes->shape[0], Hkv = codes->shape[1], M = codes->shape[3];
    const int64_t D = v->shape[3], NB = cnt->shape[2], NBT = state_blocks > NB ? state_blocks : NB;
    if (v->stride[0] % 4 || v->stride[1] % 4 || v->stride[2] % 4 || reinterpret_cast<uintptr_t>(v->ptr) % 8) return VQ_EINVAL_STRIDE;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    const size_t smem = static_cast<size_t>(kSortWarps) * 2 * (K + 1) * sizeof(int);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(sort_block_codes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return VQ_ELAUNCH;
    dim3 gs(static_cast<unsigned>((NBT * M + kSortWarps - 1) / kSortWarps), static_cast<unsigned>(B * Hkv));
    sort_block_codes_kernel<<<gs, kSortWarps * 32, smem, stream>>>(codes->ptr, codes->dtype, codes->stride[0], codes->stride[1], codes->stride[2],
                                                                    ws, static_cast<int>(Hkv), static_cast<int>(M), K, static_cast<int>(NBT), status);
    const int64_t warps = M * K / kArRows;
    dim3 grid(static_cast<unsigned>((warps + kArWarps - 1) / kArWarps), static_cast<unsigned>(B * Hkv));
    const int row_bytes = static_cast<int>(v->stride[2] * 2);
#define VQ_SORTED(DD, ST)                                                                                                          \
    build_aggregates_sorted_kernel<DD, ST><<<grid, kArWarps * 32, 0, stream>>>(                                                    \
        ws, static_cast<const __nv_bfloat16 *>(v->ptr), v->stride[0], v->stride[1], row_bytes, static_cast<float *>(cnt->ptr),    \
        static_cast<__nv_bfloat16 *>(vsum->ptr), state_cnt, state_vsum, static_cast<int>(Hkv), static_cast<int>(M), K,             \
        static_cast<int>(NB), static_cast<int>(NBT))
    const bool with_state = state_vsum != nullptr;
    if (D == 64) {
        if (with_state) VQ_SORTED(64, true);
        else VQ_SORTED(64, false);
    } else {
        if (with_state) VQ_SORTED(128, true);
        else VQ_SORTED(128, false);
    }
#undef VQ_SORTED
    return launch_status();
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
