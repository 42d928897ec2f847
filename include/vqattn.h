/*
 * vqattn.h - C ABI of the B200 (sm_100a) fused vector-quantised attention library.
 *
 * Every entry point is plain C: pointers, sizes and small structs; no C++ or framework
 * types cross the boundary.  The caller owns every buffer (inputs, outputs, workspaces);
 * the library allocates no device memory.  All calls are asynchronous on the CUDA stream
 * passed as `stream` (a cudaStream_t cast to void*; NULL = the legacy default stream) and
 * return 0 or a negative VqStatus.  All tensors must live on the same CUDA device, which
 * must be the calling thread's current device.
 *
 * Each function names the reference (LouChao98/vqtree) interface it replaces, by file:line.
 */
#ifndef VQATTN_H
#define VQATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VQATTN_VERSION 201
#define VQATTN_BLOCK 128   /* key/query block size; ops/attn_vq.py:23 BLOCK_SIZE ("MUST MATCH KERNEL") */
#define VQATTN_MAX_DIMS 5

typedef enum VqDtype {
    VQ_F32 = 0,
    VQ_BF16 = 1,
    VQ_U8 = 2,
    VQ_U16 = 3,
    VQ_I32 = 4,
    VQ_I64 = 5,
    VQ_F16 = 6   /* IEEE half: the dtype of the reference's own self-test (ops/attn_vq.py:534-556) */
} VqDtype;

typedef enum VqStatus {
    VQ_OK = 0,
    VQ_EINVAL_SHAPE = -1,   /* a shape disagrees with the others or breaks a documented constraint */
    VQ_EINVAL_DTYPE = -2,   /* unsupported dtype or dtype combination */
    VQ_EINVAL_STRIDE = -3,  /* innermost stride != 1, or a layout the kernels cannot address */
    VQ_EDEVICE = -4,        /* tensors on different devices, or not on the current device */
    VQ_ELAUNCH = -5,        /* the CUDA runtime rejected a launch or attribute call */
    VQ_ETIMEOUT = -6,       /* a bounded device-side wait expired (reported through a status word) */
    VQ_EINVAL_ARG = -7,     /* null pointer or bad scalar argument */
    VQ_EUNSUPPORTED = -8,   /* valid request outside what the kernels cover (head dim, codebook size) */
    VQ_EWORKSPACE = -9      /* workspace missing or too small */
} VqStatus;

/* Dense tensor view.  `stride` is in elements.  `device` is the CUDA ordinal. */
typedef struct VqTensorDesc {
    void *ptr;
    int32_t dtype; /* VqDtype */
    int32_t ndim;
    int64_t shape[VQATTN_MAX_DIMS];
    int64_t stride[VQATTN_MAX_DIMS];
    int32_t device;
} VqTensorDesc;

/* Which prefill kernel to run; AUTO picks the tensor-core kernel for 16-bit activations and the fp32
 * kernel for f32 (SIMT also accepts 16-bit activations: an on-device cross-check of the same arithmetic). */
typedef enum VqPrefillImpl { VQ_IMPL_AUTO = 0, VQ_IMPL_SIMT = 1, VQ_IMPL_TENSOR = 2 } VqPrefillImpl;

/*
 * Status word: kernels that can detect a problem on the device (an expired bounded wait, an input value
 * they must not use as an index) take a pointer to a device int32 (`status_word`, may be NULL).  It stays 0
 * when all is well; a kernel that finds a problem stores one of the values below, leaves the offending
 * element out and finishes normally.  The host reads the word when it wants to know (one copy per step is
 * enough), maps it with vqattn_status_from_word and resets it to 0.  Replaces the reference's Python
 * asserts, which cannot see device-side values (ops/attn_vq.py:192-198).
 */
#define VQ_WORD_TIMEOUT 1       /* a bounded device-side wait expired            -> VQ_ETIMEOUT   */
#define VQ_WORD_BAD_POSITION 2  /* vqattn_rope: position outside the cos/sin tables -> VQ_EINVAL_ARG */
#define VQ_WORD_BAD_CODE 3      /* vqattn_cache_advance: code outside [0, K)       -> VQ_EINVAL_ARG */

int vqattn_version(void);
const char *vqattn_status_string(int status);
int vqattn_status_from_word(int32_t word);

/*
 * Every wait inside a kernel (on a barrier another warp, the tensor pipe or a tile copy completes) gives up
 * after a number of SM clock cycles, raises VQ_WORD_TIMEOUT in the status word and lets the kernel end.
 * vqattn_set_wait_limit_cycles sets that number for launches made after it, process-wide (cycles <= 0:
 * the default, four thousand million cycles, about two seconds); it returns the previous value.
 * vqattn_wait_selftest launches one warp that waits on a barrier nothing arrives at, so that a host can
 * check its handling of the time-out path without any kernel misbehaving: with a limit of a few million
 * cycles it ends within milliseconds and leaves VQ_WORD_TIMEOUT in *status_word.
 * No counterpart in the reference (its Triton kernels have no device-side waits).
 */
int64_t vqattn_set_wait_limit_cycles(int64_t cycles);
int vqattn_wait_selftest(int32_t *status_word, void *stream);

/*
 * Key -> code assignment.  Replaces ops/mini_vq.py:4-18 multi_head_single_quantize (scores by
 * raw inner product, first arg-max) and generalises it to M codebooks by greedy residual
 * assignment: r0 = k; c_m = argmax_c(r_m.C_m[c] + bias_m[c]); r_{m+1} = r_m - C_m[c_m].
 * Arithmetic is fp32 with a fixed order (one fused-multiply-add chain over d = 0..D-1), so the
 * codes are reproducible bit for bit.
 *   k         [B,Hkv,L,D]  f32 | bf16 | f16  (D in {64,128})
 *   codebooks [Hkv,M,K,D]  f32             (K % 64 == 0, K <= 65536)
 *   bias      NULL or [Hkv,M,K] f32
 *   codes     [B,Hkv,L,M]  u8 (K <= 256) | u16 | i32 | i64
 */
int vqattn_assign_codes(const VqTensorDesc *k, const VqTensorDesc *codebooks, const VqTensorDesc *bias_or_null,
                        VqTensorDesc *codes, void *stream);

/*
 * The same assignment, bit for bit the same codes, with the score matrix on the tensor cores
 * (bf16 keys, K a multiple of 128 up to 512 or K = 1024, M <= 8): approximate scores by tcgen05.mma over a bf16 hi/lo split of the
 * codebook, then an exact fp32 re-score of every key whose two best approximate
 * scores are closer than the proven error bound.  Needs `workspace` (256-byte aligned) of
 * vqattn_assign_workspace_bytes(B, Hkv, L, M, K, D) bytes for the split codebook.  Inputs outside the
 * tensor-core path (fp32 or f16 keys, larger K or M) are forwarded to vqattn_assign_codes.
 * `status_word`: device int32 or NULL, raised if a bounded device-side wait expires.
 */
size_t vqattn_assign_workspace_bytes(int64_t B, int64_t Hkv, int64_t L, int64_t M, int64_t K, int64_t D);
int vqattn_assign_codes_ws(const VqTensorDesc *k, const VqTensorDesc *codebooks, const VqTensorDesc *bias_or_null,
                           VqTensorDesc *codes, void *workspace, size_t workspace_bytes, int32_t *status_word,
                           void *stream);

/*
 * Per-block aggregates.  Replaces the host preparation at ops/attn_vq.py:352-384,411-417 (one-hot
 * cumsum, argsort, gather, prefix sums): block n of the outputs describes the keys [0,128(n+1)):
 *   cnt  [B,Hkv,NB,M*K]    f32  number of those keys whose code in codebook m is c  (row m*K+c)
 *   vsum [B,Hkv,NB,M*K,D]  f32 | bf16 | f16  sum of their value rows, accumulated in fp32 in position order
 * from
 *   codes [B,Hkv,L,M] u8|u16|i32|i64,  v [B,Hkv,L,D] f32|bf16|f16,   NB <= L/128.
 * (f16 sums saturate at 65504 like the reference's cast of its prefix sums, ops/attn_vq.py:383.)
 */
int vqattn_build_aggregates(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt,
                            VqTensorDesc *vsum, void *stream);

/*
 * The same with a caller workspace of vqattn_aggregates_workspace_bytes(B, Hkv, NB, M, K) bytes (device memory,
 * 16-byte aligned; contents need not be preserved between calls): the keys of every 128-key block are sorted by
 * code once, so that the kernel that forms the sums reads each row's keys instead of scanning the block's codes.
 * Same results, bit for bit.  Used for bf16 values and sums with D = 64 or 128 and K a multiple of 8 up to 4096;
 * other inputs, a NULL workspace or one that is too small take the path of vqattn_build_aggregates.
 * A code outside [0, K) is left out and reported through status_word (VQ_WORD_BAD_CODE; may be NULL).
 */
size_t vqattn_aggregates_workspace_bytes(int64_t B, int64_t Hkv, int64_t NB, int64_t M, int64_t K);
int vqattn_build_aggregates_ws(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt,
                               VqTensorDesc *vsum, void *workspace, size_t workspace_bytes, int32_t *status_word,
                               void *stream);

/*
 * vqattn_build_aggregates_ws and, from the same pass over the values, the state a decode phase starts from
 * (what ops/attn_vq.py:89-127 update_prefill is meant to leave in the cache): the counts and the fp32 value sums
 * of the first state_blocks * 128 keys,
 *   state_cnt [B,Hkv,M*K] f32,   state_vsum [B,Hkv,M*K,D] f32   (dense),   NB <= state_blocks <= L/128, NB >= 1.
 * They equal, bit for bit, vqattn_cache_advance applied to those keys from zero.  The workspace is sized for
 * state_blocks blocks: vqattn_aggregates_workspace_bytes(B, Hkv, state_blocks, M, K).  Inputs the sorted path does
 * not cover (see above) get the snapshots from the path of vqattn_build_aggregates and the state from the
 * cache-advance kernel: same results, one more pass over the values.
 */
int vqattn_build_aggregates_state(const VqTensorDesc *codes, const VqTensorDesc *v, int32_t K, VqTensorDesc *cnt,
                                  VqTensorDesc *vsum, VqTensorDesc *state_cnt, VqTensorDesc *state_vsum,
                                  int64_t state_blocks, void *workspace, size_t workspace_bytes, int32_t *status_word,
                                  void *stream);

/*
 * Converts the reference's own aggregate format to the dense one above, for callers that already
 * hold it (the arguments of ops/triton_fused_vq_attn.py:190 vq_attn_forward):
 *   v_vq [B,H,L+1,D] f32|bf16 (sorted within-code prefix sums, ops/attn_vq.py:364-383)
 *   vi   [B,H,NBin,C] i32|i64 (row of v_vq per block and code, ops/attn_vq.py:384,412-413)
 *   ->   vsum [B,H,NB,C,D] (same dtype as v_vq), NB <= NBin
 *   cnt  [B,H,NB,C] f32 dense, optional (NULL or ptr NULL): rows of codes without members
 *        (cnt == 0) are written as zeros, which vqattn_prefill relies on (see below); the reference
 *        masks such codes inside its kernel instead (ops/triton_fused_vq_attn.py:52-56).
 */
int vqattn_gather_aggregates(const VqTensorDesc *v_vq, const VqTensorDesc *vi, const VqTensorDesc *cnt, VqTensorDesc *vsum,
                             void *stream);

/*
 * Fused prefill attention.  Replaces ops/triton_fused_vq_attn.py:190-251 vq_attn_forward, i.e. the
 * far kernel (:88-187), the local ReRoPE window kernel (ops/triton_fused_local_attn_rerope.py:121-226)
 * and the log-sum-exp merge (:246-250), as one kernel with a single online softmax.
 * For query row i, with boundary = max(0, ((i - window)/128)*128):
 *   keys j in [max(0,i-window), i]       scored q1_i.k1_j
 *   keys j in [boundary, max(0,i-window)) scored q2_i.k3_j
 *   keys j <  boundary                   through the aggregates of block boundary/128 - 1:
 *       score q2_i.codebook[r] for every row r with cnt[r] > 0, numerator weight vsum[r],
 *       denominator weight cnt[r]                         (ops/triton_fused_vq_attn.py:38-68)
 * All of q1,q2,k1,k3,v,codebook,vsum,out share one dtype (f32, bf16 or f16); math is fp32.
 * Codes with cnt == 0 are excluded from the softmax like the reference does (:44-46); their vsum rows
 * should still be zero (vqattn_build_aggregates and vqattn_gather_aggregates with cnt produce them so).
 *   q1,q2,out [B,Hq,L,D]; k1,k3,v [B,Hkv,L,D]; codebook [Hkv,MK,D]; cnt [B,Hkv,NB,MK] f32;
 *   vsum [B,Hkv,NB,MK,D]; lse2 NULL or [B,Hq,L] f32 (base-2 log-sum-exp of the scaled scores).
 * Constraints: D in {64,128}; window % 128 == 0; MK % 128 == 0; Hq % Hkv == 0;
 * NB >= L/128 - window/128 - 1 when that is positive (cnt/vsum may be NULL otherwise).
 * codebook.ptr == NULL computes the local part only (the far keys are ignored), which is what
 * ops/triton_fused_local_attn_rerope.py:287-294 flash_attn_func returns.
 * q2 may alias q1 and k3 may alias k1 (plain-RoPE mode).
 */
typedef struct VqPrefillArgs {
    VqTensorDesc q1, q2, k1, k3, v;
    VqTensorDesc codebook, cnt, vsum;
    VqTensorDesc out;
    VqTensorDesc lse2;     /* ptr may be NULL */
    int64_t window;
    float scale;           /* <= 0: 1/sqrt(D) */
    int32_t impl;          /* VqPrefillImpl */
    int32_t *status_word;  /* device int32 or NULL: set non-zero by a kernel whose bounded wait expired */
} VqPrefillArgs;

int vqattn_prefill(const VqPrefillArgs *args, void *stream);

/*
 * Single-query decode over a cache (seqlen_q == 1).  The reference promises this kernel
 * (README.md:8) but its cache update is unfinished (ops/attn_vq.py:128-165); the semantics are
 * those of prefill row n-1 for a context of n tokens.  The cache holds the newest keys in
 * k1_win/k3_win/v_win (entries [0,n_valid)); the first n_bd entries are scored q2.k3, the rest
 * q1.k1; older keys are in cnt/vsum (skipped when use_far == 0).
 *   q1,q2,out [B,Hq,D]; k1_win,k3_win,v_win [B,Hkv,Nwin,D]; codebook [Hkv,MK,D] (f32 or the
 *   activation dtype); cnt [B,Hkv,MK] f32; vsum [B,Hkv,MK,D] (activation dtype).
 * `workspace` must hold vqattn_decode_workspace_bytes(...) bytes and be zero-filled before its
 * first use; the kernel leaves it ready for the next call on the same stream.
 */
typedef struct VqDecodeArgs {
    VqTensorDesc q1, q2, k1_win, k3_win, v_win;
    VqTensorDesc codebook, cnt, vsum;
    VqTensorDesc out;
    int64_t n_valid, n_bd;
    int32_t use_far;
    float scale;
    void *workspace;
    size_t workspace_bytes;
    int32_t *status_word;  /* device int32 or NULL: set non-zero by a kernel whose bounded wait expired */
} VqDecodeArgs;

size_t vqattn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t D);
int vqattn_decode(const VqDecodeArgs *args, void *stream);

/*
 * vqattn_decode for hosts that cannot supply a workspace (no counterpart in the reference, which
 * lets PyTorch allocate freely): a server whose memory plan gives all spare HBM to its KV-cache pool,
 * or a runtime that forbids device allocation inside the serving step.  Same arguments and result as
 * vqattn_decode; `workspace` / `workspace_bytes` are ignored and the scratch is a fixed array of
 * vqattn_decode_static_capacity() bytes (16 MiB) inside the library, resident on every GPU that loads
 * it until the process exits.  The call allocates nothing, on the device or through any library.
 * Limits and rules:
 *   - returns VQ_EWORKSPACE when vqattn_decode_workspace_bytes(B,Hq,Hkv,D) exceeds the capacity;
 *   - the first call on a device looks up the array's device address (with that device current);
 *     make that first call before any stream capture begins on the device;
 *   - every call on a device shares the one array: calls whose kernels could overlap on the GPU
 *     (different streams, different host threads) race on it - issue them on one stream, or use
 *     vqattn_decode with separate workspaces.
 */
size_t vqattn_decode_static_capacity(void);
int vqattn_decode_static(const VqDecodeArgs *args, void *stream);

/*
 * Rotary position embedding of x [B,H,L,D] (f32|bf16|f16) in the HF Llama half-split convention the
 * reference applies before its kernels (ops/attn_vq.py:55-64,296-299: x*cos + rotate_half(x)*sin):
 *   out_pos   (optional) [B,H,L,D]: every row rotated to its own position, positions[b*L + l]
 *             (int64, device) or l when positions is NULL          (ops/attn_vq.py:402-404)
 *   out_const (optional) [B,H,L,D]: every row rotated to const_pos, the ReRoPE query at
 *             window + 1                                             (ops/attn_vq.py:405-407)
 * cos_tab, sin_tab: device fp32 tables [n_pos, D/2] (angle = pos * base^(-2i/D)).  Products and sum
 * are rounded separately in fp32, then once to the output dtype.  A position outside [0, n_pos)
 * sets *status_word to VQ_WORD_BAD_POSITION (status_word may be NULL) and uses the nearest table row.
 * Constraints: D % 16 == 0 (bf16) or D % 8 == 0 (f32); 16-byte aligned rows and tables.
 */
int vqattn_rope(const VqTensorDesc *x, const int64_t *positions, const float *cos_tab, const float *sin_tab, int64_t n_pos,
                int64_t const_pos, VqTensorDesc *out_pos, VqTensorDesc *out_const, int32_t *status_word, void *stream);

/*
 * The rotations of one prefill in a single launch (ops/attn_vq.py:402-407): q [B,Hq,L,D] -> q1 (each row at
 * its position) and q2 (every row at const_pos = window + 1; NULL or ptr NULL to skip), k [B,Hkv,L,D] -> k1.
 * Inputs and outputs may be strided views ([B,L,H,D] storage viewed as [B,H,L,D] included); arguments as in
 * vqattn_rope.
 */
int vqattn_rope_qk(const VqTensorDesc *q, const VqTensorDesc *k, const int64_t *positions, const float *cos_tab,
                   const float *sin_tab, int64_t n_pos, int64_t const_pos, VqTensorDesc *q1, VqTensorDesc *q2,
                   VqTensorDesc *k1, int32_t *status_word, void *stream);

/*
 * The per-token bookkeeping of a decode step in one launch: rotates the new query (q [B,Hq,1,D] -> q1, q2
 * [B,Hq,1,D]) and writes the new key and value into row `row` of the window caches: k1_win gets the key
 * rotated to its position, k3_win the key as it is, v_win the value (all [B,Hkv,Nwin,D]).  The position of
 * batch b is positions[b] (device int64) or `pos` when positions is NULL.  Stands in for the cache update the
 * reference left unfinished (ops/attn_vq.py:128-165) and its per-step rotations (:402-407).
 */
int vqattn_decode_append(const VqTensorDesc *q, const VqTensorDesc *k, const VqTensorDesc *v, const int64_t *positions,
                         int64_t pos, const float *cos_tab, const float *sin_tab, int64_t n_pos, int64_t const_pos,
                         VqTensorDesc *q1, VqTensorDesc *q2, VqTensorDesc *k1_win, VqTensorDesc *k3_win,
                         VqTensorDesc *v_win, int64_t row, int32_t *status_word, void *stream);

/*
 * One generated token in one call: vqattn_decode_append followed by vqattn_decode on the same stream (two
 * launches).  `decode.q1` / `decode.q2` must describe the [B,Hq,D] views of the scratch tensors q1 / q2
 * ([B,Hq,1,D]) that the first launch fills, `decode.k1_win` / `k3_win` / `v_win` the window caches the new
 * key and value are written into at row `row`, and `decode.n_valid` must count that row.  A host keeps one
 * such struct per layer and changes only q/k/v.ptr, pos, row, n_valid, n_bd and out.ptr from token to token.
 */
typedef struct VqDecodeStepArgs {
    VqTensorDesc q, k, v;        /* the new token: [B,Hq,1,D], [B,Hkv,1,D], [B,Hkv,1,D], un-rotated */
    const int64_t *positions;    /* device [B] or NULL */
    int64_t pos;                 /* position of the token when positions is NULL */
    const float *cos_tab, *sin_tab;
    int64_t n_pos, const_pos;
    VqTensorDesc q1, q2;         /* scratch [B,Hq,1,D] */
    int64_t row;
    VqDecodeArgs decode;
} VqDecodeStepArgs;

int vqattn_decode_step(const VqDecodeStepArgs *args, void *stream);

/*
 * Cache advance: folds `n_new` (a multiple of 128 is not required) keys that cross the boundary
 * into the running aggregates of a decode cache.  Stands in for the unfinished
 * ops/attn_vq.py:128-165 VectorQuantizedReRoPECache.update.
 *   codes [B,Hkv,n_new,M] ; v_new [B,Hkv,n_new,D] ;
 *   cnt [B,Hkv,MK] f32 (in/out) ; vsum_f32 [B,Hkv,MK,D] f32 master (in/out) ;
 *   vsum_act NULL or [B,Hkv,MK,D] 16-bit shadow (the dtype of v_new; bf16 for f32 values) refreshed for
 *   the touched rows.
 * A code outside [0,K) (a foreign quantizer, 8-bit codes with K < 256) is skipped and reported as
 * VQ_WORD_BAD_CODE in *status_word (may be NULL); nothing outside the code's own rows is written.
 */
int vqattn_cache_advance(const VqTensorDesc *codes, const VqTensorDesc *v_new, int32_t K, VqTensorDesc *cnt,
                         VqTensorDesc *vsum_f32, VqTensorDesc *vsum_act_or_null, int32_t *status_word, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* VQATTN_H */
