"""Tensor-level entry points of the fused VQ-attention path (thin wrappers over the C ABI).

Every function here allocates its outputs with torch, fills C descriptors and calls
``libvqattn.so`` on the current CUDA stream of the tensors' device.  No arithmetic of the path
is done in Python or by torch operators.  Host (CPU) tensors are accepted by the ``*_host``
helpers, which stage them through pinned memory to the device and bring the result back.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import native
from .native import BLOCK, VqDecodeArgs, VqPrefillArgs, check, desc, lib, stream_ptr

_IMPL = {"auto": native.IMPL_AUTO, "simt": native.IMPL_SIMT, "tensor": native.IMPL_TENSOR}


def _require_cuda(*ts):
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("expected CUDA tensors (use the *_host helpers for CPU tensors)")
        dev = dev or t.device
        if t.device != dev:
            raise ValueError("all tensors must be on the same device")
    return dev


_STATUS = {}


def _device_index(dev) -> int:
    """CUDA ordinal of ``dev``; a device without an index ("cuda") means the current device."""
    d = torch.device(dev)
    return torch.cuda.current_device() if d.index is None else d.index


def device_status_word(dev="cuda") -> torch.Tensor:
    """Per-device int32 word the kernels raise when they find a problem on the device (an expired bounded
    wait, a position outside the RoPE tables, a code outside its codebook)."""
    key = _device_index(dev)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _STATUS[key]


def check_status(dev="cuda") -> None:
    """Synchronises, reads the device's status word and raises VqError with the status the word maps to
    (VQ_ETIMEOUT for an expired wait, VQ_EINVAL_ARG for a bad position or code).  The word is cleared."""
    w = device_status_word(dev)
    word = int(w.item())
    if word != 0:
        w.zero_()
        raise native.VqError(lib.vqattn_status_from_word(word), f"device status word {word}")


def set_wait_limit(cycles: int) -> int:
    """Cycles a device-side wait may last before a kernel gives up (<= 0: the default); returns the old value."""
    return int(lib.vqattn_set_wait_limit_cycles(int(cycles)))


def wait_selftest(dev="cuda") -> None:
    """Launches one warp that waits on a barrier nothing arrives at (see vqattn_wait_selftest)."""
    idx = _device_index(dev)
    with torch.cuda.device(idx):
        check(lib.vqattn_wait_selftest(device_status_word(idx).data_ptr(), stream_ptr(torch.device("cuda", idx))),
              "vqattn_wait_selftest")


def code_dtype_for(K: int) -> torch.dtype:
    """uint8 when a code fits (K <= 256), else uint16."""
    return torch.uint8 if K <= 256 else torch.uint16


def assign_codes(k: torch.Tensor, codebooks: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, impl: str = "auto",
                 workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Key -> code assignment (replaces ops/mini_vq.py:4-18; greedy residual for M > 1).

    k [B,Hkv,L,D] f32|bf16, codebooks [Hkv,M,K,D] f32, bias None|[Hkv,M,K] f32 -> codes [B,Hkv,L,M].
    """
    dev = _require_cuda(k, codebooks, bias)
    B, Hkv, L, _ = k.shape
    M, K = codebooks.shape[1], codebooks.shape[2]
    codes = torch.empty((B, Hkv, L, M), dtype=out_dtype or code_dtype_for(K), device=dev)
    with torch.cuda.device(dev):
        dk, dc, db, do = desc(k), desc(codebooks), desc(bias), desc(codes)
        if impl == "simt":
            check(lib.vqattn_assign_codes(dk, dc, db if bias is not None else None, do, stream_ptr(dev)), "vqattn_assign_codes")
        else:
            # tensor-core scoring + exact re-score where it applies (bf16 keys); same codes either way
            need = lib.vqattn_assign_workspace_bytes(B, Hkv, L, M, K, k.shape[3])
            if workspace is None or workspace.numel() < need:
                workspace = torch.empty(need, dtype=torch.uint8, device=dev)
            check(lib.vqattn_assign_codes_ws(dk, dc, db if bias is not None else None, do, workspace.data_ptr(), workspace.numel(),
                                             device_status_word(dev).data_ptr(), stream_ptr(dev)), "vqattn_assign_codes_ws")
    return codes


def far_blocks(L: int, window: int) -> int:
    """Number of aggregate blocks a prefill of length L reads (0 when the far set is empty)."""
    return max(0, (L + BLOCK - 1) // BLOCK - window // BLOCK - 1)


def build_aggregates(codes: torch.Tensor, v: torch.Tensor, K: int, nb: Optional[int] = None,
                     out_dtype: Optional[torch.dtype] = None, workspace: Optional[torch.Tensor] = None,
                     impl: str = "auto", state_blocks: Optional[int] = None):
    """Per-block counts and value sums (replaces ops/attn_vq.py:352-384,411-417).

    codes [B,Hkv,L,M], v [B,Hkv,L,D] -> cnt [B,Hkv,NB,M*K] f32, vsum [B,Hkv,NB,M*K,D] (v's dtype).
    impl "auto": with a workspace (uint8, allocated here when none is passed) in which the library sorts every block's
    keys by code first; "scan": the entry point without a workspace.  Same results bit for bit.
    state_blocks (>= nb >= 1): also returns the fp32 counts [B,Hkv,M*K] and sums [B,Hkv,M*K,D] of the first
    state_blocks * 128 keys, taken from the same pass (what cache_advance over those keys gives from zero).
    """
    dev = _require_cuda(codes, v)
    B, Hkv, L, M = codes.shape
    D = v.shape[-1]
    nb = L // BLOCK if nb is None else nb
    cnt = torch.empty((B, Hkv, nb, M * K), dtype=torch.float32, device=dev)
    vsum = torch.empty((B, Hkv, nb, M * K, D), dtype=out_dtype or v.dtype, device=dev)
    if state_blocks is not None:
        assert nb >= 1 and nb <= state_blocks <= L // BLOCK, "state_blocks must lie in [nb, L // 128] and nb >= 1"
        s_cnt = torch.empty((B, Hkv, M * K), dtype=torch.float32, device=dev)
        s_vsum = torch.empty((B, Hkv, M * K, D), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            need = 0 if impl == "scan" else lib.vqattn_aggregates_workspace_bytes(B, Hkv, state_blocks, M, K)
            if need and (workspace is None or workspace.numel() < need):
                workspace = torch.empty(need, dtype=torch.uint8, device=dev)
            check(lib.vqattn_build_aggregates_state(desc(codes), desc(v), K, desc(cnt), desc(vsum), desc(s_cnt), desc(s_vsum),
                                                    state_blocks, workspace.data_ptr() if need else None, need,
                                                    device_status_word(dev).data_ptr(), stream_ptr(dev)),
                  "vqattn_build_aggregates_state")
        return cnt, vsum, s_cnt, s_vsum
    if nb > 0:
        with torch.cuda.device(dev):
            if impl == "scan":
                check(lib.vqattn_build_aggregates(desc(codes), desc(v), K, desc(cnt), desc(vsum), stream_ptr(dev)),
                      "vqattn_build_aggregates")
            else:
                need = lib.vqattn_aggregates_workspace_bytes(B, Hkv, nb, M, K)
                if workspace is None or workspace.numel() < need:
                    workspace = torch.empty(need, dtype=torch.uint8, device=dev)
                check(lib.vqattn_build_aggregates_ws(desc(codes), desc(v), K, desc(cnt), desc(vsum), workspace.data_ptr(),
                                                     workspace.numel(), device_status_word(dev).data_ptr(), stream_ptr(dev)),
                      "vqattn_build_aggregates_ws")
    return cnt, vsum


_ROPE_TABLES = {}


def rope_tables(n_pos: int, dim: int, device, base: float = 10000.0):
    """fp32 cos / sin tables [n_pos, dim/2] (angle = pos * base^(-2i/dim), evaluated in float64), cached per device."""
    dev = torch.device(device)
    key = (_device_index(dev), dim, float(base))
    have = _ROPE_TABLES.get(key)
    if have is None or have[0].shape[0] < n_pos:
        n = max(n_pos, 2 * have[0].shape[0] if have is not None else 0)
        inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64, device=dev) / dim))
        ang = torch.outer(torch.arange(n, dtype=torch.float64, device=dev), inv)
        have = _ROPE_TABLES[key] = (ang.cos().float().contiguous(), ang.sin().float().contiguous())
    return have


def rope(x: torch.Tensor, positions: Optional[torch.Tensor] = None, const_pos: Optional[int] = None,
         want_pos: bool = True, base: float = 10000.0, n_pos: Optional[int] = None):
    """RoPE of x [B,H,L,D] (ops/attn_vq.py:296-299,402-407): returns (x rotated to its positions or None,
    x rotated to ``const_pos`` or None), both from one pass.  positions: int64 [B,L] (None: 0..L-1);
    n_pos: an upper bound of the positions + 1 (None: read from ``positions``, which synchronises)."""
    dev = _require_cuda(x, positions)
    B, H, L, D = x.shape
    if x.stride(-1) != 1:
        x = x.contiguous()
    if n_pos is None:
        n_pos = L if positions is None else int(positions.max().item()) + 1
    if const_pos is not None:
        n_pos = max(n_pos, const_pos + 1)
    cos, sin = rope_tables(n_pos, D, dev, base)
    if positions is not None:
        positions = positions.to(torch.int64).expand(B, L).contiguous()
    out_pos = torch.empty((B, H, L, D), dtype=x.dtype, device=dev) if want_pos else None
    out_const = torch.empty((B, H, L, D), dtype=x.dtype, device=dev) if const_pos is not None else None
    with torch.cuda.device(dev):
        check(lib.vqattn_rope(desc(x), positions.data_ptr() if positions is not None else None, cos.data_ptr(), sin.data_ptr(),
                              cos.shape[0], const_pos if const_pos is not None else 0, desc(out_pos), desc(out_const),
                              device_status_word(dev).data_ptr(), stream_ptr(dev)), "vqattn_rope")
    return out_pos, out_const


def rope_qk(q: torch.Tensor, k: torch.Tensor, positions: Optional[torch.Tensor] = None, const_pos: Optional[int] = None,
            base: float = 10000.0, n_pos: Optional[int] = None, like_input: bool = False):
    """The rotations of one prefill in one launch (ops/attn_vq.py:402-407): returns (q1, q2 or None, k1).

    q [B,Hq,L,D], k [B,Hkv,L,D]: any strided views with a contiguous last dim.  positions int64 [B,L] (None: 0..L-1).
    like_input=True allocates the outputs with the memory layout of the inputs ([B,L,H,D] storage stays so)."""
    dev = _require_cuda(q, k, positions)
    B, Hq, L, D = q.shape
    if n_pos is None:
        n_pos = L if positions is None else int(positions.max().item()) + 1
    if const_pos is not None:
        n_pos = max(n_pos, const_pos + 1)
    cos, sin = rope_tables(n_pos, D, dev, base)
    if positions is not None:
        positions = positions.to(torch.int64).expand(B, L).contiguous()
    new = (lambda t: torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=dev)) if like_input else \
        (lambda t: torch.empty(t.shape, dtype=t.dtype, device=dev))
    q1, k1 = new(q), new(k)
    q2 = new(q) if const_pos is not None else None
    with torch.cuda.device(dev):
        check(lib.vqattn_rope_qk(desc(q), desc(k), positions.data_ptr() if positions is not None else None, cos.data_ptr(),
                                 sin.data_ptr(), cos.shape[0], const_pos if const_pos is not None else 0, desc(q1), desc(q2),
                                 desc(k1), device_status_word(dev).data_ptr(), stream_ptr(dev)), "vqattn_rope_qk")
    return q1, q2, k1


def decode_append(q, k, v, pos: int, const_pos: int, q1, q2, k1_win, k3_win, v_win, row: int, base: float = 10000.0,
                  positions: Optional[torch.Tensor] = None, n_pos: Optional[int] = None) -> None:
    """Per-token step of a decode in one launch: q [B,Hq,1,D] -> q1, q2 [B,Hq,1,D] (rotated to ``pos`` and to
    ``const_pos``); k, v [B,Hkv,1,D] -> row ``row`` of the window caches (rotated key, raw key, value)."""
    dev = _require_cuda(q, k, v, q1, q2, k1_win, k3_win, v_win, positions)
    D = q.shape[-1]
    cos, sin = rope_tables(max(n_pos or 0, pos + 1, const_pos + 1), D, dev, base)
    with torch.cuda.device(dev):
        check(lib.vqattn_decode_append(desc(q), desc(k), desc(v), positions.data_ptr() if positions is not None else None, int(pos),
                                       cos.data_ptr(), sin.data_ptr(), cos.shape[0], int(const_pos), desc(q1), desc(q2),
                                       desc(k1_win), desc(k3_win), desc(v_win), int(row), device_status_word(dev).data_ptr(),
                                       stream_ptr(dev)), "vqattn_decode_append")


def gather_aggregates(v_vq: torch.Tensor, vi: torch.Tensor, nb: int, cnt: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense value sums from the reference's sorted-prefix format (v_vq [B,H,L+1,D], vi [B,H,NB,C]).

    cnt [B,H,nb,C] f32 (optional): rows of codes with cnt == 0 are written as zeros, as the prefill
    kernels expect (the reference masks those codes inside its kernel).
    """
    dev = _require_cuda(v_vq, vi, cnt)
    B, H, _, D = v_vq.shape
    C = vi.shape[-1]
    if vi.dtype not in (torch.int32, torch.int64):
        vi = vi.to(torch.int64)
    vsum = torch.empty((B, H, nb, C, D), dtype=v_vq.dtype, device=dev)
    if nb > 0:
        with torch.cuda.device(dev):
            check(lib.vqattn_gather_aggregates(desc(v_vq), desc(vi), desc(cnt), desc(vsum), stream_ptr(dev)),
                  "vqattn_gather_aggregates")
    return vsum


def prefill_from_aggregates(q1, q2, k1, k3, v, codebook_act, cnt, vsum, window: int, scale: Optional[float] = None,
                            impl: str = "auto", return_lse: bool = False, status_word: Optional[torch.Tensor] = None,
                            out: Optional[torch.Tensor] = None):
    """Fused prefill attention from ready aggregates (replaces ops/triton_fused_vq_attn.py:190-251).

    codebook_act [Hkv,MK,D] in the activation dtype (None: local part only).
    """
    dev = _require_cuda(q1, q2, k1, k3, v, codebook_act, cnt, vsum)
    B, Hq, L, D = q1.shape
    if out is None:
        out = torch.empty((B, Hq, L, D), dtype=q1.dtype, device=dev)
    lse = torch.empty((B, Hq, L), dtype=torch.float32, device=dev) if return_lse else None
    a = VqPrefillArgs()
    a.q1, a.q2, a.k1, a.k3, a.v = desc(q1), desc(q2), desc(k1), desc(k3), desc(v)
    a.codebook, a.cnt, a.vsum = desc(codebook_act), desc(cnt), desc(vsum)
    a.out, a.lse2 = desc(out), desc(lse)
    a.window = int(window)
    a.scale = float(scale) if scale else 0.0
    a.impl = _IMPL[impl]
    a.status_word = (status_word if status_word is not None else device_status_word(dev)).data_ptr()
    with torch.cuda.device(dev):
        check(lib.vqattn_prefill(ctypes.byref(a), stream_ptr(dev)), "vqattn_prefill")
    return (out, lse) if return_lse else out


def vq_attention_prefill(q1, q2, k1, k3, v, codebooks, window: int, scale: Optional[float] = None,
                         bias: Optional[torch.Tensor] = None, impl: str = "auto", return_state: bool = False,
                         out: Optional[torch.Tensor] = None, codebook_act: Optional[torch.Tensor] = None,
                         state_blocks: Optional[int] = None):
    """The whole prefill path: assign codes to k3, build aggregates of v, fused attention.

    q1,q2 [B,Hq,L,D]; k1,k3,v [B,Hkv,L,D] (f32 or bf16); codebooks [Hkv,M,K,D] f32.
    ReRoPE mode: q1,k1 rotated by position, q2 rotated to the constant position window+1, k3 un-rotated
    (ops/attn_vq.py:402-407).  Plain-RoPE mode: pass q2 = q1 and k3 = k1.
    All five may be strided views with a contiguous last dim, and so may ``out`` ([B,Hq,L,D] view of
    [B,L,Hq,D] storage gives the layout the reference produces with a transposing copy, :442).
    codebook_act: [Hkv,M*K,D] copy of the codebooks in the activation dtype, if the caller keeps one.
    state_blocks (with return_state): the state dict also gets "state_cnt" / "state_vsum", the fp32 aggregates of
    the first state_blocks * 128 keys, when the aggregate pass can supply them (a far set exists).
    """
    B, Hq, L, D = q1.shape
    Hkv, M, K, _ = codebooks.shape
    nb = far_blocks(L, window)
    codes = cnt = vsum = cb_act = s_cnt = s_vsum = None
    if nb > 0 or return_state:
        codes = assign_codes(k3, codebooks, bias)
    if nb > 0:
        if return_state and state_blocks is not None and nb <= state_blocks <= L // BLOCK:
            cnt, vsum, s_cnt, s_vsum = build_aggregates(codes, v, K, nb, state_blocks=state_blocks)
        else:
            cnt, vsum = build_aggregates(codes, v, K, nb)
        cb_act = codebook_act if codebook_act is not None else codebooks.reshape(Hkv, M * K, D).to(q1.dtype)
    out = prefill_from_aggregates(q1, q2, k1, k3, v, cb_act, cnt, vsum, window, scale, impl, out=out)
    if return_state:
        return out, dict(codes=codes, cnt=cnt, vsum=vsum, state_cnt=s_cnt, state_vsum=s_vsum)
    return out


def decode_workspace(B: int, Hq: int, Hkv: int, D: int, device) -> torch.Tensor:
    """Zero-filled workspace for vq_attention_decode; reusable across calls on one stream."""
    n = lib.vqattn_decode_workspace_bytes(B, Hq, Hkv, D)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def vq_attention_decode(q1, q2, k1_win, k3_win, v_win, codebook, cnt, vsum, n_valid: Optional[int] = None, n_bd: int = 0,
                        scale: Optional[float] = None, workspace: Optional[torch.Tensor] = None,
                        out: Optional[torch.Tensor] = None, static_scratch: bool = False):
    """Single-query decode (seqlen_q == 1) over a window cache plus far aggregates.

    q1,q2 [B,Hq,D]; k1_win,k3_win,v_win [B,Hkv,Nwin,D]; codebook [Hkv,MK,D] (f32 or activation dtype) or None;
    cnt [B,Hkv,MK] f32; vsum [B,Hkv,MK,D].
    static_scratch=True uses ``vqattn_decode_static``: the merge scratch is a fixed 16 MiB array inside
    the library, for hosts that cannot supply a workspace; one such call at a time per device.
    """
    dev = _require_cuda(q1, q2, k1_win, k3_win, v_win, codebook, cnt, vsum)
    B, Hq, D = q1.shape
    Hkv, Nwin = k1_win.shape[1], k1_win.shape[2]
    if workspace is None and not static_scratch:
        workspace = decode_workspace(B, Hq, Hkv, D, dev)
    if out is None:
        out = torch.empty((B, Hq, D), dtype=q1.dtype, device=dev)
    a = VqDecodeArgs()
    a.q1, a.q2, a.k1_win, a.k3_win, a.v_win = desc(q1), desc(q2), desc(k1_win), desc(k3_win), desc(v_win)
    a.codebook, a.cnt, a.vsum, a.out = desc(codebook), desc(cnt), desc(vsum), desc(out)
    a.n_valid = Nwin if n_valid is None else int(n_valid)
    a.n_bd = int(n_bd)
    a.use_far = 1 if codebook is not None else 0
    a.scale = float(scale) if scale else 0.0
    a.status_word = device_status_word(dev).data_ptr()
    if static_scratch:
        # the library's built-in scratch array: nothing is allocated for this call (pass `out` too)
        with torch.cuda.device(dev):
            check(lib.vqattn_decode_static(ctypes.byref(a), stream_ptr(dev)), "vqattn_decode_static")
        return out
    a.workspace = workspace.data_ptr()
    a.workspace_bytes = workspace.numel() * workspace.element_size()
    with torch.cuda.device(dev):
        check(lib.vqattn_decode(ctypes.byref(a), stream_ptr(dev)), "vqattn_decode")
    return out


class DecodeStepCall:
    """The argument block of ``vqattn_decode_step`` for one layer of a cache, kept between tokens: the host fills
    the descriptors of the caches once and changes a handful of fields per token, so that generating a token costs
    one call into the library (two kernel launches: rotate-and-append, attention)."""

    def __init__(self, q1, q2, win_k1, win_k3, win_v, codebook, cnt, vsum, workspace, const_pos: int, base: float,
                 scale: float):
        self.dev = _require_cuda(q1, q2, win_k1, win_k3, win_v, codebook, cnt, vsum, workspace)
        self.dev_index = _device_index(self.dev)
        self.base, self.far_tensors = base, (codebook, cnt, vsum)
        self.keep = (q1, q2, win_k1, win_k3, win_v, workspace)
        a = self.args = native.VqDecodeStepArgs()
        desc(q1, a.q1)
        desc(q2, a.q2)
        a.const_pos = int(const_pos)
        d = a.decode
        desc(q1[:, :, 0], d.q1)
        desc(q2[:, :, 0], d.q2)
        self.rebind_windows(win_k1, win_k3, win_v)
        desc(codebook, d.codebook)
        desc(cnt, d.cnt)
        desc(vsum, d.vsum)
        d.scale = float(scale)
        d.workspace = workspace.data_ptr()
        d.workspace_bytes = workspace.numel() * workspace.element_size()
        d.status_word = device_status_word(self.dev).data_ptr()
        self._tables(max(const_pos + 1, 2))
        self._in = None
        self._ref = ctypes.byref(a)

    def _tables(self, n_pos):
        D = self.keep[0].shape[-1]
        self.cos, self.sin = rope_tables(n_pos, D, self.dev, self.base)
        a = self.args
        a.cos_tab, a.sin_tab, a.n_pos = self.cos.data_ptr(), self.sin.data_ptr(), self.cos.shape[0]

    def rebind_windows(self, win_k1, win_k3, win_v):
        """The window views moved (a block left the window, or the buffers were compacted)."""
        d = self.args.decode
        desc(win_k1, d.k1_win)
        desc(win_k3, d.k3_win)
        desc(win_v, d.v_win)
        self.windows = (win_k1, win_k3, win_v)

    def __call__(self, q, k, v, pos: int, row: int, n_valid: int, n_bd: int, use_far: bool, positions=None):
        a = self.args
        B, Hq, _, D = q.shape
        out = torch.empty((B, Hq, D), dtype=q.dtype, device=self.dev)
        sig = (q.shape, q.stride(), k.stride(), v.stride())
        if self._in != sig:                      # layout of the new token's tensors: usually the same every step
            desc(q, a.q)
            desc(k, a.k)
            desc(v, a.v)
            desc(out, a.decode.out)
            self._in = sig
        else:
            a.q.ptr, a.k.ptr, a.v.ptr, a.decode.out.ptr = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
        if pos + 1 > a.n_pos:
            self._tables(pos + 1)
        a.positions = positions.data_ptr() if positions is not None else None
        a.pos, a.row = int(pos), int(row)
        d = a.decode
        d.n_valid, d.n_bd, d.use_far = int(n_valid), int(n_bd), 1 if use_far else 0
        if torch.cuda.current_device() == self.dev_index:       # the usual case: no device switch around the call
            st = lib.vqattn_decode_step(self._ref, stream_ptr(self.dev_index))
        else:
            with torch.cuda.device(self.dev):
                st = lib.vqattn_decode_step(self._ref, stream_ptr(self.dev_index))
        if st != 0:
            check(st, "vqattn_decode_step")
        return out


def cache_advance(codes, v_new, K: int, cnt, vsum_f32, vsum_act=None):
    """Fold keys that crossed the boundary into a decode cache's aggregates (in place)."""
    dev = _require_cuda(codes, v_new, cnt, vsum_f32, vsum_act)
    with torch.cuda.device(dev):
        check(lib.vqattn_cache_advance(desc(codes), desc(v_new), K, desc(cnt), desc(vsum_f32),
                                       desc(vsum_act) if vsum_act is not None else None,
                                       device_status_word(dev).data_ptr(), stream_ptr(dev)), "vqattn_cache_advance")


# ---------------------------------------------------------------------------------------------
# Host-buffer entry points: CPU tensors in, CPU tensor out, copies included.

def _to_device(t, dev):
    if t is None:
        return None
    if not t.is_pinned():
        t = t.pin_memory()
    return t.to(dev, non_blocking=True)


_SIDE_STREAMS = {}


def _side_streams(dev):
    key = _device_index(dev)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _SIDE_STREAMS[key]


def vq_attention_prefill_host(q1, q2, k1, k3, v, codebooks, window: int, scale: Optional[float] = None,
                              device="cuda:0", impl: str = "auto", out: Optional[torch.Tensor] = None,
                              chunks: int = 8) -> torch.Tensor:
    """vq_attention_prefill for host tensors: host->device copies, the three kernels, device->host copy.

    (batch, kv-head) units are independent, so the work is cut into about ``chunks`` groups of kv heads
    and pipelined: a copy-in stream runs ahead of the kernels (current stream) and a copy-out stream
    behind them, so both directions of the host link and the kernels overlap.  Returns after everything
    has landed in ``out`` (pinned host memory).
    q2 / k3 may be the same objects as q1 / k1 (plain-RoPE mode): they are then copied once.
    """
    dev = torch.device(device)
    same_q, same_k = q2 is q1, k3 is k1
    hq1, hq2, hk1, hk3, hv = [t if (t is None or t.is_pinned()) else t.pin_memory() for t in (q1, q2, k1, k3, v)]
    if same_q:
        hq2 = hq1
    if same_k:
        hk3 = hk1
    B, Hq, L, D = q1.shape
    Hkv = k1.shape[1]
    group = Hq // Hkv
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream(dev)
        s_in, s_out = _side_streams(dev)
        dcb = codebooks if codebooks.is_cuda else _to_device(codebooks, dev)
        dq1 = torch.empty(q1.shape, dtype=q1.dtype, device=dev)
        dq2 = dq1 if same_q else torch.empty(q2.shape, dtype=q2.dtype, device=dev)
        dk1 = torch.empty(k1.shape, dtype=k1.dtype, device=dev)
        dk3 = dk1 if same_k else torch.empty(k3.shape, dtype=k3.dtype, device=dev)
        dv = torch.empty(v.shape, dtype=v.dtype, device=dev)
        dout = torch.empty(q1.shape, dtype=q1.dtype, device=dev)
        if out is None:
            out = torch.empty(q1.shape, dtype=q1.dtype, pin_memory=True)
        per_b = max(1, int(chunks) // B)
        hc = (Hkv + per_b - 1) // per_b
        parts = [(b, h0, min(Hkv, h0 + hc)) for b in range(B) for h0 in range(0, Hkv, hc)]
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        # copy order k, v, q: the kernels of a chunk need them in that order (codes from k, aggregates from v,
        # attention from q), so each stage waits only for what it reads
        Hkv_, M_, K_, _ = dcb.shape
        nb = far_blocks(L, window)
        arrived = []
        with torch.cuda.stream(s_in):
            for b, h0, h1 in parts:
                g0, g1 = h0 * group, h1 * group
                evs = []
                for dst, src, lo, hi, skip in ((dk1, hk1, h0, h1, False), (dk3, hk3, h0, h1, same_k), (dv, hv, h0, h1, False),
                                                (dq1, hq1, g0, g1, False), (dq2, hq2, g0, g1, same_q)):
                    if not skip:
                        dst[b, lo:hi].copy_(src[b, lo:hi], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(s_in)
                    evs.append(ev)
                arrived.append(evs)
        for (b, h0, h1), evs in zip(parts, arrived):
            g0, g1 = h0 * group, h1 * group
            sl_q, sl_k = (slice(b, b + 1), slice(g0, g1)), (slice(b, b + 1), slice(h0, h1))
            cnt = vsum = cb_act = None
            if nb > 0:
                cur.wait_event(evs[1])   # k1, k3
                codes = assign_codes(dk3[sl_k], dcb[h0:h1])
                cur.wait_event(evs[2])   # v
                cnt, vsum = build_aggregates(codes, dv[sl_k], K_, nb)
                cb_act = dcb[h0:h1].reshape(h1 - h0, M_ * K_, D).to(q1.dtype)
            cur.wait_event(evs[4])       # q1, q2 (and everything before them)
            prefill_from_aggregates(dq1[sl_q], dq2[sl_q], dk1[sl_k], dk3[sl_k], dv[sl_k], cb_act, cnt, vsum, window, scale,
                                    impl, out=dout[sl_q])
            done = torch.cuda.Event()
            done.record(cur)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                out[b, g0:g1].copy_(dout[b, g0:g1], non_blocking=True)
        cur.wait_stream(s_out)
        cur.synchronize()
    return out


def default_scale(D: int) -> float:
    return 1.0 / math.sqrt(D)
