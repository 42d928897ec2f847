"""Test double for ``vqtree_b200.api`` on machines without a GPU: the same function signatures, computed by
the CPU oracle (test infrastructure).  It exists so that the HOST logic above the C ABI - the attention module,
the cache bookkeeping, the transformers integration - can be exercised by the CPU test suite; the product
never imports it, and the GPU tests run the same scenarios against the real kernels.
"""
from __future__ import annotations

import contextlib

import numpy as np
import torch

from oracle import vq_oracle as vo


def _np(t):
    return t.detach().float().cpu().numpy()


def _rot(x, pos, base):
    """x [..., L, D] rotated to integer positions pos [L] or [B, L] (HF half-split convention), fp32 math."""
    D = x.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = pos.to(torch.float64)[..., None] * inv
    ang = torch.cat((ang, ang), -1)
    cos, sin = ang.cos().float(), ang.sin().float()
    if cos.dim() == 3:
        cos, sin = cos[:, None], sin[:, None]
    xf = x.float()
    h = D // 2
    rot = torch.cat((-xf[..., h:], xf[..., :h]), -1)
    return (xf * cos + rot * sin).to(x.dtype)


def rope_qk(q, k, positions=None, const_pos=None, base=10000.0, n_pos=None, like_input=False):
    L = q.shape[2]
    pos = positions if positions is not None else torch.arange(L)
    q2 = _rot(q, torch.full((L,), const_pos), base) if const_pos is not None else None
    return _rot(q, pos, base), q2, _rot(k, pos, base)


def decode_append(q, k, v, pos, const_pos, q1, q2, k1_win, k3_win, v_win, row, base=10000.0, positions=None, n_pos=None):
    p = positions.reshape(-1, 1) if positions is not None else torch.tensor([pos])
    q1.copy_(_rot(q, p, base))
    q2.copy_(_rot(q, torch.tensor([const_pos]), base))
    k1_win[:, :, row] = _rot(k, p, base)[:, :, 0]
    k3_win[:, :, row] = k[:, :, 0]
    v_win[:, :, row] = v[:, :, 0]


def code_dtype_for(K):
    return torch.uint8 if K <= 256 else torch.int32


def assign_codes(k, codebooks, bias=None, out_dtype=None, impl="auto", workspace=None):
    codes = vo.assign_codes(_np(k), _np(codebooks), None if bias is None else _np(bias))
    return torch.from_numpy(codes).to(out_dtype or code_dtype_for(codebooks.shape[2]))


def cache_advance(codes, v_new, K, cnt, vsum_f32, vsum_act=None):
    B, H, n, M = codes.shape
    c, vv = codes.long(), v_new.float()
    for b in range(B):
        for h in range(H):
            for j in range(n):
                for m in range(M):
                    r = m * K + int(c[b, h, j, m])
                    cnt[b, h, r] += 1
                    vsum_f32[b, h, r] += vv[b, h, j]
    if vsum_act is not None:
        vsum_act.copy_(vsum_f32.to(vsum_act.dtype))


def far_blocks(L, window):
    return max(0, (L + 127) // 128 - window // 128 - 1)


def _round(x, dtype):
    return _np(torch.from_numpy(np.ascontiguousarray(x)).to(dtype))


def vq_attention_prefill(q1, q2, k1, k3, v, codebooks, window, scale=None, bias=None, impl="auto", return_state=False,
                         out=None, codebook_act=None, state_blocks=None):
    cb = _np(codebooks)
    codes = vo.assign_codes(_np(k3), cb, None if bias is None else _np(bias))
    cb_act = cb if q1.dtype == torch.float32 else _round(cb, q1.dtype)
    res = vo.attn_naive(_np(q1), _np(q2), _np(k1), _np(k3), _np(v), cb_act, codes, window, scale)
    res = torch.from_numpy(res).to(q1.dtype)
    if out is not None:
        out.copy_(res)
        res = out
    if return_state:
        return res, dict(codes=torch.from_numpy(codes).to(code_dtype_for(codebooks.shape[2])), cnt=None, vsum=None,
                         state_cnt=None, state_vsum=None)   # the state is then summed by cache_advance
    return res


def prefill_from_aggregates(q1, q2, k1, k3, v, codebook_act, cnt, vsum, window, scale=None, impl="auto", return_lse=False,
                            status_word=None, out=None):
    assert codebook_act is None, "the test double covers the local-only call"
    Hkv, D, L = k1.shape[1], k1.shape[3], k1.shape[2]
    cb = np.zeros((Hkv, 1, 128, D), np.float32)
    codes = np.zeros(k1.shape[:3] + (1,), np.int32)
    res = torch.from_numpy(vo.attn_naive(_np(q1), _np(q2), _np(k1), _np(k3), _np(v), cb, codes, max(window, (L + 127) // 128 * 128),
                                         scale)).to(q1.dtype)
    if out is not None:
        out.copy_(res)
        res = out
    return res


def decode_workspace(B, Hq, Hkv, D, device):
    return torch.zeros(1)


def vq_attention_decode(q1, q2, k1_win, k3_win, v_win, codebook, cnt, vsum, n_valid=None, n_bd=0, scale=None, workspace=None,
                        out=None, static_scratch=False):
    B, Hq, D = q1.shape
    Hkv = k1_win.shape[1]
    far = codebook is not None
    if far:
        MK = codebook.shape[1]
        cbn, cn, vs = _np(codebook).reshape(Hkv, 1, MK, D), _np(cnt).reshape(B, Hkv, 1, MK), _np(vsum).reshape(B, Hkv, 1, MK, D)
    else:
        cbn, cn, vs = np.zeros((Hkv, 1, 128, D), np.float32), np.zeros((B, Hkv, 1, 128), np.float32), np.zeros((B, Hkv, 1, 128, D), np.float32)
    res = vo.decode(_np(q1), _np(q2), _np(k1_win), _np(k3_win), _np(v_win), cbn, cn, vs, n_valid, n_bd, scale, use_far=far)
    res = torch.from_numpy(res).to(q1.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


class DecodeStepCall:
    """Same interface as ``api.DecodeStepCall``: append, then attention, by the functions above."""

    def __init__(self, q1, q2, win_k1, win_k3, win_v, codebook, cnt, vsum, workspace, const_pos, base, scale):
        self.q1, self.q2, self.windows = q1, q2, (win_k1, win_k3, win_v)
        self.far = (codebook, cnt, vsum)
        self.const_pos, self.base, self.scale = const_pos, base, scale

    def rebind_windows(self, win_k1, win_k3, win_v):
        self.windows = (win_k1, win_k3, win_v)

    def __call__(self, q, k, v, pos, row, n_valid, n_bd, use_far, positions=None):
        decode_append(q, k, v, pos, self.const_pos, self.q1, self.q2, *self.windows, row, self.base, positions)
        cb, cnt, vsum = self.far if use_far else (None, None, None)
        return vq_attention_decode(self.q1[:, :, 0], self.q2[:, :, 0], *self.windows, cb, cnt, vsum, n_valid, n_bd, self.scale)


@contextlib.contextmanager
def installed():
    """Replaces the kernel-calling functions of ``vqtree_b200.api`` for the duration of the context."""
    from vqtree_b200 import api
    names = ("rope_qk", "decode_append", "assign_codes", "cache_advance", "vq_attention_prefill", "prefill_from_aggregates",
             "decode_workspace", "vq_attention_decode", "DecodeStepCall")
    saved = {n: getattr(api, n) for n in names}
    try:
        for n in names:
            setattr(api, n, globals()[n])
        yield
    finally:
        for n, f in saved.items():
            setattr(api, n, f)
