"""PyTorch (CPU, multi-threaded) port of the reference's naive VQ-attention path.

TEST / BASELINE INFRASTRUCTURE ONLY: this is the "reference's CPU PyTorch path" timed beside the
CUDA library by the benchmark, and a second oracle for the tests.  It restates, with dense masks
instead of Python loops, what the reference computes:

* ``quantize``  - ops/mini_vq.py:4-18 ``multi_head_single_quantize`` (einsum scores, first arg-max),
  extended to M codebooks by greedy residual assignment (no counterpart in the reference).
* ``naive_attention`` - ops/attn_vq.py:278-334 ``long_prefilling_slow_reference_impl``: per query,
  window keys scored q1.k1, boundary keys scored q2.k3, older keys scored q2.codeword(key) and
  weighted by their own values, one fp32 softmax over all of them (:331), then ``@ v`` (:332).
"""
from __future__ import annotations

import math

import torch

BLOCK = 128


def quantize(k: torch.Tensor, codebooks: torch.Tensor):
    """k [B,H,L,D], codebooks [H,M,K,D] -> codes [B,H,L,M] int64 (greedy residual, inner-product metric)."""
    r = k.float()
    out = []
    for m in range(codebooks.shape[1]):
        cb = codebooks[:, m].float()
        scores = torch.einsum("zhqx,hcx->zhqc", r, cb)           # ops/mini_vq.py:10
        ids = scores.argmax(-1)                                  # ops/mini_vq.py:11
        out.append(ids)
        picked = torch.gather(cb[None].expand(r.shape[0], -1, -1, -1), 2, ids[..., None].expand(-1, -1, -1, r.shape[-1]))
        r = r - picked
    return torch.stack(out, -1)


def naive_attention(q1, q2, k1, k3, v, codebooks, codes, window: int, scale=None, q_block: int = 512):
    """Dense-mask restatement of the naive loop; returns [B,Hq,L,D] float32."""
    B, Hq, L, D = q1.shape
    Hkv, M, K, _ = codebooks.shape
    G = Hq // Hkv
    scale = scale or 1.0 / math.sqrt(D)
    q1, q2, k1, k3, v = (t.float() for t in (q1, q2, k1, k3, v))
    cb = codebooks.float()
    rep = lambda t: t.repeat_interleave(G, dim=1) if G > 1 else t
    k1r, k3r, vr = rep(k1), rep(k3), rep(v)
    # reconstruction of every key in every codebook: khat[m] = C_m[code_m]      (ops/attn_vq.py:300)
    khat = []
    for m in range(M):
        idx = codes[..., m].long()[..., None].expand(-1, -1, -1, D)
        khat.append(rep(torch.gather(cb[None, :, m].expand(B, -1, -1, -1), 2, idx)))
    out = torch.empty(B, Hq, L, D)
    j = torch.arange(L)
    for s in range(0, L, q_block):
        e = min(L, s + q_block)
        i = torch.arange(s, e)[:, None]
        lb = (i - window).clamp(min=0)
        bd = ((i - window).clamp(min=0) // BLOCK) * BLOCK          # ops/attn_vq.py:311
        win = (j[None] >= lb) & (j[None] <= i)                      # :313-316
        bnd = (j[None] >= bd) & (j[None] < lb)                      # :317-323
        far = j[None] < bd                                          # :324-330
        neg = float("-inf")
        s1 = torch.matmul(q1[:, :, s:e], k1r.transpose(-1, -2)) * scale
        s3 = torch.matmul(q2[:, :, s:e], k3r.transpose(-1, -2)) * scale
        parts = [torch.where(win, s1, torch.where(bnd, s3, torch.full_like(s1, neg)))]
        for m in range(M):
            sf = torch.matmul(q2[:, :, s:e], khat[m].transpose(-1, -2)) * scale
            parts.append(torch.where(far, sf, torch.full_like(sf, neg)))
        p = torch.softmax(torch.cat(parts, -1), dim=-1)            # :331
        o = torch.matmul(p[..., :L], vr)
        for m in range(M):
            o = o + torch.matmul(p[..., (m + 1) * L:(m + 2) * L], vr)
        out[:, :, s:e] = o
    return out


def prefill(q1, q2, k1, k3, v, codebooks, window: int, scale=None):
    """The whole naive path on CPU: quantize, then attend."""
    codes = quantize(k3, codebooks)
    return naive_attention(q1, q2, k1, k3, v, codebooks, codes, window, scale)
