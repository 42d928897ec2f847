"""Seeded synthetic inputs shared by the tests (shapes and distributions of the benchmark configs)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import vq_oracle as vo


def make_case(B, Hq, Hkv, L, D, M, K, W, seed, rerope, dtype=torch.float32, cb_std=None):
    """q/k/v ~ N(0,1), codebooks ~ N(0, cb_std^2); RoPE (HF half-split, base 10000) applied on the host.

    rerope=True : q1,k1 rotated by position, q2 rotated to position W+1, k3 un-rotated (ops/attn_vq.py:402-407)
    rerope=False: q2 is q1 and k3 is k1.
    Returns CPU tensors in ``dtype`` plus fp32 codebooks [Hkv,M,K,D].
    """
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, L, D, generator=g)
    k = torch.randn(B, Hkv, L, D, generator=g)
    v = torch.randn(B, Hkv, L, D, generator=g)
    cb = torch.randn(Hkv, M, K, D, generator=g) * (cb_std if cb_std is not None else D ** -0.25)
    cos, sin = vo.rope_tables(max(L, W + 2), D)
    pos = np.arange(L)
    q1 = torch.from_numpy(vo.apply_rope(q.numpy(), cos, sin, pos))
    k1 = torch.from_numpy(vo.apply_rope(k.numpy(), cos, sin, pos))
    if rerope:
        q2 = torch.from_numpy(vo.apply_rope(q.numpy(), cos, sin, np.full(L, W + 1)))
        k3 = k
    else:
        q2, k3 = q1, k1
    cast = lambda t: t.to(dtype).contiguous()
    out = dict(q1=cast(q1), k1=cast(k1), v=cast(v), cb=cb.contiguous(), W=W, M=M, K=K)
    out["q2"] = out["q1"] if not rerope else cast(q2)
    out["k3"] = out["k1"] if not rerope else cast(k3)
    return out


def oracle_prefill(case, rows=None, naive=True):
    """Oracle output for a case, evaluated on the inputs as the kernel sees them (after dtype rounding)."""
    f = lambda t: t.float().numpy()
    cb = case["cb"].numpy()
    q1, q2, k1, k3, v = (f(case[n]) for n in ("q1", "q2", "k1", "k3", "v"))
    codes = vo.assign_codes(k3, cb)
    cb_act = cb if case["q1"].dtype == torch.float32 else vo.round_bf16(cb)
    if naive:
        return vo.attn_naive(q1, q2, k1, k3, v, cb_act, codes, case["W"], rows=rows), codes
    cnt, vsum = vo.build_aggregates(codes, v, case["K"])
    return vo.attn_agg(q1, q2, k1, k3, v, cb_act, cnt, vsum, case["W"], rows=rows), codes
