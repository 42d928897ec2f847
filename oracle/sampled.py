"""Sampled-row parity at full benchmark sizes (test infrastructure, like the rest of ``oracle/``).

The naive oracle (vq_oracle.attn_naive, the restatement of ops/attn_vq.py:308-333) costs O(L) per query row, so
whole outputs at L = 32768 are out of reach; single rows are not.  The helpers here pick the rows where the
kernels change behaviour - the first tile, the first tile with a far part, either side of a boundary move, the
last tile, a few random ones - run the oracle on those rows for a few (batch, kv-head) units and report the
largest absolute difference from the rows a kernel produced.
"""
from __future__ import annotations

import numpy as np
import torch

from . import vq_oracle as vo


def row_ranges(L: int, W: int, n_random: int = 4, seed: int = 0):
    """Short row ranges [r0, r1) to check for a prefill of length L with window W."""
    t_far = W // 128 + 1                       # first query tile with a far part (rows 128 * t_far ...)
    picks = [0, 127, W - 1, W + 127, 128 * t_far - 1, 128 * t_far + 126, 128 * (t_far + 1) - 1, L // 2 - 1, L - 129, L - 2]
    rng = np.random.default_rng(seed)
    picks += [int(x) for x in rng.integers(0, max(1, L - 2), size=n_random)]
    out = []
    for r in sorted(set(p for p in picks if 0 <= p < L - 1)):
        if not out or r >= out[-1][1]:
            out.append((r, r + 2))
    return out


def prefill_rows_max_err(out, q1, q2, k1, k3, v, codebooks, codes, W, units, ranges, scale=None):
    """Largest |out - oracle| over the sampled rows.

    out, q1, q2 [B,Hq,L,D]; k1, k3, v [B,Hkv,L,D] (torch, any device, as the kernel saw them);
    codebooks [Hkv,M,K,D] float32 (already rounded the way the kernel's copy is); codes [B,Hkv,L,M] integer;
    units: list of (b, kv_head).  Returns (max_abs, rows_checked)."""
    G = q1.shape[1] // k1.shape[1]
    worst, rows = 0.0, 0
    f = lambda t: t.detach().float().cpu().numpy()
    for b, h in units:
        hs = slice(h * G, (h + 1) * G)
        a = [f(t[b:b + 1, hs]) for t in (q1, q2)] + [f(t[b:b + 1, h:h + 1]) for t in (k1, k3, v)]
        cb = f(codebooks[h:h + 1])
        cd = codes[b:b + 1, h:h + 1].detach().cpu().to(torch.int32).numpy()
        got = f(out[b:b + 1, hs])
        for r0, r1 in ranges:
            want = vo.attn_naive(a[0], a[1], a[2], a[3], a[4], cb, cd, W, scale, rows=(r0, r1))
            worst = max(worst, float(np.abs(got[:, :, r0:r1] - want[:, :, r0:r1]).max()))
            rows += (r1 - r0) * G
    return worst, rows


def codes_equal_on_ranges(codes, k3, codebooks, units, ranges, bias=None):
    """True when the kernel's codes equal the oracle's on the sampled key ranges of the sampled units."""
    f = lambda t: t.detach().float().cpu().numpy()
    for b, h in units:
        for r0, r1 in ranges:
            want = vo.assign_codes(f(k3[b:b + 1, h:h + 1, r0:r1]), f(codebooks[h:h + 1]),
                                   None if bias is None else f(bias[h:h + 1]))
            got = codes[b:b + 1, h:h + 1, r0:r1].detach().cpu().to(torch.int32).numpy()
            if not np.array_equal(got, want):
                return False
    return True
