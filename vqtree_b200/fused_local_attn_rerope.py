"""Mirror of the reference's ``ops/triton_fused_local_attn_rerope.py`` entry point."""
from __future__ import annotations

import torch

from . import api


def flash_attn_func(q1, q2, k1, k2, v, window_size, softmax_scale=None, return_lse=False):
    """Same contract as ops/triton_fused_local_attn_rerope.py:287-294.

    q1,q2: (batch, seqlen_q, nheads, headdim); k1,k2,v: (batch, seqlen_k, nheads, headdim).
    Keys of the 128-block holding position i - window are scored q1.k1 when i - j <= window and
    q2.k2 otherwise (:68-75); newer blocks q1.k1, causal on the diagonal.  Returns o in the input
    layout and, if asked, the base-2 log-sum-exp [batch, nheads, seqlen_q] fp32.
    """
    q1, q2, k1, k2, v = [x if x.stride(-1) == 1 else x.contiguous() for x in (q1, q2, k1, k2, v)]
    batch, seqlen_q, nheads, d = q1.shape
    assert k1.shape == (batch, seqlen_q, nheads, d) and v.shape == k1.shape, "prefill needs seqlen_q == seqlen_k"
    assert q1.dtype == q2.dtype == k1.dtype == k2.dtype == v.dtype, "All tensors must have the same type"
    assert q1.is_cuda and q2.is_cuda and k1.is_cuda and k2.is_cuda and v.is_cuda
    o = torch.empty_like(q1, memory_format=torch.contiguous_format)
    t = lambda x: x.transpose(1, 2)
    res = api.prefill_from_aggregates(t(q1), t(q2), t(k1), t(k2), t(v), None, None, None, window_size, softmax_scale,
                                      return_lse=return_lse, out=t(o))
    if return_lse:
        return o, res[1]
    return o
