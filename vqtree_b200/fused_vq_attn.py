"""Mirror of the reference's ``ops/triton_fused_vq_attn.py`` entry point on the CUDA library."""
from __future__ import annotations

import math

import torch

from . import api

BLOCK = 128


def vq_attn_forward(q1, q2, k1, k_vq, k_vq_cnt, k3, v, v_vq, vi, window_size, softmax_scale=None):
    """Same arguments and result layout as ops/triton_fused_vq_attn.py:190-251.

    q1,q2,k1,k3,v [B,H,L,D]; k_vq [H,C,D]; k_vq_cnt [B,H,L/128,C]; v_vq [B,H,L+1,D] (within-code prefix
    sums in sorted order); vi [B,H,L/128,C] (row of v_vq per block and code).  Returns [B,H,L,D].
    The reference's sorted-prefix value format is converted to dense per-block sums by
    ``vqattn_gather_aggregates``; attention itself is one ``vqattn_prefill`` launch.
    """
    q1, q2, k1, k_vq, k_vq_cnt, k3, v, v_vq, vi = [
        x if x.stride(-1) == 1 else x.contiguous() for x in (q1, q2, k1, k_vq, k_vq_cnt, k3, v, v_vq, vi)
    ]
    batch, nheads, seqlen_q, d = q1.shape
    assert d in (64, 128), "head dimension must be 64 or 128"
    assert window_size % BLOCK == 0 and k_vq.shape[1] % BLOCK == 0
    softmax_scale = softmax_scale or 1.0 / math.sqrt(d)
    nb = api.far_blocks(seqlen_q, window_size)
    cnt = vsum = cb = None
    if nb > 0:
        assert vi.shape[2] >= nb and k_vq_cnt.shape[2] >= nb
        cnt = k_vq_cnt[:, :, :nb].float().contiguous()
        vsum = api.gather_aggregates(v_vq.to(q1.dtype), vi, nb, cnt)
        cb = k_vq.to(q1.dtype).contiguous()
    return api.prefill_from_aggregates(q1, q2, k1, k3, v, cb, cnt, vsum, window_size, softmax_scale)
