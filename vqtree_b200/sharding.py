"""Multi-GPU layout of the VQ-attention path: independent (batch, kv-head) units, no collective on
the hot path, one gather of the outputs at the end.

Every (batch, kv-head) unit - its Hq/Hkv query heads, its codebooks, codes, aggregates and window -
is self-contained (the reference's kernels already treat batch*heads as a pure grid dimension,
ops/triton_fused_vq_attn.py:111-113,222), so rank r of G simply owns a contiguous range of units.
"""
from __future__ import annotations

from typing import List, Tuple

import torch


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous range [lo, hi) of flattened units u = b * Hkv + h_kv owned by `rank` (sizes differ by at most 1)."""
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def unit_pieces(B: int, Hkv: int, lo: int, hi: int) -> List[Tuple[int, int, int, int]]:
    """The unit range [lo, hi) as at most three rectangles (b0, b1, h0, h1) of the [B, Hkv] grid: the tail of a
    first batch row, whole batch rows, the head of a last batch row.  Each rectangle is a plain slice
    x[b0:b1, h0*G:h1*G] of every tensor, with codebooks[h0:h1]."""
    pieces = []
    u = lo
    while u < hi:
        b, h = divmod(u, Hkv)
        if h == 0 and hi - u >= Hkv:
            nb = (hi - u) // Hkv
            pieces.append((b, b + nb, 0, Hkv))
            u += nb * Hkv
        else:
            h1 = min(Hkv, h + hi - u)
            pieces.append((b, b + 1, h, h1))
            u += h1 - h
    return pieces


def slice_units(q1, q2, k1, k3, v, codebooks, piece):
    """Views of the tensors of one rectangle of units (see unit_pieces); q2 / k3 aliasing q1 / k1 is kept."""
    b0, b1, h0, h1 = piece
    G = q1.shape[1] // k1.shape[1]
    sq = lambda t: t[b0:b1, h0 * G: h1 * G]
    sk = lambda t: t[b0:b1, h0:h1]
    pq1, pk1 = sq(q1), sk(k1)
    return pq1, (pq1 if q2 is q1 else sq(q2)), pk1, (pk1 if k3 is k1 else sk(k3)), sk(v), codebooks[h0:h1]


def prefill_sharded(q1, q2, k1, k3, v, codebooks, window: int, world: int, rank: int, scale=None, out=None):
    """This rank's share of one prefill job: the (batch, kv-head) units unit_range(B*Hkv, world, rank) of the
    full tensors q1,q2 [B,Hq,L,D], k1,k3,v [B,Hkv,L,D], codebooks [Hkv,M,K,D], through the same three kernels
    as the unsharded call and with no communication.  Returns [units, Hq/Hkv, L, D]; gather_outputs (or a plain
    concatenation over ranks) gives the unsharded result viewed as [B*Hkv, Hq/Hkv, L, D]."""
    from . import api
    B, Hq, L, D = q1.shape
    Hkv = k1.shape[1]
    G = Hq // Hkv
    lo, hi = unit_range(B * Hkv, world, rank)
    if out is None:
        out = torch.empty((hi - lo, G, L, D), dtype=q1.dtype, device=q1.device)
    at = 0
    for piece in unit_pieces(B, Hkv, lo, hi):
        b0, b1, h0, h1 = piece
        n = (b1 - b0) * (h1 - h0)
        pq1, pq2, pk1, pk3, pv, pcb = slice_units(q1, q2, k1, k3, v, codebooks, piece)
        dst = out[at: at + n].view(b1 - b0, (h1 - h0) * G, L, D)
        api.vq_attention_prefill(pq1, pq2, pk1, pk3, pv, pcb.contiguous(), window, scale=scale, out=dst)
        at += n
    return out


def shard_heads(x: torch.Tensor, heads_per_unit: int, world: int, rank: int) -> torch.Tensor:
    """Slice of x [B, H, ...] (H = Hkv * heads_per_unit) holding this rank's units, as [units, heads_per_unit, ...]."""
    B, H = x.shape[:2]
    n_units = B * H // heads_per_unit
    lo, hi = unit_range(n_units, world, rank)
    flat = x.reshape(n_units, heads_per_unit, *x.shape[2:])
    return flat[lo:hi]


def shard_codebooks(codebooks: torch.Tensor, B: int, world: int, rank: int) -> List[int]:
    """kv-head index of every unit this rank owns (codebooks [Hkv, M, K, D] are indexed by it)."""
    Hkv = codebooks.shape[0]
    lo, hi = unit_range(B * Hkv, world, rank)
    return [u % Hkv for u in range(lo, hi)]


def gather_outputs(local_out: torch.Tensor, n_units: int, group=None) -> torch.Tensor:
    """All-gather of per-rank outputs [units_r, heads_per_unit, L, D] into [n_units, heads_per_unit, L, D].

    The only collective of the path; runs after the attention kernels.  Ranks may own unequal
    numbers of units: shards are padded to the largest count for the collective and trimmed after.
    """
    import torch.distributed as dist
    world = dist.get_world_size(group)
    counts = [unit_range(n_units, world, r) for r in range(world)]
    most = max(hi - lo for lo, hi in counts)
    pad = torch.zeros((most,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    pad[: local_out.shape[0]] = local_out
    full = torch.empty((world * most,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(full, pad, group=group)
    parts = [full[r * most: r * most + (hi - lo)] for r, (lo, hi) in enumerate(counts)]
    return torch.cat(parts, 0)
