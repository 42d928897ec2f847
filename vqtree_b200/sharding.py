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
