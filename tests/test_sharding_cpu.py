"""The multi-GPU layer on CPU: unit partition and the final gather, with world_size-2 gloo ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vqtree_b200 import sharding


def test_unit_ranges_partition_everything():
    for n in (1, 7, 32, 64, 512):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.unit_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_units, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, Hkv, L, D = 1, 2 * n_units, n_units, 4, 8
        g = torch.Generator().manual_seed(0)
        full = torch.randn(B, Hq, L, D, generator=g)          # what a single process would produce
        mine = sharding.shard_heads(full, Hq // Hkv, world, rank).clone()
        heads = sharding.shard_codebooks(torch.zeros(Hkv, 1, 1, 1), B, world, rank)
        lo, hi = sharding.unit_range(n_units, world, rank)
        assert heads == [u % Hkv for u in range(lo, hi)] and mine.shape[0] == hi - lo
        out = sharding.gather_outputs(mine, n_units)
        ok = torch.equal(out.reshape(B, Hq, L, D), full)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_gather_reassembles_outputs_with_two_gloo_ranks():
    for n_units in (4, 5):                                     # even and uneven split
        ctx = mp.get_context("spawn")
        with ctx.Manager() as man:
            ret = man.dict()
            port = _free_port()
            procs = [ctx.Process(target=_worker, args=(r, 2, port, n_units, ret)) for r in range(2)]
            for p in procs:
                p.start()
            for p in procs:
                p.join(120)
                assert p.exitcode == 0
            assert dict(ret) == {0: True, 1: True}
