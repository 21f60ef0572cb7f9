"""Host-side logic of the multi-GPU paths, run as real world_size > 1 process groups over gloo on
the CPU: the batch split, the limb ownership rule and the (in-place or padded) limb all-gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pyPhantom.parallel import allgather_limbs, limb_range, shard_batch


def test_partitions_cover_everything_once():
    for n in (1, 5, 8, 24, 64):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                b, c = limb_range(n, r, world)
                covered += list(range(b, b + c))
                sb, se = shard_batch(n, r, world)
                assert (sb, se - sb) == (b, c)
            assert covered == list(range(n))
            sizes = [limb_range(n, r, world)[1] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_limbs, N, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(n_limbs * N, dtype=torch.int64).view(n_limbs, N) * 7 + 3
        buf = torch.full((n_limbs + 2, N), -1, dtype=torch.int64)       # two limbs of slack stay untouched
        b, c = limb_range(n_limbs, rank, world)
        buf[b:b + c] = full[b:b + c]
        allgather_limbs(buf, n_limbs, rank, world)
        ok = torch.equal(buf[:n_limbs], full) and bool((buf[n_limbs:] == -1).all())
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_limbs", [(2, 24), (2, 5), (3, 8), (4, 24)])
def test_limb_allgather_over_gloo(world, n_limbs):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_limbs, 64, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(r, True) for r in range(world)]
