"""Host-side logic of the multi-GPU paths, run as real world_size > 1 process groups over gloo on
the CPU: the batch split, the limb ownership rule and the (in-place or padded) limb all-gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pyPhantom.parallel import allgather_limbs, exchange_block, limb_range, pipeline_schedule, shard_batch


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


@pytest.mark.parametrize("n_batches", [1, 2, 3, 4, 7, 16])
def test_staggered_pipeline_schedule(n_batches):
    """the issue order of BatchedLimbShardedKeySwitch.pipeline: every batch runs phase 0, exchange 0, phase 1, exchange 1,
    phase 2 in that order; an exchange directly follows the phase that feeds it; at most three batches are between their phase 0
    and their phase 2 when a phase 0 is queued, so four workspaces suffice: everything of batch i precedes phase 0 of batch i + 4"""
    sched = pipeline_schedule(n_batches)
    pos = {item: k for k, item in enumerate(sched)}
    assert len(pos) == len(sched) == 5 * n_batches
    for i in range(n_batches):
        order = [pos[("phase", i, 0)], pos[("exchange", i, 0)], pos[("phase", i, 1)], pos[("exchange", i, 1)], pos[("phase", i, 2)]]
        assert order == sorted(order)
        assert pos[("exchange", i, 0)] == pos[("phase", i, 0)] + 1 and pos[("exchange", i, 1)] == pos[("phase", i, 1)] + 1
        if i + 4 < n_batches:
            assert pos[("phase", i, 2)] < pos[("phase", i + 4, 0)]
    # between an exchange and the phase that consumes it, phases of other batches are queued (what hides it)
    for i in range(1, n_batches - 3):
        between = sched[pos[("exchange", i, 0)] + 1: pos[("phase", i, 1)]]
        assert any(kind == "phase" and b != i for kind, b, _ in between)
        between = sched[pos[("exchange", i, 1)] + 1: pos[("phase", i, 2)]]
        assert sum(kind == "phase" and b != i for kind, b, _ in between) >= 3


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_peer_pushes_move_what_the_all_gather_moves(world):
    """every rank pushing its exchange_block into every peer's workspace leaves all workspaces equal to the one in which
    every limb row was written by its owner - the state an all-gather over the rows gives"""
    l, alpha, batch, N = 24, 8, 3, 16
    words = (l + 2 * alpha) * batch * N
    full = np.zeros(words, dtype=np.uint64)
    ws = [np.zeros(words, dtype=np.uint64) for _ in range(world)]
    for which in (0, 1):
        for r in range(world):
            off, size = exchange_block(l, alpha, batch, N, which, r, world)
            assert off % 8 == 0 and size % 8 == 0
            blk = np.arange(size // 8, dtype=np.uint64) + np.uint64(1000003 * (r + 1) + 7 * which)
            ws[r][off // 8: (off + size) // 8] = blk       # the owner computed its rows
            full[off // 8: (off + size) // 8] = blk
        for r in range(world):                              # pushes
            off, size = exchange_block(l, alpha, batch, N, which, r, world)
            for p in range(world):
                if p != r:
                    ws[p][off // 8: (off + size) // 8] = ws[r][off // 8: (off + size) // 8]
    for r in range(world):
        assert np.array_equal(ws[r], full)
    # the blocks of one exchange tile the region exactly
    for which, (lo, hi) in ((0, (0, l * batch * N * 8)), (1, (l * batch * N * 8, (l + 2 * alpha) * batch * N * 8))):
        spans = sorted(exchange_block(l, alpha, batch, N, which, r, world) for r in range(world))
        assert spans[0][0] == lo and all(a[0] + a[1] == b[0] for a, b in zip(spans, spans[1:])) and spans[-1][0] + spans[-1][1] == hi
