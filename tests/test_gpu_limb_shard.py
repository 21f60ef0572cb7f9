"""RNS-limb sharding of one key switch. On one GPU the ranks are emulated one after another on
shared buffers (the all-gathers are then implicit): the union of what the ranks compute must be the
unsharded result, bit for bit. With two or more GPUs the same thing runs as real NCCL ranks."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import pyPhantom as ph
from pyPhantom import _native
from pyPhantom._native import LIB, check
from gpu_helpers import dev, host, key_dev, make_ctx, stream


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("l", [8, 5, 2])
def test_emulated_ranks_reproduce_the_key_switch(world, l):
    N = 4096
    ctx, o = make_ctx(N, [55, 40, 41, 42, 43, 44, 45, 46, 58, 59, 60], 3)
    beta = o.beta(l)
    key = o.synth_key(beta, 61, 10)
    kt, kp = key_dev(key)
    c2_h, ct_h = o.fill(1, o.primes[:l], 61, 3)[0], o.synth_ct(l, 61, 1)
    want = o.keyswitch(l, c2_h, key, ct_h)
    c2, ct = dev(c2_h), dev(ct_h)
    ws, nb = ctx.workspace(_native.OP_KEYSWITCH, l)
    ws.zero_()
    seen_q, seen_p = [], []
    for phase in range(3):
        for r in range(world):
            check(LIB.b2_ctx_set_shard(ctx._h, r, world))
            if phase == 0:
                rg = np.zeros(4, dtype=np.uint32)
                check(LIB.b2_shard_limbs(ctx._h, l, rg.ctypes.data))
                seen_q += list(range(rg[0], rg[0] + rg[1]))
                seen_p += list(range(rg[2], rg[2] + rg[3]))
            check(LIB.b2_shard_keyswitch_phase(ctx._h, l, phase, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(),
                                               ws.data_ptr(), nb, stream()))
    assert seen_q == list(range(l)) and seen_p == list(range(o.size_P))
    assert np.array_equal(host(ct), want)
    # the unsharded entry point still works on a context that has shard lists
    ct2 = dev(ct_h)
    check(LIB.b2_keyswitch(ctx._h, l, c2.data_ptr(), kp.ctypes.data, beta, ct2.data_ptr(), ws.data_ptr(), nb, stream()))
    assert np.array_equal(host(ct2), want)


@pytest.mark.parametrize("world,batch", [(1, 3), (2, 4), (3, 2), (8, 5)])
@pytest.mark.parametrize("shape", ["n12", "n16"])
def test_emulated_ranks_reproduce_a_batch_of_key_switches(world, batch, shape):
    """the batched phases (one launch per kernel over the whole batch, limb-major exchange buffers) with the ranks run one
    after another on shared buffers: every ciphertext of the batch must come out as the unsharded key switch gives it"""
    if shape == "n12":
        N, bits, special, levels = 4096, [55, 40, 41, 42, 43, 44, 45, 46, 58, 59, 60], 3, [8, 5]
    else:
        N, bits, special, levels = 65536, [60] + [40] * 23 + [60] * 8, 8, [24]
        if world == 3:
            pytest.skip("one ragged case is enough")
    ctx, o = make_ctx(N, bits, special)
    for l in levels:
        beta = o.beta(l)
        key = o.synth_key(beta, 71, 10)
        kt, kp = key_dev(key)
        c2_h = np.stack([o.fill(1, o.primes[:l], 71, 30 + b)[0] for b in range(batch)])
        ct_h = np.stack([o.synth_ct(l, 71, 60 + b) for b in range(batch)])
        c2, ct = dev(c2_h), dev(ct_h)
        nbytes = int(LIB.b2_shard_batch_workspace_bytes(ctx._h, l, batch))
        ws = torch.zeros(nbytes // 8, dtype=torch.int64, device="cuda")
        for phase in range(3):
            for r in range(world):
                check(LIB.b2_ctx_set_shard(ctx._h, r, world))
                check(LIB.b2_shard_keyswitch_phase_batch(ctx._h, l, phase, batch, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(),
                                                         ws.data_ptr(), nbytes, stream()))
        got = host(ct)
        ref_ws, ref_nb = ctx.workspace(_native.OP_KEYSWITCH, l)
        for b in range(batch):
            one = dev(ct_h[b])
            check(LIB.b2_keyswitch(ctx._h, l, c2[b].data_ptr(), kp.ctypes.data, beta, one.data_ptr(), ref_ws.data_ptr(), ref_nb, stream()))
            assert np.array_equal(got[b], host(one)), (l, b)
        assert np.array_equal(got[0], o.keyswitch(l, c2_h[0], key, ct_h[0]))
    assert ctx.device_status() == 0


def test_staggered_pipeline_schedule_on_one_rank():
    """the software pipeline of BatchedLimbShardedKeySwitch.pipeline (phase 0 of batch s, phase 1 of batch s - 1, phase 2 of
    batch s - 3 on one stream, exchanges on a second) with a world of one rank: seven batches through five workspaces, twice,
    every ciphertext equal to the single key switch"""
    from pyPhantom.parallel import BatchedLimbShardedKeySwitch
    N, l, B, n_batches = 8192, 7, 3, 7
    ctx, o = make_ctx(N, [58, 40, 40, 40, 40, 40, 40, 60, 60, 60], 3)
    key_h = o.synth_key(o.beta(l), 71, 10)
    key = ph.relin_key.from_numpy(ctx, key_h)
    bs = BatchedLimbShardedKeySwitch(ctx, rank=0, world=1)
    lanes = bs.make_lanes(1)
    wss = [bs.batch_workspace(l, B)[0] for _ in range(5)]
    c2s = [np.stack([o.fill(1, o.primes[:l], 75, 100 * i + b)[0] for b in range(B)]) for i in range(n_batches)]
    cts = [np.stack([o.synth_ct(l, 75, 1000 + 100 * i + b) for b in range(B)]) for i in range(n_batches)]
    kt, kp = key_dev(key_h)
    ws1, nb1 = ctx.workspace(_native.OP_KEYSWITCH, l)
    for rep in range(2):
        batches = [(dev(a), dev(b)) for a, b in zip(c2s, cts)]
        bs.pipeline(l, batches, key, lanes, wss)
        torch.cuda.synchronize()
        for i, (c2d, ctd) in enumerate(batches):
            for b in range(B):
                one = dev(cts[i][b])
                check(LIB.b2_keyswitch(ctx._h, l, c2d[b].data_ptr(), kp.ctypes.data, o.beta(l), one.data_ptr(), ws1.data_ptr(), nb1, stream()))
                assert torch.equal(ctd[b], one), (rep, i, b)
    assert ctx.device_status() == 0


def test_shard_argument_checks():
    ctx, o = make_ctx(4096, [40, 40, 50], 1)
    x = ctx.empty(2, 2)
    ws, nb = ctx.workspace(_native.OP_KEYSWITCH, 2)
    kt, kp = key_dev(o.synth_key(2, 1, 10))
    with pytest.raises(ValueError, match="set_shard first"):
        check(LIB.b2_shard_keyswitch_phase(ctx._h, 2, 0, x.data_ptr(), kp.ctypes.data, 2, x.data_ptr(), ws.data_ptr(), nb, stream()))
    with pytest.raises(ValueError, match="rank must be"):
        check(LIB.b2_ctx_set_shard(ctx._h, 2, 2))
    check(LIB.b2_ctx_set_shard(ctx._h, 0, 2))
    with pytest.raises(ValueError, match="phase must be"):
        check(LIB.b2_shard_keyswitch_phase(ctx._h, 2, 3, x.data_ptr(), kp.ctypes.data, 2, x.data_ptr(), ws.data_ptr(), nb, stream()))


_NCCL_WORKER = r"""
import os, sys
sys.path.insert(0, os.path.join(os.environ["REPO"], "phantom-fhe_b200")); sys.path.insert(0, os.path.join(os.environ["REPO"], "tests"))
import numpy as np, torch, torch.distributed as dist
import pyPhantom as ph
from pyPhantom.parallel import LimbShardedKeySwitch
from gpu_helpers import make_ctx, dev, host
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
N, l = 8192, 7
ctx, o = make_ctx(N, [58, 40, 40, 40, 40, 40, 40, 60, 60, 60], 3)
key_h = o.synth_key(o.beta(l), 71, 10)
key = ph.relin_key.from_numpy(ctx, key_h)
c2_h, ct_h = o.fill(1, o.primes[:l], 71, 3)[0], o.synth_ct(l, 71, 1)
sh = LimbShardedKeySwitch(ctx)
c2, ct = dev(c2_h), dev(ct_h)
sh.keyswitch(l, c2, key, ct)
sh.allgather_ct(l, ct)
ok = np.array_equal(host(ct), o.keyswitch(l, c2_h, key_h, ct_h))
# batches of three: on two lanes (own stream and communicator each: two workspaces select that form), and as the staggered
# software pipeline (five workspaces, seven batches: workspaces are reused while three batches are in flight), twice in a row
from pyPhantom.parallel import BatchedLimbShardedKeySwitch
bs = BatchedLimbShardedKeySwitch(ctx)
lanes = bs.make_lanes(2)
B = 3
# and the staggered pipeline once more on peer-writable workspaces (exchanges as copy-engine pushes + a one-word all-reduce)
for n_ws, n_batches, repeats, peer in ((2, 4, 1, False), (5, 7, 2, False), (4, 9, 2, True)):
    c2s = [np.stack([o.fill(1, o.primes[:l], 72 + n_ws, 100 * i + b)[0] for b in range(B)]) for i in range(n_batches)]
    cts = [np.stack([o.synth_ct(l, 72 + n_ws, 1000 + 100 * i + b) for b in range(B)]) for i in range(n_batches)]
    wss = bs.peer_workspaces(l, B, n_ws) if peer else [bs.batch_workspace(l, B)[0] for _ in range(n_ws)]
    if wss is None:
        print("peer workspaces unavailable: skipped", flush=True)
        continue
    for rep in range(repeats):
        batches = [(dev(a), dev(b)) for a, b in zip(c2s, cts)]
        bs.pipeline(l, batches, key, lanes, wss)
        torch.cuda.synchronize()
        for i, (c2d, ctd) in enumerate(batches):
            for b in range(B):
                one = ctd[b]
                bs.allgather_ct(l, one)
                ok = ok and np.array_equal(host(one), o.keyswitch(l, c2s[i][b], key_h, cts[i][b]))
    if peer:
        dist.barrier()
        for w in wss:
            w.close()
ok = ok and ctx.device_status() == 0
t = torch.tensor([1 if ok else 0], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if int(t.item()) == 1 else 1)
"""


def test_two_real_ranks_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_NCCL_WORKER)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
