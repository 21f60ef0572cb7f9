"""Multi-GPU use of the key-switching path: one process per GPU, torch.distributed for plumbing.

Two ways the path shards (the reference itself has no multi-GPU code; its application runs one
independent engine per GPU from Python threads, python/llm_project/mrpc_sweep_parallel.py:1-9):

* independent ciphertexts: `shard_batch` gives each rank its slice of a batch; no collective on the
  data path (this is what bench.py measures at N > 1);
* RNS limbs of ONE ciphertext: `LimbShardedKeySwitch` - every rank owns a block of the Q and P
  limbs, transforms and the inner product are limb-local, and the two base conversions are fed by
  two all-gathers (the l scaled coefficient-form limbs of ModUp, the 2*alpha P limbs of ModDown).
  The exchanged limbs land in local HBM first; kernels only ever read local memory.
"""
import numpy as np
import torch
import torch.distributed as dist

from . import _native
from ._native import LIB, check


def shard_batch(n_items, rank, world):
    """contiguous slice [begin, end) of a batch of independent ciphertexts for this rank"""
    return n_items * rank // world, n_items * (rank + 1) // world


def limb_range(n_limbs, rank, world):
    """(first limb, count) of the block rank owns - the rule b2_ctx_set_shard uses"""
    b, e = n_limbs * rank // world, n_limbs * (rank + 1) // world
    return b, e - b


def allgather_limbs(buf, n_limbs, rank, world, group=None):
    """buf: [>= n_limbs][N] tensor whose block limb_range(n_limbs, rank, world) is valid on this
    rank; afterwards limbs [0, n_limbs) are valid on every rank. Equal blocks are gathered in place;
    ragged ones go through a padded staging buffer."""
    if world == 1:
        return
    ranges = [limb_range(n_limbs, r, world) for r in range(world)]
    b, cnt = ranges[rank]
    if n_limbs % world == 0:
        dist.all_gather_into_tensor(buf[:n_limbs], buf[b:b + cnt], group=group)
        return
    width = max(c for _, c in ranges)
    stage = torch.zeros((width,) + tuple(buf.shape[1:]), dtype=buf.dtype, device=buf.device)
    stage[:cnt].copy_(buf[b:b + cnt])
    gathered = torch.empty((world * width,) + tuple(buf.shape[1:]), dtype=buf.dtype, device=buf.device)
    dist.all_gather_into_tensor(gathered, stage, group=group)
    for r, (rb, rc) in enumerate(ranges):
        if r != rank and rc:
            buf[rb:rb + rc].copy_(gathered[r * width: r * width + rc])


class LimbShardedKeySwitch:
    """ct[2][l][N] += ModDown(<ModUp(c2), key>) with the limbs of everything spread over the ranks.

    Every rank passes full-size buffers; only its own limbs of c2, of the key digits and of ct need
    to hold data, and only its own limbs of ct are updated (gather them with `allgather_ct` if the
    whole ciphertext is wanted on every rank)."""

    def __init__(self, ctx, rank=None, world=None, group=None):
        self.ctx, self.group = ctx, group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        check(LIB.b2_ctx_set_shard(ctx._h, self.rank, self.world))

    def limbs(self, l):
        out = np.zeros(4, dtype=np.uint32)
        check(LIB.b2_shard_limbs(self.ctx._h, l, out.ctypes.data))
        return tuple(int(x) for x in out)  # q0, nq, p0, np

    def workspace(self, l):
        return self.ctx.workspace(_native.OP_KEYSWITCH, l)

    def phase(self, l, phase, c2, key_table, ct, ws, ws_bytes, stream=None):
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        check(LIB.b2_shard_keyswitch_phase(self.ctx._h, l, phase, c2.data_ptr(), key_table.ctypes.data, len(key_table),
                                           ct.data_ptr(), ws.data_ptr(), ws_bytes, s))

    def keyswitch(self, l, c2, key, ct, ws=None):
        ctx, N, a = self.ctx, self.ctx.N, self.ctx.size_P
        if ws is None:
            ws, ws_bytes = self.workspace(l)
        else:
            ws_bytes = ws.numel() * 8
        tab = key.pointer_table()
        beta, lP = ctx.beta(l), l + a
        t = ws[: l * N].view(l, N)
        cxp = ws[(l + beta * lP) * N: (l + beta * lP + 2 * a) * N].view(2, a, N)
        self.phase(l, 0, c2, tab, ct, ws, ws_bytes)
        allgather_limbs(t, l, self.rank, self.world, self.group)
        self.phase(l, 1, c2, tab, ct, ws, ws_bytes)
        for k in range(2):
            allgather_limbs(cxp[k], a, self.rank, self.world, self.group)
        self.phase(l, 2, c2, tab, ct, ws, ws_bytes)

    def allgather_ct(self, l, ct):
        for k in range(ct.shape[0]):
            allgather_limbs(ct[k], l, self.rank, self.world, self.group)


class BatchedLimbShardedKeySwitch(LimbShardedKeySwitch):
    """A batch of ciphertexts, all switched with one key, with their limbs spread over the ranks.

    c2: [batch][l][N], ct: [batch][2][l][N] (only this rank's limbs need to hold data; only they are updated).
    Every kernel of a phase covers the whole batch in one launch, and each of the two exchanges is ONE all-gather:
    the batch's scaled coefficient-form limbs T [l][batch][N] after phase 0, the P limbs CXP [alpha][2][batch][N]
    after phase 1. `pipeline` runs several batches on alternating streams, each with its own communicator, so one
    batch's all-gathers overlap another's kernels."""

    def batch_workspace(self, l, batch):
        nbytes = int(LIB.b2_shard_batch_workspace_bytes(self.ctx._h, l, batch))
        return torch.empty(nbytes // 8, dtype=torch.int64, device=torch.device("cuda", self.ctx.device)), nbytes

    def _views(self, l, batch, ws):
        N, a = self.ctx.N, self.ctx.size_P
        t = ws[: l * batch * N].view(l, batch * N)
        cxp = ws[l * batch * N: (l + 2 * a) * batch * N].view(a, 2 * batch * N)
        return t, cxp

    def phase_batch(self, l, phase, batch, c2, key_table, ct, ws, ws_bytes, stream=None):
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        check(LIB.b2_shard_keyswitch_phase_batch(self.ctx._h, l, phase, batch, c2.data_ptr(), key_table.ctypes.data, len(key_table),
                                                 ct.data_ptr(), ws.data_ptr(), ws_bytes, s))

    def keyswitch_batch(self, l, c2, key, ct, ws, group=None):
        """the three phases and two all-gathers of one batch, on the current stream"""
        batch = c2.shape[0]
        ws_bytes = ws.numel() * 8
        tab = key.pointer_table()
        t, cxp = self._views(l, batch, ws)
        g = self.group if group is None else group
        self.phase_batch(l, 0, batch, c2, tab, ct, ws, ws_bytes)
        allgather_limbs(t, l, self.rank, self.world, g)
        self.phase_batch(l, 1, batch, c2, tab, ct, ws, ws_bytes)
        allgather_limbs(cxp, self.ctx.size_P, self.rank, self.world, g)
        self.phase_batch(l, 2, batch, c2, tab, ct, ws, ws_bytes)

    def make_lanes(self, n_lanes):
        """(stream, process group) pairs for `pipeline`: every lane has its own communicator, so that collectives of
        different lanes do not queue behind one another. Collective: every rank must call it."""
        ranks = list(range(self.world))
        return [(torch.cuda.Stream(), dist.new_group(ranks) if self.world > 1 else None) for _ in range(n_lanes)]

    def pipeline(self, l, batches, key, lanes, workspaces):
        """batches: list of (c2, ct); batch i runs on lane i % len(lanes) with that lane's workspace. Returns after
        queueing everything; the caller's stream waits for every lane."""
        main = torch.cuda.current_stream()
        for st, _ in lanes:
            st.wait_stream(main)
        for i, (c2, ct) in enumerate(batches):
            st, grp = lanes[i % len(lanes)]
            with torch.cuda.stream(st):
                self.keyswitch_batch(l, c2, key, ct, workspaces[i % len(lanes)], grp)
        for st, _ in lanes:
            main.wait_stream(st)
