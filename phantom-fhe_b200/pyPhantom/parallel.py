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
import ctypes

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


def exchange_block(l, alpha, batch, N, which, rank, world):
    """(offset, size) in bytes of the block of a limb-major batch workspace T [l][batch][N] | CXP [alpha][2][batch][N] | ..
    that `rank` owns in exchange `which` (0: its Q limbs of T, 1: its P limbs of CXP): what it pushes into every peer's
    workspace, and what an all-gather over the same rows would send"""
    limb = N * 8
    first, cnt = limb_range(alpha if which else l, rank, world)
    row = (2 * batch if which else batch) * limb
    base = l * batch * limb if which else 0
    return base + first * row, cnt * row


def pipeline_schedule(n_batches):
    """Issue order of the staggered pipeline as a list of ("phase", batch, p) and ("exchange", batch, which) items: step s queues
    phase 0 of batch s and its first exchange, phase 1 of batch s - 1 and its second exchange, phase 2 of batch s - 3. Phases go
    to the compute stream in this order, exchanges to the communication stream in this order; an exchange waits for the phase
    listed just before it, a phase 1 (2) waits for exchange 0 (1) of its batch. With this order batch i + 4 may reuse the
    workspace of batch i: everything of batch i is queued before phase 0 of batch i + 4."""
    out = []
    for s in range(n_batches + 3):
        if s < n_batches:
            out += [("phase", s, 0), ("exchange", s, 0)]
        if 0 <= s - 1 < n_batches:
            out += [("phase", s - 1, 1), ("exchange", s - 1, 1)]
        if 0 <= s - 3 < n_batches:
            out.append(("phase", s - 3, 2))
    return out


class PeerWorkspace:
    """A batch workspace of the limb-sharded pipeline that the other ranks of the node can write into: device memory with a
    CUDA IPC handle (b2_peer_alloc) and, after `connect`, every peer's mapping of its own. `push` copies a block of this
    rank's buffer to the same offset of every peer's with plain asynchronous copies (DMA over NVLink: no SM, so they run
    beside the kernels of other batches). Collective: every rank creates and connects the same number of them in the same
    order."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        p, h = ctypes.c_void_p(), (ctypes.c_uint8 * 64)()
        check(LIB.b2_peer_alloc(self.nbytes, ctypes.byref(p), h))
        self.ptr, self.handle = int(p.value), bytes(h)
        self.peers = None  # device addresses of every rank's buffer as mapped into this process (own one included)

    def data_ptr(self):
        return self.ptr

    def numel(self):
        return self.nbytes // 8

    def connect(self, rank, world, group=None):
        handles = [None] * world
        dist.all_gather_object(handles, self.handle, group=group)
        self.peers = []
        for r, h in enumerate(handles):
            if r == rank:
                self.peers.append(self.ptr)
            else:
                p = ctypes.c_void_p()
                check(LIB.b2_peer_open((ctypes.c_uint8 * 64).from_buffer_copy(h), ctypes.byref(p)))
                self.peers.append(int(p.value))
        self.rank = rank
        return self

    def push(self, offset_bytes, nbytes, stream=None):
        """this rank's bytes [offset, offset + nbytes) into every peer's buffer at the same offset, ordered after the work
        queued on the current stream and before what is queued on it next. One copy per peer, spread over a few side streams
        so that several copy engines drive the links at once (one stream of seven copies in a row reached 210 GB/s on eight
        B200s)."""
        if not nbytes or len(self.peers) < 2:
            return
        cur = torch.cuda.current_stream()
        if len(self.peers) == 2:
            r = 1 - self.rank
            check(LIB.b2_peer_copy(self.peers[r] + offset_bytes, self.ptr + offset_bytes, nbytes, cur.cuda_stream))
            return
        if not hasattr(self, "_side"):
            self._side = [torch.cuda.Stream() for _ in range(min(len(self.peers) - 1, 4))]
        start = torch.cuda.Event()
        start.record(cur)
        others = [(self.rank + 1 + k) % len(self.peers) for k in range(len(self.peers) - 1)]  # start with the next rank: no hot spot
        for k, r in enumerate(others):
            st = self._side[k % len(self._side)]
            if k < len(self._side):
                st.wait_event(start)
            check(LIB.b2_peer_copy(self.peers[r] + offset_bytes, self.ptr + offset_bytes, nbytes, st.cuda_stream))
        for st in self._side:
            done = torch.cuda.Event()
            done.record(st)
            cur.wait_event(done)

    def close(self):
        if self.peers:
            for r, base in enumerate(self.peers):
                if r != self.rank:
                    LIB.b2_peer_close(base)
            self.peers = None
        if self.ptr:
            LIB.b2_peer_free(self.ptr)
            self.ptr = 0


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

    def peer_workspaces(self, l, batch, count):
        """`count` batch workspaces whose exchange blocks the peers push into directly (`pipeline` then needs no all-gather
        kernel); None when the ranks cannot map one another's memory (the caller falls back to `batch_workspace`).
        Collective: every rank must call it."""
        nbytes = int(LIB.b2_shard_batch_workspace_bytes(self.ctx._h, l, batch))
        made, ok = [], 1
        try:
            for _ in range(count):
                made.append(PeerWorkspace(nbytes))
        except ValueError:
            ok = 0
        flag = torch.tensor([ok], device=torch.device("cuda", self.ctx.device))
        if self.world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) != 1:
            for w in made:
                w.close()
            return None
        try:
            for w in made:
                w.connect(self.rank, self.world, self.group)
            ok = 1
        except ValueError:
            ok = 0
        flag.fill_(ok)
        if self.world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) != 1:
            for w in made:
                w.close()
            return None
        return made

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
        import os
        pri = -1 if os.environ.get("B2_SHARD_COMM_PRIORITY", "1") == "1" else 0
        return [(torch.cuda.Stream(priority=pri), dist.new_group(ranks) if self.world > 1 else None) for _ in range(n_lanes)]

    def exchange(self, l, batch, ws, which, group=None):
        """One exchange of a batch on the current stream. which = 0: the scaled coefficient-form limbs T [l][batch][N] after
        phase 0; 1: the P limbs CXP [alpha][2][batch][N] after phase 1. A tensor workspace goes through one NCCL all-gather; a
        PeerWorkspace pushes this rank's block into every peer's buffer with asynchronous copies and then joins a one-word
        all-reduce: a rank queues its copies before its contribution, so when the reduction completes here every peer's block
        has landed, and the kernels that read the blocks are ordered after it."""
        a = self.ctx.size_P
        if not isinstance(ws, PeerWorkspace):
            return allgather_limbs(self._views(l, batch, ws)[which], a if which else l, self.rank, self.world, group)
        ws.push(*exchange_block(l, a, batch, self.ctx.N, which, self.rank, self.world))
        if self.world > 1:
            if not hasattr(self, "_xflag"):
                self._xflag = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", self.ctx.device))
            dist.all_reduce(self._xflag, group=group)

    def pipeline_lanes(self, l, batches, key, lanes, workspaces):
        """batches: list of (c2, ct); batch i runs on lane i % len(lanes) with that lane's workspace. Returns after
        queueing everything; the caller's stream waits for every lane. (The lanes start in step and stay in step - all
        of them compute, then all of them exchange - so this form hides little of the exchanges; `pipeline` staggers.)"""
        if isinstance(workspaces[0], PeerWorkspace):
            raise ValueError("peer workspaces go with the staggered pipeline: pass four or more")
        main = torch.cuda.current_stream()
        for st, _ in lanes:
            st.wait_stream(main)
        for i, (c2, ct) in enumerate(batches):
            st, grp = lanes[i % len(lanes)]
            with torch.cuda.stream(st):
                self.keyswitch_batch(l, c2, key, ct, workspaces[i % len(lanes)], grp)
        for st, _ in lanes:
            main.wait_stream(st)

    def pipeline(self, l, batches, key, lanes, workspaces):
        """Software pipeline over the batches: all kernels go to the caller's stream in the order
        phase 0 of batch s, phase 1 of batch s - 1, phase 2 of batch s - 3 (s = 0, 1, ..), and the two exchanges of a batch go
        to the communication lane (lanes[0]: a stream and its communicator) as soon as the phase that feeds them is queued.
        An exchange thus has the kernels of the neighbouring batches to hide behind - the first one phases 1 and 2 of other
        batches, the second one two steps' worth - instead of every lane exchanging at the same moment. Batch i uses
        workspace i % len(workspaces); four or more workspaces are needed (three batches are in flight), else the lanes form
        is used. Returns after queueing everything; the caller's stream has waited for the last exchange."""
        D = len(workspaces)
        if D < 4 or len(batches) < 2:
            return self.pipeline_lanes(l, batches, key, lanes, workspaces)
        cs = torch.cuda.current_stream()
        ms, grp = lanes[0]
        ms.wait_stream(cs)
        NB = len(batches)
        tab = key.pointer_table()
        LB = batches[0][0].shape[0]
        ev_p0 = [torch.cuda.Event() for _ in range(NB)]
        ev_p1 = [torch.cuda.Event() for _ in range(NB)]
        ev_x1 = [torch.cuda.Event() for _ in range(NB)]
        ev_x2 = [torch.cuda.Event() for _ in range(NB)]

        def exchange(i, which):
            self.exchange(l, LB, workspaces[i % D], which, grp)

        def phase(i, ph):
            c2, ct = batches[i]
            w = workspaces[i % D]
            self.phase_batch(l, ph, c2.shape[0], c2, tab, ct, w, w.numel() * 8)

        waits = {1: ev_x1, 2: ev_x2}       # phase p waits for the exchange that feeds it
        after = {0: (ev_p0, ev_x1), 1: (ev_p1, ev_x2)}
        for kind, i, p in pipeline_schedule(NB):
            if kind == "phase":
                if p in waits:
                    cs.wait_event(waits[p][i])
                phase(i, p)
                if p in after:
                    after[p][0][i].record(cs)
            else:
                with torch.cuda.stream(ms):
                    ms.wait_event(after[p][0][i])
                    exchange(i, p)
                    after[p][1][i].record(ms)
        cs.wait_stream(ms)
