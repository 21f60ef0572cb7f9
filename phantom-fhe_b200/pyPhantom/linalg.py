"""Plaintext-matrix times ciphertext with the diagonals resident in HBM (no counterpart in the reference).

The reference's bsgs_matmul_preencoded (src/bsgs.cu:194-367, mirrored by pyPhantom.bsgs_matmul_preencoded) keeps
every diagonal as one int64 tower on the host and, for every giant step of every product, copies M of them to the
device and expands and transforms them again; its babies are a chain of dependent rotations and its giants a Horner
chain of dependent rotations. On a GPU with 180 GB of HBM the expanded diagonals of a 4096 x 4096 matrix at 16 limbs
(32 GB) simply stay resident, and the product becomes:

  babies   rot(x, b), b = 1 .. M-1     one hoisted call per stream (one ModUp each)
  partials sum_b pt[g][b] * baby_b      four giants per launch, every baby read once per launch
  giants   sum_g rot(partial_g, g*M)    independent, dealt over the streams, one ModDown per stream
  one rescale, scale reset to the input's

It needs a Galois key for every baby step 1..M-1 and every giant step M, 2M, .. (G-1)M (the "64 + 64 keys" form);
the result decrypts to the same product as the reference's driver but is not limb-identical to it (hoisted babies).
"""
import numpy as np
import torch

from . import _native, get_elt_from_step, rescale_to_next
from ._native import LIB, check

LANES = 3


def _stream():
    return torch.cuda.current_stream().cuda_stream


class resident_bsgs:
    def __init__(self, context, galois_key_, diags, chain_index):
        ctx = self.ctx = context
        self.M, self.G, self.d_pad = diags.baby_steps, diags.giant_steps, diags.d_pad
        if self.M * self.G != self.d_pad or len(diags.diagonals) != self.d_pad:
            raise ValueError("resident_bsgs: M*G must equal d_pad and every diagonal must be present")
        self.chain_index, self.l = chain_index, ctx.limbs_at(chain_index)
        self.pt_scale = diags.diagonals[0].scale
        l, N, M, G = self.l, ctx.N, self.M, self.G
        # expand every diagonal once: [d_pad][l][N], NTT form
        self.pts = ctx.empty(self.d_pad, l)
        for d, scp in enumerate(diags.diagonals):
            if scp.coeffs.numel() != N:
                raise ValueError("resident_bsgs: scp coeff length != N")
            stage = scp.coeffs.to(ctx.device, non_blocking=True)
            check(LIB.b2_expand_single_chain(ctx._h, l, stage.data_ptr(), self.pts[d].data_ptr(), _stream()))
        # keys by step
        self.keys = {}
        for s in list(range(1, M)) + [g * M for g in range(1, G)]:
            e = get_elt_from_step(s, N)
            if e not in ctx.galois_elts:
                raise ValueError(f"resident_bsgs: no Galois element for step {s} in the context")
            k = galois_key_.resolve(ctx.galois_elts.index(e))
            if k is None:
                raise ValueError(f"resident_bsgs: no Galois key for step {s}")
            self.keys[s] = (e, k)
        self.baby_buf = ctx.empty(M, 2, l)
        self.part_buf = ctx.empty(G, 2, l)
        self.baby_tab = torch.tensor([self.baby_buf[b].data_ptr() for b in range(M)], dtype=torch.int64, device=ctx.device)
        # giants 1..G-1 in LANES contiguous shares, each in launches of <= 4; giant 0 (no rotation) rides with lane 0
        order = list(range(1, G)) + [0]
        n_lanes = max(1, min(LANES, len(order)))
        share = -(-len(order) // n_lanes)
        self.lane_groups = []
        for k in range(n_lanes):
            mine, groups = order[k * share: (k + 1) * share], []
            for g0 in range(0, len(mine), 4):
                chunk = mine[g0: g0 + 4]
                tab = np.array([[self.pts[g * M + b].data_ptr() for b in range(M)] for g in chunk], dtype=np.int64)
                outs = [self.part_buf[g].data_ptr() for g in chunk]
                groups.append((chunk, torch.from_numpy(tab.ravel().copy()).to(ctx.device),
                               torch.tensor(outs, dtype=torch.int64, device=ctx.device)))
            self.lane_groups.append(groups)
        self.streams = [torch.cuda.Stream() for _ in range(n_lanes - 1)]
        torch.cuda.synchronize()

    def apply(self, x):
        ctx, l, N, M = self.ctx, self.l, self.ctx.N, self.M
        if x._chain_index != self.chain_index or x._size != 2:
            raise ValueError("resident_bsgs: the ciphertext is not at the level the diagonals were expanded for")
        main = torch.cuda.current_stream()
        lanes = [main] + self.streams
        n_evk = ctx.beta(l)
        self.baby_buf[0].copy_(x.data)
        for st in lanes[1:]:
            st.wait_stream(main)
        # babies: every lane hoists its share of the steps 1..M-1
        steps = list(range(1, M))
        for k, lane in enumerate(lanes):
            mine = steps[k::len(lanes)]
            if not mine:
                continue
            with torch.cuda.stream(lane):
                elts = np.array([self.keys[s][0] for s in mine], dtype=np.uint32)
                ksk = np.concatenate([self.keys[s][1].pointer_table()[:n_evk] for s in mine]).astype(np.uint64)
                outs = np.array([self.baby_buf[s].data_ptr() for s in mine], dtype=np.uint64)
                ws, nbytes = ctx.workspace(_native.OP_HOIST, l)
                check(LIB.b2_hoist_rotations(ctx._h, l, x.data.data_ptr(), elts.ctypes.data, len(mine), ksk.ctypes.data, n_evk,
                                             outs.ctypes.data, ws.data_ptr(), nbytes, _stream()))
        for st in lanes[1:]:
            main.wait_stream(st)
        for st in lanes[1:]:
            st.wait_stream(main)
        # partial sums and giant rotations per lane, one ModDown per lane
        a = ctx.size_P
        accs, plain = [None] * len(lanes), None
        for k, groups in enumerate(self.lane_groups):
            with torch.cuda.stream(lanes[k]):
                st = _stream()
                for chunk, ptab, otab in groups:
                    check(LIB.b2_bsgs_mac_multi(ctx._h, l, M, len(chunk), ptab.data_ptr(), self.baby_tab.data_ptr(), otab.data_ptr(), st))
                    for g in chunk:
                        part = self.part_buf[g]
                        if g == 0:
                            plain = (k, part)
                            continue
                        first = accs[k] is None
                        if first:
                            accs[k] = (ctx.empty(2, l), ctx.empty(2, a), ctx.workspace(_native.OP_ROTATE, l))
                        acc, accP, (ws, nbytes) = accs[k]
                        e, key = self.keys[g * M]
                        ktab = key.pointer_table()
                        check(LIB.b2_apply_galois_accumulate(ctx._h, l, e, part.data_ptr(), ktab.ctypes.data, n_evk, acc.data_ptr(),
                                                             accP.data_ptr(), 1 if first else 0, ws.data_ptr(), nbytes, st))
                if accs[k] is not None:
                    acc, accP, (ws, nbytes) = accs[k]
                    check(LIB.b2_keyswitch_finish(ctx._h, l, accP.data_ptr(), acc.data_ptr(), ws.data_ptr(), nbytes, st))
        total = ctx.empty(2, l)
        first = True
        for k, lane in enumerate(lanes[: len(self.lane_groups)]):
            if k:
                main.wait_stream(lane)
            pieces = []
            if accs[k] is not None:
                pieces.append(accs[k][0])
                if k:
                    accs[k][0].record_stream(main)
            if plain is not None and plain[0] == k:
                pieces.append(plain[1])
            for p in pieces:
                if first:
                    total.copy_(p)
                    first = False
                else:
                    check(LIB.b2_ct_op(ctx._h, 0, l, 2, total.data_ptr(), p.data_ptr(), total.data_ptr(), _stream()))
        out = rescale_to_next(ctx, x._like(total, scale=x._scale * self.pt_scale))
        out.set_scale(x._scale)
        return out
