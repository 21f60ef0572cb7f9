"""CKKS bootstrapping as a host composition over the C ABI (python/src/binding.cu:292-336;
src/bootstrap.cu:1702-1949, src/evalmod.cu).

Same surface as the reference - bootstrap_required_galois_elts, create_bootstrap_key, bootstrap -
and the same overall route: key switch to a sparse secret, raise the modulus, CoeffToSlot as layered
BSGS linear transforms, EvalRound on the real and imaginary halves, SlotToCoeff, and a final
subtraction  ct_raised - q0 * I  that leaves the message on the user levels. The linear transforms
and the polynomial evaluation are this library's own arrangement (see bootmath.py):

* the top three primes carry CoeffToSlot (three layers; they may be short primes, because EvalRound
  is flat around the integers and does not pass CoeffToSlot's rounding errors on);
* the next ten carry EvalRound: a degree-63 Chebyshev cosine by Paterson-Stockmeyer (7 levels) and
  three double-angle steps;
* the next two carry SlotToCoeff in two layers, whose last plaintext scale is chosen so that the
  result is q0 * I to the last bit that double precision can place.

Every ciphertext operation below is a call into the C ABI; numpy is used for the diagonals, the
Chebyshev coefficients and the scale bookkeeping only.
"""
import math

import numpy as np
import torch

from . import _native, bootmath
from ._native import LIB, check

C2S_LAYERS, EVAL_LEVELS, S2C_LAYERS = 3, 10, 2
BOOT_LEVELS = C2S_LAYERS + EVAL_LEVELS + S2C_LAYERS
K_RANGE, DOUBLE_ANGLES, COS_DEGREE = 28, 3, 63
SCALE_UP_MARGIN_BITS = 10  # the raised message stays below q0 / 2^10
GIANT_LANES = 3            # streams the giant steps of a linear transform are dealt over
FORK_LANES = 6             # extra streams shared by the two EvalRound tracks for their independent pieces


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _elt(step, N):
    return int(LIB.b2_galois_elt_from_step(int(step), N))


def bootstrap_required_galois_elts(log_n, stages_per_layer=(5, 5, 5)):
    """python/src/binding.cu:301-318: Galois elements of every rotation CoeffToSlot and SlotToCoeff use,
    plus the conjugation 2N - 1. `stages_per_layer` is CoeffToSlot's grouping of the log2(N/2) radix-2
    stages; SlotToCoeff always runs in two layers. On chains with short CoeffToSlot primes the key runs CoeffToSlot
    in two layers as well (see create_bootstrap_key), whatever the grouping given here: the list covers both."""
    N = 1 << log_n
    stages = list(stages_per_layer)
    if sum(stages) != log_n - 1:
        stages = bootmath.split_stages(log_n - 1, C2S_LAYERS)
    two = bootmath.split_stages(log_n - 1, S2C_LAYERS)
    steps = set(bootmath.required_rotation_steps(log_n, stages, two))
    steps.update(bootmath.required_rotation_steps(log_n, stages if len(stages) == 2 else two, two))
    return [_elt(s, N) for s in sorted(steps)] + [2 * N - 1]


# ---- arithmetic on ciphertexts with (level, scale) bookkeeping: the `ops` of bootmath ---------------------
class CtOps:
    def __init__(self, ctx, rlk, counts=None):
        self.ctx, self.rlk = ctx, rlk
        self.counts = {"mul": 0, "rescale": 0} if counts is None else counts
        self.stream = _stream()  # the stream current when the ops object is made: one lookup, not one per call
        self.tab = rlk.pointer_table()
        self.pool = []           # free streams that fork() may use
        self.keep = []           # results that crossed streams during a graph capture (see fork)

    def on_current_stream(self):
        """the same arithmetic bound to whatever stream is current now (shares the counters and the lane pool)"""
        o = CtOps(self.ctx, self.rlk, self.counts)
        o.pool, o.keep = self.pool, self.keep
        return o

    def fork(self, thunks):
        """independent pieces of work: all but the first go to free streams of the pool (if any are left), the first
        runs here; everything joins before this returns. Each thunk gets the arithmetic bound to its stream."""
        pool = self.pool
        here = torch.cuda.current_stream()
        capturing = torch.cuda.is_current_stream_capturing()
        results, lanes = [None] * len(thunks), []
        for i in range(1, len(thunks)):
            if not pool:
                break
            lane = pool.pop()
            lanes.append((i, lane))
            lane.wait_stream(here)
            with torch.cuda.stream(lane):
                results[i] = thunks[i](self.on_current_stream())
        for i, t in enumerate(thunks):
            if results[i] is None:
                results[i] = t(self)
        for i, lane in lanes:
            here.wait_stream(lane)
            if hasattr(results[i], "data"):
                if capturing:
                    # record_stream does nothing for the allocator of a capture: once freed, this block could be
                    # handed to the lane's next user - which may hang off another stream, unordered with the reads
                    # that follow here. Keep it allocated until the whole pipeline has been issued.
                    self.keep.append(results[i])
                else:
                    results[i].data.record_stream(here)
            pool.append(lane)
        return results

    def prime(self, level):
        return float(self.ctx.primes[level - 1])

    def level(self, x):
        return x._limbs

    def scale(self, x):
        return x._scale

    def with_scale(self, x, s):
        return x._like(x.data, scale=float(s))

    def drop(self, x, level):
        if level == x._limbs:
            return x
        if level > x._limbs:
            raise ValueError("cannot raise a level")
        return x._like(x.data[:, :level].contiguous(), chain_index=x._chain_index + (x._limbs - level))

    def mul(self, x, y):
        ctx, l = self.ctx, x._limbs
        if y._limbs != l:
            raise ValueError("operands at different levels")
        out = ctx.empty(2, l)
        ws, nbytes = ctx.workspace(_native.OP_MUL_RELIN, l)
        tab = self.tab
        check(LIB.b2_multiply_and_relin(ctx._h, l, x.data.data_ptr(), y.data.data_ptr(), tab.ctypes.data, len(tab),
                                        out.data_ptr(), ws.data_ptr(), nbytes, self.stream))
        self.counts["mul"] += 1
        return x._like(out, scale=x._scale * y._scale)

    def rescale(self, x):
        ctx, l = self.ctx, x._limbs
        if l < 2:
            raise ValueError("out of levels")
        out = ctx.empty(x._size, l - 1)
        ws, nbytes = ctx.workspace(_native.OP_RESCALE, l)
        check(LIB.b2_rescale_rounded(ctx._h, l, x._size, x.data.data_ptr(), out.data_ptr(), ws.data_ptr(), nbytes, self.stream))
        self.counts["rescale"] += 1
        return x._like(out, chain_index=x._chain_index + 1, scale=x._scale / self.prime(l))

    def _scalars(self, k, l):
        return np.array([k % int(q) for q in self.ctx.primes[:l]], dtype=np.uint64)

    def mul_const(self, x, c, const_scale):
        k = int(round(c * const_scale))
        sc = self._scalars(k, x._limbs)
        out = torch.empty_like(x.data)
        check(LIB.b2_ct_scalar(self.ctx._h, x._limbs, x._size, x.data.data_ptr(), sc.ctypes.data, out.data_ptr(), self.stream))
        return x._like(out, scale=x._scale * const_scale)

    def lincomb(self, terms, c0, level, scale):
        """sum_i round(c_i * s_i) * x_i + round(c0 * scale) at `level`; x_i may sit higher, every x_i.scale * s_i ~ scale"""
        n = len(terms)
        if n > 8 or level > 32:
            acc = None
            for x, c, cs in terms:
                t = self.mul_const(self.drop(x, level), c, cs)
                acc = t if acc is None else self.add(acc, t)
            return self.add_const(acc, c0)
        ptrs = np.array([x.data.data_ptr() for x, _, _ in terms], dtype=np.uint64)
        limbs = np.array([x._limbs for x, _, _ in terms], dtype=np.uint32)
        sc = np.concatenate([self._scalars(int(round(c * cs)), level) for _, c, cs in terms])
        c0v = self._scalars(int(round(c0 * scale)), level)
        x0 = terms[0][0]
        out = self.ctx.empty(x0._size, level)
        check(LIB.b2_ct_lincomb(self.ctx._h, level, x0._size, n, ptrs.ctypes.data, limbs.ctypes.data, sc.ctypes.data, c0v.ctypes.data,
                                out.data_ptr(), self.stream))
        return x0._like(out, chain_index=x0._chain_index + (x0._limbs - level), scale=scale)

    def add_const(self, x, c):
        sc = self._scalars(int(round(c * x._scale)), x._limbs)
        out = x.data.clone()
        check(LIB.b2_poly_scalar(self.ctx._h, 0, x._limbs, x.data[0].data_ptr(), sc.ctypes.data, out[0].data_ptr(), self.stream))
        return x._like(out)

    def _lin(self, op, x, y):
        if x._limbs != y._limbs or x._size != y._size:
            raise ValueError("operands at different levels")
        if abs(x._scale / y._scale - 1.0) > 2.0 ** -40:
            raise ValueError("scale mismatch")
        out = torch.empty_like(x.data)
        check(LIB.b2_ct_op(self.ctx._h, op, x._limbs, x._size, x.data.data_ptr(), y.data.data_ptr(), out.data_ptr(), self.stream))
        return x._like(out)

    def add(self, x, y):
        return self._lin(0, x, y)

    def sub(self, x, y):
        return self._lin(1, x, y)


# ---- one layer of a linear transform, compiled to device plaintexts ----------------------------------------
class _Layer:
    """the LayerPlan of bootmath with every pre-rotated diagonal encoded at (limbs, scale) and resident in HBM"""

    def __init__(self, ctx, encoder, plan, limbs, scale, value_factor=1.0, rescales=1):
        self.limbs, self.scale, self.n = limbs, float(scale), plan.n
        self.rescales = rescales  # primes the layer's plaintext scale spans: that many rescales end the transform
        self.baby_steps = [(b, (b * plan.unit) % plan.n) for b in plan.babies]
        chain_index = ctx.size_Q - limbs + 1
        self.giants = []  # (rotation step, [baby position], device pointer table, plaintext tensors)
        pos = {b: i for i, (b, _) in enumerate(self.baby_steps)}
        for g in plan.giants:
            pts, idx = [], []
            for b, d in plan.terms[g]:
                pts.append(encoder.encode_complex_vector(ctx, d * value_factor, self.scale, chain_index).data)
                idx.append(pos[b])
            tab = torch.tensor([p.data_ptr() for p in pts], dtype=torch.int64, device=ctx.device)
            self.giants.append(((g * plan.n1 * plan.unit) % plan.n, idx, tab, pts))
        # the baby rotations land in buffers owned by the layer, so the pointer tables of the fused
        # multiply-accumulate are built once
        self.baby_buf = ctx.empty(len(self.baby_steps), 2, limbs)
        self.baby_tabs = [torch.tensor([self.baby_buf[i].data_ptr() for i in idx], dtype=torch.int64, device=ctx.device)
                          for _, idx, _, _ in self.giants]

    def steps(self):
        return [s for _, s in self.baby_steps if s] + [s for s, _, _, _ in self.giants if s]


class small_bootstrap_key:
    """the two switching keys of the sparse-secret encapsulation (include/bootstrap.h SmallBootstrapKey)"""

    def __init__(self):
        self.to_sparse = None
        self.to_dense = None


class bootstrap_key:
    def __init__(self):
        self.small = small_bootstrap_key()
        self.relin = None
        self.rot = {}     # slot rotation step -> switching key
        self.conj = None
        self.c2s, self.s2c = [], []
        self._streams = []
        self._fork_streams = None
        self.use_graph = True   # replay a captured CUDA graph per (input limbs, input scale) after the first call
        self._graphs = {}

    def fork_pool(self):
        """streams for the independent sub-computations inside EvalRound (disjoint from side_streams)"""
        if self._fork_streams is None:
            self._fork_streams = [torch.cuda.Stream() for _ in range(FORK_LANES)]
        return list(self._fork_streams)

    def side_streams(self, n):
        while len(self._streams) < n:
            self._streams.append(torch.cuda.Stream())
        return self._streams[:n]
        self.user_limbs = 0
        self.user_scale, self.up_bits, self.down_const, self.final_target = 0.0, 0, 0, 0.0
        self.eval_scale = 0.0
        self.mono_i = None      # NTT form of X^(N/2): multiplication by i on the slots
        self.mono_i_neg = None  # -X^(N/2)


def _key_for_elt(sk, ctx, elt, limbs=0):
    check(LIB.b2_galois_prepare(ctx._h, elt))
    rot = ctx.empty(ctx.size_QP)
    check(LIB.b2_galois_permute(ctx._h, elt, sk.data.data_ptr(), rot.data_ptr(), ctx.size_QP, _stream()))
    # `limbs`: the most limbs any ciphertext has when this key switches it: only that level's digits are generated
    # (the reference's per-level bootstrap keys, src/bootstrap.cu:1040-1158, src/secretkey.cu:400-472)
    return sk._kswitch_key(ctx, rot, ctx.size_Q - limbs + 1 if limbs else 0)


def _configure_scale(ctx, encoder, bk, user_scale):
    """scale_up_for_bootstrap (src/bootstrap.cu:1435-1512): every error of EvalRound comes back multiplied by
    q0 / scale, so a ciphertext at `user_scale` is first raised by 2^up_bits to about q0 / 2^10. The way back costs
    no user level: the raised ciphertext is multiplied by down_const ~ p_x / 2^up_bits and rescaled by p_x (the prime
    just above the user levels), and the last SlotToCoeff layer is encoded at the scale that makes the transform
    deliver q0 * I * down_const / p_x to the last bit double precision can place. Re-run when the scale changes."""
    plan, s2c_top, pa, pb = bk._s2c_last
    q0 = float(ctx.primes[0])
    bk.user_scale = float(user_scale) if user_scale and user_scale > 0 else 0.0
    bk.up_bits = max(0, int(math.floor(math.log2(q0 / bk.user_scale))) - SCALE_UP_MARGIN_BITS) if bk.user_scale else 0
    p_x = int(ctx.primes[bk.user_limbs])
    bk.down_const = int(round(p_x / 2.0 ** bk.up_bits)) if bk.up_bits else 0
    bk.final_target = q0 * (bk.down_const / p_x) if bk.up_bits else q0
    e1 = bk.final_target * pa * pb / (bk.eval_scale * pa)
    bk.s2c[1] = _Layer(ctx, encoder, plan, s2c_top - 1, e1)
    bk._graphs = {}


def create_bootstrap_key(context, encoder, dense_sk, sparse_hamming_weight=128, eval_mod_levels=0, user_scale=0.0,
                         split_scale_down=False, stages_per_layer=None):
    """python/src/binding.cu:320-327; src/bootstrap.cu:895-1199.

    The chain must hold q0, at least one user level and BOOT_LEVELS = 15 further primes above them.
    `eval_mod_levels` is accepted for compatibility (the reference spends 9 levels on EvalMod and 3 on
    SlotToCoeff, this pipeline 10 and 2: the same 12 primes)."""
    from .keys import secret_key
    ctx = context
    if eval_mod_levels not in (0, 9, EVAL_LEVELS):
        raise ValueError("eval_mod_levels: this pipeline uses the 12 primes below CoeffToSlot as 10 + 2")
    if ctx.size_Q < BOOT_LEVELS + 2:
        raise ValueError("the modulus chain is too short for bootstrapping")
    N, n, sQ = ctx.N, ctx.N // 2, ctx.size_Q
    logn = n.bit_length() - 1
    bk = bootstrap_key()
    bk.user_limbs = sQ - BOOT_LEVELS
    # sparse-secret encapsulation: s -> s' at the bottom prime, s' -> s at the top (src/bootstrap.cu:183-216)
    sparse = secret_key(seed=None)
    sparse._rng, sparse._rng_pub = dense_sk._rng, dense_sk._rng_pub
    sparse.generate_sparse(ctx, sparse_hamming_weight)
    bk.small.to_sparse = sparse._kswitch_key(ctx, dense_sk.data)
    bk.small.to_dense = dense_sk._kswitch_key(ctx, sparse.data)
    bk.relin = dense_sk.gen_relinkey(ctx)
    # linear transforms
    q0 = float(ctx.primes[0])
    eval_top = sQ - C2S_LAYERS                     # limbs at EvalRound's input
    bk.eval_scale = float(ctx.primes[eval_top - 1])
    # CoeffToSlot: slots of the raised ciphertext read at scale q0*K are t/(q0 K); the unnormalised inverse
    # FFT multiplies by n and the real/imaginary split wants another 1/2: that factor, eval_scale / (2 n q0 K) (about
    # 2^-21 at N = 2^16), has to come out of the plaintext scales, i.e. out of the bits the three primes provide.
    sigma0 = q0 * K_RANGE
    whole = bk.eval_scale / (2.0 * n * sigma0)
    wide = float(ctx.primes[sQ - 1]) * float(ctx.primes[sQ - 2]) * whole
    user_split = list(stages_per_layer) if stages_per_layer and sum(stages_per_layer) == logn else None
    if (user_split is None or len(user_split) == 2) and wide < 2.0 ** 60:
        # Short CoeffToSlot primes (the reference's chains give it three 29-bit ones): three even layers would encode
        # their diagonals with (87 - 21) / 3 = 22 bits each, and the 2e-6 error that leaves in u = t/(q0 K) is what
        # EvalRound's second-order terms turn into most of the bootstrap's final error. Two layers instead: the first
        # spends two primes (plaintext scale p p' 2^-21, about 2^37, two rescales), the second the third prime at
        # its full 29 bits - 2^-27 in u, at the price of more diagonals per layer.
        c2s_stages = user_split or bootmath.split_stages(logn, 2)
        la, lb = bootmath.fft_layers(n, c2s_stages, True)
        bk.c2s.append(_Layer(ctx, encoder, bootmath.LayerPlan(la, n), sQ, wide, rescales=2))
        bk.c2s.append(_Layer(ctx, encoder, bootmath.LayerPlan(lb, n), sQ - 2, float(ctx.primes[sQ - 3])))
    else:
        c2s_stages = user_split if user_split and len(user_split) == C2S_LAYERS else bootmath.split_stages(logn, C2S_LAYERS)
        ratio = whole ** (1.0 / C2S_LAYERS)
        for i, layer in enumerate(bootmath.fft_layers(n, c2s_stages, True)):
            limbs = sQ - i
            bk.c2s.append(_Layer(ctx, encoder, bootmath.LayerPlan(layer, n), limbs, float(ctx.primes[limbs - 1]) * ratio))
    s2c_stages = bootmath.split_stages(logn, S2C_LAYERS)
    # SlotToCoeff: the first layer at its own prime; the scale of the last one depends on the caller's scale
    # (see _configure_scale), so its plan is kept for re-encoding
    s2c_top = eval_top - EVAL_LEVELS
    layers = bootmath.fft_layers(n, s2c_stages, False)
    pa, pb = float(ctx.primes[s2c_top - 1]), float(ctx.primes[s2c_top - 2])
    bk._s2c_last = (bootmath.LayerPlan(layers[1], n), s2c_top, pa, pb)
    bk.s2c.append(_Layer(ctx, encoder, bootmath.LayerPlan(layers[0], n), s2c_top, pa))
    bk.s2c.append(None)
    _configure_scale(ctx, encoder, bk, user_scale)
    # rotation keys
    # one key per rotation step, generated once at the shallowest level that uses it and shared by the deeper layers
    need = {}
    for layer in bk.c2s + bk.s2c:
        for s in layer.steps():
            need[s] = max(need.get(s, 0), layer.limbs)
    for s in sorted(need):
        bk.rot[s] = _key_for_elt(dense_sk, ctx, _elt(s, N), need[s])
    bk.conj = _key_for_elt(dense_sk, ctx, 2 * N - 1, eval_top)
    bk.key_bytes = sum(k.device_bytes() for k in bk.rot.values()) + bk.conj.device_bytes() + bk.relin.device_bytes()
    mono = np.zeros(N, dtype=np.int64)
    mono[N // 2] = 1
    d = torch.from_numpy(mono).to(ctx.device)
    bk.mono_i, bk.mono_i_neg = ctx.empty(sQ), ctx.empty(sQ)
    check(LIB.b2_expand_signed(ctx._h, 0, sQ, d.data_ptr(), bk.mono_i.data_ptr(), 1, _stream()))
    check(LIB.b2_expand_signed(ctx._h, 0, sQ, (-d).data_ptr(), bk.mono_i_neg.data_ptr(), 1, _stream()))
    torch.cuda.synchronize()
    return bk


# ---- the pipeline --------------------------------------------------------------------------------------------
def _keyswitch_c1(ctx, ct, key):
    """(c0, c1) under one secret -> (c0 + ks0, ks1) under the other"""
    l = ct._limbs
    out = torch.stack([ct.data[0], torch.zeros_like(ct.data[1])])
    ws, nbytes = ctx.workspace(_native.OP_KEYSWITCH, l)
    tab = key.pointer_table()
    check(LIB.b2_keyswitch(ctx._h, l, ct.data[1].data_ptr(), tab.ctypes.data, len(tab), out.data_ptr(), ws.data_ptr(), nbytes, _stream()))
    return ct._like(out)


def _galois(ctx, ct, elt, key):
    l = ct._limbs
    out = ctx.empty(2, l)
    ws, nbytes = ctx.workspace(_native.OP_ROTATE, l)
    tab = key.pointer_table()
    check(LIB.b2_apply_galois(ctx._h, l, int(elt), ct.data.data_ptr(), tab.ctypes.data, len(tab), out.data_ptr(), ws.data_ptr(), nbytes, _stream()))
    return ct._like(out)


def mod_raise(ctx, bk, ct):
    """src/bootstrap.cu:105-216: a ciphertext on q0 alone -> the same c0 + c1 s = t over every Q prime, where
    now t = scale*m + q0*I with |I| bounded by the sparse secret's weight"""
    if ct._limbs != 1:
        raise ValueError("mod_raise wants a ciphertext on the bottom prime only")
    sQ, N = ctx.size_Q, ctx.N
    x = _keyswitch_c1(ctx, ct, bk.small.to_sparse)
    coeff = x.data.clone()
    for p in range(2):
        check(LIB.b2_ntt_inverse(ctx._h, coeff[p].data_ptr(), 1, 0, _stream()))
    q0 = int(ctx.primes[0])
    centred = torch.where(coeff > q0 // 2, coeff - q0, coeff)  # residues of one 58-bit prime fit int64
    out = ctx.empty(2, sQ)
    for p in range(2):
        check(LIB.b2_expand_signed(ctx._h, 0, sQ, centred[p, 0].data_ptr(), out[p].data_ptr(), 1, _stream()))
    raised = ct._like(out, chain_index=1)
    return _keyswitch_c1(ctx, raised, bk.small.to_dense)


def linear_transform(ctx, bk, ct, layer, ops):
    """one BSGS layer: hoisted baby rotations, a fused multiply-accumulate per giant, giant rotations, one rescale
    (src/bootstrap.cu:1201-1353 does the same with one key switch per baby)"""
    ct = ops.drop(ct, layer.limbs)
    l, N = layer.limbs, ctx.N
    steps = [(i, s) for i, (_, s) in enumerate(layer.baby_steps) if s]
    for i, (_, s) in enumerate(layer.baby_steps):
        if s == 0:
            layer.baby_buf[i].copy_(ct.data)
    main = torch.cuda.current_stream()
    lanes = [main] + bk.side_streams(GIANT_LANES - 1)
    for st in lanes[1:]:
        st.wait_stream(main)
    if steps:
        # the babies are independent too: each lane hoists its share (its own ModUp of c1 - cheaper than waiting
        # for the other lanes' steps, since one lane alone leaves most of the GPU idle at these sizes)
        n_evk = ctx.beta(l)
        n_lanes = min(len(lanes), max(1, len(steps) // 2))
        for k in range(n_lanes):
            mine = steps[k::n_lanes]
            with torch.cuda.stream(lanes[k]):
                elts = np.array([_elt(s, N) for _, s in mine], dtype=np.uint32)
                ksk = np.concatenate([bk.rot[s].pointer_table()[:n_evk] for _, s in mine]).astype(np.uint64)
                outs = np.array([layer.baby_buf[i].data_ptr() for i, _ in mine], dtype=np.uint64)
                ws, nbytes = ctx.workspace(_native.OP_HOIST, l)
                check(LIB.b2_hoist_rotations(ctx._h, l, ct.data.data_ptr(), elts.ctypes.data, len(mine), ksk.ctypes.data, n_evk,
                                             outs.ctypes.data, ws.data_ptr(), nbytes, _stream()))
        for st in lanes[1:n_lanes]:   # every giant reads every baby: join, then fork again
            main.wait_stream(st)
        for st in lanes[1:]:
            st.wait_stream(main)
    # the giants are independent until the final sum: deal them round-robin over the key's streams
    # Giants on one lane are summed anyway, so they share one ModDown: every rotation adds its Q limbs to the lane's
    # ciphertext accumulator and its P limbs to accP, and b2_keyswitch_finish converts the P limbs once per lane.
    capturing = torch.cuda.is_current_stream_capturing()
    a = ctx.size_P
    accs, plain = [None] * len(lanes), None
    n_evk = ctx.beta(l)
    for gi, ((step, idx, tab, _), btab) in enumerate(zip(layer.giants, layer.baby_tabs)):
        k = gi % len(lanes)
        with torch.cuda.stream(lanes[k]):
            st = _stream()
            part = ctx.empty(2, l)
            check(LIB.b2_bsgs_mac(ctx._h, l, len(idx), tab.data_ptr(), btab.data_ptr(), part.data_ptr(), st))
            if not step:
                plain = (k, part)  # the giant without rotation
                continue
            first = accs[k] is None
            if first:
                accs[k] = (ctx.empty(2, l), ctx.empty(2, a), ctx.workspace(_native.OP_ROTATE, l))
            acc, accP, (ws, nbytes) = accs[k]
            ktab = bk.rot[step].pointer_table()
            check(LIB.b2_apply_galois_accumulate(ctx._h, l, _elt(step, N), part.data_ptr(), ktab.ctypes.data, n_evk, acc.data_ptr(),
                                                 accP.data_ptr(), 1 if first else 0, ws.data_ptr(), nbytes, st))
    total = None
    for k, lane in enumerate(lanes):
        if accs[k] is None:
            continue
        acc, accP, (ws, nbytes) = accs[k]
        with torch.cuda.stream(lane):
            check(LIB.b2_keyswitch_finish(ctx._h, l, accP.data_ptr(), acc.data_ptr(), ws.data_ptr(), nbytes, _stream()))
        if k:
            main.wait_stream(lane)
            if not capturing:
                acc.record_stream(main)
        piece = ct._like(acc, scale=ct._scale * layer.scale)
        total = piece if total is None else ops.add(total, piece)
    if plain is not None:
        k, part = plain
        if k:
            main.wait_stream(lanes[k])
            if not capturing:
                part.record_stream(main)
        piece = ct._like(part, scale=ct._scale * layer.scale)
        total = piece if total is None else ops.add(total, piece)
    for _ in range(layer.rescales):
        total = ops.rescale(total)
    return total


def _times_i(ctx, bk, ct, negate=False):
    """multiply the slots by i (or -i): the monomial X^(N/2), exact and free of levels (shift_poly_N2_kernel,
    src/bootstrap.cu:76-98, does it in coefficient form)"""
    l = ct._limbs
    out = torch.empty_like(ct.data)
    mono = bk.mono_i_neg if negate else bk.mono_i
    check(LIB.b2_ct_op(ctx._h, 2, l, 2, ct.data.data_ptr(), mono.data_ptr(), out.data_ptr(), _stream()))
    return ct._like(out)


def coeff_to_slot(ctx, bk, raised, ops):
    """-> (u_lo, u_hi): slots t_k / (q0 K) and t_(k+N/2) / (q0 K) in bit-reversed order, at bk.eval_scale"""
    x = ops.with_scale(raised, float(ctx.primes[0]) * K_RANGE)
    for layer in bk.c2s:
        x = linear_transform(ctx, bk, x, layer, ops)
    x = ops.with_scale(x, x._scale * 2.0 * layer.n)  # the same integers read as w/2, w = (t_lo + i t_hi)/(q0 K)
    xc = _galois(ctx, x, 2 * ctx.N - 1, bk.conj)
    return ops.add(x, xc), _times_i(ctx, bk, ops.sub(x, xc), negate=True)


def slot_to_coeff(ctx, bk, lo, hi, ops):
    x = ops.add(lo, _times_i(ctx, bk, hi))
    for layer in bk.s2c:
        x = linear_transform(ctx, bk, x, layer, ops)
    return x


def _eval_round_pair(ops, bk, lo, hi):
    """the real and the imaginary track are independent: the second one runs on a side stream, with its own
    scratch (everything it allocates belongs to that stream), and joins before SlotToCoeff"""
    main = torch.cuda.current_stream()
    side = bk.side_streams(1)[0]
    side.wait_stream(main)
    with torch.cuda.stream(side):
        b = bootmath.eval_round(ops.on_current_stream(), hi, K_RANGE, DOUBLE_ANGLES, COS_DEGREE, bk.eval_scale)
    a = bootmath.eval_round(ops, lo, K_RANGE, DOUBLE_ANGLES, COS_DEGREE, bk.eval_scale)
    main.wait_stream(side)
    if not torch.cuda.is_current_stream_capturing():
        for t in (b.data, hi.data):
            t.record_stream(main)
    return a, b


def bootstrap(context, encoder, ct, bk, user_scale, split_scale_down=False, stats=None):
    """python/src/binding.cu:329-336; src/bootstrap.cu:1702-1949: see bootstrap_eager for the pipeline. The
    sequence of launches depends only on the input's level and scale, so after one eager run (which also
    warms every lazily built table) the whole pipeline is captured into a CUDA graph - its streams become
    parallel branches - and later calls copy the input into the graph's buffer and replay it."""
    if not bk.use_graph or stats is not None or torch.cuda.is_current_stream_capturing():
        return bootstrap_eager(context, encoder, ct, bk, user_scale, split_scale_down, stats)
    key = (ct._limbs, ct._chain_index, ct._scale, ct._size, bool(split_scale_down), torch.cuda.current_device())
    entry = bk._graphs.get(key)
    if entry is None:
        out = bootstrap_eager(context, encoder, ct, bk, user_scale, split_scale_down)
        bk._graphs[key] = "warm"
        return out
    if entry == "warm":
        static_in = ct._like(ct.data.clone())
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = bootstrap_eager(context, encoder, static_in, bk, user_scale, split_scale_down)
        entry = bk._graphs[key] = (graph, static_in, static_out)
    graph, static_in, static_out = entry
    static_in.data.copy_(ct.data)
    graph.replay()
    return static_out._like(static_out.data.clone())


def bootstrap_eager(context, encoder, ct, bk, user_scale, split_scale_down=False, stats=None):
    """python/src/binding.cu:329-336; src/bootstrap.cu:1702-1949. `ct`: any level, scale about user_scale with
    |message| <= 1 and at least two limbs; returns a ciphertext at the input's scale with bk.user_limbs limbs
    (q0 and every user prime: the reference's "freshest" chain index); with split_scale_down one limb fewer, where the
    reference's split mode returns."""
    ctx = context
    if ct._size != 2 or not ct._is_ntt_form:
        raise ValueError("bootstrap wants a 2-polynomial ciphertext in NTT form")
    ops = CtOps(ctx, bk.relin)
    ops.pool = bk.fork_pool()
    scale_in = ct._scale
    x = ct
    if bk.user_scale == 0.0 or abs(scale_in / bk.user_scale - 1.0) > 2.0 ** -20:
        _configure_scale(ctx, encoder, bk, scale_in)  # first use at this scale: re-encode the last SlotToCoeff layer
    if bk.up_bits:
        if x._limbs < 2:
            raise ValueError("bootstrap wants the prime above q0 still present (two limbs or more)")
        x = ops.rescale(ops.mul_const(ops.drop(x, 2), 1.0, ops.prime(2) * 2.0 ** bk.up_bits))
    raised = mod_raise(ctx, bk, ops.drop(x, 1))
    lo, hi = coeff_to_slot(ctx, bk, raised, ops)
    ints = _eval_round_pair(ops, bk, lo, hi)
    qi = slot_to_coeff(ctx, bk, ints[0], ints[1], ops)  # the integers q0 * I (times down_const / p_x) in the coefficients
    if bk.up_bits:
        out = ops.rescale(ops.mul_const(ops.drop(raised, qi._limbs + 1), 1.0, float(bk.down_const)))
    else:
        out = ops.drop(raised, qi._limbs)
    res = torch.empty_like(out.data)
    check(LIB.b2_ct_op(ctx._h, 1, out._limbs, 2, out.data.data_ptr(), qi.data.data_ptr(), res.data_ptr(), _stream()))
    if stats is not None:
        stats.update(ops.counts)
        stats["final_scale_over_target"] = qi._scale / bk.final_target
        stats["raised_scale_log2"] = math.log2(x._scale)
    out = out._like(res, scale=scale_in)
    if split_scale_down:
        # the reference's split mode gives up the top user prime for precision (src/ckks_engine.cu:563-566); this
        # pipeline has that precision already, so the flag only selects where the result is handed over
        out = out._like(out.data[:, : out._limbs - 1].contiguous(), chain_index=out._chain_index + 1)
    return out
