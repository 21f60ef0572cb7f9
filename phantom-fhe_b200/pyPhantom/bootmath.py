"""Host mathematics of CKKS bootstrapping: numpy only, no device work.

What the reference builds on the host for the same purpose (src/bootstrap.cu:271-434, butterfly
factors collapsed into layers of diagonals; src/evalmod.cu:76-112, Chebyshev coefficients of the
scaled cosine) - restated here from the published algorithms, in a form the device pipeline and the
CPU tests share:

* the "special" FFT over the rotation group 5^j (the CKKS embedding), one radix-2 stage at a time,
  each stage written as three generalised diagonals;
* composition of consecutive stages into layers and a baby-step/giant-step plan per layer;
* Chebyshev interpolation of a_0 cos((2 pi K u - pi/2) / 2^r) and a Paterson-Stockmeyer evaluator
  in the Chebyshev basis that is generic over the arithmetic (`ops`), so that the same recursion
  runs on floats in the CPU tests and on ciphertexts on the device.

Slot convention: rot(x, r)[p] = x[(p + r) mod n], the effect of `rotate(ct, r)` on the slots.
A linear map in diagonal form is {r: d_r} with  (A x)[p] = sum_r d_r[p] * x[(p + r) mod n].
"""
import math

import numpy as np


# ---- the special FFT as stages of diagonals -------------------------------------------------------
def rot_group(n):
    m = 4 * n
    out, g = np.empty(n, dtype=np.int64), 1
    for j in range(n):
        out[j] = g
        g = (g * 5) % m
    return out


def bit_reverse_perm(n):
    bits = n.bit_length() - 1
    idx = np.arange(n)
    rev = np.zeros(n, dtype=np.int64)
    for b in range(bits):
        rev |= ((idx >> b) & 1) << (bits - 1 - b)
    return rev


def embedding_matrix(n):
    """U0[j][k] = zeta^(5^j k), zeta = exp(2 pi i / 4n): slots = U0 (m_lo + i m_hi)"""
    return np.exp(2j * np.pi * np.outer(rot_group(n), np.arange(n)) / (4 * n))


def stage_diagonals(n, ln, inverse):
    """one radix-2 stage of block length ln (2 <= ln <= n) as {offset: diagonal}.

    forward (decimation in time, input bit-reversed):  lower: x[p] + w_j x[p+h];  upper: x[p-h] - w_j x[p]
    inverse (decimation in frequency, output bit-reversed): lower: x[p] + x[p+h];  upper: w'_j (x[p-h] - x[p])
    with h = ln/2, j = p mod h, w_j = exp(2 pi i (5^j mod 4 ln) / (4 ln)), w'_j = conj(w_j)."""
    h, lenq = ln >> 1, ln << 2
    j = np.arange(n) % h
    upper = (np.arange(n) % ln) >= h
    e = (rot_group(n)[:h] % lenq)[j]
    w = np.exp(2j * np.pi * e / lenq)
    if inverse:
        w = np.conj(w)
        d0 = np.where(upper, -w, 1.0)
        dp = np.where(upper, 0.0, 1.0)
        dm = np.where(upper, w, 0.0)
    else:
        d0 = np.where(upper, -w, 1.0)
        dp = np.where(upper, 0.0, w)
        dm = np.where(upper, 1.0, 0.0)
    out = {}
    for r, d in ((0, d0), (h % n, dp), ((-h) % n, dm)):
        out[r] = out.get(r, 0) + d.astype(np.complex128)
    return out


def compose(a, b, n):
    """diagonal form of x -> A(B x)"""
    out = {}
    for ra, da in a.items():
        for rb, db in b.items():
            r = (ra + rb) % n
            term = da * np.roll(db, -ra)
            out[r] = out[r] + term if r in out else term
    return out


def apply_diagonals(diags, x):
    n = len(x)
    out = np.zeros(n, dtype=np.complex128)
    for r, d in diags.items():
        out += d * np.roll(x, -r)
    return out


def fft_layers(n, stages_per_layer, inverse):
    """the log2(n) stages grouped into len(stages_per_layer) layers, in order of application.

    inverse: block lengths n, n/2, ..., 2 (no final bit reversal, no 1/n);
    forward: block lengths 2, 4, ..., n (expects bit-reversed input).
    The composition is  P U0^H  (inverse) or  U0 P  (forward), P the bit-reversal permutation."""
    logn = n.bit_length() - 1
    if sum(stages_per_layer) != logn:
        raise ValueError("stages_per_layer must sum to log2(slots)")
    lens = [n >> s for s in range(logn)] if inverse else [2 << s for s in range(logn)]
    layers, at = [], 0
    for cnt in stages_per_layer:
        acc = None
        for ln in lens[at: at + cnt]:
            st = stage_diagonals(n, ln, inverse)
            acc = st if acc is None else compose(st, acc, n)
        layers.append({r: d for r, d in acc.items() if np.any(d != 0)})
        at += cnt
    return layers


def split_stages(logn, n_layers):
    """stages per layer, larger groups first: 15 -> [5,5,5] / [8,7]; 11 -> [4,4,3] / [6,5]"""
    base, extra = divmod(logn, n_layers)
    return [base + (1 if i < extra else 0) for i in range(n_layers)]


# ---- baby-step / giant-step plan of one layer ----------------------------------------------------------
class LayerPlan:
    """diagonals at offsets k*unit, k = g*n1 + b (0 <= b < n1): out = sum_g rot( sum_b pt[g][b] * rot(x, b*unit), g*n1*unit )
    with pt[g][b] = rot(d_k, -g*n1*unit) - the pre-rotation that lets the giant rotation act last."""

    def __init__(self, diags, n, n1=None):
        offs = sorted(diags)
        self.n = n
        nz = [r for r in offs if r]
        unit = 0
        for r in nz:
            unit = math.gcd(unit, r)
        unit = math.gcd(unit, n) if unit else 1
        self.unit = unit
        span = n // unit
        ks = []
        for r in offs:
            k = r // unit
            if len(offs) < span and k > span // 2:
                k -= span  # a layer that does not wrap: signed indices keep the giant steps few
            ks.append(k)
        if n1 is None:
            # baby rotations share one ModUp (hoisting) and cost about two thirds of a giant rotation: lean to babies
            n1 = 1 << max(1, math.ceil(math.log2(math.sqrt(max(len(ks), 4)))))
        self.n1 = n1
        self.terms = {}  # g -> [(b, diagonal pre-rotated)]
        for r, k in zip(offs, ks):
            g, b = divmod(k, n1)  # floor division: b in [0, n1) also for negative k
            shift = (g * n1 * unit) % n
            self.terms.setdefault(g, []).append((b, np.roll(diags[r], shift)))
        self.babies = sorted({b for t in self.terms.values() for b, _ in t})
        self.giants = sorted(self.terms)

    def baby_steps(self):
        return [(b * self.unit) % self.n for b in self.babies if b]

    def giant_steps(self):
        return [(g * self.n1 * self.unit) % self.n for g in self.giants if g]

    def apply(self, x):
        """the plan on a plain vector (what the device pipeline does on ciphertexts)"""
        rots = {b: np.roll(x, -((b * self.unit) % self.n)) for b in self.babies}
        out = np.zeros(self.n, dtype=np.complex128)
        for g in self.giants:
            part = np.zeros(self.n, dtype=np.complex128)
            for b, d in self.terms[g]:
                part += d * rots[b]
            out += np.roll(part, -((g * self.n1 * self.unit) % self.n))
        return out


def required_rotation_steps(log_n, c2s_stages, s2c_stages):
    """every slot rotation the two linear transforms use (bootstrap_required_galois_elts,
    python/src/binding.cu:301-318, adds the conjugation element to these)"""
    n = 1 << (log_n - 1)
    steps = set()
    for stages, inverse in ((c2s_stages, True), (s2c_stages, False)):
        for layer in fft_layers(n, stages, inverse):
            plan = LayerPlan(layer, n)
            steps.update(plan.baby_steps())
            steps.update(plan.giant_steps())
    return sorted(steps)


# ---- EvalRound: u -> the integer part of K u through a scaled cosine -----------------------------------
def cosine_chebyshev(K, r, degree):
    """Chebyshev coefficients on [-1, 1] of a_0 cos((2 pi K u - pi/2) / 2^r), a_0 = (2 pi)^(-1/2^r).

    r double-angle steps D <- 2 D^2 - a_j, a_j = a_{j-1}^2, turn it into sin(2 pi K u) / (2 pi)
    (the scaled double-angle recurrence of src/evalmod.cu:604-618)."""
    a0 = (2.0 * math.pi) ** (-1.0 / (1 << r))
    f = lambda u: a0 * np.cos((2.0 * math.pi * K * u - math.pi / 2.0) / (1 << r))
    return np.polynomial.chebyshev.chebinterpolate(f, degree), a0


def cheb_divide(c, g):
    """p = q T_g + r for deg p <= 2g, all in the Chebyshev basis: T_{g+j} = 2 T_j T_g - T_{g-j}"""
    d = len(c) - 1
    if not g <= d <= 2 * g:
        raise ValueError("cheb_divide needs g <= deg <= 2g")
    q = np.zeros(d - g + 1)
    r = np.array(c[:g], dtype=np.float64)
    q[0] = c[g]
    for j in range(1, d - g + 1):
        q[j] = 2.0 * c[g + j]
        r[g - j] -= c[g + j]
    return q, r


class ChebyshevEvaluator:
    """Paterson-Stockmeyer evaluation of sum_i c_i T_i(u) with exact scale bookkeeping.

    `ops` supplies the arithmetic on values that carry (level, scale): level = number of RNS limbs,
    rescale goes from `level` to `level - 1` and divides the scale by ops.prime(level). Products are
    relinearised by ops.mul and rescaled here; constants enter as integers round(c * const_scale), so
    every sum is between operands of equal level whose scales agree to about 2^-52."""

    def __init__(self, ops, u, babies=8, tight=False):
        """tight: T_m also serves in the leaves and the giants stop below the degree, so that a polynomial of degree
        2^k m (not only 2^k m - 1) fits k giants, and the output level is the smallest the coefficients allow"""
        self.ops, self.m, self.tight = ops, babies, tight
        self.T = {1: u}
        self.giants = None

    def match(self, x, level, scale, ops=None):
        """bring x down to (level, scale): free if it is already there, else one integer multiply and rescale"""
        ops = ops or self.ops
        if ops.level(x) == level:
            if abs(ops.scale(x) / scale - 1.0) > 2.0 ** -40:
                raise ValueError("operand already at the target level with a different scale")
            return x
        if ops.level(x) < level:
            raise ValueError("operand is below the target level")
        x = ops.drop(x, level + 1)
        x = ops.mul_const(x, 1.0, scale * ops.prime(level + 1) / ops.scale(x))
        return ops.rescale(x)

    def _power(self, k, ops):
        """T_k from T_ceil(k/2), T_floor(k/2), both already there: 2 T_a T_b - T_(a-b), a - b in {0, 1}"""
        a, b = (k + 1) // 2, k // 2
        xa, xb = self.T[a], self.T[b]
        lvl = min(ops.level(xa), ops.level(xb))
        prod = ops.mul(ops.drop(xa, lvl), ops.drop(xb, lvl))
        prod = ops.rescale(ops.add(prod, prod))
        if a == b:
            return ops.add_const(prod, -1.0)
        return ops.sub(prod, self.match(self.T[1], ops.level(prod), ops.scale(prod), ops))

    def prepare(self, degree):
        """T_2 .. T_(m-1) and the giants T_m, T_2m, ...: powers of equal depth ceil(log2 k) only need shallower ones,
        so each depth is one fork (independent work the arithmetic may spread over streams)"""
        if getattr(self, "giants", None) is not None:
            return
        g, giants = self.m, []
        while g < degree or (g == degree and not self.tight):
            giants.append(g)
            g *= 2
        top = min(self.m, degree) + 1 if self.tight else min(self.m, degree + 1)
        need = sorted(set(range(2, top)) | set(giants))
        by_depth = {}
        for k in need:
            by_depth.setdefault((k - 1).bit_length(), []).append(k)
        for depth in sorted(by_depth):
            ks = by_depth[depth]
            outs = self.ops.fork([(lambda o, k=k: self._power(k, o)) for k in ks])
            for k, v in zip(ks, outs):
                self.T[k] = v
        self.giants = giants

    def _leaf(self, c, level, scale, ops):
        up = level + 1
        target = scale * ops.prime(up)
        if hasattr(ops, "lincomb"):  # one fused launch where the arithmetic has it
            terms = [(self.T[i], float(c[i]), target / ops.scale(self.T[i])) for i in range(1, len(c)) if c[i] != 0.0]
            if terms:
                return ops.rescale(ops.lincomb(terms, float(c[0]), up, target))
        acc = None
        for i in range(1, len(c)):
            if c[i] == 0.0 and not (acc is None and i == len(c) - 1):
                continue
            x = ops.drop(self.T[i], up)
            term = ops.mul_const(x, float(c[i]), target / ops.scale(x))
            acc = term if acc is None else ops.add(acc, term)
        if acc is None:  # a bare constant: carry it on 0 * T_1
            x = ops.drop(self.T[1], up)
            acc = ops.mul_const(x, 0.0, target / ops.scale(x))
        acc = ops.add_const(acc, float(c[0]))
        return ops.rescale(acc)

    def _eval(self, c, level, scale, ops=None):
        ops = ops or self.ops
        c = np.asarray(c, dtype=np.float64)
        d = len(c) - 1
        while d > 0 and c[d] == 0.0:
            d -= 1
        c = c[: d + 1]
        if d < self.m or (self.tight and d == self.m):
            return self._leaf(c, level, scale, ops)
        g = max(x for x in self.giants if x <= d)
        q, r = cheb_divide(c, g)
        tg = ops.drop(self.T[g], level + 1)
        q_scale = scale * ops.prime(level + 1) / ops.scale(tg)
        # quotient and remainder are independent until the final sum
        qv, rv = ops.fork([lambda o: self._eval(q, level + 1, q_scale, o), lambda o: self._eval(r, level, scale, o)])
        prod = ops.rescale(ops.mul(qv, tg))
        return ops.add(prod, rv)

    def _depth(self, c):
        """levels below T_1 that _eval needs for these coefficients (a dry run of its recursion)"""
        ops = self.ops
        c = np.asarray(c, dtype=np.float64)
        d = len(c) - 1
        while d > 0 and c[d] == 0.0:
            d -= 1
        c = c[: d + 1]
        top = ops.level(self.T[1])
        if d < self.m or (self.tight and d == self.m):
            return 1 + max([top - ops.level(self.T[i]) for i in range(1, d + 1) if c[i] != 0.0], default=0)
        g = max(x for x in self.giants if x <= d)
        q, r = cheb_divide(c, g)
        return max(max(self._depth(q), top - ops.level(self.T[g])) + 1, self._depth(r))

    def evaluate(self, coeffs, scale):
        """-> value at level (input level - depth) whose scale is `scale` to about 2^-50"""
        degree = len(coeffs) - 1
        self.prepare(degree)
        ops = self.ops
        if self.tight:
            return self._eval(coeffs, ops.level(self.T[1]) - self._depth(coeffs), scale)
        lb = min(ops.level(self.T[k]) for k in range(1, min(self.m, degree + 1)))
        out_level = lb - 1 - len(self.giants)
        return self._eval(coeffs, out_level, scale)


def eval_round(ops, u, K, r, degree, out_scale, babies=8):
    """u (slots t / (q0 K), |u| <= 1) -> K u - sin(2 pi K u) / (2 pi): the integer part of K u wherever K u
    is close to an integer, flat to second order around it (so errors of u do not pass through)."""
    coeffs, a = cosine_chebyshev(K, r, degree)
    ev = ChebyshevEvaluator(ops, u, babies)
    # every double-angle step squares the scale and divides by one prime: start so that it ends at out_scale
    lvl_poly = None
    ev.prepare(degree)
    lb = min(ops.level(ev.T[k]) for k in range(1, min(babies, degree + 1)))
    lvl_poly = lb - 1 - len(ev.giants)
    s = out_scale
    for j in range(r):  # walk back from the last squaring: s_j = sqrt(s_{j+1} * prime)
        s = math.sqrt(s * ops.prime(lvl_poly - (r - 1 - j)))
    D = ev._eval(coeffs, lvl_poly, s)
    for _ in range(r):
        a = a * a
        sq = ops.mul(D, D)
        D = ops.add_const(ops.rescale(ops.add(sq, sq)), -a)
    Ku = ev.match(ops.with_scale(u, ops.scale(u) / K), ops.level(D), ops.scale(D))
    return ops.sub(Ku, D)


class FloatOps:
    """the `ops` protocol on plain numpy values: an (array, level, scale) triple stands for the integers
    array * scale, so that a scale mismatch in an addition shows up as the error it would cause."""

    class V:
        __slots__ = ("v", "level", "scale")

        def __init__(self, v, level, scale):
            self.v, self.level, self.scale = v, level, scale

    def __init__(self, primes):
        self.primes = [int(p) for p in primes]
        self.muls = 0

    def prime(self, level):
        return float(self.primes[level - 1])

    def fork(self, thunks):
        """independent pieces of work, each given the arithmetic to use: here simply one after the other"""
        return [t(self) for t in thunks]

    def level(self, x):
        return x.level

    def scale(self, x):
        return x.scale

    def with_scale(self, x, s):
        return self.V(x.v * (x.scale / s), x.level, s)

    def drop(self, x, level):
        if level > x.level:
            raise ValueError("cannot raise a level")
        return self.V(x.v, level, x.scale)

    def mul(self, x, y):
        assert x.level == y.level
        self.muls += 1
        return self.V(x.v * y.v, x.level, x.scale * y.scale)

    def rescale(self, x):
        if x.level < 2:
            raise ValueError("out of levels")
        return self.V(x.v, x.level - 1, x.scale / self.prime(x.level))

    def mul_const(self, x, c, const_scale):
        k = float(round(c * const_scale))
        return self.V(x.v * (k / const_scale), x.level, x.scale * const_scale)

    def add(self, x, y):
        assert x.level == y.level
        return self.V(x.v + y.v * (y.scale / x.scale), x.level, x.scale)

    def sub(self, x, y):
        assert x.level == y.level
        return self.V(x.v - y.v * (y.scale / x.scale), x.level, x.scale)

    def add_const(self, x, c):
        return self.V(x.v + round(c * x.scale) / x.scale, x.level, x.scale)
