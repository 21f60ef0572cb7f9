"""The transformer-layer compositions the reference binds next to its evaluator (python/src/binding.cu:595-724;
src/rmsnorm.cu, src/softmax.cu, src/mlp.cu, src/attention.cu): RMSNorm, the exp / squaring / Goldschmidt pieces of
softmax, the SwiGLU MLP (real and complex-folded) and the two attention products. Every one of them is a sequence of
calls into the evaluator (key switches, rescales, limb arithmetic); nothing here touches a limb on the host.

Same names, arguments, level consumption and error behaviour as the reference. What differs, on purpose:

  * a real constant c at scale q is the integer round(c q) on every limb (one `b2_ct_scalar` launch), not an encoded
    constant vector and a plaintext product; a constant added is one `b2_poly_scalar` launch, not ceil(|c|/0.1) of them;
  * multiplication of the slots by +-i is the monomial +-X^(N/2): exact; the level the reference spends on it is
    dropped without scaling so that the chain indices still agree;
  * the 1/sqrt polynomial of RMSNorm is evaluated in the Chebyshev basis of the interval it was fitted on (the affine
    map onto [-1, 1] rides on the scalar product that forms the mean), never expanded into monomials of z;
  * independent pieces (the K-cache ciphertexts of QK^T, the chunks of score x V, gate / up tracks of the MLP) are
    issued on separate CUDA streams.
"""
import math

import numpy as np
import torch

from . import (_native, add, bsgs_apply_giants_with_babies, compute_bsgs_babies, mod_switch_to, mod_switch_to_next,
               multiply_and_relin, multiply_plain, rescale_to_next, rotate, sub)
from ._native import LIB, check
from .blocks import eval_chebyshev_series, eval_polynomial, inner_sum, schedule_chain_index

MAX_LANES = 3          # side streams next to the caller's
_LANES = {}            # device index -> list of side streams
_FORKED = [False]      # forks do not nest: an inner fork runs in order on its lane


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _is_pow2(v):
    return v != 0 and (v & (v - 1)) == 0


def _record(result, stream):
    if isinstance(result, (list, tuple)):
        for r in result:
            _record(r, stream)
    elif hasattr(result, "data") and isinstance(result.data, torch.Tensor):
        result.data.record_stream(stream)


def _fork(thunks):
    """run independent thunks, dealt round-robin over the caller's stream and up to MAX_LANES side streams; all of
    them have joined the caller's stream when this returns"""
    if len(thunks) < 2 or _FORKED[0]:
        return [t() for t in thunks]
    here = torch.cuda.current_stream()
    pool = _LANES.setdefault(torch.cuda.current_device(), [])
    n_side = min(len(thunks) - 1, MAX_LANES)
    while len(pool) < n_side:
        pool.append(torch.cuda.Stream())
    side = pool[:n_side]
    for s in side:
        s.wait_stream(here)
    results = [None] * len(thunks)
    _FORKED[0] = True
    try:
        for i, t in enumerate(thunks):
            k = i % (n_side + 1)
            if k == 0:
                results[i] = t()
            else:
                with torch.cuda.stream(side[k - 1]):
                    results[i] = t()
                _record(results[i], here)
    finally:
        _FORKED[0] = False
        for s in side:
            here.wait_stream(s)
    return results


def _assign(dst, src):
    dst.__dict__.update(src.__dict__)


def _last_prime(ctx, ct):
    return int(ctx.primes[ct._limbs - 1])


def _scalars(ctx, k, l):
    return np.array([k % int(q) for q in ctx.primes[:l]], dtype=np.uint64)


def _mul_scalar(ctx, ct, c, nominal):
    """ct * c at one level: the constant carries the scale of the prime that the rescale removes
    (mul_scalar_inplace of src/rmsnorm.cu:28-40, src/softmax.cu:52-64)"""
    q = _last_prime(ctx, ct)
    sc = _scalars(ctx, int(round(c * q)), ct._limbs)
    out = torch.empty_like(ct.data)
    check(LIB.b2_ct_scalar(ctx._h, ct._limbs, ct._size, ct.data.data_ptr(), sc.ctypes.data, out.data_ptr(), _stream()))
    r = rescale_to_next(ctx, ct._like(out, scale=ct._scale * float(q)))
    r.set_scale(nominal)
    return r


def _add_scalar(ctx, ct, c):
    """ct + c on every slot (add_scalar_split_inplace, src/rmsnorm.cu:42-56, without the split)"""
    if c == 0.0:
        return ct
    sc = _scalars(ctx, int(round(c * ct._scale)), ct._limbs)
    out = ct.data.clone()
    check(LIB.b2_poly_scalar(ctx._h, 0, ct._limbs, ct.data[0].data_ptr(), sc.ctypes.data, out[0].data_ptr(), _stream()))
    return ct._like(out)


def _times_i(ctx, ct, negate=False):
    """slots times +-i: the monomial +-X^(N/2), kept in NTT form on the context"""
    mono = getattr(ctx, "_mono_i", None)
    if mono is None:
        d = torch.zeros(ctx.N, dtype=torch.int64, device=ctx.device)
        d[ctx.N // 2] = 1
        pos, neg = ctx.empty(ctx.size_Q), ctx.empty(ctx.size_Q)
        check(LIB.b2_expand_signed(ctx._h, 0, ctx.size_Q, d.data_ptr(), pos.data_ptr(), 1, _stream()))
        check(LIB.b2_expand_signed(ctx._h, 0, ctx.size_Q, (-d).data_ptr(), neg.data_ptr(), 1, _stream()))
        torch.cuda.current_stream().synchronize()
        mono = ctx._mono_i = (pos, neg)
    out = torch.empty_like(ct.data)
    check(LIB.b2_ct_op(ctx._h, 2, ct._limbs, ct._size, ct.data.data_ptr(), mono[1 if negate else 0].data_ptr(), out.data_ptr(), _stream()))
    return ct._like(out)


def _mul_relin_rescale(ctx, a, b, rlk, nominal):
    r = rescale_to_next(ctx, multiply_and_relin(ctx, a, b, rlk))
    r.set_scale(nominal)
    return r


# ---- RMSNorm (include/rmsnorm.h, src/rmsnorm.cu) ------------------------------------------------------------------
class rmsnorm_params:
    def __init__(self):
        self.d_model, self.epsilon, self.z_min, self.z_max, self.poly_degree = 0, 0.0, 0.0, 0.0, 0


class rmsnorm_weights:
    def __init__(self, g_tiled_real=(), g=()):
        self._g_tiled_real, self._g = [float(v) for v in g_tiled_real], [float(v) for v in g]

    @property
    def g_tiled_real(self):
        return list(self._g_tiled_real)

    @property
    def g(self):
        return list(self._g)


def _power_fit(z_min, z_max, exponent, degree):
    """Chebyshev interpolant of z^exponent on [z_min, z_max] at degree + 1 Chebyshev nodes, as coefficients of
    T_k(t), t = (2 z - z_min - z_max) / (z_max - z_min) (steps 1-2 of chebyshev_monomial_coeffs_local,
    src/rmsnorm.cu:90-131; its steps 3-4, the expansion into monomials of z, are not needed here)"""
    if z_min <= 0.0:
        raise ValueError("chebyshev_monomial_coeffs: z_min must be positive")
    if z_max <= z_min:
        raise ValueError("chebyshev_monomial_coeffs: z_max must exceed z_min")
    if degree < 1:
        raise ValueError("chebyshev_monomial_coeffs: degree must be >= 1")
    n = degree + 1
    theta = np.pi * (np.arange(n) + 0.5) / n
    z = 0.5 * (z_min + z_max) + 0.5 * (z_max - z_min) * np.cos(theta)
    f = z ** exponent
    c = np.array([np.sum(f * np.cos(k * theta)) for k in range(n)]) * (2.0 / n)
    c[0] *= 0.5
    return c


def rmsnorm_forward(context, encoder, relin_key, galois_key, x, weights, params):
    """x in period-d_model replicated layout -> rmsnorm(x) * g in the same layout (src/rmsnorm.cu:249-296):
    sum of squares over each period, mean + epsilon prescaled by alpha = 1/sqrt(z_min z_max), 1/sqrt by a polynomial
    of degree poly_degree fitted on [alpha z_min, alpha z_max], x * w, times the tiled gain (which already holds
    1/sqrt(sqrt(z_min z_max)))."""
    d_model = int(params.d_model)
    if not _is_pow2(d_model):
        raise ValueError("rmsnorm_forward: d_model must be a power of 2")
    nominal = x.scale()
    # 1: sum of squares, broadcast over each period
    acc = _mul_relin_rescale(context, x, x, relin_key, nominal)
    acc = inner_sum(context, galois_key, acc, d_model)
    # 2 + 3: zp = (alpha/d) sum + alpha eps lives in [zp_min, zp_max]; the polynomial wants t = a zp + b in [-1, 1],
    # so the one scalar product forms t directly
    zgeo = math.sqrt(params.z_min * params.z_max)
    alpha = 1.0 / zgeo
    if abs(alpha * params.epsilon) > 0.5:
        raise ValueError("mean_squares_plus_eps_alpha: |alpha*epsilon| must be <= 0.5")
    if params.z_min <= 0.0:
        raise ValueError("invsqrt_direct_prescaled: z_min must be positive")
    if params.z_max <= params.z_min:
        raise ValueError("invsqrt_direct_prescaled: z_max must exceed z_min")
    if params.poly_degree < 1:
        raise ValueError("invsqrt_direct_prescaled: degree must be >= 1")
    zp_min, zp_max = params.z_min * alpha, params.z_max * alpha
    cheb = _power_fit(zp_min, zp_max, -0.5, int(params.poly_degree))
    a, b = 2.0 / (zp_max - zp_min), -(zp_min + zp_max) / (zp_max - zp_min)
    t = _mul_scalar(context, acc, a * alpha / d_model, nominal)
    t = _add_scalar(context, t, a * alpha * params.epsilon + b)
    w = eval_chebyshev_series(context, relin_key, t, cheb, schedule_chain_index(t, int(params.poly_degree)))
    # 4: x * w
    xw = _mul_relin_rescale(context, mod_switch_to(context, x, w.chain_index()), w, relin_key, nominal)
    # 5: times the tiled gain, encoded at the scale of the prime the rescale removes
    q = float(_last_prime(context, xw))
    g_pt = encoder.encode_double_vector(context, weights.g_tiled_real, q, xw.chain_index())
    out = rescale_to_next(context, multiply_plain(context, xw, g_pt))
    out.set_scale(nominal)
    return out


# ---- softmax pieces (include/softmax.h, src/softmax.cu) -------------------------------------------------------------
def _exp_fit(degree=8):
    """monomial coefficients of the Chebyshev interpolant of exp(y) on [-1, 1] at degree + 1 nodes (the table
    EXP_CHEB_COEFFS_DEG4_R2 of src/softmax.cu:19-29 holds the same fit, written out)"""
    n = degree + 1
    theta = np.pi * (np.arange(n) + 0.5) / n
    f = np.exp(np.cos(theta))
    c = np.array([np.sum(f * np.cos(k * theta)) for k in range(n)]) * (2.0 / n)
    c[0] *= 0.5
    return np.polynomial.chebyshev.cheb2poly(c)


def ps_exp_init(context, encoder, relin_key, scores, num_tokens, num_squarings, extra_scale):
    """extra_scale * T^(-1/2^k) * exp(x / 2^k), k = num_squarings, T = num_tokens (src/softmax.cu:102-141): the
    division by 2^k and the leading factor are folded into the coefficients, so the polynomial runs on the scores
    as they come; valid for |x| <= 2^k"""
    scale_exp = 2.0 ** num_squarings
    lead = extra_scale * float(num_tokens) ** (-1.0 / scale_exp)
    base = _exp_fit()
    coeffs = [lead * base[i] * scale_exp ** (-i) for i in range(base.size)]
    return eval_polynomial(context, encoder, relin_key, scores, coeffs)


def square_iterations_inplace(context, relin_key, ct, num_squarings):
    """src/softmax.cu:143-154"""
    nominal = ct.scale()
    cur = ct
    for _ in range(int(num_squarings)):
        cur = _mul_relin_rescale(context, cur, cur, relin_key, nominal)
    _assign(ct, cur)


def square_iterations_damped_inplace(context, encoder, relin_key, ct, damps):
    """src/softmax.cu:156-171: after every squaring a scalar damps[i] (one more level unless it is 1)"""
    nominal = ct.scale()
    cur = ct
    for d in damps:
        cur = _mul_relin_rescale(context, cur, cur, relin_key, nominal)
        if abs(d - 1.0) > 1e-12:
            cur = _mul_scalar(context, cur, float(d), nominal)
    _assign(ct, cur)


def softmax_correct(context, encoder, relin_key, e_ct, a_ct, iters):
    """joint Goldschmidt steps (x, a) -> (2x - x a, 2a - a a): a -> 1, x -> e / a0 (src/softmax.cu:173-213);
    one level per step"""
    nominal = e_ct.scale()
    x, a = e_ct, a_ct
    for _ in range(int(iters)):
        def step_x(x=x, a=a):
            xa = _mul_relin_rescale(context, x, a, relin_key, nominal)
            return sub(context, mod_switch_to(context, add(context, x, x), xa.chain_index()), xa)

        def step_a(a=a):
            aa = _mul_relin_rescale(context, a, a, relin_key, nominal)
            return sub(context, mod_switch_to(context, add(context, a, a), aa.chain_index()), aa)

        x, a = _fork([step_x, step_a])
    return x


def _sum_reduce_stride(context, galois_key, ct, num_tokens, stride):
    """src/softmax.cu:72-98: sum over num_tokens positions that lie `stride` slots apart"""
    if not _is_pow2(num_tokens):
        raise ValueError("sum_reduce_stride: num_tokens must be a power of 2")
    if stride == 0:
        raise ValueError("sum_reduce_stride: stride must be > 0")
    acc, step, reach = ct, int(stride), 1
    while reach < num_tokens:
        acc = add(context, acc, rotate(context, acc, step, galois_key))
        step <<= 1
        reach <<= 1
    return acc


def finalize_softmax(context, encoder, relin_key, galois_key, e_ct, num_tokens, stride, iters):
    """src/softmax.cu:215-226"""
    a = _sum_reduce_stride(context, galois_key, e_ct, int(num_tokens), int(stride))
    return softmax_correct(context, encoder, relin_key, e_ct, a, iters)


# ---- SwiGLU MLP (include/mlp.h, src/mlp.cu) ---------------------------------------------------------------------
def _silu_fit(degree=8, radius=2.0):
    """monomial coefficients of the Chebyshev interpolant of x * sigmoid(x) on [-radius, radius] at degree + 1 nodes
    (SILU_COEFFS_DEG5_R2 of src/mlp.cu:15-25 holds the same fit, written out)"""
    n = degree + 1
    theta = np.pi * (np.arange(n) + 0.5) / n
    xs = radius * np.cos(theta)
    f = xs / (1.0 + np.exp(-xs))
    c = np.array([np.sum(f * np.cos(k * theta)) for k in range(n)]) * (2.0 / n)
    c[0] *= 0.5
    mono_t = np.polynomial.chebyshev.cheb2poly(c)
    return mono_t * radius ** (-np.arange(n, dtype=np.float64))


def _silu(context, encoder, relin_key, ct):
    return eval_polynomial(context, encoder, relin_key, ct, _silu_fit())


class mlp_weights:
    def __init__(self, w_gate=None, w_up=None, w_down=None):
        self.w_gate, self.w_up, self.w_down = w_gate, w_up, w_down


class mlp_weights_complex:
    def __init__(self, w_gate=None, w_up=None, w_down=None, d_model=0, d_hidden=0, d_pad=0):
        self.w_gate, self.w_up, self.w_down = w_gate, w_up, w_down
        self._d_model, self._d_hidden, self._d_pad = int(d_model), int(d_hidden), int(d_pad)

    d_model = property(lambda self: self._d_model)
    d_hidden = property(lambda self: self._d_hidden)
    d_pad = property(lambda self: self._d_pad)


def mlp_forward(context, encoder, relin_key, galois_key, x, w):
    """W_down (silu(W_gate x) * (W_up x)) (src/mlp.cu:38-70). The gate and up products share the baby rotations of
    x (the reference computes them twice; the ciphertexts are the same)."""
    nominal = x.scale()
    if w.w_gate.baby_steps == w.w_up.baby_steps:
        babies = compute_bsgs_babies(context, galois_key, x, w.w_gate.baby_steps)
        up_babies = babies
    else:
        babies = compute_bsgs_babies(context, galois_key, x, w.w_gate.baby_steps)
        up_babies = compute_bsgs_babies(context, galois_key, x, w.w_up.baby_steps)
    gate = bsgs_apply_giants_with_babies(context, galois_key, babies, w.w_gate)
    up = bsgs_apply_giants_with_babies(context, galois_key, up_babies, w.w_up)
    gate_silu = _silu(context, encoder, relin_key, gate)
    up = mod_switch_to(context, up, gate_silu.chain_index())
    h = _mul_relin_rescale(context, gate_silu, up, relin_key, nominal)
    babies = compute_bsgs_babies(context, galois_key, h, w.w_down.baby_steps)
    return bsgs_apply_giants_with_babies(context, galois_key, babies, w.w_down)


def _half_parts(context, galois_key, z):
    """(re(z), im(z)) of the slots, both real-valued, two levels below z: (z +- conj z)/2 costs one level; the
    imaginary part comes out as i*im and is turned by -i, the level the reference spends on that product
    (extract_real_part_ct, extract_imag_i_form_ct and the (0, -1) product of src/mlp.cu:105-170) is dropped unscaled"""
    nominal = z.scale()
    cj = rotate(context, z, 0, galois_key)
    re = _mul_scalar(context, add(context, z, cj), 0.5, nominal)
    im = _mul_scalar(context, sub(context, z, cj), 0.5, nominal)
    im = mod_switch_to_next(context, _times_i(context, im, negate=True))
    return re, im


def mlp_forward_complex(context, encoder, relin_key, galois_key, x, w):
    """the MLP with complex-folded weights (src/mlp.cu:174-236): gate and up each come out as top + i bottom halves
    of the hidden vector, SiLU and the product run on the real-valued halves, h is packed again as top + i bottom and
    the column-folded W_down returns the full real output"""
    nominal = x.scale()
    babies = compute_bsgs_babies(context, galois_key, x, w.w_gate.inner.baby_steps)
    gate_c = bsgs_apply_giants_with_babies(context, galois_key, babies, w.w_gate.inner)
    up_c = bsgs_apply_giants_with_babies(context, galois_key, babies, w.w_up.inner)
    (gate_top, gate_bot), (up_top, up_bot) = _fork([lambda: _half_parts(context, galois_key, gate_c),
                                                    lambda: _half_parts(context, galois_key, up_c)])

    def track(gate, up):
        s = _silu(context, encoder, relin_key, gate)
        return _mul_relin_rescale(context, s, mod_switch_to(context, up, s.chain_index()), relin_key, nominal)

    h_top, h_bot = _fork([lambda: track(gate_top, up_top), lambda: track(gate_bot, up_bot)])
    h_bot = mod_switch_to_next(context, _times_i(context, h_bot))
    h_top = mod_switch_to(context, h_top, h_bot.chain_index())
    h = add(context, h_top, h_bot)
    babies = compute_bsgs_babies(context, galois_key, h, w.w_down.inner.baby_steps)
    return bsgs_apply_giants_with_babies(context, galois_key, babies, w.w_down.inner)


# ---- attention products (include/attention.h, src/attention.cu) ---------------------------------------------------
def compute_qkt(context, relin_key, galois_key, q, packed_k, d_head):
    """per K-cache ciphertext: q * k, one rescale, sum over each d_head block (src/attention.cu:10-28); slot
    t*d_total + h*d_head of result j holds Q[h] . K[t_j + t][h]"""
    nominal = q.scale()

    def one(k_ct):
        return inner_sum(context, galois_key, _mul_relin_rescale(context, q, k_ct, relin_key, nominal), d_head)

    return _fork([lambda k_ct=k_ct: one(k_ct) for k_ct in packed_k])


def score_times_v(context, relin_key, galois_key, score_cts, v_cts, mask_pt, d_head, d_total, positions_per_ct):
    """sum_t score[t] V[t] (src/attention.cu:30-98): per chunk mask the score slot of every head, spread it over the
    head's d_head slots (rotations by -d_head/2 .. -1), multiply with V, fold the positions of the chunk (rotations by
    d_total, 2 d_total, ..); chunks add up"""
    if len(score_cts) == 0:
        raise ValueError("score_times_v: score_cts is empty")
    if len(score_cts) != len(v_cts):
        raise ValueError("score_times_v: score_cts and v_cts size mismatch")
    if not _is_pow2(d_head):
        raise ValueError("score_times_v: d_head must be a power of 2")
    if not _is_pow2(positions_per_ct):
        raise ValueError("score_times_v: positions_per_ct must be a power of 2")
    nominal = score_cts[0].scale()
    reach = positions_per_ct * d_total

    def chunk(score, v):
        m = rescale_to_next(context, multiply_plain(context, score, mask_pt))
        m.set_scale(nominal)
        b = d_head // 2
        while b >= 1:
            m = add(context, m, rotate(context, m, -b, galois_key))
            b >>= 1
        prod = _mul_relin_rescale(context, m, mod_switch_to(context, v, m.chain_index()), relin_key, nominal)
        stride = d_total
        while stride < reach:
            prod = add(context, prod, rotate(context, prod, stride, galois_key))
            stride <<= 1
        return prod

    parts = _fork([lambda s=s, v=v: chunk(s, v) for s, v in zip(score_cts, v_cts)])
    total = parts[0]
    for p in parts[1:]:
        total = add(context, total, p)
    return total
