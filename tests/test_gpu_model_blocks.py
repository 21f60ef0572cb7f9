"""The transformer-layer compositions (RMSNorm, softmax pieces, SwiGLU MLP real and complex-folded, the attention
products) against numpy, with the layouts, parameter bands and tolerances of the reference's own block tests
(python/llm_project/blocks/rmsnorm_test.py, softmax_test.py, mlp_test.py, mlp_complex_test.py, sdpa_test.py)
on a smaller ring."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ph = pytest.importorskip("pyPhantom")

N = 1 << 12
SLOTS = N // 2
SCALE = 2.0 ** 40


@pytest.fixture(scope="module")
def kit():
    steps = sorted({s for k in range(11) for s in (1 << k, -(1 << k))} | {3, 0})
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(N)
    parms.set_coeff_modulus(ph.create_coeff_modulus(N, [60] + [40] * 14 + [60] * 3))
    parms.set_special_modulus_size(3)
    parms.set_galois_elts(sorted(set(ph.get_elts_from_steps(steps, N))))
    ctx = ph.context(parms)
    sk = ph.secret_key(ctx, seed=99)
    enc = ph.ckks_encoder(ctx)
    return dict(ctx=ctx, sk=sk, enc=enc, rlk=sk.gen_relinkey(ctx), glk=sk.create_galois_keys(ctx))


def _enc(kit, v, chain=1):
    return kit["sk"].encrypt_symmetric(kit["ctx"], kit["enc"].encode_double_vector(kit["ctx"], v, SCALE, chain))


def _dec(kit, ct):
    return np.asarray(kit["enc"].decode_complex_vector(kit["ctx"], kit["sk"].decrypt(kit["ctx"], ct)))


def test_rmsnorm_forward(kit):
    ctx, enc = kit["ctx"], kit["enc"]
    d_model = 16
    rng = np.random.default_rng(5)
    x, g = rng.uniform(-0.5, 0.5, d_model), rng.uniform(0.5, 1.5, d_model)
    p = ph.rmsnorm_params()
    p.d_model, p.epsilon, p.z_min, p.z_max, p.poly_degree = d_model, 1e-5, 0.05, 0.15, 8
    zgeo = math.sqrt(p.z_min * p.z_max)
    w = ph.rmsnorm_weights(np.tile(g / math.sqrt(zgeo), SLOTS // d_model), g)
    assert len(w.g_tiled_real) == SLOTS and len(w.g) == d_model
    cx = _enc(kit, np.tile(x, SLOTS // d_model))
    y = ph.rmsnorm_forward(ctx, enc, kit["rlk"], kit["glk"], cx, w, p)
    # 1 square + 1 scalar + (m + l - 2 = 4 for degree 8) + 1 product + 1 gain
    assert y.chain_index() == 1 + 8 and y.scale() == SCALE
    got = _dec(kit, y)[:d_model].real
    want = x / math.sqrt(np.mean(x * x) + p.epsilon) * g
    assert np.max(np.abs(got - want)) < 1e-3          # python/llm_project/blocks/rmsnorm_test.py:21
    assert np.max(np.abs(_dec(kit, y)[SLOTS - d_model:].real - want)) < 1e-3
    p.d_model = 12
    with pytest.raises(ValueError, match="power of 2"):
        ph.rmsnorm_forward(ctx, enc, kit["rlk"], kit["glk"], cx, w, p)
    p.d_model, p.z_max = 16, 0.01
    with pytest.raises(ValueError, match="z_max must exceed z_min"):
        ph.rmsnorm_forward(ctx, enc, kit["rlk"], kit["glk"], cx, w, p)


def test_softmax_pipeline(kit):
    ctx, enc, rlk, glk = kit["ctx"], kit["enc"], kit["rlk"], kit["glk"]
    tokens, stride, k, iters = 8, SLOTS // 8, 2, 4
    rng = np.random.default_rng(6)
    x = rng.uniform(-1.0, 0.5, SLOTS)
    cx = _enc(kit, x)
    e = ph.ps_exp_init(ctx, enc, rlk, cx, tokens, k, 1.0)
    assert e.chain_index() == 1 + 4 and e.scale() == SCALE
    assert np.max(np.abs(_dec(kit, e).real - tokens ** (-1 / 2 ** k) * np.exp(x / 2 ** k))) < 1e-6
    ph.square_iterations_inplace(ctx, rlk, e, k)
    assert e.chain_index() == 1 + 4 + k
    assert np.max(np.abs(_dec(kit, e).real - np.exp(x) / tokens)) < 1e-5
    out = ph.finalize_softmax(ctx, enc, rlk, glk, e, tokens, stride, iters)
    assert out.chain_index() == 1 + 4 + k + iters and out.scale() == SCALE
    ex = np.exp(x).reshape(tokens, stride)
    # the recurrence itself (tight) and the softmax it converges to (as far as 4 steps go from |1 - a| <= 0.65)
    xs, a = ex / tokens, np.tile(ex.sum(0) / tokens, (tokens, 1))
    for _ in range(iters):
        xs, a = 2 * xs - xs * a, 2 * a - a * a
    got = _dec(kit, out).real.reshape(tokens, stride)
    assert np.max(np.abs(got - xs)) < 1e-4
    assert np.max(np.abs(got - ex / ex.sum(0))) < 5e-3
    # damped squarings: a level more for every factor that is not 1
    e2 = ph.ps_exp_init(ctx, enc, rlk, cx, tokens, k, 1.0)
    ph.square_iterations_damped_inplace(ctx, enc, rlk, e2, [0.5, 1.0])
    assert e2.chain_index() == 1 + 4 + 3
    assert np.max(np.abs(_dec(kit, e2).real - (0.5 * (tokens ** -0.25 * np.exp(x / 4)) ** 2) ** 2)) < 1e-5
    with pytest.raises(ValueError, match="power of 2"):
        ph.finalize_softmax(ctx, enc, rlk, glk, e, 6, stride, 1)


def _silu(v):
    return v / (1.0 + np.exp(-v))


def test_mlp_forward_real_and_complex(kit):
    ctx, enc, rlk, glk = kit["ctx"], kit["enc"], kit["rlk"], kit["glk"]
    d_model, d_hidden, M = 8, 16, 4
    rng = np.random.default_rng(8)
    Wg, Wu = rng.uniform(-0.4, 0.4, (d_hidden, d_model)), rng.uniform(-0.4, 0.4, (d_hidden, d_model))
    Wd = rng.uniform(-0.4, 0.4, (d_model, d_hidden))
    x = rng.uniform(-0.5, 0.5, d_model)
    want = Wd @ (_silu(Wg @ x) * (Wu @ x))
    # real: d_pad covers d_hidden
    d_pad = 16
    w = ph.mlp_weights(ph.pre_encode_bsgs_diagonals(ctx, enc, Wg.ravel(), d_hidden, d_model, d_pad, M, SCALE),
                       ph.pre_encode_bsgs_diagonals(ctx, enc, Wu.ravel(), d_hidden, d_model, d_pad, M, SCALE),
                       ph.pre_encode_bsgs_diagonals(ctx, enc, Wd.ravel(), d_model, d_hidden, d_pad, M, SCALE))
    xp = np.zeros(d_pad)
    xp[:d_model] = x
    y = ph.mlp_forward(ctx, enc, rlk, glk, _enc(kit, np.tile(xp, SLOTS // d_pad)), w)
    assert y.chain_index() == 1 + 1 + 4 + 1 + 1 and y.scale() == SCALE
    assert np.max(np.abs(_dec(kit, y)[:d_model].real - want)) < 2e-3     # the fit of SiLU is good to 3e-5 on [-2, 2]
    # complex-folded: d_pad halves
    d_pad = 8
    fold = ph.pre_encode_bsgs_diagonals_complex
    wc = ph.mlp_weights_complex(fold(ctx, enc, Wg.ravel(), d_hidden, d_model, d_pad, M, SCALE, ph.complex_fold_mode.Rows),
                                fold(ctx, enc, Wu.ravel(), d_hidden, d_model, d_pad, M, SCALE, ph.complex_fold_mode.Rows),
                                fold(ctx, enc, Wd.ravel(), d_model, d_hidden, d_pad, M, SCALE, ph.complex_fold_mode.ColsConj),
                                d_model, d_hidden, d_pad)
    assert (wc.d_model, wc.d_hidden, wc.d_pad) == (8, 16, 8)
    yc = ph.mlp_forward_complex(ctx, enc, rlk, glk, _enc(kit, np.tile(x, SLOTS // d_pad)), wc)
    # matmul 1, halves 1 (+1 on the lower track), SiLU 4, product 1, repack 1, matmul 1
    assert yc.chain_index() == 1 + 1 + 2 + 4 + 1 + 1 + 1 and yc.scale() == SCALE
    assert np.max(np.abs(_dec(kit, yc)[:d_model].real - want)) < 2e-3


def test_attention_products(kit):
    ctx, enc, rlk, glk = kit["ctx"], kit["enc"], kit["rlk"], kit["glk"]
    heads, d_head = 2, 4
    d_total = heads * d_head
    positions = SLOTS // d_total                      # token positions in one ciphertext
    chunks = 3
    rng = np.random.default_rng(9)
    q = rng.uniform(-1, 1, (heads, d_head))
    K = rng.uniform(-1, 1, (chunks, positions, heads, d_head))
    V = rng.uniform(-1, 1, (chunks, positions, heads, d_head))
    cq = _enc(kit, np.tile(q.ravel(), positions))
    scores = ph.compute_qkt(ctx, rlk, glk, cq, [_enc(kit, K[c].ravel()) for c in range(chunks)], d_head)
    assert len(scores) == chunks and all(s.chain_index() == 2 and s.scale() == SCALE for s in scores)
    want_s = np.einsum("hi,cthi->cth", q, K)
    for c in range(chunks):
        got = _dec(kit, scores[c]).real.reshape(positions, heads, d_head)[:, :, 0]
        assert np.max(np.abs(got - want_s[c])) < 1e-5
    # score x V: the mask keeps slot 0 of every head block
    mask = np.zeros((positions, heads, d_head))
    mask[:, :, 0] = 1.0
    q_last = float(ctx.primes[ctx.limbs_at(2) - 1])
    mask_pt = enc.encode_double_vector(ctx, mask.ravel(), q_last, 2)
    out = ph.score_times_v(ctx, rlk, glk, scores, [_enc(kit, V[c].ravel()) for c in range(chunks)], mask_pt,
                           d_head, d_total, positions)
    assert out.chain_index() == 4 and out.scale() == SCALE
    want = np.einsum("cth,cthi->hi", want_s, V)
    got = _dec(kit, out).real
    assert np.max(np.abs(got[:d_total] - want.ravel())) < 1e-3
    assert np.max(np.abs(got[-d_total:] - want.ravel())) < 1e-3     # every d_total block carries the result
    with pytest.raises(ValueError, match="size mismatch"):
        ph.score_times_v(ctx, rlk, glk, scores, [], mask_pt, d_head, d_total, positions)
    with pytest.raises(ValueError, match="empty"):
        ph.score_times_v(ctx, rlk, glk, [], [], mask_pt, d_head, d_total, positions)
    with pytest.raises(ValueError, match="d_head must be a power of 2"):
        ph.score_times_v(ctx, rlk, glk, scores, scores, mask_pt, 3, d_total, positions)


def test_streams_do_not_change_the_limbs(kit, monkeypatch):
    """the pieces issued on side streams give the limbs the same calls give one after the other"""
    import torch
    from pyPhantom import model_blocks as mb
    ctx, enc, rlk, glk = kit["ctx"], kit["enc"], kit["rlk"], kit["glk"]
    rng = np.random.default_rng(10)
    d_head, d_total = 4, 8
    positions = SLOTS // d_total
    cq = _enc(kit, rng.uniform(-1, 1, SLOTS))
    ks = [_enc(kit, rng.uniform(-1, 1, SLOTS)) for _ in range(5)]
    vs = [_enc(kit, rng.uniform(-1, 1, SLOTS)) for _ in range(5)]
    mask = np.zeros((positions, 2, d_head))
    mask[:, :, 0] = 1.0
    mask_pt = enc.encode_double_vector(ctx, mask.ravel(), float(ctx.primes[ctx.limbs_at(2) - 1]), 2)

    def run():
        scores = ph.compute_qkt(ctx, rlk, glk, cq, ks, d_head)
        out = ph.score_times_v(ctx, rlk, glk, scores, vs, mask_pt, d_head, d_total, positions)
        sm = ph.softmax_correct(ctx, enc, rlk, scores[0], scores[1], 2)
        torch.cuda.synchronize()
        return [s.data.clone() for s in scores] + [out.data.clone(), sm.data.clone()]

    forked = [run() for _ in range(3)]
    monkeypatch.setattr(mb, "MAX_LANES", 0)
    plain = run()
    for got in forked:
        assert len(got) == len(plain) and all(torch.equal(a, b) for a, b in zip(got, plain))
