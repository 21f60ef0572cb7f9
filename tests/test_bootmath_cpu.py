"""Host mathematics of bootstrapping on plain numbers (no device): the layered special FFT, the
BSGS plans, the Chebyshev evaluator and EvalRound with the float stand-in for ciphertexts."""
import importlib.util
import math
import os

import numpy as np
import pytest

_spec = importlib.util.spec_from_file_location(
    "bootmath", os.path.join(os.path.dirname(__file__), "..", "phantom-fhe_b200", "pyPhantom", "bootmath.py"))
bm = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bm)


@pytest.mark.parametrize("n,c2s,s2c", [(64, [2, 2, 2], [3, 3]), (2048, [4, 4, 3], [6, 5])])
def test_layers_compose_to_the_embedding(n, c2s, s2c):
    U0, P = bm.embedding_matrix(n), bm.bit_reverse_perm(n)
    rng = np.random.default_rng(1)
    z = rng.normal(size=n) + 1j * rng.normal(size=n)
    x = z.copy()
    for layer in bm.fft_layers(n, c2s, True):
        plan = bm.LayerPlan(layer, n)
        y = bm.apply_diagonals(layer, x)
        assert np.allclose(plan.apply(x), y, atol=1e-9)
        x = y
    w = U0.conj().T @ z  # n times the coefficients
    assert np.max(np.abs(x - w[P])) < 1e-9 * n
    x = x / n
    for layer in bm.fft_layers(n, s2c, False):
        assert max(np.max(np.abs(d)) for d in layer.values()) < 1.0 + 1e-9  # encodable at a 2^58 scale
        x = bm.LayerPlan(layer, n).apply(x)
    assert np.max(np.abs(x - z)) < 1e-10


def test_plan_sizes_at_full_size():
    # logN = 16: what the key generator has to provide
    steps = bm.required_rotation_steps(16, [5, 5, 5], [8, 7])
    assert len(steps) == len(set(steps)) and 60 <= len(steps) <= 120
    assert bm.split_stages(15, 3) == [5, 5, 5] and bm.split_stages(15, 2) == [8, 7] and bm.split_stages(11, 3) == [4, 4, 3]


def test_chebyshev_division_and_evaluator():
    primes = [2 ** 58 - 27] + [2 ** 58 - (2 * i + 1) * 2 ** 17 + 1 for i in range(12)]
    ops = bm.FloatOps(primes)
    x = np.linspace(-1, 1, 1001)
    c = np.random.default_rng(0).normal(size=64)
    q, r = bm.cheb_divide(c, 32)
    cheb = np.polynomial.chebyshev.chebval
    assert np.max(np.abs(cheb(x, q) * np.cos(32 * np.arccos(x)) + cheb(x, r) - cheb(x, c))) < 1e-11
    ev = bm.ChebyshevEvaluator(ops, ops.V(x, 13, 2.0 ** 58), 8)
    out = ev.evaluate(c, 2.0 ** 58)
    assert out.level == 13 - 7 and abs(out.scale / 2.0 ** 58 - 1) < 2.0 ** -45
    assert np.max(np.abs(out.v - cheb(x, c))) < 1e-11
    for k, t in ev.T.items():
        assert np.max(np.abs(t.v - np.cos(k * np.arccos(x)))) < 1e-12
    with pytest.raises(ValueError):
        bm.cheb_divide(c, 16)


@pytest.mark.parametrize("degree", [55, 63])
def test_eval_round_on_floats(degree):
    primes = [2 ** 58 - 27] + [2 ** 40 - 87] * 2 + [2 ** 58 - (2 * i + 1) * 2 ** 17 + 1 for i in range(12)]
    ops = bm.FloatOps(primes)
    K = 28
    rng = np.random.default_rng(0)
    I = rng.integers(-K + 1, K, size=4096)
    y = I + rng.uniform(-2.0 ** -11, 2.0 ** -11, size=4096)   # message part
    u = ops.V(y / K + rng.normal(size=4096) * 2.0 ** -24, 15, 2.0 ** 58 * (1 + 1e-7))  # CoeffToSlot's rounding
    out = bm.eval_round(ops, u, K, 3, degree, 2.0 ** 58)
    assert out.level == 5                      # 7 levels of polynomial + 3 double angles
    assert abs(out.scale / 2.0 ** 58 - 1) < 2.0 ** -45
    assert np.max(np.abs(out.v - I)) < 2e-9    # cubic in the distance to the integer: (2 pi)^2 (2^-11)^3 / 6
    assert ops.muls <= 19


@pytest.mark.parametrize("degree,babies,depth", [(3, 2, 2), (7, 4, 4), (8, 4, 4), (9, 4, 4), (15, 4, 5), (16, 4, 5), (4, 4, 3), (1, 2, 1)])
def test_tight_evaluator_depth_and_value(degree, babies, depth):
    """tight mode: T_m serves in the leaves, degree 2^k m fits k giants, the output sits at the smallest depth"""
    primes = [2 ** 58 - 27] + [2 ** 58 - (2 * i + 1) * 2 ** 17 + 1 for i in range(12)]
    ops = bm.FloatOps(primes)
    x = np.linspace(-1, 1, 501)
    c = np.random.default_rng(degree).normal(size=degree + 1)
    ev = bm.ChebyshevEvaluator(ops, ops.V(x, 13, 2.0 ** 58), babies, tight=True)
    out = ev.evaluate(c, 2.0 ** 58)
    assert out.level == 13 - depth and abs(out.scale / 2.0 ** 58 - 1) < 2.0 ** -45
    assert np.max(np.abs(out.v - np.polynomial.chebyshev.chebval(x, c))) < 1e-11
    q, r = bm.cheb_divide(np.arange(1.0, 10.0), 4)      # degree exactly 2g
    assert np.max(np.abs(np.polynomial.chebyshev.chebval(x, q) * np.cos(4 * np.arccos(x)) + np.polynomial.chebyshev.chebval(x, r)
                         - np.polynomial.chebyshev.chebval(x, np.arange(1.0, 10.0)))) < 1e-12
