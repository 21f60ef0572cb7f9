"""Bootstrapping end to end through the pyPhantom surface (python/examples/bootstrap.py is the model):
deplete a ciphertext, bootstrap it, decrypt and compare with the message. N = 2^12 and 2^13 keep most
tests short; test_full_size_bootstrap_meets_the_reference_bar runs N = 2^16 against the reference test's
own bar."""
import importlib
import math

import numpy as np
import pytest

import encoder_ref
import torch

pytestmark = pytest.mark.gpu

import pyPhantom as ph

boot = importlib.import_module("pyPhantom.boot")
bm = importlib.import_module("pyPhantom.bootmath")


def _setup(log_n, n_user, alpha, c2s_bits, sparse_main, user_scale=2.0 ** 40):
    N = 1 << log_n
    bits = [58] + [40] * n_user + [58] * 12 + [c2s_bits] * 3 + [58] * alpha
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(N)
    parms.set_special_modulus_size(alpha)
    parms.set_coeff_modulus(ph.create_coeff_modulus(N, bits))
    parms.set_galois_elts(ph.bootstrap_required_galois_elts(log_n, bm.split_stages(log_n - 1, 3)))
    ctx = ph.context(parms)
    sk = ph.secret_key(ctx, seed=11)
    if sparse_main:
        sk.generate_sparse(ctx, 128)
    enc = ph.ckks_encoder(ctx)
    bk = ph.create_bootstrap_key(ctx, enc, sk, sparse_hamming_weight=128, eval_mod_levels=9, user_scale=user_scale)
    return ctx, sk, enc, bk


@pytest.mark.parametrize("log_n,n_user,alpha,c2s_bits,sparse_main", [(12, 3, 6, 29, True), (13, 2, 3, 58, False)])
def test_bootstrap_round_trip(log_n, n_user, alpha, c2s_bits, sparse_main):
    ctx, sk, enc, bk = _setup(log_n, n_user, alpha, c2s_bits, sparse_main)
    n = ctx.N // 2
    rng = np.random.default_rng(0xB007B007)
    msg = rng.uniform(-0.4, 0.4, n)
    scale = 2.0 ** 40
    ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, msg, scale, chain_index=1))
    ph.mod_switch_to_inplace(ctx, ct, ctx.total_parm_size() - 2)   # two limbs left, as the example does
    assert ct.coeff_modulus_size() == 2
    stats = {}
    out = ph.bootstrap(ctx, enc, ct, bk, scale, stats=stats)
    assert out.coeff_modulus_size() == bk.user_limbs == n_user + 1  # q0 and every user prime
    assert out.scale() == scale
    got = enc.decode_double_vector(ctx, sk.decrypt(ctx, out))
    err = np.max(np.abs(got - msg))
    assert err < 2e-5, err            # the reference's example accepts 1e-3, its C++ test 5e-6 at N = 2^16
    assert abs(stats["final_scale_over_target"] - 1.0) < 2.0 ** -45
    # second call captures the CUDA graph, third replays it: both must reproduce the eager result bit for bit
    for _ in range(2):
        again = ph.bootstrap(ctx, enc, ct, bk, scale)
        assert torch.equal(again.data, out.data)
    other = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, -msg, scale, chain_index=ctx.total_parm_size() - 2))
    replayed = ph.bootstrap(ctx, enc, other, bk, scale)
    assert torch.equal(replayed.data, ph.bootstrap_eager(ctx, enc, other, bk, scale).data)
    assert np.max(np.abs(enc.decode_double_vector(ctx, sk.decrypt(ctx, replayed)) + msg)) < 2e-5
    # the refreshed ciphertext computes: one multiplication and a rescale on the new levels
    sq = ph.rescale_to_next(ctx, ph.multiply_and_relin(ctx, out, out, bk.relin))
    got2 = enc.decode_double_vector(ctx, sk.decrypt(ctx, sq))
    assert np.max(np.abs(got2 - msg * msg)) < 1e-4


@pytest.mark.parametrize("chain", ["example", "bench"])
def test_full_size_bootstrap_meets_the_reference_bar(chain):
    """N = 2^16 with the inputs of the reference's own round-trip test (test/bootstrap_test.cu:517-662): 2^15 real slots
    uniform in (-0.5, 0.5) from mt19937_64(0xB007B007), scale 2^40, encapsulation weight 128, input left on two primes,
    and its bar, max |error| <= 5e-6 (:654). "example": the chain and sparse secret (weight 128) of
    python/examples/bootstrap.py, 58 | 40x4 | 58x12 | 29x3 | P 58x4; "bench": the 24-limb dnum-3 chain of bench.py,
    58 | 40x8 | 58x12 | 29x3 | P 58x8, sparse secret of weight 192. tests/golden/bootstrap/ref_bootstrap_n16.json holds what the
    reference itself gives on the example chain on a B200 (8.6e-5, 125 ms) beside this pipeline."""
    from gpu_helpers import mt19937_64_doubles
    log_n = 16
    N, n = 1 << log_n, 1 << (log_n - 1)
    n_user, alpha, hw = (4, 4, 128) if chain == "example" else (8, 8, 192)
    bits = [58] + [40] * n_user + [58] * 12 + [29] * 3 + [58] * alpha
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(N)
    parms.set_special_modulus_size(alpha)
    parms.set_coeff_modulus(ph.create_coeff_modulus(N, bits))
    parms.set_galois_elts(ph.bootstrap_required_galois_elts(log_n, [5, 5, 5]))
    ctx = ph.context(parms)
    sk = ph.secret_key(ctx, seed=2026)
    sk.generate_sparse(ctx, hw)
    enc = ph.ckks_encoder(ctx)
    scale = 2.0 ** 40
    bk = ph.create_bootstrap_key(ctx, enc, sk, sparse_hamming_weight=128, eval_mod_levels=9, user_scale=scale)
    msg = mt19937_64_doubles(0xB007B007, n, -0.5, 0.5)
    ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, msg, scale, chain_index=1))
    ph.mod_switch_to_inplace(ctx, ct, ctx.total_parm_size() - 2)
    out = ph.bootstrap(ctx, enc, ct, bk, scale)
    assert out.coeff_modulus_size() == n_user + 1 and out.scale() == scale
    err = np.abs(enc.decode_double_vector(ctx, sk.decrypt(ctx, out)) - msg)
    assert err.max() <= 5e-6, err.max()
    assert ctx.device_status() == 0


def test_stages_against_the_plain_computation():
    ctx, sk, enc, bk = _setup(12, 2, 6, 29, False)
    N, n = ctx.N, ctx.N // 2
    ops = boot.CtOps(ctx, bk.relin)
    rng = np.random.default_rng(3)
    msg = rng.uniform(-0.5, 0.5, n)
    scale = 2.0 ** 47
    ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, msg, scale, chain_index=ctx.size_Q))
    raised = boot.mod_raise(ctx, bk, ct)
    assert raised.coeff_modulus_size() == ctx.size_Q
    coef = encoder_ref.centred_coefficients(ctx, sk.decrypt(ctx, raised))
    q0 = int(ctx.primes[0])
    I = np.array([(2 * int(v) + q0) // (2 * q0) for v in coef])
    assert np.abs(I).max() < boot.K_RANGE                       # the sparse secret keeps q0*I small
    frac = np.array([float(int(v) - int(i) * q0) for v, i in zip(coef, I)]) / scale
    b = np.zeros(2 * N, dtype=np.complex128)
    b[:N] = frac
    assert np.max(np.abs((np.fft.ifft(b) * 2 * N)[enc._pos].real - msg)) < 1e-6  # t = scale*m + e + q0*I
    lo, hi = boot.coeff_to_slot(ctx, bk, raised, ops)
    P = bm.bit_reverse_perm(n)
    t = np.array([float(int(v)) for v in coef]) / (float(q0) * boot.K_RANGE)
    dec = lambda c: enc.decode_complex_vector(ctx, sk.decrypt(ctx, c))
    assert np.max(np.abs(dec(lo) - t[:n][P])) < 1e-5            # 29-bit primes: coarse on purpose
    assert np.max(np.abs(dec(hi) - t[n:][P])) < 1e-5
    ints = [bm.eval_round(ops, u, boot.K_RANGE, boot.DOUBLE_ANGLES, boot.COS_DEGREE, bk.eval_scale) for u in (lo, hi)]
    assert np.max(np.abs(dec(ints[0]) - I[:n][P])) < 1e-8
    assert np.max(np.abs(dec(ints[1]) - I[n:][P])) < 1e-8
    qi = boot.slot_to_coeff(ctx, bk, ints[0], ints[1], ops)
    cq = encoder_ref.centred_coefficients(ctx, sk.decrypt(ctx, qi))
    # the coefficients hold I times the key's target scale (q0, times down_const / p_x when the key scales the input up)
    assert max(abs(float(int(a)) / bk.final_target - float(i)) for a, i in zip(cq, I)) < 1e-8


def test_errors():
    ctx, sk, enc, bk = _setup(12, 2, 6, 29, True)
    ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, np.full(8, 0.25), 2.0 ** 40, chain_index=ctx.size_Q - 1))
    split = ph.bootstrap(ctx, enc, ct, bk, 2.0 ** 40, True)      # the reference's split mode hands back one level lower
    assert split.coeff_modulus_size() == bk.user_limbs - 1 and split.chain_index() == ctx.size_Q - bk.user_limbs + 2
    assert np.max(np.abs(enc.decode_double_vector(ctx, sk.decrypt(ctx, split))[:8] - 0.25)) < 1e-5
    with pytest.raises(ValueError):
        ph.create_bootstrap_key(ctx, enc, sk, eval_mod_levels=5)
    assert len(ph.bootstrap_required_galois_elts(12, [4, 4, 3])) == len(set(ph.bootstrap_required_galois_elts(12, [4, 4, 3])))
    assert (2 * ctx.N - 1) in ph.bootstrap_required_galois_elts(12)
    pt = enc.encode_double_vector(ctx, np.zeros(4), 2.0 ** 40, chain_index=ctx.size_Q)
    with pytest.raises(ValueError):     # one limb: the prime needed for the scale-up is gone
        ph.bootstrap(ctx, enc, sk.encrypt_symmetric(ctx, pt), bk, 2.0 ** 40)


def test_scale_follows_the_input():
    # a key made without user_scale, then used at 2^40 and at 2^36: the last SlotToCoeff layer is re-encoded
    ctx, sk, enc, bk = _setup(12, 2, 6, 29, True, user_scale=0.0)
    msg = np.random.default_rng(2).uniform(-0.5, 0.5, ctx.N // 2)
    for scale in (2.0 ** 40, 2.0 ** 36):
        ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, msg, scale, chain_index=ctx.size_Q - 1))
        out = ph.bootstrap(ctx, enc, ct, bk, scale)
        assert bk.user_scale == scale and out.scale() == scale and out.coeff_modulus_size() == bk.user_limbs
        assert np.max(np.abs(enc.decode_double_vector(ctx, sk.decrypt(ctx, out)) - msg)) < 5e-5
