"""b2_sample (ChaCha20 keystream samplers on the device) against the host restatement, word for word"""
import numpy as np
import pytest
import torch

import pyPhantom as ph
from pyPhantom._native import LIB, check
from gpu_helpers import make_ctx, stream
import chacha_ref

pytestmark = pytest.mark.gpu


def _draw(ctx, kind, key, nonce, first, n_limbs, out):
    k = np.frombuffer(key + nonce, dtype=np.uint8).copy()
    check(LIB.b2_sample(ctx._h, kind, k.ctypes.data, k[32:].ctypes.data, first, n_limbs, out.data_ptr(), stream()))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_samplers_match_the_host_restatement():
    N = 4096
    ctx, o = make_ctx(N, [60, 40, 50, 33, 60], 1)
    primes = [int(q) for q in o.primes]
    rng = np.random.default_rng(11)
    for first, n in ((0, 5), (1, 3), (4, 1)):
        key, nonce = rng.bytes(32), rng.bytes(12)
        got = _draw(ctx, 0, key, nonce, first, n, torch.empty(n, N, dtype=torch.int64, device="cuda")).view(np.uint64)
        assert np.array_equal(got, chacha_ref.uniform(key, nonce, primes[first:first + n], N))
    key, nonce = rng.bytes(32), rng.bytes(12)
    e = _draw(ctx, 1, key, nonce, 0, 1, torch.empty(N, dtype=torch.int64, device="cuda"))
    assert np.array_equal(e, chacha_ref.cbd(key, nonce, N))
    t = _draw(ctx, 2, key, nonce, 0, 1, torch.empty(N, dtype=torch.int64, device="cuda"))
    assert np.array_equal(t, chacha_ref.ternary(key, nonce, N))
    assert LIB.b2_sample(ctx._h, 0, 0, 0, 0, 1, 0, stream()) != 0          # null pointers
    k = np.zeros(44, dtype=np.uint8)
    out = torch.empty(N, dtype=torch.int64, device="cuda")
    assert LIB.b2_sample(ctx._h, 0, k.ctypes.data, k[32:].ctypes.data, 4, 2, out.data_ptr(), stream()) != 0   # past the chain
    assert LIB.b2_sample(ctx._h, 3, k.ctypes.data, k[32:].ctypes.data, 0, 1, out.data_ptr(), stream()) != 0   # unknown kind


def test_full_size_draw_statistics():
    """N = 2^16 over the headline chain: every residue below its prime, 60-bit limbs (1 word in 16 rejected) included;
    error and ternary moments"""
    N = 65536
    ctx, o = make_ctx(N, [60] + [40] * 3 + [60] * 2, 2)
    primes = [int(q) for q in o.primes]
    key, nonce = bytes(range(32)), bytes(range(12))
    u = _draw(ctx, 0, key, nonce, 0, len(primes), torch.empty(len(primes), N, dtype=torch.int64, device="cuda")).view(np.uint64)
    for j, q in enumerate(primes):
        assert (u[j] < np.uint64(q)).all()
        assert abs(u[j].astype(np.float64).mean() / q - 0.5) < 0.01
    # spot check of a 60-bit limb against the restatement (a slice: the host loop is slow)
    w = chacha_ref.uniform(key, nonce, primes[:1], N)
    assert np.array_equal(u[0], w[0])
    e = _draw(ctx, 1, key, nonce, 0, 1, torch.empty(N, dtype=torch.int64, device="cuda"))
    assert abs(e.mean()) < 0.06 and abs(e.var() - 10.5) < 0.4
    t = _draw(ctx, 2, key, nonce, 0, 1, torch.empty(N, dtype=torch.int64, device="cuda"))
    assert np.abs(np.bincount(t + 1, minlength=3) - N / 3).max() < 5 * np.sqrt(N * 2 / 9)
