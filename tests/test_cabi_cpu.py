"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, its
host-only entry points agree with the oracle, and it refuses to work without a CUDA device."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import pyPhantom as ph
from pyPhantom import _native
from oracle_lib import LIB as ORA, create_coeff_modulus

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported():
    header = open(os.path.join(ROOT, "include", "b200fhe.h")).read()
    declared = set(re.findall(r"\b(b2_[a-zA-Z0-9_]+)\s*\(", header))
    assert len(declared) >= 25
    lib = ctypes.CDLL(_native.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/b200fhe.h but not exported"
    assert declared == set(_native.SIGNATURES), "python binding and header disagree"


@pytest.mark.parametrize("N,bits", [(1 << 14, [50] * 8), (1 << 16, [60] + [40] * 23 + [60] * 8),
                                    (1 << 12, [50, 36, 36, 36, 36, 36, 50, 50]), (1 << 13, [60, 40, 40, 58, 58])])
def test_create_coeff_modulus_matches_oracle(N, bits):
    got = [m.value() for m in ph.create_coeff_modulus(N, bits)]
    assert got == [int(x) for x in create_coeff_modulus(N, bits)]


def test_create_coeff_modulus_rejects_bad_input():
    with pytest.raises(ValueError):
        ph.create_coeff_modulus(1000, [30])  # not a power of two
    with pytest.raises(ValueError):
        ph.create_coeff_modulus(4096, [61])  # above USER_MOD_BIT_COUNT_MAX
    with pytest.raises(ValueError):
        ph.create_coeff_modulus(1 << 16, [18] * 3)  # no room for primes = 1 mod 2N


@pytest.mark.parametrize("N", [4096, 65536])
def test_galois_elt_from_step_matches_oracle(N):
    for step in [0, 1, 2, 3, -1, -7, 64, N // 2 - 1, -(N // 2 - 1)]:
        assert ph.get_elt_from_step(step, N) == ORA.ora_galois_elt_from_step(step, N)
    with pytest.raises(ValueError):
        ph.get_elt_from_step(N // 2, N)


def test_naf_matches_definition():
    for v in [3, 5, 7, 11, 100, -13, 12345]:
        terms = ph._naf(v)
        assert sum(terms) == v
        mags = sorted(abs(t).bit_length() - 1 for t in terms)
        assert all(b - a >= 2 for a, b in zip(mags, mags[1:]))  # no two adjacent non-zero digits


def test_context_fails_loudly_without_gpu():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    primes = create_coeff_modulus(4096, [40, 40, 50])
    h = ctypes.c_void_p()
    rc = _native.LIB.b2_ctx_create(4096, primes.ctypes.data, 3, 1, 0, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert b"no CUDA device" in _native.LIB.b2_last_error() or rc > 0
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(4096)
    parms.set_coeff_modulus(ph.create_coeff_modulus(4096, [40, 40, 50]))
    with pytest.raises(RuntimeError):
        ph.context(parms)


def test_unsupported_schemes_are_refused():
    for s in (ph.scheme_type.bfv, ph.scheme_type.bgv):
        with pytest.raises(ValueError):
            ph.context(ph.params(s))


def test_serialisation_header_layout():
    # include/ciphertext.h:173-191: four size_t, double, u64, size_t, two bools = 58 bytes
    assert ph.ciphertext._HDR.size == 58
    assert ph.plaintext._HDR.size == 32


def test_numpy_generator_matches_the_golden_generator():
    import synth
    from oracle_lib import Oracle
    N = 4096
    pr = create_coeff_modulus(N, [60, 36, 50])
    o = Oracle(N, pr, 1)
    assert np.array_equal(synth.poly(N, pr, 2, 7, 3), o.fill(2, pr, 7, 3))
    assert np.array_equal(synth.fill_limbs(N, pr[:2], 9, 50), o.fill(1, pr[:2], 9, 50)[0])


def test_key_sampling_uses_a_cryptographic_generator():
    """secret material and public masks come from independent AES-CTR streams keyed from os.urandom unless a test seed is
    given; the draws keep their distributions (exactly uniform below a bound, fair-coin binomial, distinct positions)"""
    from pyPhantom import keys
    a, b = keys._rng_pair(None)
    assert isinstance(a, keys._CtrDrbg) and isinstance(b, keys._CtrDrbg) and a is not b
    q = 1152921504606584833
    x, y = a.integers(0, q, 1 << 16, dtype=np.uint64), b.integers(0, q, 1 << 16, dtype=np.uint64)
    assert x.dtype == np.uint64 and int(x.max()) < q and not np.array_equal(x, y)
    assert abs(float(x.astype(np.float64).mean()) / q - 0.5) < 0.01
    t = a.integers(-1, 2, 1 << 16)
    assert set(np.unique(t)) == {-1, 0, 1} and abs(np.bincount(t + 1) / (1 << 16) - 1 / 3).max() < 0.01
    e = a.binomial(21, 0.5, 1 << 16) - a.binomial(21, 0.5, 1 << 16)
    assert abs(e.mean()) < 0.05 and abs(e.var() - 10.5) < 0.3 and np.abs(e).max() <= 21
    pos = a.choice(4096, size=128, replace=False)
    assert len(set(pos.tolist())) == 128 and pos.min() >= 0 and pos.max() < 4096
    assert set(np.unique(a.choice(np.array([-1, 1]), size=256))) == {-1, 1}
    s1, s2 = keys._rng_pair(7)   # the reproducible test hook
    assert isinstance(s1, np.random.Generator) and s1.integers(0, 10, 4).tolist() == keys._rng_pair(7)[0].integers(0, 10, 4).tolist()


def test_batched_wrappers_check_their_arguments_before_any_device_call():
    """relinearize_batch and multiply_relin_rescale_batch want contiguous [batch][3 or 2][limbs][N] tensors: a wrong shape is a
    ValueError raised on the host (no GPU needed to see it)"""
    import torch
    import pyPhantom as ph
    with pytest.raises(ValueError, match="contiguous"):
        ph.relinearize_batch(None, torch.zeros(2, 2, 3, 8, dtype=torch.int64), None)
    with pytest.raises(ValueError, match="contiguous"):
        ph.relinearize_batch(None, torch.zeros(2, 3, 3, 8, dtype=torch.int64).transpose(2, 3), None)
    with pytest.raises(ValueError, match="one shape"):
        ph.multiply_relin_rescale_batch(None, torch.zeros(2, 2, 3, 8, dtype=torch.int64), torch.zeros(2, 2, 4, 8, dtype=torch.int64), None)
