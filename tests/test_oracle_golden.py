"""Pins the CPU oracle to the reference: every stage of the key-switching path, recomputed by
oracle/ckks_oracle.c on the seeded synthetic limbs, must reproduce the per-limb hashes that the
unmodified reference library produced on a GPU (tests/golden/*.json, made by make_golden.sh)."""
import glob
import json
import os

import numpy as np
import pytest

from oracle_lib import Oracle, create_coeff_modulus, golden_case_stages, LIB

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.json")))


def test_golden_records_present():
    assert len(GOLDEN) >= 9


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-5] for p in GOLDEN])
def test_oracle_reproduces_reference(path):
    case = json.load(open(path))
    assert case["host_tables_match_oracle"] is True and case["cuda_error"] == "no error"
    N = 1 << case["logn"]
    primes = create_coeff_modulus(N, case["bits"])
    assert [int(p) for p in primes] == case["primes"]
    o = Oracle(N, primes, case["special"])
    got = golden_case_stages(o, case)
    assert set(got) == set(case["hashes"])
    for name, want in case["hashes"].items():
        assert got[name] == want, f"{name} differs from the reference"


def test_prime_and_root_facts():
    # the published parameter facts of the two headline configurations
    p1 = create_coeff_modulus(1 << 14, [50] * 8)
    assert int(p1[0]) == 1125899901665281 and int(p1[7]) == 1125899904679937
    roots = [int(LIB.ora_minimal_primitive_root(1 << 15, int(q))) for q in p1]
    assert roots[:3] == [9625540990, 584428750, 32853495844]
    p2 = create_coeff_modulus(1 << 16, [60] + [40] * 23 + [60] * 8)
    assert int(p2[0]) == 1152921504583647233 and int(p2[1]) == 1099468505089
    assert int(p2[31]) == 1152921504606584833


def test_negacyclic_convolution_small():
    N = 64
    pr = create_coeff_modulus(N, [30, 30, 30])
    o = Oracle(N, pr, 1)
    rng = np.random.default_rng(0)
    a = np.stack([rng.integers(0, int(q), N, dtype=np.uint64) for q in pr])
    b = np.stack([rng.integers(0, int(q), N, dtype=np.uint64) for q in pr])
    A, B = o.ntt_forward(a), o.ntt_forward(b)
    C = np.stack([np.array([int(x) * int(y) % int(q) for x, y in zip(A[l], B[l])], dtype=np.uint64)
                  for l, q in enumerate(pr)])
    c = o.ntt_inverse(C)
    for l, q in enumerate(pr):
        q = int(q)
        ref = [0] * N
        for i in range(N):
            for j in range(N):
                v = int(a[l][i]) * int(b[l][j])
                if i + j >= N:
                    ref[i + j - N] = (ref[i + j - N] - v) % q
                else:
                    ref[i + j] = (ref[i + j] + v) % q
        assert ref == [int(x) for x in c[l]]
    assert np.array_equal(o.ntt_inverse(A), a)
