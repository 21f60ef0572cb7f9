"""The host restatement of the device samplers: its ChaCha20 block function against the `cryptography` package, and the
distributions it draws."""
import os

import numpy as np
import pytest

import chacha_ref


def test_block_function_matches_a_library_chacha20():
    algorithms = pytest.importorskip("cryptography.hazmat.primitives.ciphers.algorithms")
    from cryptography.hazmat.primitives.ciphers import Cipher
    rng = np.random.default_rng(3)
    for first in (0, 1, 7, 0xFFFFFFF0):
        key, nonce = rng.bytes(32), rng.bytes(12)
        n = 9
        # the library takes the 32-bit block counter (little endian) in front of the 12-byte nonce
        enc = Cipher(algorithms.ChaCha20(key, int(first).to_bytes(4, "little") + nonce), mode=None).encryptor()
        want = np.frombuffer(enc.update(bytes(64 * n)), dtype="<u4").reshape(n, 16)
        got = chacha_ref.blocks(key, nonce, (np.arange(n, dtype=np.uint64) + first).astype(np.uint32))
        assert np.array_equal(got, want)


def test_uniform_is_below_the_prime_and_rejects_exactly():
    key, nonce = bytes(range(32)), bytes(12)
    # a prime just above 2^63 rejects almost every second word: the reserve blocks are exercised
    primes = [(1 << 63) + 29, 1099511627689, 97]
    N = 64
    u = chacha_ref.uniform(key, nonce, primes, N)
    assert u.shape == (3, N) and all((u[j] < np.uint64(q)).all() for j, q in enumerate(primes))
    w = chacha_ref.words(chacha_ref.blocks(key, nonce, np.arange(3 * N // 8)))
    # where the first word is accepted it is the one reduced
    limit = (1 << 64) - ((1 << 64) % primes[1])
    first = [int(x) for x in w[N // 8:2 * N // 8].reshape(-1)]
    assert all(int(u[1, i]) == x % primes[1] for i, x in enumerate(first) if x < limit)
    rejected = sum(int(x) >= (1 << 64) - ((1 << 64) % primes[0]) for x in w[:N // 8].reshape(-1))
    assert rejected > N // 4


def test_small_distributions():
    key, nonce = os.urandom(32), os.urandom(12)
    N = 1 << 16
    e = chacha_ref.cbd(key, nonce, N)
    assert abs(e.mean()) < 0.06 and abs(e.var() - 10.5) < 0.4 and np.abs(e).max() <= 21
    t = chacha_ref.ternary(key, nonce, N)
    assert set(np.unique(t)) == {-1, 0, 1}
    counts = np.array([(t == v).sum() for v in (-1, 0, 1)])
    assert np.abs(counts - N / 3).max() < 5 * np.sqrt(N * 2 / 9)
