"""Deterministic synthetic limbs: uniform residues addressed by (seed, index).

Element i of stream `seed` for prime q is the first of the 64-bit draws mix(seed, i, 0),
mix(seed, i, 1), ... (masked to bitlen(q) bits) that falls below q - exactly uniform in [0, q)
and independent of evaluation order. The test-suite checks that this numpy statement produces
the same words as the generator the golden records were made with.
"""
import numpy as np

_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_G = np.uint64(0x9E3779B97F4A7C15)
_C0 = np.uint64(0x632BE59BD9B4E019)
_C1 = np.uint64(0xD1342543DE82EF95)


def _mix64(z):
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def uniform(n, q, seed):
    """n residues in [0, q) of stream `seed`"""
    q = int(q)
    mask = np.uint64((1 << q.bit_length()) - 1)
    with np.errstate(over="ignore"):
        s = np.array([seed & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64)
        base = _mix64(s * _G + _C0)[0] + np.arange(n, dtype=np.uint64) * _C1
        out = np.empty(n, dtype=np.uint64)
        todo = np.arange(n)
        k = 0
        while todo.size:
            v = _mix64(base[todo] + np.uint64(k) * _G) & mask
            ok = v < np.uint64(q)
            out[todo[ok]] = v[ok]
            todo = todo[~ok]
            k += 1
    return out


def fill_limbs(N, primes, case_seed, buf, limb0=0):
    """[len(primes)][N]: limb l takes stream (case_seed << 40) ^ (buf << 16) ^ (limb0 + l)"""
    return np.stack([uniform(N, q, (case_seed << 40) ^ (buf << 16) ^ (limb0 + l)) for l, q in enumerate(primes)])


def poly(N, primes, n_poly, case_seed, buf):
    """[n_poly][len(primes)][N] with the limb numbering continuing across polynomials"""
    return np.stack([fill_limbs(N, primes, case_seed, buf, p * len(primes)) for p in range(n_poly)])
