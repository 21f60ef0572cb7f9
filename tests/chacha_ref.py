"""Host restatement (test infrastructure) of the device samplers of phantom-fhe_b200/csrc/sampler.cuh: the ChaCha20 block
function of RFC 8439 vectorised over block counters with numpy, and the three draws made from it word for word as the
kernels make them. The GPU tests compare the kernels' output with this; test_sampler_cpu.py checks the block function
against the `cryptography` package's ChaCha20."""
import numpy as np

RESERVE = 64


def _rotl(x, r):
    return (x << np.uint32(r)) | (x >> np.uint32(32 - r))


def _qr(s, a, b, c, d):
    s[a] += s[b]; s[d] ^= s[a]; s[d] = _rotl(s[d], 16)
    s[c] += s[d]; s[b] ^= s[c]; s[b] = _rotl(s[b], 12)
    s[a] += s[b]; s[d] ^= s[a]; s[d] = _rotl(s[d], 8)
    s[c] += s[d]; s[b] ^= s[c]; s[b] = _rotl(s[b], 7)


def blocks(key32, nonce12, counters):
    """keystream blocks for the given 32-bit counters: uint32 [len(counters)][16]"""
    counters = np.asarray(counters, dtype=np.uint32)
    k = np.frombuffer(bytes(key32), dtype="<u4")
    n = np.frombuffer(bytes(nonce12), dtype="<u4")
    init = [np.full(counters.shape, v, dtype=np.uint32) for v in (0x61707865, 0x3320646E, 0x79622D32, 0x6B206574, *k)]
    init += [counters.copy()] + [np.full(counters.shape, v, dtype=np.uint32) for v in n]
    s = [x.copy() for x in init]
    with np.errstate(over="ignore"):
        for _ in range(10):
            _qr(s, 0, 4, 8, 12); _qr(s, 1, 5, 9, 13); _qr(s, 2, 6, 10, 14); _qr(s, 3, 7, 11, 15)
            _qr(s, 0, 5, 10, 15); _qr(s, 1, 6, 11, 12); _qr(s, 2, 7, 8, 13); _qr(s, 3, 4, 9, 14)
        out = np.stack([a + b for a, b in zip(s, init)], axis=1)
    return out


def words(blk):
    """the eight little-endian 64-bit words of each block"""
    return blk[:, 0::2].astype(np.uint64) | (blk[:, 1::2].astype(np.uint64) << np.uint64(32))


def uniform(key32, nonce12, primes, N):
    """[len(primes)][N] residues: limb j's coefficients 8t..8t+7 from block j*N/8 + t, rejected words replaced from the
    thread's reserve blocks"""
    total = len(primes) * (N // 8)
    w = words(blocks(key32, nonce12, np.arange(total)))
    out = np.empty((len(primes), N), dtype=np.uint64)
    for j, q in enumerate(primes):
        q = int(q)
        limit = (1 << 64) - ((1 << 64) % q)
        for tt in range(N // 8):
            t = j * (N // 8) + tt
            row = [int(x) for x in w[t]]
            pool, r = [], 0
            for i in range(8):
                x = row[i]
                while x >= limit and (pool or r < RESERVE):
                    if not pool:
                        r += 1
                        pool = [int(v) for v in words(blocks(key32, nonce12, [(t + r * total) & 0xFFFFFFFF]))[0]]
                    x = pool.pop(0)
                out[j, 8 * tt + i] = x % q
    return out


def cbd(key32, nonce12, N):
    w = words(blocks(key32, nonce12, np.arange(N // 8))).reshape(-1)
    lo = (w & np.uint64(0x1FFFFF)).astype(np.uint32)
    hi = ((w >> np.uint64(32)) & np.uint64(0x1FFFFF)).astype(np.uint32)
    pc = lambda v: np.unpackbits(v.view(np.uint8).reshape(-1, 4), axis=1).sum(axis=1).astype(np.int64)
    return pc(lo) - pc(hi)


def ternary(key32, nonce12, N):
    w = words(blocks(key32, nonce12, np.arange(N // 8))).reshape(-1)
    by = w.view(np.uint8).reshape(-1, 8)  # least significant byte first on a little-endian host
    out = np.zeros(N, dtype=np.int64)
    done = np.zeros(N, dtype=bool)
    for b in range(8):
        ok = (~done) & (by[:, b] < 252)
        out[ok] = by[ok, b].astype(np.int64) % 3 - 1
        done |= ok
    return out
