"""Key generation, symmetric encryption and decryption (binding.cu:77-98; src/secretkey.cu).

The secret itself (one polynomial, a choice of positions for the sparse form) is drawn on the host; the uniform masks,
the errors and the ternary encryption randomness - the bulk: gigabytes for a bootstrapping key set - are drawn on the
device by b2_sample from ChaCha20 keystreams whose keys and nonces come from the host generator; every polynomial
operation - reduction into the limbs, NTT, products, sums - is a call into the C ABI.
The host generator is cryptographic: an AES-256-CTR keystream keyed from os.urandom,
one stream for secret material (secrets, error and encryption-randomness keys) and an independent one for
the public uniform masks, as the reference draws from a salsa20 stream seeded from
std::random_device (src/prng.cu, include/prng.cuh:12-21). `seed=` swaps in numpy's PCG64 so that
tests and benchmarks are reproducible: it is NOT secure and is meant for nothing else.
Keys are not reproducible in the reference either: what is kept is the distributions (ternary or fixed-Hamming-weight
secret, centred-binomial error with 21 coin pairs, uniform masks), the algebra
(pk = (-(a s + e), a); digit d of a switching key adds P s' on the Q limbs of digit d,
src/secretkey.cu:354-398, src/polymath.cu:317-337) and the save()/load() byte layouts, so keys and
ciphertexts made here work with the reference's evaluator and the other way round.
"""
import os
import struct

import numpy as np
import torch

from ._native import LIB, check


class _CtrDrbg:
    """The sampling calls this module makes (integers, binomial, choice) on an AES-256-CTR keystream keyed from
    os.urandom. Uniform draws below a bound use rejection on words masked to the bound's bit length, so they are exactly
    uniform; nothing here depends on a value already drawn except how many more words are fetched."""

    def __init__(self):
        from cryptography.hazmat.primitives.ciphers import Cipher, algorithms, modes
        self._enc = Cipher(algorithms.AES(os.urandom(32)), modes.CTR(os.urandom(16))).encryptor()

    def _words(self, n):
        return np.frombuffer(self._enc.update(bytes(8 * int(n))), dtype=np.uint64)

    def bytes(self, n):
        return self._enc.update(bytes(int(n)))

    def _below(self, bound, size):
        bound = int(bound)
        mask = np.uint64((1 << max(1, (bound - 1).bit_length())) - 1)
        out = np.empty(size, dtype=np.uint64)
        have = 0
        while have < size:
            w = self._words(max(64, int(1.25 * (size - have)) + 16)) & mask
            w = w[w < np.uint64(bound)][: size - have]
            out[have: have + w.size] = w
            have += w.size
        return out

    def integers(self, low, high=None, size=None, dtype=np.int64):
        if high is None:
            low, high = 0, low
        v = self._below(int(high) - int(low), int(size))
        if np.dtype(dtype) == np.uint64:
            return v + np.uint64(int(low))
        return v.astype(np.int64) + int(low)

    def binomial(self, n, p, size):
        """number of heads in n <= 32 fair coins per sample (p must be 0.5)"""
        if p != 0.5 or not 0 < n <= 32:
            raise ValueError("fair coins only")
        w = self._words((int(size) + 1) // 2).view(np.uint32)[: int(size)] & np.uint32((1 << n) - 1)
        return np.unpackbits(w.view(np.uint8).reshape(-1, 4), axis=1).sum(axis=1).astype(np.int64)

    def choice(self, a, size, replace=True):
        if isinstance(a, (int, np.integer)):
            if replace:
                return self.integers(0, int(a), size)
            keys = self._words(int(a))          # a uniform random subset: the positions of the `size` smallest keys
            return np.argpartition(keys, int(size))[: int(size)]
        a = np.asarray(a)
        return a[self.integers(0, len(a), size)]


def _rng_pair(seed):
    """(secret stream, public-mask stream): cryptographic unless a test seed is given"""
    if seed is None:
        return _CtrDrbg(), _CtrDrbg()
    a, b = np.random.SeedSequence(seed).spawn(2)
    return np.random.default_rng(a), np.random.default_rng(b)

_SK_HDR = struct.Struct("<QQQ")  # sk_max_power, N, coeff_mod_size (include/secretkey.h:537-554)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _poly(ctx, op, n_limbs, a, b, out):
    check(LIB.b2_poly_op(ctx._h, op, n_limbs, a.data_ptr(), 0 if b is None else b.data_ptr(), out.data_ptr(), _stream()))


def _expand(ctx, coeffs_i64, n_limbs, ntt=True):
    """signed int64[N] on the host -> [n_limbs][N] residues (limb i <-> prime i), NTT form by default"""
    d = torch.from_numpy(np.ascontiguousarray(coeffs_i64, dtype=np.int64)).to(ctx.device)
    out = ctx.empty(n_limbs)
    check(LIB.b2_expand_signed(ctx._h, 0, n_limbs, d.data_ptr(), out.data_ptr(), 1 if ntt else 0, _stream()))
    return out


def _device_draw(ctx, rng, kind, n_limbs, out):
    """one draw of b2_sample (src/prng.cu:142-240's three samplers): a fresh ChaCha20 key and nonce from the host
    generator, the polynomial itself made on the device"""
    kn = np.frombuffer(rng.bytes(44), dtype=np.uint8).copy()
    check(LIB.b2_sample(ctx._h, kind, kn.ctypes.data, kn[32:].ctypes.data, 0, n_limbs, out.data_ptr(), _stream()))
    return out


def _signed_draw(ctx, rng, kind, n_limbs, ntt=True):
    """kind 1: centred-binomial error, kind 2: uniform ternary; the same integer in every limb, NTT form by default"""
    d = _device_draw(ctx, rng, kind, 1, torch.empty(ctx.N, dtype=torch.int64, device=ctx.device))
    out = ctx.empty(n_limbs)
    check(LIB.b2_expand_signed(ctx._h, 0, n_limbs, d.data_ptr(), out.data_ptr(), 1 if ntt else 0, _stream()))
    return out


def _uniform(ctx, rng, n_limbs):
    """[n_limbs][N] uniform residues (already a valid NTT-form polynomial)"""
    return _device_draw(ctx, rng, 0, n_limbs, ctx.empty(n_limbs))


def _error(ctx, rng, n_limbs):
    """centred binomial, 21 coin pairs: standard deviation sqrt(21/2) = 3.24 (include/prng.cuh:67-76)"""
    return _signed_draw(ctx, rng, 1, n_limbs)


class public_key:
    def __init__(self):
        self.pk = None  # ciphertext at the key level

    def encrypt_asymmetric(self, ctx, pt, seed=None):
        """src/secretkey.cu:20-175: (u pk0 + e0, u pk1 + e1) over all QP primes with a ternary u, ModDown by P,
        then the plaintext added to c0. Levels below the first are reached by dropping limbs."""
        from . import _native, ciphertext
        if self.pk is None:
            raise ValueError("PhantomPublicKey has not been generated")
        rng, _ = _rng_pair(seed)
        n_all, sQ = ctx.size_QP, ctx.size_Q
        u = _signed_draw(ctx, rng, 2, n_all)
        cx = ctx.empty(2, n_all)
        for i in range(2):
            _poly(ctx, 2, n_all, self.pk.data[i], u, cx[i])
            _poly(ctx, 0, n_all, cx[i], _error(ctx, rng, n_all), cx[i])
        out = ctx.empty(2, sQ)
        ws, nbytes = ctx.workspace(_native.OP_MODDOWN, sQ)
        check(LIB.b2_moddown(ctx._h, sQ, 2, cx.data_ptr(), out.data_ptr(), ws.data_ptr(), nbytes, _stream()))
        l = pt._limbs
        data = out[:, :l].contiguous()
        _poly(ctx, 0, l, data[0], pt.data, data[0])
        ct = ciphertext()
        ct._chain_index, ct._size, ct._N, ct._limbs, ct._scale = pt._chain_index, 2, ctx.N, l, pt._scale
        ct._is_asymmetric = True
        ct.data = data
        return ct

    def save(self, stream):
        if self.pk is None:
            raise ValueError("PhantomPublicKey has not been generated")
        self.pk.save(stream)

    def load(self, stream, device=None):
        from . import ciphertext
        self.pk = ciphertext().load(stream, device)
        return self


class secret_key:
    """binding.cu:77-98. `secret_key(ctx)` draws a uniform ternary secret; `generate_sparse` replaces it
    by one with exactly `hamming_weight` non-zero (+-1) coefficients (src/secretkey.cu:513-590)."""

    def __init__(self, ctx=None, seed=None):
        self._rng, self._rng_pub = _rng_pair(seed)  # secret material / public masks
        self.data = None  # [size_QP][N], NTT form, key level
        self.coeffs = None
        if ctx is not None:
            self._set(ctx, self._rng.integers(-1, 2, ctx.N).astype(np.int64))

    def _set(self, ctx, coeffs):
        self.coeffs = coeffs
        self.data = _expand(ctx, coeffs, ctx.size_QP)

    def generate_sparse(self, context, hamming_weight):
        ctx, h = context, int(hamming_weight)
        if not 0 < h <= ctx.N:
            raise ValueError("hamming_weight out of range")
        c = np.zeros(ctx.N, dtype=np.int64)
        pos = self._rng.choice(ctx.N, size=h, replace=False)
        c[pos] = self._rng.choice(np.array([-1, 1], dtype=np.int64), size=h)
        self._set(ctx, c)

    # ---- encryption of zero under this secret: (-(a s + e), a) over the first n_limbs primes -------
    def _encrypt_zero(self, ctx, n_limbs):
        a = _uniform(ctx, self._rng_pub, n_limbs)
        e = _error(ctx, self._rng, n_limbs)
        c0 = ctx.empty(n_limbs)
        _poly(ctx, 2, n_limbs, a, self.data[:n_limbs], c0)
        _poly(ctx, 0, n_limbs, c0, e, c0)
        _poly(ctx, 3, n_limbs, c0, None, c0)
        return torch.stack([c0, a])

    def gen_publickey(self, ctx):
        from . import ciphertext
        pk = public_key()
        ct = ciphertext()
        ct._chain_index, ct._size, ct._N, ct._limbs = 0, 2, ctx.N, ctx.size_QP
        ct.data = self._encrypt_zero(ctx, ctx.size_QP)
        pk.pk = ct
        return pk

    def _kswitch_key(self, ctx, new_key, target_chain_index=0):
        """src/secretkey.cu:354-398: one (-(a s + e) + P s' [limb in digit d], a) per digit. With a target chain index
        (src/secretkey.cu:400-472) only the ceil(size_Ql / alpha) digits a key switch at that level or deeper reads are
        made; each is still a key-level ciphertext, the missing ones are never materialised."""
        from . import ciphertext, relin_key
        a, sQ, N = ctx.size_P, ctx.size_Q, ctx.N
        dnum = (sQ + a - 1) // a
        if target_chain_index:
            if target_chain_index < 1 or target_chain_index > sQ:
                raise ValueError("generate_one_kswitch_key_at_level: target_chain_index out of range")
            dnum = ctx.beta(ctx.limbs_at(target_chain_index))
        P = 1
        for p in ctx.primes[sQ:]:
            P *= int(p)
        out = relin_key()
        for d in range(dnum):
            data = self._encrypt_zero(ctx, ctx.size_QP)
            lo, hi = d * a, min((d + 1) * a, sQ)
            fac = torch.from_numpy(np.stack([np.full(N, P % int(ctx.primes[i]), dtype=np.uint64) for i in range(lo, hi)])
                                   .view(np.int64)).to(ctx.device)
            # multiply limb i of new_key by (P mod q_i) and add into c0's limb i
            self._scaled_add(ctx, data[0], new_key, fac, lo, hi)
            ct = ciphertext()
            ct._chain_index, ct._size, ct._N, ct._limbs = 0, 2, N, ctx.size_QP
            ct.data = data
            out.public_keys.append(ct)
        return out

    @staticmethod
    def _scaled_add(ctx, c0, new_key, fac, lo, hi):
        # b2_poly_op works on limbs [0, n): operate on the prefix [0, hi) of scratch copies so that limb i
        # meets prime i, then keep only [lo, hi)
        N = ctx.N
        full_fac = torch.zeros(hi, N, dtype=torch.int64, device=ctx.device)
        full_fac[lo:hi] = fac
        prod = ctx.empty(hi)
        _poly(ctx, 2, hi, new_key[:hi].contiguous(), full_fac, prod)
        summed = ctx.empty(hi)
        _poly(ctx, 0, hi, c0[:hi].contiguous(), prod, summed)
        c0[lo:hi] = summed[lo:hi]

    def gen_relinkey(self, ctx):
        s2 = ctx.empty(ctx.size_QP)
        _poly(ctx, 2, ctx.size_QP, self.data, self.data, s2)
        return self._kswitch_key(ctx, s2)

    def create_one_galois_key(self, ctx, galois_elt_idx, target_chain_index=0):
        """src/secretkey.cu:684-724: the key of one Galois element, with only the digits `target_chain_index` needs
        (0: every digit)"""
        elt = ctx.galois_elts[galois_elt_idx]
        rot = ctx.empty(ctx.size_QP)
        check(LIB.b2_galois_permute(ctx._h, elt, self.data.data_ptr(), rot.data_ptr(), ctx.size_QP, _stream()))
        return self._kswitch_key(ctx, rot, target_chain_index)

    def create_galois_keys(self, ctx):
        """one key per Galois element of the context, same order (src/secretkey.cu:642-682)"""
        from . import galois_key
        return galois_key.from_keys([self.create_one_galois_key(ctx, i) for i in range(len(ctx.galois_elts))])

    def create_galois_keys_per_level(self, ctx, indices, target_chain_indices):
        """src/secretkey.cu:726-775: keys only for the listed Galois-element indices, each with the digits its target
        chain index needs (0: all of them); the other slots stay empty (to be served by fallbacks)."""
        from . import galois_key, relin_key
        if len(indices) != len(target_chain_indices):
            raise ValueError("create_galois_keys_per_level: indices and target_chain_indices must have the same length")
        out = galois_key.from_keys([relin_key() for _ in ctx.galois_elts])
        for idx, target in zip(indices, target_chain_indices):
            if idx >= len(ctx.galois_elts):
                raise IndexError("create_galois_keys_per_level: index out of range")
            out.relin_keys[idx] = self.create_one_galois_key(ctx, idx, int(target))
        return out

    # ---- data path ------------------------------------------------------------------------------------
    def encrypt_symmetric(self, ctx, pt):
        """(c0, c1) = (-(a s + e) + m, a) at the plaintext's level (src/secretkey.cu:236-299, 771-812)"""
        from . import ciphertext
        l = pt._limbs
        data = self._encrypt_zero(ctx, l)
        _poly(ctx, 0, l, data[0], pt.data, data[0])
        ct = ciphertext()
        ct._chain_index, ct._size, ct._N, ct._limbs, ct._scale = pt._chain_index, 2, ctx.N, l, pt._scale
        ct.data = data
        return ct

    def decrypt(self, ctx, ct):
        """m = c0 + c1 s (+ c2 s^2) on the first l limbs of the key-level secret (src/secretkey.cu:883-919)"""
        from . import plaintext
        l = ct._limbs
        s = self.data[:l]
        acc = ct.data[0].clone()
        t = ctx.empty(l)
        sp = s
        for k in range(1, ct._size):
            _poly(ctx, 2, l, ct.data[k], sp, t)
            _poly(ctx, 0, l, acc, t, acc)
            if k + 1 < ct._size:
                nxt = ctx.empty(l)
                _poly(ctx, 2, l, sp.contiguous(), s, nxt)
                sp = nxt
        pt = plaintext()
        pt._chain_index, pt._N, pt._limbs, pt._scale = ct._chain_index, ctx.N, l, ct._scale
        pt.data = acc
        return pt

    # ---- serialisation ------------------------------------------------------------------------------------
    def save(self, stream):
        n_limbs, N = self.data.shape
        stream.write(_SK_HDR.pack(1, N, n_limbs))
        stream.write(self.data.cpu().numpy().view(np.uint64).tobytes())

    def load(self, stream, device=None):
        powers, N, n_limbs = _SK_HDR.unpack(stream.read(_SK_HDR.size))
        # the reference keeps s, s^2, ... once it has made relinearisation keys; only s is needed here
        arr = np.frombuffer(stream.read(powers * n_limbs * N * 8), dtype=np.uint64).reshape(powers, n_limbs, N)[0]
        self.data = torch.from_numpy(arr.view(np.int64).copy()).to(torch.cuda.current_device() if device is None else device)
        return self
