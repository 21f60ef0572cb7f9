"""ctypes binding of the CPU oracle (oracle/libckks_oracle.so) for the test-suite.

The oracle is test infrastructure: it restates the reference's arithmetic for the
key-switching path on the CPU and is pinned by the records in tests/golden/, which were
produced by the unmodified reference library on a GPU (tests/golden/make_golden.sh).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_DIR = os.path.join(os.path.dirname(_HERE), "oracle")
_LIB_PATH = os.path.join(_ORACLE_DIR, "libckks_oracle.so")

_c = ctypes
_sz, _u64, _vp, _int, _u32 = _c.c_size_t, _c.c_uint64, _c.c_void_p, _c.c_int, _c.c_uint32


def _build():
    src = os.path.join(_ORACLE_DIR, "ckks_oracle.c")
    if (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _ORACLE_DIR, "oracle"], stdout=subprocess.DEVNULL)


def _load():
    _build()
    L = ctypes.CDLL(_LIB_PATH)
    sig = {
        "ora_create_coeff_modulus": (_int, [_sz, _vp, _sz, _vp]),
        "ora_minimal_primitive_root": (_u64, [_u64, _u64]),
        "ora_fill_uniform": (None, [_vp, _sz, _u64, _u64]),
        "ora_fill_limbs": (None, [_vp, _sz, _vp, _sz, _u64, _u64, _u64]),
        "ora_limb_hash": (_u64, [_vp, _sz]),
        "ora_ctx_create": (_vp, [_sz, _vp, _sz, _sz]),
        "ora_ctx_destroy": (None, [_vp]),
        "ora_ctx_twiddle": (_vp, [_vp, _sz]),
        "ora_ctx_itwiddle": (_vp, [_vp, _sz]),
        "ora_ctx_root": (_u64, [_vp, _sz]),
        "ora_beta": (_sz, [_vp, _sz]),
        "ora_ntt_forward": (None, [_vp, _vp, _sz, _sz]),
        "ora_ntt_inverse": (None, [_vp, _vp, _sz, _sz]),
        "ora_modup": (None, [_vp, _sz, _vp, _vp]),
        "ora_ks_inner_prod": (None, [_vp, _sz, _vp, _vp, _vp]),
        "ora_moddown": (None, [_vp, _sz, _vp, _vp]),
        "ora_keyswitch": (None, [_vp, _sz, _vp, _vp, _vp]),
        "ora_tensor_mul": (None, [_vp, _sz, _vp, _vp, _vp]),
        "ora_multiply_and_relin": (None, [_vp, _sz, _vp, _vp, _vp, _vp]),
        "ora_rescale": (None, [_vp, _sz, _sz, _vp, _vp]),
        "ora_rescale_rounded": (None, [_vp, _sz, _sz, _vp, _vp]),
        "ora_galois_elt_from_step": (_u32, [_int, _sz]),
        "ora_galois_perm": (None, [_sz, _u32, _vp]),
        "ora_apply_galois": (None, [_vp, _sz, _u32, _vp, _vp]),
        "ora_hoist_rotations": (None, [_vp, _sz, _vp, _vp, _sz, _vp, _vp]),
        "ora_hoisting_sum": (None, [_vp, _sz, _vp, _vp, _sz, _vp, _vp]),
        "ora_bsgs_mac": (None, [_vp, _sz, _sz, _vp, _vp, _vp]),
        "ora_expand_single_chain": (None, [_vp, _sz, _vp, _vp]),
        "ora_add": (None, [_vp, _sz, _vp, _vp, _vp]),
        "ora_sub": (None, [_vp, _sz, _vp, _vp, _vp]),
        "ora_mul": (None, [_vp, _sz, _vp, _vp, _vp]),
        "ora_num_threads": (_int, []),
        "ora_set_threads": (None, [_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    return L


LIB = _load()


def use_all_cores():
    """Pins the oracle's OpenMP thread count to the cores this process may run on (a launcher's OMP_NUM_THREADS=1 does
    not apply to the timed CPU baseline) and returns that count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    LIB.ora_set_threads(n)
    return int(LIB.ora_num_threads())


def _p(a):
    return a.ctypes.data


def _ptr_array(arrs):
    return np.array([a.ctypes.data for a in arrs], dtype=np.uint64)


def create_coeff_modulus(N, bits):
    b = np.asarray(bits, dtype=np.int32)
    out = np.zeros(len(bits), dtype=np.uint64)
    rc = LIB.ora_create_coeff_modulus(N, _p(b), len(bits), _p(out))
    if rc != 0:
        raise ValueError(f"ora_create_coeff_modulus failed: {rc}")
    return out


def limb_hashes(a, N):
    """per-limb content hashes of a C-contiguous uint64 array viewed as [limbs][N]"""
    a = np.ascontiguousarray(a, dtype=np.uint64).reshape(-1, N)
    return [f"{LIB.ora_limb_hash(_p(a[i]), N):016x}" for i in range(a.shape[0])]


class Oracle:
    """CPU oracle context: Q primes first, then size_P special primes."""

    def __init__(self, N, primes, size_P):
        self.N = int(N)
        self.primes = np.ascontiguousarray(primes, dtype=np.uint64)
        self.size_QP = len(self.primes)
        self.size_P = int(size_P)
        self.size_Q = self.size_QP - self.size_P
        self.h = LIB.ora_ctx_create(self.N, _p(self.primes), self.size_QP, self.size_P)
        if not self.h:
            raise ValueError("ora_ctx_create failed")

    def __del__(self):
        if getattr(self, "h", None):
            LIB.ora_ctx_destroy(self.h)
            self.h = None

    def beta(self, l):
        return int(LIB.ora_beta(self.h, l))

    def twiddle(self, i, inverse=False):
        fn = LIB.ora_ctx_itwiddle if inverse else LIB.ora_ctx_twiddle
        ptr = fn(self.h, i)
        return np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctypes.c_uint64)), shape=(self.N,)).copy()

    # ---- synthetic data -------------------------------------------------------------------
    def fill(self, n_poly, limb_primes, seed, buf):
        """[n_poly][len(limb_primes)][N] synthetic limbs, the rule ref_harness.cu uses"""
        pr = np.ascontiguousarray(limb_primes, dtype=np.uint64)
        out = np.empty((n_poly, len(pr), self.N), dtype=np.uint64)
        for p in range(n_poly):
            LIB.ora_fill_limbs(_p(out[p]), self.N, _p(pr), len(pr), seed, buf, p * len(pr))
        return out

    def synth_ct(self, l, seed, buf, n_poly=2):
        return self.fill(n_poly, self.primes[:l], seed, buf)

    def synth_key(self, beta, seed, buf0):
        """relin-style key: beta digits, each [2][size_QP][N]"""
        return [self.fill(2, self.primes, seed, buf0 + d) for d in range(beta)]

    # ---- ops ------------------------------------------------------------------------------
    def ntt_forward(self, data, first_prime=0):
        d = np.ascontiguousarray(data, dtype=np.uint64).copy().reshape(-1, self.N)
        LIB.ora_ntt_forward(self.h, _p(d), d.shape[0], first_prime)
        return d

    def ntt_inverse(self, data, first_prime=0):
        d = np.ascontiguousarray(data, dtype=np.uint64).copy().reshape(-1, self.N)
        LIB.ora_ntt_inverse(self.h, _p(d), d.shape[0], first_prime)
        return d

    def modup(self, l, c2):
        c2 = np.ascontiguousarray(c2, dtype=np.uint64)
        out = np.empty((self.beta(l), l + self.size_P, self.N), dtype=np.uint64)
        LIB.ora_modup(self.h, l, _p(c2), _p(out))
        return out

    def ks_inner_prod(self, l, digits, key):
        digits = np.ascontiguousarray(digits, dtype=np.uint64)
        ptrs = _ptr_array(key)
        out = np.empty((2, l + self.size_P, self.N), dtype=np.uint64)
        LIB.ora_ks_inner_prod(self.h, l, _p(digits), _p(ptrs), _p(out))
        return out

    def moddown(self, l, cx):
        cx = np.ascontiguousarray(cx, dtype=np.uint64)
        out = np.empty((l, self.N), dtype=np.uint64)
        LIB.ora_moddown(self.h, l, _p(cx), _p(out))
        return out

    def keyswitch(self, l, c2, key, ct):
        c2 = np.ascontiguousarray(c2, dtype=np.uint64)
        ct = np.ascontiguousarray(ct, dtype=np.uint64).copy()
        ptrs = _ptr_array(key)
        LIB.ora_keyswitch(self.h, l, _p(c2), _p(ptrs), _p(ct))
        return ct

    def tensor_mul(self, l, a, b):
        a = np.ascontiguousarray(a, dtype=np.uint64)
        b = np.ascontiguousarray(b, dtype=np.uint64)
        out = np.empty((3, l, self.N), dtype=np.uint64)
        LIB.ora_tensor_mul(self.h, l, _p(a), _p(b), _p(out))
        return out

    def multiply_and_relin(self, l, a, b, key):
        a = np.ascontiguousarray(a, dtype=np.uint64)
        b = np.ascontiguousarray(b, dtype=np.uint64)
        ptrs = _ptr_array(key)
        out = np.empty((2, l, self.N), dtype=np.uint64)
        LIB.ora_multiply_and_relin(self.h, l, _p(a), _p(b), _p(ptrs), _p(out))
        return out

    def rescale(self, l, ct):
        ct = np.ascontiguousarray(ct, dtype=np.uint64)
        n_poly = ct.shape[0]
        out = np.empty((n_poly, l - 1, self.N), dtype=np.uint64)
        LIB.ora_rescale(self.h, l, n_poly, _p(ct), _p(out))
        return out

    def rescale_rounded(self, l, ct):
        ct = np.ascontiguousarray(ct, dtype=np.uint64)
        n_poly = ct.shape[0]
        out = np.empty((n_poly, l - 1, self.N), dtype=np.uint64)
        LIB.ora_rescale_rounded(self.h, l, n_poly, _p(ct), _p(out))
        return out

    def galois_elt(self, step):
        return int(LIB.ora_galois_elt_from_step(step, self.N))

    def galois_perm(self, elt):
        perm = np.empty(self.N, dtype=np.uint32)
        LIB.ora_galois_perm(self.N, elt, _p(perm))
        return perm

    def apply_galois(self, l, elt, key, ct):
        ct = np.ascontiguousarray(ct, dtype=np.uint64).copy()
        ptrs = _ptr_array(key)
        LIB.ora_apply_galois(self.h, l, elt, _p(ptrs), _p(ct))
        return ct

    def hoist_rotations(self, l, ct, elts, keys):
        ct = np.ascontiguousarray(ct, dtype=np.uint64)
        e = np.asarray(elts, dtype=np.uint32)
        tabs = [_ptr_array(k) for k in keys]
        tabptrs = _ptr_array(tabs)
        outs = [np.empty((2, l, self.N), dtype=np.uint64) for _ in elts]
        outptrs = _ptr_array(outs)
        LIB.ora_hoist_rotations(self.h, l, _p(ct), _p(e), len(e), _p(tabptrs), _p(outptrs))
        return outs

    def hoisting_sum(self, l, ct, elts, keys):
        ct = np.ascontiguousarray(ct, dtype=np.uint64)
        e = np.asarray(elts, dtype=np.uint32)
        tabs = [_ptr_array(k) for k in keys]
        tabptrs = _ptr_array(tabs)
        out = np.empty((2, l, self.N), dtype=np.uint64)
        LIB.ora_hoisting_sum(self.h, l, _p(ct), _p(e), len(e), _p(tabptrs), _p(out))
        return out

    def bsgs_mac(self, l, pts, babies):
        pts = [np.ascontiguousarray(p, dtype=np.uint64) for p in pts]
        babies = [np.ascontiguousarray(b, dtype=np.uint64) for b in babies]
        pp, bp = _ptr_array(pts), _ptr_array(babies)
        out = np.empty((2, l, self.N), dtype=np.uint64)
        LIB.ora_bsgs_mac(self.h, l, len(pts), _p(pp), _p(bp), _p(out))
        return out

    def expand_single_chain(self, l, coeffs):
        coeffs = np.ascontiguousarray(coeffs, dtype=np.int64)
        out = np.empty((l, self.N), dtype=np.uint64)
        LIB.ora_expand_single_chain(self.h, l, _p(coeffs), _p(out))
        return out

    def synth_signed(self, seed, buf, bits=40):
        """signed centred coefficients in [-2^(bits-1), 2^(bits-1)): uniform draw minus the offset"""
        u = np.empty(self.N, dtype=np.uint64)
        LIB.ora_fill_uniform(_p(u), self.N, 1 << bits, (seed << 40) ^ (buf << 16))
        return (u.astype(np.int64) - (1 << (bits - 1))).astype(np.int64)

    def bsgs_matmul(self, l, x, diag_coeffs, M, G, keys_by_step):
        """src/bsgs.cu:194-359 composed from the oracle's pieces; keys_by_step: step -> key digits"""
        def rot(ct, step):
            return self.apply_galois(l, self.galois_elt(step), keys_by_step[step], ct)
        babies = [x]
        for b in range(1, M):
            bit = 1 << (b.bit_length() - 1)
            babies.append(rot(babies[b - bit], bit))
        def partial(g):
            pts = [self.expand_single_chain(l, diag_coeffs[g * M + b]) for b in range(M)]
            return self.bsgs_mac(l, pts, babies)
        acc = partial(G - 1)
        for g in range(G - 2, -1, -1):
            acc = rot(acc, M)
            p = partial(g)
            acc = np.stack([self.add(acc[k], p[k]) for k in range(2)])
        return self.rescale(l, acc)

    def add(self, a, b):
        a = np.ascontiguousarray(a, dtype=np.uint64)
        b = np.ascontiguousarray(b, dtype=np.uint64)
        out = np.empty_like(a)
        LIB.ora_add(self.h, a.reshape(-1, self.N).shape[0], _p(a), _p(b), _p(out))
        return out


def golden_case_stages(o, case):
    """Recomputes with the oracle every record of one tests/golden/*.json case.

    Returns {record name: [per-limb hash]} following oracle/ref_harness.cu step by step.
    """
    N, l, seed = o.N, case["level"], case["seed"]
    beta = o.beta(l)
    res = {}
    x = o.fill(1, o.primes, seed, 50)[0]
    res["ntt_fwd"] = limb_hashes(o.ntt_forward(x), N)
    res["ntt_inv"] = limb_hashes(o.ntt_inverse(x), N)
    rlk = o.synth_key(beta, seed, 10)
    c2 = o.fill(1, o.primes[:l], seed, 3)[0]
    up = o.modup(l, c2)
    res["modup"] = limb_hashes(up, N)
    cx = o.ks_inner_prod(l, up, rlk)
    res["inner_prod"] = limb_hashes(cx, N)
    res["moddown0"] = limb_hashes(o.moddown(l, cx[0]), N)
    res["moddown1"] = limb_hashes(o.moddown(l, cx[1]), N)
    a = o.synth_ct(l, seed, 1)
    b = o.synth_ct(l, seed, 2)
    res["keyswitch"] = limb_hashes(o.keyswitch(l, c2, rlk, a), N)
    m = o.multiply_and_relin(l, a, b, rlk)
    res["mul_relin"] = limb_hashes(m, N)
    if l >= 2:
        res["mul_relin_rescale"] = limb_hashes(o.rescale(l, m), N)
        res["rescale"] = limb_hashes(o.rescale(l, a), N)
    keys = [o.synth_key(beta, seed, 100 + 8 * e) for e in range(len(case["elts"]))]
    for e, (step, elt) in enumerate(zip(case["steps"], case["elts"])):
        assert o.galois_elt(step) == elt
        res[f"rotate_{step}"] = limb_hashes(o.apply_galois(l, elt, keys[e], a), N)
    outs = o.hoist_rotations(l, a, case["elts"], keys)
    for step, out in zip(case["steps"], outs):
        res[f"hoist_{step}"] = limb_hashes(out, N)
    res["hoisting_sum"] = limb_hashes(o.hoisting_sum(l, a, case["elts"], keys), N)
    if case.get("bsgs"):
        M, G = case["bsgs"]
        diags = [o.synth_signed(seed, 3000 + d) for d in range(M * G)]
        by_step = dict(zip(case["steps"], keys))
        res["bsgs"] = limb_hashes(o.bsgs_matmul(l, a, diags, M, G, by_step), N)
        res["expand_single_chain"] = limb_hashes(o.expand_single_chain(l, diags[0]), N)
    return res
