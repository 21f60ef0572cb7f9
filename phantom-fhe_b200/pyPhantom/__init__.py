"""pyPhantom - the reference's Python surface (python/src/binding.cu) over libb200fhe.so.

Same names, argument meaning and error behaviour as the pybind11 module of the reference for
the CKKS key-switching path: `params`, `create_coeff_modulus`, `context`, `ciphertext`,
`plaintext`, `relin_key`, `galois_key`, and the evaluator functions `multiply`,
`multiply_and_relin`, `relinearize`, `rescale_to_next`, `mod_switch_to_next`, `rotate`,
`rotate_with_key`, `apply_galois`, `apply_galois_with_key`, `hoist_rotations`, `add`, `sub`,
`negate`, `multiply_plain`, `add_plain`, `sub_plain` (binding.cu:56-290). Objects keep the
reference's memory layout ([poly][limb][N] uint64 on the device) and its save()/load() byte
layout (include/ciphertext.h:173-212, include/secretkey.h:192-226, 290-313), so ciphertexts
and keys produced by either library load in the other.

PyTorch is used only for device memory and streams; every computation is a call into the
C ABI. There is no CPU path.
"""
import enum
import io
import struct

import numpy as np
import torch

from . import _native
from ._native import LIB, check

__version__ = "b200-dev"


# ---------------------------------------------------------------------------------------------
# enums and parameter objects (binding.cu:31-67)
# ---------------------------------------------------------------------------------------------
class scheme_type(enum.IntEnum):
    none = 0
    bgv = 1
    bfv = 2
    ckks = 3


none, bgv, bfv, ckks = scheme_type.none, scheme_type.bgv, scheme_type.bfv, scheme_type.ckks


class mul_tech_type(enum.IntEnum):
    none = 0
    behz = 1
    hps = 2
    hps_overq = 3
    hps_overq_leveled = 4


class modulus:
    def __init__(self, value):
        value = int(value)
        if value == 1 or value >> 61:
            raise ValueError("value can be at most 61-bit and cannot be 1")
        self._value = value

    def value(self):
        return self._value

    def __repr__(self):
        return f"modulus({self._value})"


def create_coeff_modulus(poly_modulus_degree, bit_sizes):
    """CoeffModulus::Create (src/host/modulus.cu:80-111)"""
    bits = np.asarray(list(bit_sizes), dtype=np.int32)
    out = np.zeros(len(bits), dtype=np.uint64)
    check(LIB.b2_create_coeff_modulus(int(poly_modulus_degree), bits.ctypes.data, len(bits), out.ctypes.data))
    return [modulus(v) for v in out]


class params:
    def __init__(self, scheme):
        self._scheme = scheme_type(scheme)
        self._N = 0
        self._coeff_modulus = []
        self._special = 1
        self._galois_elts = []
        self._mul_tech = mul_tech_type.behz

    def set_mul_tech(self, t):
        self._mul_tech = mul_tech_type(t)

    def set_poly_modulus_degree(self, n):
        self._N = int(n)

    def set_special_modulus_size(self, s):
        self._special = int(s)

    def set_galois_elts(self, elts):
        self._galois_elts = [int(e) for e in elts]

    def set_coeff_modulus(self, mods):
        self._coeff_modulus = [m if isinstance(m, modulus) else modulus(m) for m in mods]

    def set_plain_modulus(self, m):
        raise ValueError("plain modulus belongs to BFV/BGV, which this engine does not implement")


def get_elt_from_step(step, coeff_count):
    """include/galois.cuh:16-49"""
    elt = int(LIB.b2_galois_elt_from_step(int(step), int(coeff_count)))
    if elt == 0:
        raise ValueError("step count too large")
    return elt


def get_elts_from_steps(steps, coeff_count):
    return [get_elt_from_step(s, coeff_count) for s in steps]


def set_cuda_device(i):
    torch.cuda.set_device(int(i))


def get_cuda_device_count():
    return torch.cuda.device_count()


def _stream():
    return torch.cuda.current_stream().cuda_stream


# ---------------------------------------------------------------------------------------------
# context (binding.cu:72-75; src/context.cu:125-232)
# ---------------------------------------------------------------------------------------------
class context:
    def __init__(self, parms):
        if not isinstance(parms, params):
            raise TypeError("context(params)")
        if parms._scheme != scheme_type.ckks:
            raise ValueError("unsupported scheme")
        if len(parms._coeff_modulus) == 1:
            raise ValueError("The coefficient modulus must be a vector of at least two primes")
        if not torch.cuda.is_available():
            raise RuntimeError("pyPhantom needs a CUDA device: there is no CPU path")
        self.device = torch.cuda.current_device()
        self.N = parms._N
        self.primes = np.array([m.value() for m in parms._coeff_modulus], dtype=np.uint64)
        self.size_QP = len(self.primes)
        self.size_P = parms._special
        self.size_Q = self.size_QP - self.size_P
        h = _native._vp()
        check(LIB.b2_ctx_create(self.N, self.primes.ctypes.data, self.size_QP, self.size_P, self.device,
                                _native.ctypes.byref(h)))
        self._h = h
        # Galois elements: as given, else the power-of-two set (src/galois.cu:52-76)
        self.galois_elts = list(parms._galois_elts) or self._elts_all()
        for e in self.galois_elts:
            check(LIB.b2_galois_prepare(self._h, e))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and LIB is not None:  # LIB is already gone when the interpreter shuts down
            LIB.b2_ctx_destroy(h)
            self._h = None

    def _elts_all(self):
        m = 2 * self.N
        elts = [m - 1]
        pos, neg = 5, pow(5, -1, m)
        for _ in range(self.N.bit_length() - 2):
            elts.append(pos)
            pos = (pos * pos) & (m - 1)
            elts.append(neg)
            neg = (neg * neg) & (m - 1)
        return elts

    def total_parm_size(self):
        return self.size_Q + 1

    def get_first_index(self):
        return 1

    # ---- helpers ----------------------------------------------------------------------------
    def limbs_at(self, chain_index):
        """number of limbs a ciphertext at `chain_index` holds (src/context.cu:145-168)"""
        if chain_index == 0:
            return self.size_QP
        if not 1 <= chain_index <= self.size_Q:
            raise ValueError("chain index out of range")
        return self.size_Q - (chain_index - 1)

    def beta(self, l):
        return int(LIB.b2_ctx_beta(self._h, l))

    def device_status(self):
        """Synchronises the device and returns the status word its kernels set (0 = no bounded wait ran out)."""
        st = _native.ctypes.c_uint32(0)
        check(LIB.b2_device_status(self._h, _native.ctypes.byref(st)))
        return int(st.value)

    def workspace(self, op, l):
        nbytes = int(LIB.b2_workspace_bytes(self._h, op, l))
        return torch.empty(max(nbytes // 8, 1), dtype=torch.int64, device=self.device), nbytes

    def table(self, which, prime_idx):
        out = np.empty(self.N, dtype=np.uint64)
        check(LIB.b2_ctx_get_table(self._h, which, prime_idx, out.ctypes.data))
        return out

    def empty(self, *shape):
        return torch.empty(*shape, self.N, dtype=torch.int64, device=self.device)


# ---------------------------------------------------------------------------------------------
# data carriers (include/ciphertext.h, include/plaintext.h, include/secretkey.h)
# ---------------------------------------------------------------------------------------------
def _to_device(arr, device):
    a = np.array(arr, dtype=np.uint64, order="C", copy=True).view(np.int64)  # own, writable copy for torch
    return torch.from_numpy(a).to(device=device, non_blocking=False)


def _read_exact(stream, n):
    b = stream.read(n)
    if len(b) != n:
        raise ValueError("truncated stream")
    return b


class ciphertext:
    _HDR = struct.Struct("<QQQQdQQ??")  # chain, size, N, limbs, scale, correction, noiseScaleDeg, ntt, asym

    def __init__(self):
        self._chain_index = 0
        self._size = 0
        self._N = 0
        self._limbs = 0
        self._scale = 1.0
        self._correction_factor = 1
        self._noise_scale_deg = 1
        self._is_ntt_form = True
        self._is_asymmetric = False
        self.data = None  # torch.int64 [size][limbs][N] on the device

    # reference surface (binding.cu:192-196)
    def set_scale(self, s):
        self._scale = float(s)

    def chain_index(self):
        return self._chain_index

    def scale(self):
        return self._scale

    # extras shared with the C++ class
    def size(self):
        return self._size

    def coeff_modulus_size(self):
        return self._limbs

    def poly_modulus_degree(self):
        return self._N

    def is_ntt_form(self):
        return self._is_ntt_form

    @classmethod
    def from_numpy(cls, ctx, arr, chain_index, scale=1.0, ntt=True):
        arr = np.ascontiguousarray(arr, dtype=np.uint64)
        if arr.ndim != 3 or arr.shape[2] != ctx.N or arr.shape[1] != ctx.limbs_at(chain_index):
            raise ValueError("array must be [size][limbs at chain_index][N]")
        ct = cls()
        ct._chain_index, ct._size, ct._N, ct._limbs = chain_index, arr.shape[0], ctx.N, arr.shape[1]
        ct._scale, ct._is_ntt_form = float(scale), bool(ntt)
        ct.data = _to_device(arr, ctx.device)
        return ct

    def numpy(self):
        return self.data.cpu().numpy().view(np.uint64)

    def _like(self, data, chain_index=None, scale=None):
        ct = ciphertext()
        ct.__dict__.update(self.__dict__)
        ct.data = data
        ct._size, ct._limbs = data.shape[0], data.shape[1]
        if chain_index is not None:
            ct._chain_index = chain_index
        if scale is not None:
            ct._scale = scale
        return ct

    def clone(self):
        return self._like(self.data.clone())

    def save(self, stream):
        """include/ciphertext.h:173-191"""
        stream.write(self._HDR.pack(self._chain_index, self._size, self._N, self._limbs, self._scale,
                                    self._correction_factor, self._noise_scale_deg, self._is_ntt_form,
                                    self._is_asymmetric))
        stream.write(self.numpy().tobytes())

    def load(self, stream, device=None):
        """include/ciphertext.h:193-212"""
        (self._chain_index, self._size, self._N, self._limbs, self._scale, self._correction_factor,
         self._noise_scale_deg, self._is_ntt_form, self._is_asymmetric) = self._HDR.unpack(
            _read_exact(stream, self._HDR.size))
        n = self._size * self._limbs * self._N
        arr = np.frombuffer(_read_exact(stream, n * 8), dtype=np.uint64).reshape(self._size, self._limbs, self._N)
        self.data = _to_device(arr, torch.cuda.current_device() if device is None else device)
        return self


class plaintext:
    _HDR = struct.Struct("<QQQd")  # chain, N, limbs, scale (include/plaintext.h:73-85)

    def __init__(self):
        self._chain_index = 0
        self._N = 0
        self._limbs = 0
        self._scale = 1.0
        self.data = None  # [limbs][N]

    def chain_index(self):
        return self._chain_index

    def scale(self):
        return self._scale

    def set_scale(self, s):
        self._scale = float(s)

    @classmethod
    def from_numpy(cls, ctx, arr, chain_index, scale=1.0):
        arr = np.ascontiguousarray(arr, dtype=np.uint64)
        pt = cls()
        pt._chain_index, pt._N, pt._limbs, pt._scale = chain_index, ctx.N, arr.shape[0], float(scale)
        pt.data = _to_device(arr, ctx.device)
        return pt

    def save(self, stream):
        stream.write(self._HDR.pack(self._chain_index, self._N, self._limbs, self._scale))
        stream.write(self.data.cpu().numpy().view(np.uint64).tobytes())

    def load(self, stream, device=None):
        self._chain_index, self._N, self._limbs, self._scale = self._HDR.unpack(_read_exact(stream, self._HDR.size))
        arr = np.frombuffer(_read_exact(stream, self._limbs * self._N * 8), dtype=np.uint64).reshape(self._limbs, self._N)
        self.data = _to_device(arr, torch.cuda.current_device() if device is None else device)
        return self


class relin_key:
    """dnum public keys, each a 2-polynomial ciphertext at the key level (include/secretkey.h:116-226)."""

    def __init__(self):
        self.public_keys = []  # list of ciphertext
        self._ptrs = None

    def dnum(self):
        return len(self.public_keys)

    @classmethod
    def from_numpy(cls, ctx, digits):
        k = cls()
        k.public_keys = [ciphertext.from_numpy(ctx, d, 0) for d in digits]
        return k

    def pointer_table(self):
        if self._ptrs is None or len(self._ptrs) != len(self.public_keys):
            self._ptrs = np.array([pk.data.data_ptr() for pk in self.public_keys], dtype=np.uint64)
        return self._ptrs

    def mod_drop_to_inplace(self, context, target_chain_index):
        """src/secretkey.cu:301-352: keep only the ceil(size_Ql / alpha) digits a key switch at `target_chain_index` (or any
        deeper level) reads; the digits beyond are released. A key that already has that many digits is left alone."""
        if not self.public_keys:
            raise ValueError("mod_drop_to_inplace: KSK not generated")
        ctx = context
        if target_chain_index < 1 or target_chain_index > ctx.size_Q:
            raise ValueError("mod_drop_to_inplace: target_chain_index out of range")
        beta_k = ctx.beta(ctx.limbs_at(target_chain_index))
        if beta_k > len(self.public_keys):
            raise RuntimeError("mod_drop_to_inplace: target chain requires more dnum entries than KSK has")
        if beta_k < len(self.public_keys):
            del self.public_keys[beta_k:]
            self._ptrs = None

    def device_bytes(self):
        return sum(pk.data.numel() * 8 for pk in self.public_keys)

    def save(self, stream):
        if not self.public_keys:
            raise ValueError("PhantomRelinKey has not been generated")
        stream.write(struct.pack("<Q", len(self.public_keys)))
        for pk in self.public_keys:
            pk.save(stream)

    def load(self, stream, device=None):
        (dnum,) = struct.unpack("<Q", _read_exact(stream, 8))
        self.public_keys = [ciphertext().load(stream, device) for _ in range(dnum)]
        self._ptrs = None
        return self


class galois_key:
    """one relin-style key per Galois element of the context, same order (include/secretkey.h:231-316)."""

    def __init__(self):
        self.relin_keys = []
        self.fallback_relin_keys = []  # non-owning, indexed like relin_keys (include/secretkey.h:236-246)

    @classmethod
    def from_keys(cls, keys):
        g = cls()
        g.relin_keys = list(keys)
        return g

    def get_relin_keys(self, index):
        return self.relin_keys[index]

    def resolve(self, index):
        """owned key if populated, else the registered fallback, else None (include/secretkey.h:266-274)"""
        if index < len(self.relin_keys) and self.relin_keys[index].dnum() > 0:
            return self.relin_keys[index]
        if index < len(self.fallback_relin_keys) and self.fallback_relin_keys[index] is not None:
            return self.fallback_relin_keys[index]
        return None

    def set_fallback(self, index, ksk):
        """include/secretkey.h:278-286"""
        if len(self.fallback_relin_keys) < len(self.relin_keys):
            self.fallback_relin_keys += [None] * (len(self.relin_keys) - len(self.fallback_relin_keys))
        if index >= len(self.fallback_relin_keys):
            raise IndexError("PhantomGaloisKey::set_fallback: index out of range")
        self.fallback_relin_keys[index] = ksk

    def save(self, stream):
        if not self.relin_keys:
            raise ValueError("PhantomGaloisKey has not been generated")
        stream.write(struct.pack("<Q", len(self.relin_keys)))
        for k in self.relin_keys:
            k.save(stream)  # an empty slot throws, like the reference (include/secretkey.h:290-302)

    def load(self, stream, device=None):
        (n,) = struct.unpack("<Q", _read_exact(stream, 8))
        self.relin_keys = [relin_key().load(stream, device) for _ in range(n)]
        return self


# ---------------------------------------------------------------------------------------------
# evaluator (binding.cu:198-290; src/evaluate.cu)
# ---------------------------------------------------------------------------------------------
def _are_close(a, b):
    # src/evaluate.cu:80-83 (are_close<double>)
    scale = max(abs(a), abs(b), 1.0)
    return abs(a - b) < np.finfo(np.float64).eps * scale


def _check_pair(a, b):
    if a._chain_index != b._chain_index:
        raise ValueError("encrypted1 and encrypted2 parameter mismatch")
    if a._is_ntt_form != b._is_ntt_form:
        raise ValueError("NTT form mismatch")
    if not _are_close(a._scale, b._scale):
        raise ValueError("scale mismatch")
    if a._size != b._size:
        raise ValueError("poly number mismatch")


def _limb_op(ctx, op, a, b, out):
    """a, b, out: [size][l][N] tensors; the library maps limb i to prime i, so go per polynomial"""
    if a.is_contiguous() and out.is_contiguous() and (b is None or b.is_contiguous()) and a.shape[0] <= 3:
        check(LIB.b2_ct_op(ctx._h, op, a.shape[1], a.shape[0], a.data_ptr(), 0 if b is None else b.data_ptr(), out.data_ptr(), _stream()))
        return
    for p in range(a.shape[0]):
        check(LIB.b2_poly_op(ctx._h, op, a.shape[1], a[p].data_ptr(), 0 if b is None else b[p].data_ptr(),
                             out[p].data_ptr(), _stream()))


def negate(ctx, ct):
    out = torch.empty_like(ct.data)
    _limb_op(ctx, 3, ct.data, None, out)
    return ct._like(out)


def add(ctx, a, b):
    _check_pair(a, b)
    out = torch.empty_like(a.data)
    _limb_op(ctx, 0, a.data, b.data, out)
    return a._like(out)


def sub(ctx, a, b, negate=False):
    _check_pair(a, b)
    out = torch.empty_like(a.data)
    if negate:
        _limb_op(ctx, 1, b.data, a.data, out)
    else:
        _limb_op(ctx, 1, a.data, b.data, out)
    return a._like(out)


def add_many(ctx, cts):
    if not cts:
        raise ValueError("encrypteds cannot be empty")
    acc = cts[0]
    for c in cts[1:]:
        acc = add(ctx, acc, c)
    return acc


def _check_plain(ct, pt):
    if ct._chain_index != pt._chain_index:
        raise ValueError("encrypted and plain parameter mismatch")


def multiply_plain(ctx, ct, pt):
    _check_plain(ct, pt)
    out = torch.empty_like(ct.data)
    l = ct._limbs
    if ct.data.is_contiguous() and ct._size <= 3:
        check(LIB.b2_ct_op(ctx._h, 2, l, ct._size, ct.data.data_ptr(), pt.data.data_ptr(), out.data_ptr(), _stream()))
    else:
        for p in range(ct._size):
            check(LIB.b2_poly_op(ctx._h, 2, l, ct.data[p].data_ptr(), pt.data.data_ptr(), out[p].data_ptr(), _stream()))
    return ct._like(out, scale=ct._scale * pt._scale)


def add_plain(ctx, ct, pt):
    _check_plain(ct, pt)
    if not _are_close(ct._scale, pt._scale):
        raise ValueError("scale mismatch")
    out = ct.data.clone()
    check(LIB.b2_poly_op(ctx._h, 0, ct._limbs, ct.data[0].data_ptr(), pt.data.data_ptr(), out[0].data_ptr(), _stream()))
    return ct._like(out)


def sub_plain(ctx, ct, pt):
    _check_plain(ct, pt)
    if not _are_close(ct._scale, pt._scale):
        raise ValueError("scale mismatch")
    out = ct.data.clone()
    check(LIB.b2_poly_op(ctx._h, 1, ct._limbs, ct.data[0].data_ptr(), pt.data.data_ptr(), out[0].data_ptr(), _stream()))
    return ct._like(out)


def multiply(ctx, a, b):
    """src/evaluate.cu:345-397 (CKKS branch): 2x2 tensor product, scale multiplied"""
    _check_pair(a, b)
    if not (a._is_ntt_form and b._is_ntt_form):
        raise ValueError("encrypted1 and encrypted2 must be in NTT form")
    if a._size != 2:
        raise ValueError("only 2-polynomial operands are built")
    l = a._limbs
    out = ctx.empty(3, l)
    check(LIB.b2_tensor_mul(ctx._h, l, a.data.data_ptr(), b.data.data_ptr(), out.data_ptr(), _stream()))
    return a._like(out, scale=a._scale * b._scale)


def _key_table(ctx, key, l):
    if key.dnum() < ctx.beta(l):
        raise ValueError("key has fewer digits than this level needs")
    return key.pointer_table()


def relinearize(ctx, ct, rlk):
    """src/evaluate.cu:1342-1374"""
    if ct._size != 3:
        raise ValueError("destination_size must be 3")
    if not ct._is_ntt_form:
        raise ValueError("CKKS encrypted must be in NTT form")
    l = ct._limbs
    out = ct.data[:2].clone()
    ws, nbytes = ctx.workspace(_native.OP_KEYSWITCH, l)
    tab = _key_table(ctx, rlk, l)
    check(LIB.b2_keyswitch(ctx._h, l, ct.data[2].data_ptr(), tab.ctypes.data, len(tab), out.data_ptr(),
                           ws.data_ptr(), nbytes, _stream()))
    return ct._like(out)


def relinearize_batch(ctx, data, rlk, ws=None):
    """relinearize (src/evaluate.cu:1342-1374) for a batch of three-polynomial ciphertexts held in one tensor
    data [batch][3][limbs][N], all with the one relinearisation key: data[:, :2] += KeySwitch(data[:, 2]) in place, every
    kernel one launch over the batch (b2_keyswitch_batch). Returns the view data[:, :2]; `ws` (from
    `keyswitch_batch_workspace`) may be passed to keep the call allocation-free."""
    if data.dim() != 4 or data.shape[1] != 3 or not data.is_contiguous():
        raise ValueError("data must be a contiguous [batch][3][limbs][N] tensor")
    batch, l = int(data.shape[0]), int(data.shape[2])
    if ws is None:
        ws = keyswitch_batch_workspace(ctx, l, batch)
    tab = _key_table(ctx, rlk, l)
    check(LIB.b2_keyswitch_batch(ctx._h, l, batch, data[0, 2].data_ptr(), 3 * l, tab.ctypes.data, len(tab), data.data_ptr(), 3 * l,
                                 ws.data_ptr(), ws.numel() * 8, _stream()))
    return data[:, :2]


def multiply_relin_rescale_batch(ctx, a, b, rlk, rescale=True, out=None, ws=None):
    """multiply_and_relin (src/evaluate.cu:1061-1104) followed, if `rescale`, by rescale_to_next (src/evaluate.cu:1413-1464) for a
    batch of ciphertext pairs held as tensors a, b [batch][2][limbs][N], all relinearised with the one key; every kernel is
    one launch over the batch (b2_multiply_relin_rescale_batch). Returns [batch][2][limbs - 1 or limbs][N]; the caller
    keeps track of scale and chain index as for the single calls."""
    if a.dim() != 4 or a.shape != b.shape or a.shape[1] != 2 or not (a.is_contiguous() and b.is_contiguous()):
        raise ValueError("a and b must be contiguous [batch][2][limbs][N] tensors of one shape")
    batch, l = int(a.shape[0]), int(a.shape[2])
    lo = l - 1 if rescale else l
    if out is None:
        out = torch.empty(batch, 2, lo, ctx.N, dtype=torch.int64, device=a.device)
    if ws is None:
        nbytes = int(LIB.b2_multiply_relin_batch_workspace_bytes(ctx._h, l, batch))
        ws = torch.empty(max(nbytes // 8, 1), dtype=torch.int64, device=a.device)
    tab = _key_table(ctx, rlk, l)
    check(LIB.b2_multiply_relin_rescale_batch(ctx._h, l, batch, a.data_ptr(), 2 * l, b.data_ptr(), 2 * l, tab.ctypes.data, len(tab),
                                              out.data_ptr(), 2 * lo, 1 if rescale else 0, ws.data_ptr(), ws.numel() * 8, _stream()))
    return out


def keyswitch_batch_workspace(ctx, l, batch):
    """scratch tensor for `relinearize_batch` / b2_keyswitch_batch at `l` limbs"""
    nbytes = int(LIB.b2_keyswitch_batch_workspace_bytes(ctx._h, l, batch))
    return torch.empty(max(nbytes // 8, 1), dtype=torch.int64, device=ctx.device)


def multiply_and_relin(ctx, a, b, rlk):
    """src/evaluate.cu:1061-1104"""
    _check_pair(a, b)
    if not (a._is_ntt_form and b._is_ntt_form):
        raise ValueError("encrypted1 and encrypted2 must be in NTT form")
    if a._size != 2:
        raise ValueError("only 2-polynomial operands are built")
    l = a._limbs
    out = ctx.empty(2, l)
    ws, nbytes = ctx.workspace(_native.OP_MUL_RELIN, l)
    tab = _key_table(ctx, rlk, l)
    check(LIB.b2_multiply_and_relin(ctx._h, l, a.data.data_ptr(), b.data.data_ptr(), tab.ctypes.data, len(tab),
                                    out.data_ptr(), ws.data_ptr(), nbytes, _stream()))
    return a._like(out, scale=a._scale * b._scale)


def rescale_to_next(ctx, ct):
    """src/evaluate.cu:1582-1602, 1413-1464: drop the last prime with scaling; scale /= q_last"""
    if ct._chain_index == ctx.size_Q:
        raise ValueError("end of modulus switching chain reached")
    l = ct._limbs
    out = ctx.empty(ct._size, l - 1)
    ws, nbytes = ctx.workspace(_native.OP_RESCALE, l)
    check(LIB.b2_rescale(ctx._h, l, ct._size, ct.data.data_ptr(), out.data_ptr(), ws.data_ptr(), nbytes, _stream()))
    return ct._like(out, chain_index=ct._chain_index + 1, scale=ct._scale / float(ctx.primes[l - 1]))


def mod_switch_to_next(ctx, x):
    """src/evaluate.cu:1466-1560: CKKS drops the last limb without scaling"""
    if x._chain_index == ctx.size_Q:
        raise ValueError("end of modulus switching chain reached")
    if isinstance(x, plaintext):
        pt = plaintext()
        pt.__dict__.update(x.__dict__)
        pt.data = x.data[: x._limbs - 1].clone()
        pt._limbs -= 1
        pt._chain_index += 1
        return pt
    if not x._is_ntt_form:
        raise ValueError("CKKS encrypted must be in NTT form")
    return x._like(x.data[:, : x._limbs - 1].contiguous(), chain_index=x._chain_index + 1)


def mod_switch_to(ctx, x, chain_index):
    if x._chain_index > chain_index:
        raise ValueError("cannot switch to higher level modulus")
    while x._chain_index != chain_index:
        x = mod_switch_to_next(ctx, x)
    return x


def mod_switch_to_inplace(ctx, x, chain_index):
    y = mod_switch_to(ctx, x, chain_index)
    x.__dict__.update(y.__dict__)


def _galois_index(ctx, elt):
    try:
        return ctx.galois_elts.index(int(elt))
    except ValueError:
        raise ValueError("Galois elt not present") from None


def apply_galois_with_key(ctx, ct, galois_elt, ksk):
    """src/evaluate.cu:1607-1656"""
    if ct._size > 2:
        raise ValueError("encrypted size must be 2")
    _galois_index(ctx, galois_elt)
    l = ct._limbs
    out = ctx.empty(2, l)
    ws, nbytes = ctx.workspace(_native.OP_ROTATE, l)
    tab = _key_table(ctx, ksk, l)
    check(LIB.b2_apply_galois(ctx._h, l, int(galois_elt), ct.data.data_ptr(), tab.ctypes.data, len(tab),
                              out.data_ptr(), ws.data_ptr(), nbytes, _stream()))
    return ct._like(out)


def apply_galois(ctx, ct, galois_elt, glk):
    """src/evaluate.cu:1658-1675"""
    idx = _galois_index(ctx, galois_elt)
    ksk = glk.resolve(idx)
    if ksk is None:
        raise ValueError("Galois key not present (no owned key, no fallback)")
    return apply_galois_with_key(ctx, ct, galois_elt, ksk)


def _naf(value):
    """non-adjacent form, least significant term first (SEAL's naf(), used by rotate_internal)"""
    res = []
    sign = value < 0
    value = abs(value)
    i = 0
    while value:
        if value & 1:
            zi = 2 - (value & 3)
            value -= zi
            res.append((-zi if sign else zi) * (1 << i))
        value >>= 1
        i += 1
    return res


def rotate(ctx, ct, step, glk):
    """src/evaluate.cu:1683-1713: exact key if present, else a chain of power-of-two rotations"""
    elt = get_elt_from_step(step, ctx.N)
    if elt in ctx.galois_elts:
        return apply_galois(ctx, ct, elt, glk)
    steps = _naf(int(step))
    if len(steps) == 1:
        raise ValueError("Galois key not present")
    for s in steps:
        if abs(s) != ctx.N >> 1:
            ct = rotate(ctx, ct, s, glk)
    return ct


def rotate_with_key(ctx, ct, step, ksk):
    """src/evaluate.cu:1720-1730: direct rotation with a single key"""
    elt = get_elt_from_step(step, ctx.N)
    check(LIB.b2_galois_prepare(ctx._h, elt))
    if elt not in ctx.galois_elts:
        ctx.galois_elts.append(elt)
    return apply_galois_with_key(ctx, ct, elt, ksk)


def hoist_rotations(context, ct, glk, steps):
    """src/evaluate.cu:1929-2082: one ModUp shared by all steps; returns one ciphertext per step"""
    ctx = context
    if ct._size > 2:
        raise ValueError("ciphertext size must be 2")
    steps = list(steps)
    if not steps:
        return []
    l = ct._limbs
    elts = np.array([get_elt_from_step(s, ctx.N) for s in steps], dtype=np.uint32)
    tabs = []
    for e in elts:
        if int(e) not in ctx.galois_elts:
            raise RuntimeError("Galois key not present in hoist_rotations")
        tabs.append(_key_table(ctx, glk.get_relin_keys(ctx.galois_elts.index(int(e))), l))
    n_evk = ctx.beta(l)
    ksk = np.concatenate([t[:n_evk] for t in tabs]).astype(np.uint64)
    outs = [ctx.empty(2, l) for _ in steps]
    out_ptrs = np.array([o.data_ptr() for o in outs], dtype=np.uint64)
    ws, nbytes = ctx.workspace(_native.OP_HOIST, l)
    check(LIB.b2_hoist_rotations(ctx._h, l, ct.data.data_ptr(), elts.ctypes.data, len(steps), ksk.ctypes.data, n_evk,
                                 out_ptrs.ctypes.data, ws.data_ptr(), nbytes, _stream()))
    return [ct._like(o) for o in outs]


def hoisting(context, ct, glk, steps):
    """python/src/binding.cu:285; src/evaluate.cu:1732-1927: the SUM of the rotations of ct by `steps`, from one ModUp and
    one ModDown per polynomial"""
    ctx = context
    if ct._size > 2:
        raise ValueError("ciphertext size must be 2")
    steps = list(steps)
    if not steps:
        raise ValueError("steps cannot be empty")
    l = ct._limbs
    elts = np.array([get_elt_from_step(s, ctx.N) for s in steps], dtype=np.uint32)
    tabs = []
    for e in elts:
        if int(e) not in ctx.galois_elts:
            raise RuntimeError("Galois key not present in hoisting")
        tabs.append(_key_table(ctx, glk.get_relin_keys(ctx.galois_elts.index(int(e))), l))
    n_evk = ctx.beta(l)
    ksk = np.concatenate([t[:n_evk] for t in tabs]).astype(np.uint64)
    out = ctx.empty(2, l)
    ws, nbytes = ctx.workspace(_native.OP_HOIST, l)
    check(LIB.b2_hoisting_sum(ctx._h, l, ct.data.data_ptr(), elts.ctypes.data, len(steps), ksk.ctypes.data, n_evk,
                              out.data_ptr(), ws.data_ptr(), nbytes, _stream()))
    return ct._like(out)


from .keys import public_key, secret_key  # noqa: E402,F401
from .encoder import ckks_encoder  # noqa: E402,F401
from .boot import (bootstrap, bootstrap_eager, bootstrap_key, bootstrap_required_galois_elts, create_bootstrap_key,  # noqa: E402,F401
                        small_bootstrap_key)


# ---------------------------------------------------------------------------------------------
# single-chain plaintexts and the BSGS matrix-vector driver (binding.cu:405-568; src/bsgs.cu)
# ---------------------------------------------------------------------------------------------
class single_chain_plaintext:
    """N signed, centred int64 coefficients in pinned host memory plus a scale
    (include/single_chain_plaintext.h:40-43)."""

    def __init__(self, coeffs=None, scale=1.0):
        self.scale = float(scale)
        self.coeffs = None
        if coeffs is not None:
            t = torch.from_numpy(np.ascontiguousarray(coeffs, dtype=np.int64).copy())
            self.coeffs = t.pin_memory() if torch.cuda.is_available() else t

    def coeffs_bytes(self):
        return self.coeffs.numpy().tobytes()

    def get_scale(self):
        return self.scale

    @property
    def nbytes(self):
        return 0 if self.coeffs is None else self.coeffs.numel() * 8

    @property
    def N(self):
        return 0 if self.coeffs is None else self.coeffs.numel()


def scp_from_bytes(raw, scale):
    """binding.cu:416-516: rebuild a single-chain plaintext from its int64 little-endian bytes"""
    return single_chain_plaintext(np.frombuffer(raw, dtype=np.int64), scale)


def expand_single_chain_to_full(ctx, scp, target_chain_index):
    """src/single_chain_plaintext.cu:93-192: residues in every limb of the level, NTT form"""
    l = ctx.limbs_at(target_chain_index)
    if scp.coeffs.numel() != ctx.N:
        raise ValueError("scp coeff length != N")
    pt = plaintext()
    pt._chain_index, pt._N, pt._limbs, pt._scale = target_chain_index, ctx.N, l, scp.scale
    pt.data = ctx.empty(l)
    d = scp.coeffs.to(ctx.device, non_blocking=True)
    check(LIB.b2_expand_single_chain(ctx._h, l, d.data_ptr(), pt.data.data_ptr(), _stream()))
    return pt


class bsgs_diagonals:
    """include/bsgs.h:14-19: d_pad = baby_steps * giant_steps diagonals, diagonal g*M + b pre-rotated"""

    def __init__(self, diagonals, d_pad, baby_steps, giant_steps):
        self.diagonals, self.d_pad = list(diagonals), int(d_pad)
        self.baby_steps, self.giant_steps = int(baby_steps), int(giant_steps)


def encode_single_chain_plaintext(context, encoder, slots, scale):
    """python/src/binding.cu:405-470; src/single_chain_plaintext.cu:93-192: encode, then keep one signed, centred int64
    coefficient vector instead of the residues in every limb"""
    arr = np.asarray(slots)
    if arr.ndim != 1:
        raise RuntimeError("encode_single_chain_plaintext: array must be 1-D")
    return single_chain_plaintext(encoder.signed_coefficients(context, arr, scale, 1), scale)


def pre_encode_bsgs_diagonals(context, encoder, matrix, num_rows, num_cols, d_pad, baby_steps, scale):
    """python/src/binding.cu:542-553; src/bsgs.cu:100-178: diag[d][t] = padded[t][(t + d) mod d_pad]; diagonal g*M + b is
    pre-rotated by -g*M, tiled over the slots and kept as one signed int64 coefficient vector"""
    m = np.asarray(matrix, dtype=np.float64).ravel()
    if num_rows == 0 or num_cols == 0:
        raise ValueError("pre_encode_bsgs_diagonals: dimensions must be non-zero")
    if m.size != num_rows * num_cols:
        raise ValueError("pre_encode_bsgs_diagonals: matrix size mismatch")
    if d_pad & (d_pad - 1) or d_pad == 0:
        raise ValueError("pre_encode_bsgs_diagonals: d_pad must be a power of 2")
    if d_pad < num_rows or d_pad < num_cols:
        raise ValueError("pre_encode_bsgs_diagonals: d_pad must be >= max(num_rows, num_cols)")
    if baby_steps == 0 or d_pad % baby_steps:
        raise ValueError("pre_encode_bsgs_diagonals: baby_steps must divide d_pad")
    slots = encoder.slot_count()
    if slots % d_pad:
        raise ValueError("pre_encode_bsgs_diagonals: num_slots must be multiple of d_pad")
    padded = np.zeros((d_pad, d_pad))
    padded[:num_rows, :num_cols] = m.reshape(num_rows, num_cols)
    t = np.arange(d_pad)
    out = []
    for g in range(d_pad // baby_steps):
        for b in range(baby_steps):
            d = g * baby_steps + b
            diag = padded[t, (t + d) % d_pad]
            row = np.tile(np.roll(diag, g * baby_steps), slots // d_pad)  # entry i takes diag[(i - g*M) mod d_pad]
            out.append(single_chain_plaintext(encoder.signed_coefficients(context, row, scale, 1), scale))
    return bsgs_diagonals(out, d_pad, baby_steps, d_pad // baby_steps)


class complex_fold_mode(enum.IntEnum):
    """include/bsgs.h:81-96"""
    Rows = 0      # rows i and i + ceil(rows/2) become the real and imaginary part of one row
    ColsConj = 1  # columns j and j + ceil(cols/2) become one complex column, imaginary part negated


class complex_bsgs_diagonals:
    """include/bsgs.h:77-79: the same container, its plaintexts carry complex slots"""

    def __init__(self, inner):
        self.inner = inner


def pre_encode_bsgs_diagonals_complex(ctx, encoder, matrix, num_rows, num_cols, d_pad, baby_steps, scale, fold_mode):
    """python/src/binding.cu:574-587; src/bsgs.cu:373-515: fold the real matrix into a complex one of half the rows (or
    half the columns), then the diagonals as in pre_encode_bsgs_diagonals with complex slot values"""
    m = np.asarray(matrix, dtype=np.float64).ravel()
    if num_rows == 0 or num_cols == 0:
        raise ValueError("pre_encode_bsgs_diagonals_complex: dimensions must be non-zero")
    if m.size != num_rows * num_cols:
        raise ValueError("pre_encode_bsgs_diagonals_complex: matrix size mismatch")
    if d_pad & (d_pad - 1) or d_pad == 0:
        raise ValueError("pre_encode_bsgs_diagonals_complex: d_pad must be a power of 2")
    if baby_steps == 0 or d_pad % baby_steps:
        raise ValueError("pre_encode_bsgs_diagonals_complex: baby_steps must divide d_pad")
    m = m.reshape(num_rows, num_cols)
    if complex_fold_mode(fold_mode) == complex_fold_mode.Rows:
        half = (num_rows + 1) // 2
        w = np.zeros((half, num_cols), dtype=np.complex128)
        w.real = m[:half]
        w.imag[: num_rows - half] = m[half:]
    else:
        half = (num_cols + 1) // 2
        w = np.zeros((num_rows, half), dtype=np.complex128)
        w.real = m[:, :half]
        w.imag[:, : num_cols - half] = -m[:, half:]
    if d_pad < w.shape[0] or d_pad < w.shape[1]:
        raise ValueError("pre_encode_bsgs_diagonals_complex: d_pad must be >= max(folded_rows, folded_cols)")
    slots = encoder.slot_count()
    if slots % d_pad:
        raise ValueError("pre_encode_bsgs_diagonals_complex: num_slots must be multiple of d_pad")
    padded = np.zeros((d_pad, d_pad), dtype=np.complex128)
    padded[: w.shape[0], : w.shape[1]] = w
    t = np.arange(d_pad)
    out = []
    for g in range(d_pad // baby_steps):
        for b in range(baby_steps):
            diag = padded[t, (t + g * baby_steps + b) % d_pad]
            row = np.tile(np.roll(diag, g * baby_steps), slots // d_pad)
            out.append(single_chain_plaintext(encoder.signed_coefficients(ctx, row, scale, 1), scale))
    return complex_bsgs_diagonals(bsgs_diagonals(out, d_pad, baby_steps, d_pad // baby_steps))


def bsgs_required_steps(baby_steps):
    """src/bsgs.cu:180-191"""
    if baby_steps <= 1:
        return []
    steps, s = [], 1
    while s < baby_steps:
        steps.append(s)
        s <<= 1
    steps.append(int(baby_steps))
    return steps


def compute_bsgs_babies(ctx, galois_key_, x, baby_steps):
    """src/bsgs.cu:194-214: babies[b] = rotate(babies[b - msb(b)], msb(b)) - chained, not hoisted"""
    if baby_steps == 0:
        raise ValueError("compute_bsgs_babies: baby_steps must be > 0")
    babies = [x]
    for b in range(1, baby_steps):
        bit = 1 << (b.bit_length() - 1)
        babies.append(rotate(ctx, babies[b - bit], bit, galois_key_))
    return babies


def bsgs_apply_giants_with_babies(ctx, galois_key_, babies, diags):
    """src/bsgs.cu:216-359: per giant expand M plaintexts and run the fused MAC; Horner
    acc = rotate(acc, M) + partial_g from the last giant down; one rescale; scale reset to x's."""
    M, G = diags.baby_steps, diags.giant_steps
    if M == 0 or G == 0 or M * G != diags.d_pad:
        raise ValueError("bsgs_apply_giants_with_babies: M*G must equal d_pad")
    if len(babies) != M:
        raise ValueError("bsgs_apply_giants_with_babies: babies size != baby_steps")
    if len(diags.diagonals) != diags.d_pad:
        raise ValueError("bsgs_apply_giants_with_babies: diagonals size mismatch")
    x = babies[0]
    l, N = x._limbs, ctx.N
    # Two pools of M expanded plaintexts: while the multiply-accumulate and the rotation of one giant run on the
    # caller's stream, the next giant's diagonals are copied in and expanded on a second stream.
    main = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    pools = [ctx.empty(M, l) for _ in range(2)]
    stages = [torch.empty(M, N, dtype=torch.int64, device=ctx.device) for _ in range(2)]
    pt_ptrs = [torch.tensor([p[b].data_ptr() for b in range(M)], dtype=torch.int64, device=ctx.device) for p in pools]
    baby_ptrs = torch.tensor([c.data.data_ptr() for c in babies], dtype=torch.int64, device=ctx.device)
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]
    side.wait_stream(main)

    def prepare(g, slot, wait_free):
        with torch.cuda.stream(side):
            if wait_free:
                side.wait_event(free[slot])
            for b in range(M):
                scp = diags.diagonals[g * M + b]
                if scp.coeffs.numel() != N:
                    raise ValueError("bsgs_apply_giants_with_babies: scp coeff length != N")
                stages[slot][b].copy_(scp.coeffs, non_blocking=True)
            check(LIB.b2_expand_single_chain_batch(ctx._h, l, M, stages[slot].data_ptr(), pools[slot].data_ptr(), side.cuda_stream))
            ready[slot].record(side)

    def partial(g, slot):
        main.wait_event(ready[slot])
        out = ctx.empty(2, l)
        check(LIB.b2_bsgs_mac(ctx._h, l, M, pt_ptrs[slot].data_ptr(), baby_ptrs.data_ptr(), out.data_ptr(), _stream()))
        free[slot].record(main)
        return x._like(out, scale=x._scale * diags.diagonals[g * M].scale)

    order = list(range(G - 1, -1, -1))
    prepare(order[0], 0, False)
    acc = None
    for i, g in enumerate(order):
        if i + 1 < len(order):
            prepare(order[i + 1], (i + 1) & 1, i >= 1)
        part = partial(g, i & 1)
        acc = part if acc is None else add(ctx, rotate(ctx, acc, M, galois_key_), part)
    main.wait_stream(side)
    acc = rescale_to_next(ctx, acc)
    acc.set_scale(x._scale)
    return acc


def bsgs_matmul_preencoded(ctx, galois_key_, x, diags):
    """src/bsgs.cu:361-367"""
    return bsgs_apply_giants_with_babies(ctx, galois_key_, compute_bsgs_babies(ctx, galois_key_, x, diags.baby_steps), diags)


def bsgs_matmul_preencoded_complex(ctx, galois_key_, x, diags):
    """src/bsgs.cu:517-524: the BSGS structure does not change for complex diagonals"""
    return bsgs_matmul_preencoded(ctx, galois_key_, x, diags.inner)


def bsgs_apply_giants_with_babies_complex(ctx, galois_key_, babies, diags):
    return bsgs_apply_giants_with_babies(ctx, galois_key_, babies, diags.inner)


from .engine import ckks_engine, ckks_engine_config  # noqa: E402,F401
from .blocks import eval_polynomial, inner_sum, replicate  # noqa: E402,F401
from .model_blocks import (compute_qkt, finalize_softmax, mlp_forward, mlp_forward_complex, mlp_weights,  # noqa: E402,F401
                           mlp_weights_complex, ps_exp_init, rmsnorm_forward, rmsnorm_params, rmsnorm_weights,
                           score_times_v, softmax_correct, square_iterations_damped_inplace, square_iterations_inplace)
