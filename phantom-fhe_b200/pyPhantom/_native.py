"""ctypes binding of libb200fhe.so (the C ABI declared in include/b200fhe.h).

There is no CPU fallback: if the shared library is missing or has no CUDA device to run on,
importing or creating a context raises.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libb200fhe.so")

_sz, _u64, _vp, _int, _u32 = ctypes.c_size_t, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32

# name -> (restype, argtypes); mirrors include/b200fhe.h declaration by declaration
SIGNATURES = {
    "b2_last_error": (ctypes.c_char_p, []),
    "b2_version": (_int, []),
    "b2_create_coeff_modulus": (_int, [_sz, _vp, _sz, _vp]),
    "b2_ctx_create": (_int, [_sz, _vp, _sz, _sz, _int, ctypes.POINTER(_vp)]),
    "b2_ctx_destroy": (None, [_vp]),
    "b2_ctx_N": (_sz, [_vp]),
    "b2_ctx_size_Q": (_sz, [_vp]),
    "b2_ctx_size_P": (_sz, [_vp]),
    "b2_ctx_beta": (_sz, [_vp, _sz]),
    "b2_ctx_get_table": (_int, [_vp, _int, _sz, _vp]),
    "b2_workspace_bytes": (_sz, [_vp, _int, _sz]),
    "b2_ntt_forward": (_int, [_vp, _vp, _sz, _sz, _vp]),
    "b2_ntt_inverse": (_int, [_vp, _vp, _sz, _sz, _vp]),
    "b2_modup": (_int, [_vp, _sz, _vp, _vp, _vp, _sz, _vp]),
    "b2_ks_inner_prod": (_int, [_vp, _sz, _vp, _vp, _sz, _vp, _vp]),
    "b2_moddown": (_int, [_vp, _sz, _sz, _vp, _vp, _vp, _sz, _vp]),
    "b2_keyswitch": (_int, [_vp, _sz, _vp, _vp, _sz, _vp, _vp, _sz, _vp]),
    "b2_keyswitch_batch_workspace_bytes": (_sz, [_vp, _sz, _sz]),
    "b2_keyswitch_batch": (_int, [_vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp]),
    "b2_multiply_relin_batch_workspace_bytes": (_sz, [_vp, _sz, _sz]),
    "b2_multiply_relin_rescale_batch": (_int, [_vp, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _int, _vp, _sz, _vp]),
    "b2_special_fft": (_int, [_vp, _vp, _vp, _vp, _vp, _int, ctypes.c_double, _vp]),
    "b2_encode_round": (_int, [_vp, _vp, _vp, _vp]),
    "b2_decode_compose": (_int, [_vp, _sz, _vp, _vp, ctypes.c_double, _vp, _vp]),
    "b2_peer_alloc": (_int, [_sz, ctypes.POINTER(_vp), _vp]),
    "b2_peer_open": (_int, [_vp, ctypes.POINTER(_vp)]),
    "b2_peer_close": (_int, [_vp]),
    "b2_peer_free": (_int, [_vp]),
    "b2_peer_copy": (_int, [_vp, _vp, _sz, _vp]),
    "b2_sample": (_int, [_vp, _int, _vp, _vp, _sz, _sz, _vp, _vp]),
    "b2_tensor_mul": (_int, [_vp, _sz, _vp, _vp, _vp, _vp]),
    "b2_multiply_and_relin": (_int, [_vp, _sz, _vp, _vp, _vp, _sz, _vp, _vp, _sz, _vp]),
    "b2_rescale": (_int, [_vp, _sz, _sz, _vp, _vp, _vp, _sz, _vp]),
    "b2_rescale_rounded": (_int, [_vp, _sz, _sz, _vp, _vp, _vp, _sz, _vp]),
    "b2_rescale_static": (_int, [_vp, _sz, _sz, _vp, _vp, _vp]),
    "b2_galois_elt_from_step": (_u32, [_int, _sz]),
    "b2_galois_prepare": (_int, [_vp, _u32]),
    "b2_galois_permute": (_int, [_vp, _u32, _vp, _vp, _sz, _vp]),
    "b2_apply_galois": (_int, [_vp, _sz, _u32, _vp, _vp, _sz, _vp, _vp, _sz, _vp]),
    "b2_apply_galois_accumulate": (_int, [_vp, _sz, _u32, _vp, _vp, _sz, _vp, _vp, _int, _vp, _sz, _vp]),
    "b2_keyswitch_finish": (_int, [_vp, _sz, _vp, _vp, _vp, _sz, _vp]),
    "b2_hoist_rotations": (_int, [_vp, _sz, _vp, _vp, _sz, _vp, _sz, _vp, _vp, _sz, _vp]),
    "b2_hoisting_sum": (_int, [_vp, _sz, _vp, _vp, _sz, _vp, _sz, _vp, _vp, _sz, _vp]),
    "b2_bsgs_mac": (_int, [_vp, _sz, _sz, _vp, _vp, _vp, _vp]),
    "b2_bsgs_mac_multi": (_int, [_vp, _sz, _sz, _sz, _vp, _vp, _vp, _vp]),
    "b2_expand_single_chain": (_int, [_vp, _sz, _vp, _vp, _vp]),
    "b2_expand_single_chain_batch": (_int, [_vp, _sz, _sz, _vp, _vp, _vp]),
    "b2_expand_signed": (_int, [_vp, _sz, _sz, _vp, _vp, _int, _vp]),
    "b2_poly_op": (_int, [_vp, _int, _sz, _vp, _vp, _vp, _vp]),
    "b2_ct_op": (_int, [_vp, _int, _sz, _sz, _vp, _vp, _vp, _vp]),
    "b2_ct_scalar": (_int, [_vp, _sz, _sz, _vp, _vp, _vp, _vp]),
    "b2_ct_lincomb": (_int, [_vp, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b2_poly_scalar": (_int, [_vp, _int, _sz, _vp, _vp, _vp, _vp]),
    "b2_ctx_set_shard": (_int, [_vp, _int, _int]),
    "b2_shard_limbs": (_int, [_vp, _sz, _vp]),
    "b2_shard_keyswitch_phase": (_int, [_vp, _sz, _int, _vp, _vp, _sz, _vp, _vp, _sz, _vp]),
    "b2_shard_batch_workspace_bytes": (_sz, [_vp, _sz, _sz]),
    "b2_shard_keyswitch_phase_batch": (_int, [_vp, _sz, _int, _sz, _vp, _vp, _sz, _vp, _vp, _sz, _vp]),
    "b2_launch_count": (_u64, []),
    "b2_device_status": (_int, [_vp, _vp]),
    "b2_profile_start": (_int, [_vp]),
    "b2_profile_stop": (_int, [_vp, _vp, _sz, _vp, _vp, _sz, _vp]),
}

OP_MODUP, OP_MODDOWN, OP_KEYSWITCH, OP_RESCALE, OP_MUL_RELIN, OP_ROTATE, OP_HOIST = 1, 2, 3, 4, 5, 6, 7


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype, fn.argtypes = res, args
    return lib


LIB = load()


def check(rc):
    """0 -> ok; negative -> ValueError (the reference throws std::invalid_argument for the same
    misuse, which pybind11 turns into ValueError); positive -> RuntimeError (CUDA failure)."""
    if rc == 0:
        return
    msg = LIB.b2_last_error().decode()
    if rc < 0:
        raise ValueError(msg)
    raise RuntimeError(f"CUDA error {rc}: {msg}")
