"""Shared helpers of the GPU tests: contexts built from a golden case, device upload, hashing."""
import ctypes
import json

import numpy as np
import torch

import pyPhantom as ph
from pyPhantom import _native
from pyPhantom._native import LIB, check
from oracle_lib import Oracle, create_coeff_modulus, limb_hashes


def make_ctx(N, bits, special, galois_elts=()):
    mods = ph.create_coeff_modulus(N, bits)
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(N)
    parms.set_coeff_modulus(mods)
    parms.set_special_modulus_size(special)
    if galois_elts:
        parms.set_galois_elts(list(galois_elts))
    ctx = ph.context(parms)
    o = Oracle(N, [m.value() for m in mods], special)
    return ctx, o


def load_case(path):
    case = json.load(open(path))
    ctx, o = make_ctx(1 << case["logn"], case["bits"], case["special"], case["elts"])
    return case, ctx, o


def dev(arr):
    a = np.ascontiguousarray(arr, dtype=np.uint64).view(np.int64)
    return torch.from_numpy(a).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy().view(np.uint64)


def stream():
    return torch.cuda.current_stream().cuda_stream


def key_dev(key):
    """key: list of [2][size_QP][N] arrays -> (device tensors kept alive, pointer table)"""
    tens = [dev(d) for d in key]
    return tens, np.array([t.data_ptr() for t in tens], dtype=np.uint64)


def hashes(t, N):
    return limb_hashes(host(t), N)
