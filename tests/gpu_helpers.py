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


def mt19937_64_doubles(seed, count, lo, hi):
    """std::mt19937_64(seed) drawn through std::uniform_real_distribution<double>(lo, hi) the way libstdc++ does it
    (one 64-bit draw per value, divided by 2^64): the generator the reference's bootstrap test takes its message from
    (test/bootstrap_test.cu:575-583)"""
    nn, mm, mask = 312, 156, (1 << 64) - 1
    mt = [0] * nn
    mt[0] = seed & mask
    for i in range(1, nn):
        mt[i] = (6364136223846793005 * (mt[i - 1] ^ (mt[i - 1] >> 62)) + i) & mask
    out, idx = np.empty(count), nn
    for k in range(count):
        if idx >= nn:
            for i in range(nn):
                x = (mt[i] & 0xFFFFFFFF80000000) | (mt[(i + 1) % nn] & 0x7FFFFFFF)
                mt[i] = mt[(i + mm) % nn] ^ (x >> 1) ^ (0xB5026F5AA96619E9 if x & 1 else 0)
            idx = 0
        y = mt[idx]
        idx += 1
        y ^= (y >> 29) & 0x5555555555555555
        y ^= (y << 17) & 0x71D67FFFEDA60000
        y ^= (y << 37) & 0xFFF7EEE000000000
        y ^= y >> 43
        u = float(y) / 18446744073709551616.0
        if u >= 1.0:
            u = float(np.nextafter(1.0, 0.0))
        out[k] = u * (hi - lo) + lo
    return out
