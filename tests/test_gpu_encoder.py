"""The encoder's device kernels (special FFT over the rotation group, rounding, CRT composition) against the host
restatement in encoder_ref.py: coefficients equal up to the rounding of the last bit, composed values exact."""
import numpy as np
import pytest
import torch

import pyPhantom as ph
from pyPhantom._native import LIB, check
from gpu_helpers import make_ctx, stream
import encoder_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,count", [(4096, 2048), (4096, 5), (65536, 32768), (65536, 1000)])
def test_encoded_coefficients_match_the_host_formula(N, count):
    ctx, o = make_ctx(N, [60, 40, 40, 60], 1)
    enc = ph.ckks_encoder(ctx)
    rng = np.random.default_rng(N + count)
    z = rng.uniform(-1, 1, count) + 1j * rng.uniform(-1, 1, count)
    scale = 2.0 ** 40
    got = enc.signed_coefficients(ctx, z, scale, 1)
    want = encoder_ref.signed_coefficients(N, z, scale)
    assert got.dtype == np.int64 and got.shape == (N,)
    # both are double-precision evaluations of the same sums of up to N/2 terms of size 2^40 / (N/2) each
    assert np.abs(got - want).max() <= 1
    assert (got != want).mean() < 0.01
    pt = enc.encode_complex_vector(ctx, z, scale, 1)
    back = enc.decode_complex_vector(ctx, pt)
    assert np.abs(back[:count] - z).max() < 1e-8 and (count == N // 2 or np.abs(back[count:]).max() < 1e-8)
    assert np.abs(back - encoder_ref.decode(ctx, pt)).max() < 1e-10
    # a tensor on the device is taken as it is
    pt2 = enc.encode_complex_vector(ctx, torch.from_numpy(z).cuda(), scale, 1)
    assert torch.equal(pt2.data, pt.data)


@pytest.mark.parametrize("l", [1, 2, 7, 12])
def test_crt_composition_is_exact(l):
    """signed coefficients of up to 62 bits (and the extremes) spread over l limbs come back as exactly those doubles; a
    second plaintext holds values near +-Q/2, where the centring decides the sign"""
    N = 4096
    bits = [60, 40, 41, 42, 43, 44, 45, 46, 58, 59, 50, 36, 60]
    ctx, o = make_ctx(N, bits, 1)
    enc = ph.ckks_encoder(ctx)
    rng = np.random.default_rng(l)
    mag = min(62, sum(bits[:l]) - 2)
    c = rng.integers(-(1 << mag), 1 << mag, N, dtype=np.int64)
    c[:6] = [0, 1, -1, (1 << mag) - 1, -(1 << mag), 12345]
    d = torch.from_numpy(c).cuda()
    res = ctx.empty(l)
    check(LIB.b2_expand_signed(ctx._h, 0, l, d.data_ptr(), res.data_ptr(), 0, stream()))
    out = torch.empty(N // 2, dtype=torch.complex128, device="cuda")
    check(LIB.b2_decode_compose(ctx._h, l, res.data_ptr(), enc._crt_table(ctx, l).data_ptr(), 1.0, out.data_ptr(), stream()))
    got = torch.view_as_real(out).cpu().numpy()
    assert np.array_equal(got[:, 0], c[: N // 2].astype(np.float64)) and np.array_equal(got[:, 1], c[N // 2:].astype(np.float64))
    # values next to the centring threshold: x = floor(Q/2) + delta, residues computed on the host
    primes = [int(q) for q in o.primes[:l]]
    Q = int(np.prod([int(q) for q in primes], dtype=object))
    deltas = [-2, -1, 0, 1, 2, 3]
    xs = [(Q // 2 + dl) % Q for dl in deltas] + [Q - 1, 0, 1]
    host = np.zeros((l, N), dtype=np.uint64)
    for k, x in enumerate(xs):
        for i, q in enumerate(primes):
            host[i, k] = x % q
    res = torch.from_numpy(host.view(np.int64)).cuda()
    check(LIB.b2_decode_compose(ctx._h, l, res.data_ptr(), enc._crt_table(ctx, l).data_ptr(), 1.0, out.data_ptr(), stream()))
    got = torch.view_as_real(out).cpu().numpy()[: len(xs), 0]
    want = [float(x - Q) if x > Q // 2 else float(x) for x in xs]
    assert np.allclose(got, want, rtol=2e-16, atol=0) and all(np.sign(g) == np.sign(w) for g, w in zip(got, want))


def test_decode_at_a_high_level_and_errors():
    N = 8192
    ctx, o = make_ctx(N, [60] + [40] * 9 + [60], 1)
    enc = ph.ckks_encoder(ctx)
    rng = np.random.default_rng(4)
    z = rng.uniform(-8, 8, N // 2) + 1j * rng.uniform(-8, 8, N // 2)
    for chain_index, scale in ((1, 2.0 ** 40), (1, 2.0 ** 55), (6, 2.0 ** 30)):
        pt = enc.encode_complex_vector(ctx, z, scale, chain_index)
        back = enc.decode_complex_vector(ctx, pt)
        assert np.abs(back - z).max() < 1e-5 * (2.0 ** 30 / scale) + 1e-9
        assert np.abs(back - encoder_ref.decode(ctx, pt)).max() < 1e-9
    assert np.abs(enc.decode_double_vector(ctx, enc.encode_double_vector(ctx, z.real, 2.0 ** 40)) - z.real).max() < 1e-7
    with pytest.raises(ValueError, match="empty"):
        enc.encode_complex_vector(ctx, [], 2.0 ** 40)
    with pytest.raises(ValueError, match="exceeds"):
        enc.encode_complex_vector(ctx, np.zeros(N // 2 + 1), 2.0 ** 40)
    with pytest.raises(ValueError, match="scale out of bounds"):
        enc.encode_complex_vector(ctx, z, 2.0 ** 60, ctx.size_Q)   # one 60-bit limb cannot take a 60-bit scale
    with pytest.raises(ValueError, match="too large|above 62 bits"):
        enc.encode_complex_vector(ctx, z * 1e9, 2.0 ** 50, 1)
