"""Host restatement (test infrastructure) of the CKKS encoder's arithmetic, independent of the device kernels: the
embedding as one length-2N complex FFT in numpy, and CRT composition in Python integers
(src/ckks.cu:68-190, src/rns_base.cu:173-234 of the reference)."""
import numpy as np
import torch

from pyPhantom._native import LIB, check


def rotation_positions(N):
    pos, g = np.empty(N // 2, dtype=np.int64), 1
    for j in range(N // 2):
        pos[j] = g
        g = (g * 5) % (2 * N)
    return pos


def signed_coefficients(N, values, scale):
    """coefficient k < N/2 = round(Re u_k), coefficient k + N/2 = round(Im u_k), u_k = (scale/slots) sum_j z_j zeta^(-5^j k)"""
    z = np.asarray(values, dtype=np.complex128).ravel()
    a = np.zeros(2 * N, dtype=np.complex128)
    a[rotation_positions(N)[: z.size]] = z
    u = np.fft.fft(a)[: N // 2] * (scale / (N // 2))
    return np.rint(np.concatenate([u.real, u.imag])).astype(np.int64)


def centred_coefficients(ctx, pt):
    """INTT on the device, then CRT-compose and centre around zero in Python integers"""
    l = pt._limbs
    t = pt.data.clone()
    check(LIB.b2_ntt_inverse(ctx._h, t.data_ptr(), l, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    res = t.cpu().numpy().view(np.uint64)
    primes = [int(q) for q in ctx.primes[:l]]
    Q = 1
    for q in primes:
        Q *= q
    acc = np.zeros(ctx.N, dtype=object)
    for i, q in enumerate(primes):
        hat = Q // q
        y = (res[i].astype(object) * pow(hat % q, -1, q)) % q
        acc = acc + y * hat
    acc = acc % Q
    half = (Q + 1) // 2
    return np.where(acc >= half, acc - Q, acc)


def decode(ctx, pt):
    m = centred_coefficients(ctx, pt)
    N = ctx.N
    b = np.zeros(2 * N, dtype=np.complex128)
    b[:N] = np.array([float(v) for v in m], dtype=np.float64) / pt._scale
    return (np.fft.ifft(b) * (2 * N))[rotation_positions(N)]
