"""b2_rescale_static: the rescale for callers that cannot provide scratch and must not allocate
(their device memory is already reserved by someone else, or they are not allowed into an
allocating CUDA call at that point). It works out of a fixed array inside the library, so its
result must equal b2_rescale's limb for limb - on the first call on the device, which also looks
up the array's address, and again on a second call that finds the first one's leftovers in it.
Collected last on purpose: a failure here cannot hide any other test under `pytest -x`."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from pyPhantom import _native
from pyPhantom._native import LIB, check
from gpu_helpers import dev, host, make_ctx, stream


def _reference_rescale(ctx, l, x):
    out = ctx.empty(x.shape[0], l - 1)
    ws, nb = ctx.workspace(_native.OP_RESCALE, l)
    check(LIB.b2_rescale(ctx._h, l, x.shape[0], x.data_ptr(), out.data_ptr(), ws.data_ptr(), nb, stream()))
    return host(out).copy()


def test_static_rescale_matches_rescale_twice_in_a_row():
    N, l = 1 << 14, 5
    ctx, o = make_ctx(N, [58, 40, 40, 45, 50, 59, 60], 2)
    a = dev(o.fill(2, o.primes[:l], 91, 1))
    b = dev(o.fill(3, o.primes[:l], 92, 2))
    want_a, want_b = _reference_rescale(ctx, l, a), _reference_rescale(ctx, l, b)
    assert np.array_equal(want_a, o.rescale(l, host(a)))  # and both agree with the oracle
    free_before = torch.cuda.mem_get_info()[0]
    out_a, out_b = ctx.empty(2, l - 1), ctx.empty(3, l - 1)
    torch.cuda.synchronize()
    check(LIB.b2_rescale_static(ctx._h, l, 2, a.data_ptr(), out_a.data_ptr(), stream()))
    check(LIB.b2_rescale_static(ctx._h, l, 3, b.data_ptr(), out_b.data_ptr(), stream()))  # reuses the dirty scratch
    assert np.array_equal(host(out_a), want_a)
    assert np.array_equal(host(out_b), want_b)
    # a third call on the first input again, after the 3-polynomial call dirtied all of the array
    check(LIB.b2_rescale_static(ctx._h, l, 2, a.data_ptr(), out_a.data_ptr(), stream()))
    assert np.array_equal(host(out_a), want_a)
    assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20), "the static variant must not allocate"


def test_static_rescale_rejects_what_does_not_fit():
    ctx, o = make_ctx(4096, [40, 40, 40, 50], 1)
    x = ctx.empty(2, 3)
    with pytest.raises(ValueError, match="at most 3 polynomials"):
        check(LIB.b2_rescale_static(ctx._h, 3, 4, x.data_ptr(), x.data_ptr(), stream()))
    with pytest.raises(ValueError, match="no prime left"):
        check(LIB.b2_rescale_static(ctx._h, 1, 2, x.data_ptr(), x.data_ptr(), stream()))
    with pytest.raises(ValueError, match="null"):
        check(LIB.b2_rescale_static(ctx._h, 3, 2, 0, x.data_ptr(), stream()))
