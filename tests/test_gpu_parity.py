"""GPU parity: every C-ABI entry point against (a) the hashes the unmodified reference library
recorded on a B200 (tests/golden/*.json) and (b) the CPU oracle, bit for bit, on the same seeded
synthetic limbs. Integer work only: equality is exact, there is no tolerance anywhere."""
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import pyPhantom as ph
from pyPhantom import _native
from pyPhantom._native import LIB, check
from gpu_helpers import dev, hashes, host, key_dev, load_case, make_ctx, stream
from oracle_lib import limb_hashes

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.json")))
IDS = [os.path.basename(p)[:-5] for p in GOLDEN]


def _ws(ctx, op, l):
    return ctx.workspace(op, l)


@pytest.mark.parametrize("logn", [12, 13, 14, 15, 16])
def test_tables_match_oracle(logn):
    N = 1 << logn
    ctx, o = make_ctx(N, [50, 40, 60], 1)
    for i in range(3):
        assert np.array_equal(ctx.table(0, i), o.twiddle(i))
        assert np.array_equal(ctx.table(1, i), o.twiddle(i, inverse=True))
        q = int(o.primes[i])
        w = ctx.table(0, i)[:64]
        ws = ctx.table(2, i)[:64]
        assert [int(x) for x in ws] == [(int(v) << 64) // q for v in w]  # src/host/ntt.cu compute_shoup


@pytest.mark.parametrize("logn", [12, 13, 14, 15, 16, 17])
def test_ntt_against_oracle_and_roundtrip(logn):
    N = 1 << logn
    ctx, o = make_ctx(N, [60, 30, 40, 50, 59, 60], 2)
    x = o.fill(1, o.primes, 5, 50)[0]
    d = dev(x)
    check(LIB.b2_ntt_forward(ctx._h, d.data_ptr(), 6, 0, stream()))
    fwd = host(d).copy()
    assert np.array_equal(fwd, o.ntt_forward(x))
    check(LIB.b2_ntt_inverse(ctx._h, d.data_ptr(), 6, 0, stream()))
    assert np.array_equal(host(d), x)
    # a sub-range of the chain: limbs 2..4 only
    d = dev(x[2:5])
    check(LIB.b2_ntt_inverse(ctx._h, d.data_ptr(), 3, 2, stream()))
    assert np.array_equal(host(d), o.ntt_inverse(x[2:5], first_prime=2))
    # edge values: all zero, all q-1
    edge = np.stack([np.zeros(N, dtype=np.uint64), np.full(N, int(o.primes[1]) - 1, dtype=np.uint64)])
    d = dev(edge)
    check(LIB.b2_ntt_forward(ctx._h, d.data_ptr(), 1, 0, stream()))
    check(LIB.b2_ntt_forward(ctx._h, d[1].data_ptr(), 1, 1, stream()))
    got = host(d)
    assert not got[0].any()
    assert np.array_equal(got[1], o.ntt_forward(edge[1:2], first_prime=1)[0])


def test_largest_degree_key_switch_and_rescale():
    """N = 2^17 (the reference's largest degree, include/host/defines.h:18-23): 17 butterfly stages stretch the lazy
    ranges of every arithmetic class, so the chain holds primes at the top of each class (41 bits: FP64, 46 bits: integer
    without corrections, 60 bits) and the inputs include the all-(q-1) polynomial; transforms, a key switch with a ragged
    last digit, and both rescales against the oracle"""
    N = 131072
    ctx, o = make_ctx(N, [60, 41, 46, 45, 30, 60, 59], 2)
    nq = o.size_Q
    x = o.fill(1, o.primes, 9, 50)[0]
    x[:, 0] = [int(q) - 1 for q in o.primes]
    x[1] = int(o.primes[1]) - 1
    x[2] = int(o.primes[2]) - 1
    d = dev(x)
    check(LIB.b2_ntt_forward(ctx._h, d.data_ptr(), o.size_QP, 0, stream()))
    assert np.array_equal(host(d), o.ntt_forward(x))
    check(LIB.b2_ntt_inverse(ctx._h, d.data_ptr(), o.size_QP, 0, stream()))
    assert np.array_equal(host(d), x)
    for l in (nq, 3):
        beta = o.beta(l)
        key = o.synth_key(beta, 3, 10)
        kt, kp = key_dev(key)
        c2_h, ct_h = o.fill(1, o.primes[:l], 3, 3)[0], o.synth_ct(l, 3, 1)
        c2, ct = dev(c2_h), dev(ct_h)
        ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
        check(LIB.b2_keyswitch(ctx._h, l, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, stream()))
        assert np.array_equal(host(ct), o.keyswitch(l, c2_h, key, ct_h))
        r = ctx.empty(2, l - 1)
        ws, nb = _ws(ctx, _native.OP_RESCALE, l)
        check(LIB.b2_rescale(ctx._h, l, 2, dev(ct_h).data_ptr(), r.data_ptr(), ws.data_ptr(), nb, stream()))
        assert np.array_equal(host(r), o.rescale(l, ct_h))
        check(LIB.b2_rescale_rounded(ctx._h, l, 2, dev(ct_h).data_ptr(), r.data_ptr(), ws.data_ptr(), nb, stream()))
        assert np.array_equal(host(r), o.rescale_rounded(l, ct_h))
    assert ctx.device_status() == 0


@pytest.mark.parametrize("path", GOLDEN, ids=IDS)
def test_every_stage_matches_the_reference(path):
    case, ctx, o = load_case(path)
    N, l, seed, h = o.N, case["level"], case["seed"], ctx._h
    beta, lP, want = o.beta(l), l + o.size_P, case["hashes"]
    s = stream()

    # transforms over the whole chain
    x = o.fill(1, o.primes, seed, 50)[0]
    d = dev(x)
    check(LIB.b2_ntt_forward(h, d.data_ptr(), o.size_QP, 0, s))
    assert hashes(d, N) == want["ntt_fwd"]
    d = dev(x)
    check(LIB.b2_ntt_inverse(h, d.data_ptr(), o.size_QP, 0, s))
    assert hashes(d, N) == want["ntt_inv"]

    # the three stages of the key switch
    rlk = o.synth_key(beta, seed, 10)
    rlk_t, rlk_p = key_dev(rlk)
    c2 = dev(o.fill(1, o.primes[:l], seed, 3)[0])
    up = ctx.empty(beta, lP)
    ws, nb = _ws(ctx, _native.OP_MODUP, l)
    check(LIB.b2_modup(h, l, c2.data_ptr(), up.data_ptr(), ws.data_ptr(), nb, s))
    assert hashes(up, N) == want["modup"]
    cx = ctx.empty(2, lP)
    check(LIB.b2_ks_inner_prod(h, l, up.data_ptr(), rlk_p.ctypes.data, beta, cx.data_ptr(), s))
    assert hashes(cx, N) == want["inner_prod"]
    dn = ctx.empty(2, l)
    ws, nb = _ws(ctx, _native.OP_MODDOWN, l)
    check(LIB.b2_moddown(h, l, 2, cx.data_ptr(), dn.data_ptr(), ws.data_ptr(), nb, s))
    assert hashes(dn[0], N) == want["moddown0"]
    assert hashes(dn[1], N) == want["moddown1"]
    # one polynomial at a time gives the same limbs
    check(LIB.b2_ks_inner_prod(h, l, up.data_ptr(), rlk_p.ctypes.data, beta, cx.data_ptr(), s))
    dn1 = ctx.empty(1, l)
    check(LIB.b2_moddown(h, l, 1, cx[1].data_ptr(), dn1.data_ptr(), ws.data_ptr(), nb, s))
    assert hashes(dn1, N) == want["moddown1"]

    # whole key switch, HMult + relin, rescale
    a_h, b_h = o.synth_ct(l, seed, 1), o.synth_ct(l, seed, 2)
    ct = dev(a_h)
    ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
    check(LIB.b2_keyswitch(h, l, c2.data_ptr(), rlk_p.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, s))
    assert hashes(ct, N) == want["keyswitch"]
    a, b = dev(a_h), dev(b_h)
    m = ctx.empty(2, l)
    ws, nb = _ws(ctx, _native.OP_MUL_RELIN, l)
    check(LIB.b2_multiply_and_relin(h, l, a.data_ptr(), b.data_ptr(), rlk_p.ctypes.data, beta, m.data_ptr(),
                                    ws.data_ptr(), nb, s))
    assert hashes(m, N) == want["mul_relin"]
    if l >= 2:
        ws, nb = _ws(ctx, _native.OP_RESCALE, l)
        r = ctx.empty(2, l - 1)
        check(LIB.b2_rescale(h, l, 2, m.data_ptr(), r.data_ptr(), ws.data_ptr(), nb, s))
        assert hashes(r, N) == want["mul_relin_rescale"]
        check(LIB.b2_rescale(h, l, 2, a.data_ptr(), r.data_ptr(), ws.data_ptr(), nb, s))
        assert hashes(r, N) == want["rescale"]

    # rotations: permute-then-switch, and hoisted (ModUp first, then permute)
    keys = [o.synth_key(beta, seed, 100 + 8 * e) for e in range(len(case["elts"]))]
    kd = [key_dev(k) for k in keys]
    ws, nb = _ws(ctx, _native.OP_ROTATE, l)
    for e, (step, elt) in enumerate(zip(case["steps"], case["elts"])):
        assert ph.get_elt_from_step(step, N) == elt
        out = ctx.empty(2, l)
        check(LIB.b2_apply_galois(h, l, elt, a.data_ptr(), kd[e][1].ctypes.data, beta, out.data_ptr(), ws.data_ptr(), nb, s))
        assert hashes(out, N) == want[f"rotate_{step}"]
    outs = [ctx.empty(2, l) for _ in keys]
    optr = np.array([t.data_ptr() for t in outs], dtype=np.uint64)
    ksk = np.concatenate([k[1] for k in kd])
    elts = np.array(case["elts"], dtype=np.uint32)
    ws, nb = _ws(ctx, _native.OP_HOIST, l)
    check(LIB.b2_hoist_rotations(h, l, a.data_ptr(), elts.ctypes.data, len(elts), ksk.ctypes.data, beta,
                                 optr.ctypes.data, ws.data_ptr(), nb, s))
    for step, out in zip(case["steps"], outs):
        assert hashes(out, N) == want[f"hoist_{step}"]
    summed = ctx.empty(2, l)
    check(LIB.b2_hoisting_sum(h, l, a.data_ptr(), elts.ctypes.data, len(elts), ksk.ctypes.data, beta, summed.data_ptr(), ws.data_ptr(), nb, s))
    assert hashes(summed, N) == want["hoisting_sum"]
    assert np.array_equal(host(a), a_h), "inputs must stay untouched"


@pytest.mark.parametrize("l", [1, 2, 3, 5, 8])
def test_levels_and_ragged_digits_against_oracle(l):
    # alpha = 3 over 8 Q limbs: levels with 1, 2 and 3 digits, last digit of size 1, 2 or 3
    N = 4096
    ctx, o = make_ctx(N, [55, 40, 41, 42, 43, 44, 45, 46, 58, 59, 60], 3)
    beta = o.beta(l)
    key = o.synth_key(beta, 21, 10)
    kt, kp = key_dev(key)
    c2_h, ct_h = o.fill(1, o.primes[:l], 21, 3)[0], o.synth_ct(l, 21, 1)
    c2, ct = dev(c2_h), dev(ct_h)
    ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
    check(LIB.b2_keyswitch(ctx._h, l, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, stream()))
    assert np.array_equal(host(ct), o.keyswitch(l, c2_h, key, ct_h))
    if l >= 2:
        for n_poly in (1, 2, 3):
            x_h = o.fill(n_poly, o.primes[:l], 22, 4)
            r = ctx.empty(n_poly, l - 1)
            ws, nb = _ws(ctx, _native.OP_RESCALE, l)
            check(LIB.b2_rescale(ctx._h, l, n_poly, dev(x_h).data_ptr(), r.data_ptr(), ws.data_ptr(), nb, stream()))
            assert np.array_equal(host(r), o.rescale(l, x_h))
            check(LIB.b2_rescale_rounded(ctx._h, l, n_poly, dev(x_h).data_ptr(), r.data_ptr(), ws.data_ptr(), nb, stream()))
            assert np.array_equal(host(r), o.rescale_rounded(l, x_h))


def test_rounded_rescale_rounds_to_nearest():
    # a small integer polynomial v lifted as v * q_last + e: flooring gives v or v - 1, rounding gives v for |e| < q_last / 2
    N, l = 4096, 3
    ctx, o = make_ctx(N, [50, 40, 40, 60], 1)
    primes = [int(q) for q in o.primes[:l]]
    rng = np.random.default_rng(5)
    v = rng.integers(-1000, 1000, N)
    e = rng.integers(-(primes[-1] // 2) + 1, primes[-1] // 2, N)
    val = [int(a) * primes[-1] + int(b) for a, b in zip(v, e)]
    x_h = np.array([[c % q for c in val] for q in primes], dtype=np.uint64)[None]
    x = dev(x_h)
    check(LIB.b2_ntt_forward(ctx._h, x.data_ptr(), l, 0, stream()))
    r = ctx.empty(1, l - 1)
    ws, nb = _ws(ctx, _native.OP_RESCALE, l)
    check(LIB.b2_rescale_rounded(ctx._h, l, 1, x.data_ptr(), r.data_ptr(), ws.data_ptr(), nb, stream()))
    check(LIB.b2_ntt_inverse(ctx._h, r.data_ptr(), l - 1, 0, stream()))
    want = np.array([[int(a) % q for a in v] for q in primes[:-1]], dtype=np.uint64)[None]
    assert np.array_equal(host(r), want)


def test_per_limb_scalars():
    N, l = 4096, 4
    ctx, o = make_ctx(N, [60, 29, 40, 58, 60], 1)
    a_h = o.fill(1, o.primes[:l], 41, 1)[0]
    a = dev(a_h)
    sc = np.array([int(q) - 3 - i for i, q in enumerate(o.primes[:l])], dtype=np.uint64)
    out = ctx.empty(l)
    check(LIB.b2_poly_scalar(ctx._h, 0, l, a.data_ptr(), sc.ctypes.data, out.data_ptr(), stream()))
    want = np.stack([(a_h[i].astype(object) + int(sc[i])) % int(o.primes[i]) for i in range(l)]).astype(np.uint64)
    assert np.array_equal(host(out), want)
    check(LIB.b2_poly_scalar(ctx._h, 1, l, a.data_ptr(), sc.ctypes.data, out.data_ptr(), stream()))
    want = np.stack([(a_h[i].astype(object) * int(sc[i])) % int(o.primes[i]) for i in range(l)]).astype(np.uint64)
    assert np.array_equal(host(out), want)
    bad = sc.copy()
    bad[1] = o.primes[1]
    with pytest.raises(ValueError):
        check(LIB.b2_poly_scalar(ctx._h, 1, l, a.data_ptr(), bad.ctypes.data, out.data_ptr(), stream()))


def test_ciphertext_wide_ops_and_weighted_sum():
    N, l = 4096, 4
    ctx, o = make_ctx(N, [60, 29, 40, 58, 50, 60], 1)
    primes = [int(q) for q in o.primes]
    a_h, b_h, pt_h = o.synth_ct(l, 51, 1), o.synth_ct(l, 51, 2), o.fill(1, o.primes[:l], 51, 3)[0]
    a, b, pt = dev(a_h), dev(b_h), dev(pt_h)
    out, ref = ctx.empty(2, l), ctx.empty(2, l)
    for op, second in ((0, b), (1, b), (2, pt), (3, None)):
        check(LIB.b2_ct_op(ctx._h, op, l, 2, a.data_ptr(), 0 if second is None else second.data_ptr(), out.data_ptr(), stream()))
        for p in range(2):
            other = 0 if second is None else (second.data_ptr() if op == 2 else second[p].data_ptr())
            check(LIB.b2_poly_op(ctx._h, op, l, a[p].data_ptr(), other, ref[p].data_ptr(), stream()))
        assert torch.equal(out, ref), op
    sc = np.array([q - 5 - i for i, q in enumerate(primes[:l])], dtype=np.uint64)
    check(LIB.b2_ct_scalar(ctx._h, l, 2, a.data_ptr(), sc.ctypes.data, out.data_ptr(), stream()))
    for p in range(2):
        check(LIB.b2_poly_scalar(ctx._h, 1, l, a[p].data_ptr(), sc.ctypes.data, ref[p].data_ptr(), stream()))
    assert torch.equal(out, ref)
    # weighted sum of three terms, one of them held at a higher level (5 limbs per polynomial)
    hi_h = o.synth_ct(5, 51, 4)
    terms_h, limbs = [a_h, b_h, hi_h], np.array([l, l, 5], dtype=np.uint32)
    terms = [dev(t) for t in terms_h]
    ptrs = np.array([t.data_ptr() for t in terms], dtype=np.uint64)
    rng = np.random.default_rng(9)
    w = np.array([[int(rng.integers(0, q)) for q in primes[:l]] for _ in terms], dtype=np.uint64)
    c0 = np.array([int(rng.integers(0, q)) for q in primes[:l]], dtype=np.uint64)
    check(LIB.b2_ct_lincomb(ctx._h, l, 2, 3, ptrs.ctypes.data, limbs.ctypes.data, w.ctypes.data, c0.ctypes.data, out.data_ptr(), stream()))
    want = np.zeros((2, l, N), dtype=object)
    for t, th in enumerate(terms_h):
        for i in range(l):
            want[:, i] += th[:, i].astype(object) * int(w[t, i])
    for i in range(l):
        want[0, i] += int(c0[i])
        want[:, i] %= primes[i]
    assert np.array_equal(host(out), want.astype(np.uint64))
    with pytest.raises(ValueError):
        check(LIB.b2_ct_lincomb(ctx._h, l, 2, 9, ptrs.ctypes.data, limbs.ctypes.data, w.ctypes.data, c0.ctypes.data, out.data_ptr(), stream()))
    low = np.array([l, l - 1, 5], dtype=np.uint32)
    with pytest.raises(ValueError):
        check(LIB.b2_ct_lincomb(ctx._h, l, 2, 3, ptrs.ctypes.data, low.ctypes.data, w.ctypes.data, c0.ctypes.data, out.data_ptr(), stream()))


def test_multi_giant_mac_equals_single_giant_calls():
    N, l, M = 4096, 3, 5
    ctx, o = make_ctx(N, [60, 58, 40, 50, 60], 1)
    babies = [dev(o.synth_ct(l, 71, 10 + b)) for b in range(M)]
    pts = [[dev(o.fill(1, o.primes[:l], 71, 100 + 10 * g + b)[0]) for b in range(M)] for g in range(3)]
    tab = np.zeros((3, M), dtype=np.int64)
    for g in range(3):
        for b in range(M):
            if (g, b) not in ((1, 0), (2, 4)):      # ragged: two giants lack one diagonal each
                tab[g, b] = pts[g][b].data_ptr()
    outs = [ctx.empty(2, l) for _ in range(3)]
    d_tab = torch.from_numpy(tab.ravel().copy()).cuda()
    d_bab = torch.tensor([t.data_ptr() for t in babies], dtype=torch.int64, device="cuda")
    d_out = torch.tensor([t.data_ptr() for t in outs], dtype=torch.int64, device="cuda")
    check(LIB.b2_bsgs_mac_multi(ctx._h, l, M, 3, d_tab.data_ptr(), d_bab.data_ptr(), d_out.data_ptr(), stream()))
    for g in range(3):
        keep = [b for b in range(M) if tab[g, b]]
        p1 = torch.tensor([pts[g][b].data_ptr() for b in keep], dtype=torch.int64, device="cuda")
        b1 = torch.tensor([babies[b].data_ptr() for b in keep], dtype=torch.int64, device="cuda")
        ref = ctx.empty(2, l)
        check(LIB.b2_bsgs_mac(ctx._h, l, len(keep), p1.data_ptr(), b1.data_ptr(), ref.data_ptr(), stream()))
        assert torch.equal(outs[g], ref)
    with pytest.raises(ValueError):
        check(LIB.b2_bsgs_mac_multi(ctx._h, l, M, 5, d_tab.data_ptr(), d_bab.data_ptr(), d_out.data_ptr(), stream()))


def test_batched_expansion_equals_single_calls():
    N, l, M = 4096, 4, 5
    ctx, o = make_ctx(N, [60, 29, 40, 58, 50, 60], 1)
    src_h = np.stack([o.synth_signed(81, 10 + m) for m in range(M)])
    src = torch.from_numpy(src_h).cuda()
    out = ctx.empty(M, l)
    check(LIB.b2_expand_single_chain_batch(ctx._h, l, M, src.data_ptr(), out.data_ptr(), stream()))
    one = ctx.empty(l)
    for m in range(M):
        check(LIB.b2_expand_single_chain(ctx._h, l, src[m].data_ptr(), one.data_ptr(), stream()))
        assert torch.equal(out[m], one)
        assert np.array_equal(host(one), o.expand_single_chain(l, src_h[m]))


def test_rotations_sharing_one_moddown():
    # two rotations accumulated and converted once == the oracle's ModDown of the summed inner products;
    # a single accumulate + finish == b2_apply_galois
    N, l = 4096, 5
    ctx, o = make_ctx(N, [55, 40, 41, 42, 43, 44, 45, 46, 58, 59, 60], 3)
    beta, a, sQ = o.beta(l), o.size_P, 8
    ext_primes = [int(q) for q in o.primes[:l]] + [int(q) for q in o.primes[sQ:]]
    cts = [o.synth_ct(l, 61, 1), o.synth_ct(l, 61, 2)]
    elts = [o.galois_elt(1), o.galois_elt(3)]
    keys = [o.synth_key(beta, 61, 10), o.synth_key(beta, 61, 40)]
    kd = [key_dev(k) for k in keys]
    for e in elts:
        check(LIB.b2_galois_prepare(ctx._h, e))
    want_c0 = np.zeros((l, N), dtype=np.uint64)
    cx_sum = np.zeros((2, l + a, N), dtype=np.uint64)
    for ct_h, e, key in zip(cts, elts, keys):
        perm = o.galois_perm(e)
        pc = ct_h[:, :, perm]
        cx = o.ks_inner_prod(l, o.modup(l, pc[1]), key)
        for t, q in enumerate(ext_primes):
            cx_sum[:, t] = (cx_sum[:, t] + cx[:, t]) % np.uint64(q)
        for t in range(l):
            want_c0[t] = (want_c0[t] + pc[0, t]) % np.uint64(ext_primes[t])
    want = np.stack([o.moddown(l, cx_sum[0]), o.moddown(l, cx_sum[1])])
    for t in range(l):
        want[0, t] = (want[0, t] + want_c0[t]) % np.uint64(ext_primes[t])
    acc, accP = ctx.empty(2, l), ctx.empty(2, a)
    ws, nb = _ws(ctx, _native.OP_ROTATE, l)
    for i, (ct_h, e) in enumerate(zip(cts, elts)):
        check(LIB.b2_apply_galois_accumulate(ctx._h, l, e, dev(ct_h).data_ptr(), kd[i][1].ctypes.data, beta, acc.data_ptr(), accP.data_ptr(),
                                             1 if i == 0 else 0, ws.data_ptr(), nb, stream()))
    check(LIB.b2_keyswitch_finish(ctx._h, l, accP.data_ptr(), acc.data_ptr(), ws.data_ptr(), nb, stream()))
    assert np.array_equal(host(acc), want)
    # one rotation alone
    check(LIB.b2_apply_galois_accumulate(ctx._h, l, elts[0], dev(cts[0]).data_ptr(), kd[0][1].ctypes.data, beta, acc.data_ptr(), accP.data_ptr(), 1,
                                         ws.data_ptr(), nb, stream()))
    check(LIB.b2_keyswitch_finish(ctx._h, l, accP.data_ptr(), acc.data_ptr(), ws.data_ptr(), nb, stream()))
    assert np.array_equal(host(acc), o.apply_galois(l, elts[0], keys[0], cts[0]))


def test_elementwise_tensor_and_bsgs_mac():
    N, l = 8192, 5
    ctx, o = make_ctx(N, [60, 40, 40, 50, 59, 60, 60], 2)
    a_h, b_h = o.synth_ct(l, 31, 1), o.synth_ct(l, 31, 2)
    a, b = dev(a_h), dev(b_h)
    out = ctx.empty(3, l)
    check(LIB.b2_tensor_mul(ctx._h, l, a.data_ptr(), b.data_ptr(), out.data_ptr(), stream()))
    assert np.array_equal(host(out), o.tensor_mul(l, a_h, b_h))
    r = torch.empty_like(a)
    for p in range(2):
        check(LIB.b2_poly_op(ctx._h, 0, l, a[p].data_ptr(), b[p].data_ptr(), r[p].data_ptr(), stream()))
    assert np.array_equal(host(r), np.stack([o.add(a_h[p], b_h[p]) for p in range(2)]))
    # negate: 0 stays 0
    z = dev(np.zeros((1, N), dtype=np.uint64))
    check(LIB.b2_poly_op(ctx._h, 3, 1, z.data_ptr(), 0, z.data_ptr(), stream()))
    assert not host(z).any()
    for M in (1, 3, 40):  # 40 > 32 exercises the mid-sum reduction
        pts_h = [o.fill(1, o.primes[:l], 32, 1000 + i)[0] for i in range(M)]
        bab_h = [o.synth_ct(l, 32, 2000 + i) for i in range(M)]
        pts, bab = [dev(p) for p in pts_h], [dev(x) for x in bab_h]
        pp = torch.tensor([t.data_ptr() for t in pts], dtype=torch.int64).cuda()
        bp = torch.tensor([t.data_ptr() for t in bab], dtype=torch.int64).cuda()
        acc = ctx.empty(2, l)
        check(LIB.b2_bsgs_mac(ctx._h, l, M, pp.data_ptr(), bp.data_ptr(), acc.data_ptr(), stream()))
        assert np.array_equal(host(acc), o.bsgs_mac(l, pts_h, bab_h))


def test_galois_permute_matches_oracle_table():
    N = 4096
    ctx, o = make_ctx(N, [40, 40, 50], 1)
    x_h = o.fill(1, o.primes[:2], 41, 1)[0]
    for step in (1, -1, 5, 0):
        elt = ph.get_elt_from_step(step, N)
        check(LIB.b2_galois_prepare(ctx._h, elt))
        out = ctx.empty(2)
        check(LIB.b2_galois_permute(ctx._h, elt, dev(x_h).data_ptr(), out.data_ptr(), 2, stream()))
        perm = o.galois_perm(elt)
        assert np.array_equal(host(out), x_h[:, perm])


def test_error_behaviour():
    N = 4096
    ctx, o = make_ctx(N, [40, 40, 40, 50, 50], 2)
    h, s = ctx._h, stream()
    x = ctx.empty(2, 3)
    ws, nb = _ws(ctx, _native.OP_KEYSWITCH, 3)
    kt, kp = key_dev(o.synth_key(2, 1, 10))
    with pytest.raises(ValueError, match="size_Ql"):
        check(LIB.b2_keyswitch(h, 4, x.data_ptr(), kp.ctypes.data, 2, x.data_ptr(), ws.data_ptr(), nb, s))
    with pytest.raises(ValueError, match="workspace"):
        check(LIB.b2_keyswitch(h, 3, x[0].data_ptr(), kp.ctypes.data, 2, x.data_ptr(), ws.data_ptr(), 16, s))
    with pytest.raises(ValueError, match="fewer digits"):
        check(LIB.b2_keyswitch(h, 3, x[0].data_ptr(), kp.ctypes.data, 1, x.data_ptr(), ws.data_ptr(), nb, s))
    with pytest.raises(ValueError, match="null"):
        check(LIB.b2_keyswitch(h, 3, 0, kp.ctypes.data, 2, x.data_ptr(), ws.data_ptr(), nb, s))
    with pytest.raises(ValueError, match="limb range"):
        check(LIB.b2_ntt_forward(h, x.data_ptr(), 6, 0, s))
    with pytest.raises(ValueError, match="no prime left"):
        check(LIB.b2_rescale(h, 1, 2, x.data_ptr(), x.data_ptr(), ws.data_ptr(), nb, s))
    with pytest.raises(ValueError, match="not present"):
        check(LIB.b2_galois_permute(h, 12345, x.data_ptr(), ws.data_ptr(), 1, s))
    import ctypes
    hh = ctypes.c_void_p()
    for bad_n in (2048, 1 << 18, 5000):
        assert LIB.b2_ctx_create(bad_n, o.primes.ctypes.data, 5, 2, 0, ctypes.byref(hh)) == -2
    comp = np.array([4097 * 3, int(o.primes[1])], dtype=np.uint64)
    assert LIB.b2_ctx_create(4096, comp.ctypes.data, 2, 1, 0, ctypes.byref(hh)) == -1
    # a buffer that is only 16-byte aligned is refused before any kernel touches it (256-bit accesses)
    with pytest.raises(ValueError, match="32-byte aligned"):
        check(LIB.b2_ntt_forward(h, x.data_ptr() + 16, 1, 0, s))
    torch.cuda.synchronize()


def test_full_size_properties():
    """N = 2^16, 24+8 limbs: size-independent properties on the headline configuration."""
    N = 1 << 16
    bits = [60] + [40] * 23 + [60] * 8
    ctx, o = make_ctx(N, bits, 8)
    h, s = ctx._h, stream()
    x_h = o.fill(1, o.primes, 77, 1)[0]
    y_h = o.fill(1, o.primes, 77, 2)[0]
    x, y = dev(x_h), dev(y_h)
    # round trip
    t = x.clone()
    check(LIB.b2_ntt_forward(h, t.data_ptr(), 32, 0, s))
    fx = t.clone()
    check(LIB.b2_ntt_inverse(h, t.data_ptr(), 32, 0, s))
    assert torch.equal(t, x)
    # linearity: NTT(x + y) = NTT(x) + NTT(y)
    sxy = torch.empty_like(x)
    check(LIB.b2_poly_op(h, 0, 32, x.data_ptr(), y.data_ptr(), sxy.data_ptr(), s))
    check(LIB.b2_ntt_forward(h, sxy.data_ptr(), 32, 0, s))
    fy = y.clone()
    check(LIB.b2_ntt_forward(h, fy.data_ptr(), 32, 0, s))
    lin = torch.empty_like(x)
    check(LIB.b2_poly_op(h, 0, 32, fx.data_ptr(), fy.data_ptr(), lin.data_ptr(), s))
    assert torch.equal(lin, sxy)
    # canonical outputs: every residue below its prime
    fxh = host(fx)
    for i in range(32):
        assert int(fxh[i].max()) < int(o.primes[i])


@pytest.mark.parametrize("env", ["B2_NTT_CLUSTER", "B2_NTT_PIPE"])
def test_optional_transform_kernels(monkeypatch, env):
    """the single-launch cluster transforms and the cp.async-pipelined passes (both opt-in: measured slower than the
    default two-pass kernels) give the same limbs as the reference"""
    monkeypatch.setenv(env, "1")
    path = [p for p in GOLDEN if p.endswith("n16_l5_a8.json")][0]
    case, ctx, o = load_case(path)
    N, l, seed, h = o.N, case["level"], case["seed"], ctx._h
    x = o.fill(1, o.primes, seed, 50)[0]
    d = dev(x)
    check(LIB.b2_ntt_forward(h, d.data_ptr(), o.size_QP, 0, stream()))
    assert hashes(d, N) == case["hashes"]["ntt_fwd"]
    d = dev(x)
    check(LIB.b2_ntt_inverse(h, d.data_ptr(), o.size_QP, 0, stream()))
    assert hashes(d, N) == case["hashes"]["ntt_inv"]
    beta = o.beta(l)
    kt, kp = key_dev(o.synth_key(beta, seed, 10))
    c2 = dev(o.fill(1, o.primes[:l], seed, 3)[0])
    ct = dev(o.synth_ct(l, seed, 1))
    ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
    check(LIB.b2_keyswitch(h, l, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, stream()))
    assert hashes(ct, N) == case["hashes"]["keyswitch"]


@pytest.mark.parametrize("fused", ["all", "fp64", "0"])
@pytest.mark.parametrize("name", ["n16_l5_a8.json", "n16_l24_a8.json"])
def test_inner_product_inside_the_last_forward_pass(monkeypatch, name, fused):
    """At N = 2^16 ModUp's last forward pass multiplies the key in and never stores the digits: for every limb ("all"),
    only for the limbs on FP64 primes (the default; the 60-bit limbs keep the stored pass and the stand-alone
    inner product), or not at all (B2_KS_FUSED_IP=0). All three give the reference's limbs"""
    monkeypatch.setenv("B2_KS_FUSED_IP", "0" if fused == "0" else "1")
    monkeypatch.setenv("B2_KS_FUSED_WIDE", "1" if fused == "all" else "0")
    path = [p for p in GOLDEN if p.endswith(name)][0]
    case, ctx, o = load_case(path)
    N, l, seed, h = o.N, case["level"], case["seed"], ctx._h
    beta = o.beta(l)
    kt, kp = key_dev(o.synth_key(beta, seed, 10))
    c2 = dev(o.fill(1, o.primes[:l], seed, 3)[0])
    ct = dev(o.synth_ct(l, seed, 1))
    ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
    check(LIB.b2_keyswitch(h, l, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, stream()))
    assert hashes(ct, N) == case["hashes"]["keyswitch"]


@pytest.mark.parametrize("case", ["n16_headline", "n16_wide", "n16_l11", "n16_l5", "n16_l1", "n13_fallback"])
def test_batched_key_switch_equals_single_ones(case, monkeypatch):
    """b2_keyswitch_batch (every kernel one launch over a batch that shares the key; strided sets) gives, set by set, the limbs
    of b2_keyswitch - at the headline shape also the oracle's - with the stand-alone inner product for the 60-bit limbs and
    with every limb in the fused pass, at a level with a ragged last digit, and where the fused pipeline does not apply
    (N = 2^13: the sets run one after another)"""
    if case in ("n16_l11", "n16_l5", "n16_l1"):
        monkeypatch.delenv("B2_KS_FUSED_WIDE", raising=False)  # the default: every limb in the fused pass for batched calls only
    else:
        monkeypatch.setenv("B2_KS_FUSED_WIDE", "1" if case == "n16_wide" else "0")
    if case == "n13_fallback":
        N, bits, special, l, batch = 8192, [55, 40, 41, 42, 43, 44, 45, 46, 58, 59, 60], 3, 7, 3
    else:
        N, bits, special, batch = 65536, [60] + [40] * 23 + [60] * 8, 8, 5
        l = {"n16_l11": 11, "n16_l5": 5, "n16_l1": 1}.get(case, 24)  # 5 and 1: a single digit, every Q limb its own
    ctx, o = make_ctx(N, bits, special)
    beta = o.beta(l)
    key = o.synth_key(beta, 5, 10)
    kt, kp = key_dev(key)
    g = torch.Generator(device="cuda")
    g.manual_seed(17)
    # sets of three polynomials (c0, c1, c2) with a gap of one limb between sets: strides are not the packed ones
    stride = 3 * l + 1
    buf = torch.stack([torch.randint(0, int(q), (batch, 4, N), dtype=torch.int64, device="cuda", generator=g) for q in o.primes[:l]], dim=2)
    flat = torch.zeros(batch, stride, N, dtype=torch.int64, device="cuda")
    flat[:, :3 * l] = buf[:, :3].reshape(batch, 3 * l, N)
    want = []
    ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
    for b in range(batch):
        ct = flat[b, :2 * l].clone()
        check(LIB.b2_keyswitch(ctx._h, l, flat[b, 2 * l].data_ptr(), kp.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, stream()))
        want.append(ct)
    if case == "n16_headline":
        c2_h, ct_h = host(flat[0, 2 * l:3 * l]), host(flat[0, :2 * l]).reshape(2, l, N)
        assert np.array_equal(host(want[0]).reshape(2, l, N), o.keyswitch(l, c2_h, key, ct_h))
    nbytes = int(LIB.b2_keyswitch_batch_workspace_bytes(ctx._h, l, batch))
    wsb = torch.empty(nbytes // 8, dtype=torch.int64, device="cuda")
    check(LIB.b2_keyswitch_batch(ctx._h, l, batch, flat[0, 2 * l].data_ptr(), stride, kp.ctypes.data, beta, flat.data_ptr(), stride,
                                 wsb.data_ptr(), nbytes, stream()))
    torch.cuda.synchronize()
    for b in range(batch):
        assert torch.equal(flat[b, :2 * l], want[b]), f"set {b}"
        assert not flat[b, 3 * l].any(), "the gap between sets must stay untouched"
    assert ctx.device_status() == 0
    # a batch of one takes the single-call path and gives the same limbs
    one = torch.zeros(1, stride, N, dtype=torch.int64, device="cuda")
    one[0, :3 * l] = buf[0, :3].reshape(3 * l, N)
    check(LIB.b2_keyswitch_batch(ctx._h, l, 1, one[0, 2 * l].data_ptr(), stride, kp.ctypes.data, beta, one.data_ptr(), stride,
                                 wsb.data_ptr(), nbytes, stream()))
    assert torch.equal(one[0, :2 * l], want[0])
    # a workspace one byte short is refused, as is a stride smaller than the set
    assert LIB.b2_keyswitch_batch(ctx._h, l, batch, flat[0, 2 * l].data_ptr(), stride, kp.ctypes.data, beta, flat.data_ptr(), stride,
                                  wsb.data_ptr(), nbytes - 8, stream()) != 0
    assert LIB.b2_keyswitch_batch(ctx._h, l, batch, flat[0, 2 * l].data_ptr(), l - 1, kp.ctypes.data, beta, flat.data_ptr(), stride,
                                  wsb.data_ptr(), nbytes, stream()) != 0


@pytest.mark.parametrize("shape", ["n16_headline", "n13"])
@pytest.mark.parametrize("rescale", [1, 0])
def test_batched_multiply_relin_rescale_equals_single_calls(shape, rescale):
    """b2_multiply_relin_rescale_batch (tensor product, key switch and rescale each one launch over the batch) against
    b2_multiply_and_relin + b2_rescale pair by pair, whose limbs the reference's hashes pin (mul_relin, mul_relin_rescale)"""
    if shape == "n13":
        N, bits, special, l, batch = 8192, [55, 40, 41, 42, 43, 44, 45, 46, 58, 59, 60], 3, 6, 3
    else:
        N, bits, special, l, batch = 65536, [60] + [40] * 23 + [60] * 8, 8, 24, 4
    ctx, o = make_ctx(N, bits, special)
    beta = o.beta(l)
    kt, kp = key_dev(o.synth_key(beta, 9, 10))
    g = torch.Generator(device="cuda")
    g.manual_seed(23)
    a = torch.stack([torch.randint(0, int(q), (batch, 2, N), dtype=torch.int64, device="cuda", generator=g) for q in o.primes[:l]], dim=2).contiguous()
    b = torch.stack([torch.randint(0, int(q), (batch, 2, N), dtype=torch.int64, device="cuda", generator=g) for q in o.primes[:l]], dim=2).contiguous()
    lo = l - 1 if rescale else l
    want = []
    ws, nb = _ws(ctx, _native.OP_MUL_RELIN, l)
    wr, nr = _ws(ctx, _native.OP_RESCALE, l)
    for i in range(batch):
        m = ctx.empty(2, l)
        check(LIB.b2_multiply_and_relin(ctx._h, l, a[i].data_ptr(), b[i].data_ptr(), kp.ctypes.data, beta, m.data_ptr(), ws.data_ptr(), nb, stream()))
        if rescale:
            r = ctx.empty(2, lo)
            check(LIB.b2_rescale(ctx._h, l, 2, m.data_ptr(), r.data_ptr(), wr.data_ptr(), nr, stream()))
            m = r
        want.append(m)
    stride = 2 * lo + 3  # pairs of the result are not packed
    out = torch.zeros(batch, stride, N, dtype=torch.int64, device="cuda")
    nbytes = int(LIB.b2_multiply_relin_batch_workspace_bytes(ctx._h, l, batch))
    wsb = torch.empty(nbytes // 8, dtype=torch.int64, device="cuda")
    check(LIB.b2_multiply_relin_rescale_batch(ctx._h, l, batch, a.data_ptr(), 2 * l, b.data_ptr(), 2 * l, kp.ctypes.data, beta, out.data_ptr(), stride,
                                              rescale, wsb.data_ptr(), nbytes, stream()))
    torch.cuda.synchronize()
    for i in range(batch):
        assert torch.equal(out[i, :2 * lo].reshape(2, lo, N), want[i]), f"pair {i}"
        assert not out[i, 2 * lo:].any(), "the gap between pairs must stay untouched"
    assert LIB.b2_multiply_relin_rescale_batch(ctx._h, l, batch, a.data_ptr(), 2 * l, b.data_ptr(), 2 * l, kp.ctypes.data, beta, out.data_ptr(), stride,
                                               rescale, wsb.data_ptr(), nbytes - 8, stream()) != 0


@pytest.mark.parametrize("l", [7, 4])
def test_fused_pass_on_every_prime_class(l, monkeypatch):
    """N = 2^16 with Q and P limbs on primes of every arithmetic class (FP64 below 2^41, the lazy integer path below
    2^46, Harvey butterflies above), a ragged last digit at l = 4: the key switch, and the sum of hoisted rotations
    (whose second and later rotations add into the P limbs kept for the shared ModDown), against the oracle"""
    N = 65536
    monkeypatch.setenv("B2_KS_FUSED_WIDE", "1")
    ctx, o = make_ctx(N, [60, 45, 38, 52, 43, 40, 30, 60, 44, 39], 3)
    beta = o.beta(l)
    key = o.synth_key(beta, 77, 10)
    kt, kp = key_dev(key)
    c2_h, ct_h = o.fill(1, o.primes[:l], 77, 3)[0], o.synth_ct(l, 77, 1)
    c2, ct = dev(c2_h), dev(ct_h)
    ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
    check(LIB.b2_keyswitch(ctx._h, l, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, stream()))
    assert np.array_equal(host(ct), o.keyswitch(l, c2_h, key, ct_h))
    elts = [ph.get_elt_from_step(s, N) for s in (1, 5)]
    for e in elts:
        check(LIB.b2_galois_prepare(ctx._h, e))
    keys = [o.synth_key(beta, 77, 100 + 8 * e) for e in range(len(elts))]
    kd = [key_dev(k) for k in keys]
    ksk = np.concatenate([k[1] for k in kd])
    e32 = np.array(elts, dtype=np.uint32)
    summed = ctx.empty(2, l)
    ws, nb = _ws(ctx, _native.OP_HOIST, l)
    check(LIB.b2_hoisting_sum(ctx._h, l, ct.data_ptr(), e32.ctypes.data, len(elts), ksk.ctypes.data, beta, summed.data_ptr(),
                              ws.data_ptr(), nb, stream()))
    assert np.array_equal(host(summed), o.hoisting_sum(l, host(ct), elts, keys))


@pytest.mark.parametrize("mode", ["tc:1", "tc:2", "tc:4", "tcs:1", "tcs:4", "fp", "int"])
@pytest.mark.parametrize("shape", ["n12_ragged", "n16_headline", "n13_many_limbs"])
def test_base_conversion_kernels_agree(mode, shape, monkeypatch):
    """ModUp, ModDown (one and two polynomials) and the whole key switch through each base-conversion kernel - tensor
    cores (persistent pipelined kernel, and "tcs": one CTA per tile) with 1, 2 and 4 warpgroups per CTA, FP64 pieces,
    128-bit integers - against the oracle. The context reads the selection from the environment when it is created."""
    kind, _, wg = mode.partition(":")
    monkeypatch.setenv("B2_BCONV_TC_SIMPLE", "1" if kind == "tcs" else "0")
    monkeypatch.setenv("B2_BCONV", "tc" if kind == "tcs" else kind)
    if wg:
        monkeypatch.setenv("B2_BCONV_WG", wg)
    if shape == "n12_ragged":
        N, bits, special, levels = 4096, [55, 40, 41, 42, 43, 44, 45, 46, 58, 59, 60], 3, [1, 5, 8]
    elif shape == "n16_headline":
        N, bits, special, levels = 65536, [60] + [40] * 23 + [60] * 8, 8, [24, 11]
    else:  # 50 Q limbs in digits of 5: ModDown has 100 outputs (two jobs per polynomial), ModUp digits 50
        N, bits, special, levels = 8192, [60] + [36, 50, 44, 58, 30, 52, 40] * 7 + [60] * 5, 5, [50, 23]
    ctx, o = make_ctx(N, bits, special)
    for l in levels:
        beta, lP = o.beta(l), l + o.size_P
        c2_h, ct_h = o.fill(1, o.primes[:l], 31, 3)[0], o.synth_ct(l, 31, 1)
        c2 = dev(c2_h)
        up = ctx.empty(beta, lP)
        ws, nb = _ws(ctx, _native.OP_MODUP, l)
        check(LIB.b2_modup(ctx._h, l, c2.data_ptr(), up.data_ptr(), ws.data_ptr(), nb, stream()))
        up_h = o.modup(l, c2_h)
        assert np.array_equal(host(up).reshape(up_h.shape), up_h), (mode, l, "modup")
        cx_h = o.fill(2, list(o.primes[:l]) + list(o.primes[o.size_QP - o.size_P:]), 32, 5)
        want = np.stack([o.moddown(l, cx_h[0]), o.moddown(l, cx_h[1])])
        ws, nb = _ws(ctx, _native.OP_MODDOWN, l)
        dn = ctx.empty(2, l)
        check(LIB.b2_moddown(ctx._h, l, 2, dev(cx_h).data_ptr(), dn.data_ptr(), ws.data_ptr(), nb, stream()))
        assert np.array_equal(host(dn), want), (mode, l, "moddown")
        dn1 = ctx.empty(1, l)
        check(LIB.b2_moddown(ctx._h, l, 1, dev(cx_h[1]).data_ptr(), dn1.data_ptr(), ws.data_ptr(), nb, stream()))
        assert np.array_equal(host(dn1)[0], want[1]), (mode, l, "moddown, one polynomial")
        key = o.synth_key(beta, 31, 10)
        kt, kp = key_dev(key)
        ct = dev(ct_h)
        ws, nb = _ws(ctx, _native.OP_KEYSWITCH, l)
        check(LIB.b2_keyswitch(ctx._h, l, c2.data_ptr(), kp.ctypes.data, beta, ct.data_ptr(), ws.data_ptr(), nb, stream()))
        assert np.array_equal(host(ct), o.keyswitch(l, c2_h, key, ct_h)), (mode, l, "keyswitch")
    assert ctx.device_status() == 0
