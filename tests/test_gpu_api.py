"""GPU tests of the pyPhantom mirror (the reference's Python surface): same results as the oracle,
same errors as the reference, and the reference's save()/load() byte layout."""
import io
import struct

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import pyPhantom as ph
from gpu_helpers import make_ctx

N, BITS, SPECIAL = 4096, [55, 40, 41, 42, 43, 44, 58, 59], 2
SCALE = 2.0 ** 40


@pytest.fixture(scope="module")
def env():
    steps = [1, 2, 4, -1]
    elts = [ph.get_elt_from_step(s, N) for s in steps]
    ctx, o = make_ctx(N, BITS, SPECIAL, elts)
    l = o.size_Q
    rlk_h = o.synth_key(o.beta(l), 5, 10)
    glk_h = [o.synth_key(o.beta(l), 5, 100 + 8 * e) for e in range(len(elts))]
    rlk = ph.relin_key.from_numpy(ctx, rlk_h)
    glk = ph.galois_key.from_keys([ph.relin_key.from_numpy(ctx, k) for k in glk_h])
    a_h, b_h = o.synth_ct(l, 5, 1), o.synth_ct(l, 5, 2)
    a = ph.ciphertext.from_numpy(ctx, a_h, 1, SCALE)
    b = ph.ciphertext.from_numpy(ctx, b_h, 1, SCALE)
    return dict(ctx=ctx, o=o, l=l, steps=steps, elts=elts, rlk=rlk, rlk_h=rlk_h, glk=glk, glk_h=glk_h, a=a, b=b,
                a_h=a_h, b_h=b_h)


def test_context_shape(env):
    ctx = env["ctx"]
    assert ctx.total_parm_size() == 7 and ctx.get_first_index() == 1
    assert ctx.limbs_at(0) == 8 and ctx.limbs_at(1) == 6 and ctx.limbs_at(6) == 1


def test_multiply_relin_rescale_chain(env):
    ctx, o, l = env["ctx"], env["o"], env["l"]
    m = ph.multiply_and_relin(ctx, env["a"], env["b"], env["rlk"])
    want = o.multiply_and_relin(l, env["a_h"], env["b_h"], env["rlk_h"])
    assert np.array_equal(m.numpy(), want)
    assert m.scale() == SCALE * SCALE and m.chain_index() == 1
    # multiply + relinearize is the same thing in two calls
    m3 = ph.multiply(ctx, env["a"], env["b"])
    assert m3.size() == 3
    assert np.array_equal(ph.relinearize(ctx, m3, env["rlk"]).numpy(), want)
    r = ph.rescale_to_next(ctx, m)
    assert np.array_equal(r.numpy(), o.rescale(l, want))
    assert r.chain_index() == 2 and r.coeff_modulus_size() == l - 1
    assert r.scale() == pytest.approx(SCALE * SCALE / float(o.primes[l - 1]))
    # a level down the same key still works (fewer digits needed)
    r2 = ph.multiply_and_relin(ctx, r, r, env["rlk"])
    assert np.array_equal(r2.numpy(), o.multiply_and_relin(l - 1, r.numpy(), r.numpy(), env["rlk_h"]))
    # the batched forms: pairs (a, b) and (b, a) in one call; three-polynomial products relinearised in one call
    import torch
    A, B = torch.stack([env["a"].data, env["b"].data]), torch.stack([env["b"].data, env["a"].data])
    got = ph.multiply_relin_rescale_batch(ctx, A, B, env["rlk"], rescale=True)
    assert np.array_equal(got[0].cpu().numpy().astype(np.uint64), r.numpy()) and torch.equal(got[0], got[1])
    got = ph.multiply_relin_rescale_batch(ctx, A, B, env["rlk"], rescale=False)
    assert np.array_equal(got[1].cpu().numpy().astype(np.uint64), want)
    m3b = torch.stack([m3.data, m3.data]).contiguous()
    two = ph.relinearize_batch(ctx, m3b, env["rlk"])
    assert np.array_equal(two[1].cpu().numpy().astype(np.uint64), want) and torch.equal(two[0], two[1])


def test_add_sub_negate_plain(env):
    ctx, o, l = env["ctx"], env["o"], env["l"]
    a, b = env["a"], env["b"]
    s = ph.add(ctx, a, b)
    assert np.array_equal(s.numpy(), np.stack([o.add(env["a_h"][p], env["b_h"][p]) for p in range(2)]))
    d = ph.sub(ctx, s, b)
    assert np.array_equal(d.numpy(), env["a_h"])
    z = ph.add(ctx, a, ph.negate(ctx, a))
    assert not z.numpy().any()
    assert np.array_equal(ph.sub(ctx, a, b, True).numpy(), ph.negate(ctx, ph.sub(ctx, a, b)).numpy())
    assert np.array_equal(ph.add_many(ctx, [a, b, a]).numpy(), ph.add(ctx, s, a).numpy())
    pt_h = o.fill(1, o.primes[:l], 6, 9)[0]
    pt = ph.plaintext.from_numpy(ctx, pt_h, 1, SCALE)
    mp = ph.multiply_plain(ctx, a, pt)
    q = [int(x) for x in o.primes[:l]]
    want0 = np.stack([np.array([int(x) * int(y) % q[i] for x, y in zip(env["a_h"][0][i][:64], pt_h[i][:64])], dtype=np.uint64)
                      for i in range(l)])
    assert np.array_equal(mp.numpy()[0][:, :64], want0)
    assert mp.scale() == SCALE * SCALE
    ap = ph.add_plain(ctx, a, pt)
    assert np.array_equal(ap.numpy()[1], env["a_h"][1])
    assert np.array_equal(ph.sub_plain(ctx, ap, pt).numpy(), env["a_h"])


def test_rotations(env):
    ctx, o, l = env["ctx"], env["o"], env["l"]
    for step, elt, key in zip(env["steps"], env["elts"], env["glk_h"]):
        got = ph.rotate(ctx, env["a"], step, env["glk"])
        assert np.array_equal(got.numpy(), o.apply_galois(l, elt, key, env["a_h"]))
    # no key for step 3: the reference chains power-of-two rotations in NAF order (4, then -1)
    got = ph.rotate(ctx, env["a"], 3, env["glk"])
    t = o.apply_galois(l, env["elts"][3], env["glk_h"][3], env["a_h"])        # -1 first (least significant term)
    want = o.apply_galois(l, env["elts"][2], env["glk_h"][2], t)               # then +4
    assert np.array_equal(got.numpy(), want)
    outs = ph.hoist_rotations(ctx, env["a"], env["glk"], env["steps"][:3])
    want = o.hoist_rotations(l, env["a_h"], env["elts"][:3], env["glk_h"][:3])
    for g, w in zip(outs, want):
        assert np.array_equal(g.numpy(), w)
    assert ph.hoist_rotations(ctx, env["a"], env["glk"], []) == []
    k = ph.rotate_with_key(ctx, env["a"], 2, env["glk"].get_relin_keys(1))
    assert np.array_equal(k.numpy(), o.apply_galois(l, env["elts"][1], env["glk_h"][1], env["a_h"]))


def test_mod_switch(env):
    ctx = env["ctx"]
    a = env["a"]
    n = ph.mod_switch_to_next(ctx, a)
    assert n.chain_index() == 2 and np.array_equal(n.numpy(), env["a_h"][:, :-1])
    t = ph.mod_switch_to(ctx, a, 4)
    assert t.chain_index() == 4 and np.array_equal(t.numpy(), env["a_h"][:, :3])
    with pytest.raises(ValueError, match="higher level"):
        ph.mod_switch_to(ctx, t, 2)
    c = a.clone()
    ph.mod_switch_to_inplace(ctx, c, 3)
    assert c.chain_index() == 3 and c.coeff_modulus_size() == 4


def test_reference_error_behaviour(env):
    ctx, a, b = env["ctx"], env["a"], env["b"]
    lower = ph.mod_switch_to_next(ctx, b)
    with pytest.raises(ValueError, match="parameter mismatch"):
        ph.multiply_and_relin(ctx, a, lower, env["rlk"])
    c = b.clone()
    c.set_scale(SCALE * 2)
    with pytest.raises(ValueError, match="scale mismatch"):
        ph.multiply_and_relin(ctx, a, c, env["rlk"])
    with pytest.raises(ValueError, match="destination_size must be 3"):
        ph.relinearize(ctx, a, env["rlk"])
    last = ph.mod_switch_to(ctx, a, ctx.size_Q)
    with pytest.raises(ValueError, match="end of modulus switching chain"):
        ph.rescale_to_next(ctx, last)
    with pytest.raises(ValueError, match="step count too large"):
        ph.rotate(ctx, a, N // 2, env["glk"])
    with pytest.raises(ValueError, match="Galois key not present"):
        ph.rotate(ctx, a, 8, env["glk"])  # a single power of two without a key
    with pytest.raises(ValueError, match="Galois elt not present"):
        ph.apply_galois(ctx, a, 12345, env["glk"])
    short = ph.relin_key()
    short.public_keys = env["rlk"].public_keys[:1]
    with pytest.raises(ValueError, match="fewer digits"):
        ph.relinearize(ctx, ph.multiply(ctx, a, b), short)


def test_serialisation_round_trip_and_layout(env):
    ctx, a = env["ctx"], env["a"]
    buf = io.BytesIO()
    a.save(buf)
    raw = buf.getvalue()
    # include/ciphertext.h:173-191: chain, size, N, limbs (u64), scale (f64), correction, noiseScaleDeg, 2 bools
    chain, size, n, limbs = struct.unpack_from("<QQQQ", raw, 0)
    assert (chain, size, n, limbs) == (1, 2, N, env["l"])
    assert struct.unpack_from("<d", raw, 32)[0] == SCALE
    assert len(raw) == 58 + 2 * env["l"] * N * 8
    assert raw[58:58 + 64] == env["a_h"].tobytes()[:64]
    back = ph.ciphertext().load(io.BytesIO(raw))
    assert np.array_equal(back.numpy(), env["a_h"]) and back.scale() == SCALE and back.is_ntt_form()
    kb = io.BytesIO()
    env["rlk"].save(kb)
    k2 = ph.relin_key().load(io.BytesIO(kb.getvalue()))
    assert k2.dnum() == env["rlk"].dnum()
    m1 = ph.multiply_and_relin(ctx, a, env["b"], env["rlk"]).numpy()
    assert np.array_equal(ph.multiply_and_relin(ctx, a, env["b"], k2).numpy(), m1)
    gb = io.BytesIO()
    env["glk"].save(gb)
    g2 = ph.galois_key().load(io.BytesIO(gb.getvalue()))
    assert np.array_equal(ph.rotate(ctx, a, 1, g2).numpy(), ph.rotate(ctx, a, 1, env["glk"]).numpy())
    with pytest.raises(ValueError, match="truncated"):
        ph.ciphertext().load(io.BytesIO(raw[:100]))
    with pytest.raises(ValueError):
        ph.relin_key().save(io.BytesIO())


def test_bsgs_driver_matches_the_reference():
    """bsgs_matmul_preencoded on synthetic single-chain diagonals against the reference's hashes"""
    import glob, json, os
    from gpu_helpers import load_case, hashes
    paths = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*bsgs*.json")))
    assert paths, "no BSGS golden record"
    for path in paths:
        case, ctx, o = load_case(path)
        N, l, seed = o.N, case["level"], case["seed"]
        M, G = case["bsgs"]
        chain = o.size_Q - l + 1
        keys = [ph.relin_key.from_numpy(ctx, o.synth_key(o.beta(l), seed, 100 + 8 * e)) for e in range(len(case["elts"]))]
        glk = ph.galois_key.from_keys(keys)
        x = ph.ciphertext.from_numpy(ctx, o.synth_ct(l, seed, 1), chain, SCALE)
        diag_h = [o.synth_signed(seed, 3000 + d) for d in range(M * G)]
        diags = ph.bsgs_diagonals([ph.single_chain_plaintext(c, SCALE) for c in diag_h], M * G, M, G)
        assert ph.bsgs_required_steps(M) == case["steps"]
        y = ph.bsgs_matmul_preencoded(ctx, glk, x, diags)
        assert hashes(y.data, N) == case["hashes"]["bsgs"]
        assert y.chain_index() == chain + 1 and y.scale() == SCALE
        full = ph.expand_single_chain_to_full(ctx, diags.diagonals[0], chain)
        assert hashes(full.data, N) == case["hashes"]["expand_single_chain"]
        # round trip of the on-disk form of a single-chain plaintext
        back = ph.scp_from_bytes(diags.diagonals[1].coeffs_bytes(), SCALE)
        assert np.array_equal(back.coeffs.numpy(), diag_h[1])
        assert (back.N, back.nbytes, back.get_scale(), back.scale) == (N, 8 * N, SCALE, SCALE)
        with pytest.raises(ValueError, match="M\\*G must equal d_pad"):
            ph.bsgs_apply_giants_with_babies(ctx, glk, [x] * M, ph.bsgs_diagonals(diags.diagonals, M * G + 1, M, G))


def test_bsgs_driver_matches_the_reference_at_full_size():
    """the 4096 x 4096 product (N = 2^16, 16 limbs, M = G = 64): same limbs as the reference's bsgs_matmul_preencoded"""
    import glob, json, os
    from gpu_helpers import load_case, hashes
    paths = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "full", "*bsgs*.json")))
    assert paths, "no full-size BSGS record"
    case, ctx, o = load_case(paths[0])
    N, l, seed = o.N, case["level"], case["seed"]
    M, G = case["bsgs"]
    chain = o.size_Q - l + 1
    keys = [ph.relin_key.from_numpy(ctx, o.synth_key(o.beta(l), seed, 100 + 8 * e)) for e in range(len(case["elts"]))]
    glk = ph.galois_key.from_keys(keys)
    x = ph.ciphertext.from_numpy(ctx, o.synth_ct(l, seed, 1), chain, SCALE)
    diags = ph.bsgs_diagonals([ph.single_chain_plaintext(o.synth_signed(seed, 3000 + d), SCALE) for d in range(M * G)], M * G, M, G)
    y = ph.bsgs_matmul_preencoded(ctx, glk, x, diags)
    assert hashes(y.data, N) == case["hashes"]["bsgs"]


def test_galois_key_fallback(env):
    ctx, a = env["ctx"], env["a"]
    g = ph.galois_key.from_keys([ph.relin_key() for _ in env["elts"]])  # every owned slot empty
    with pytest.raises(ValueError, match="no owned key, no fallback"):
        ph.rotate(ctx, a, 1, g)
    g.set_fallback(0, env["glk"].get_relin_keys(0))
    assert np.array_equal(ph.rotate(ctx, a, 1, g).numpy(), ph.rotate(ctx, a, 1, env["glk"]).numpy())
    with pytest.raises(IndexError):
        g.set_fallback(99, env["glk"].get_relin_keys(0))
