"""End-to-end CKKS on the GPU through the pyPhantom surface: encode, encrypt, evaluate, decrypt,
decode, compared with the same arithmetic on the clear vectors. Floating point enters only through
the encoder, so the tolerances are the reference's own for the same flows: round trip 1e-7 and
multiply+rescale 1e-5 (test/ckks_engine_test.cu:56, :96), rotations and matrix-vector products 1e-3
(examples/3_ckks.cu:18-25, python/llm_project/blocks/bsgs_test.py:84-89)."""
import io

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import pyPhantom as ph

N = 1 << 13
SCALE = 2.0 ** 40


@pytest.fixture(scope="module")
def kit():
    steps = [1, 2, 4, 8, -1]
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(N)
    parms.set_coeff_modulus(ph.create_coeff_modulus(N, [60, 40, 40, 40, 40, 60, 60]))
    parms.set_special_modulus_size(2)
    parms.set_galois_elts(ph.get_elts_from_steps(steps, N) + [2 * N - 1])
    ctx = ph.context(parms)
    sk = ph.secret_key(ctx, seed=1234)
    enc = ph.ckks_encoder(ctx)
    rng = np.random.default_rng(7)
    x = rng.uniform(-1, 1, enc.slot_count()) + 1j * rng.uniform(-1, 1, enc.slot_count())
    y = rng.uniform(-1, 1, enc.slot_count()) + 1j * rng.uniform(-1, 1, enc.slot_count())
    return dict(ctx=ctx, sk=sk, enc=enc, rlk=sk.gen_relinkey(ctx), glk=sk.create_galois_keys(ctx), x=x, y=y, steps=steps,
                cx=sk.encrypt_symmetric(ctx, enc.encode_complex_vector(ctx, x, SCALE)),
                cy=sk.encrypt_symmetric(ctx, enc.encode_complex_vector(ctx, y, SCALE)))


def _dec(kit, ct):
    return kit["enc"].decode_complex_vector(kit["ctx"], kit["sk"].decrypt(kit["ctx"], ct))


def test_encode_decode_and_encrypt_decrypt_round_trip(kit):
    ctx, enc = kit["ctx"], kit["enc"]
    assert enc.slot_count() == N // 2
    pt = enc.encode_complex_vector(ctx, kit["x"], SCALE)
    assert np.max(np.abs(enc.decode_complex_vector(ctx, pt) - kit["x"])) < 1e-9
    assert np.max(np.abs(_dec(kit, kit["cx"]) - kit["x"])) < 1e-7
    short = enc.encode_double_vector(ctx, [1.0, 2.0, 3.0], SCALE)
    d = enc.decode_double_vector(ctx, short)
    assert np.allclose(d[:3], [1, 2, 3], atol=1e-9) and np.max(np.abs(d[3:])) < 1e-9
    with pytest.raises(ValueError, match="exceeds max slots"):
        enc.encode_double_vector(ctx, np.zeros(N), SCALE)
    with pytest.raises(ValueError, match="empty"):
        enc.encode_double_vector(ctx, [], SCALE)


def test_add_multiply_rescale(kit):
    ctx = kit["ctx"]
    assert np.max(np.abs(_dec(kit, ph.add(ctx, kit["cx"], kit["cy"])) - (kit["x"] + kit["y"]))) < 1e-7
    m = ph.rescale_to_next(ctx, ph.multiply_and_relin(ctx, kit["cx"], kit["cy"], kit["rlk"]))
    assert m.chain_index() == 2 and abs(np.log2(m.scale()) - 40) < 0.01
    assert np.max(np.abs(_dec(kit, m) - kit["x"] * kit["y"])) < 1e-5
    # depth 3: ((x*y)*x) then squared, all the way down the chain
    x2 = ph.mod_switch_to(ctx, kit["cx"], 2)
    x2.set_scale(m.scale())  # same level; scales differ by a factor 2^40 / q_last, keep it exact in the reference sense
    x2 = kit["sk"].encrypt_symmetric(ctx, kit["enc"].encode_complex_vector(ctx, kit["x"], m.scale(), 2))
    m3 = ph.rescale_to_next(ctx, ph.multiply_and_relin(ctx, m, x2, kit["rlk"]))
    assert np.max(np.abs(_dec(kit, m3) - kit["x"] * kit["y"] * kit["x"])) < 1e-4
    # unrelinearised product decrypts with s^2 as well
    m_raw = ph.multiply(ctx, kit["cx"], kit["cy"])
    assert np.max(np.abs(_dec(kit, m_raw) - kit["x"] * kit["y"])) < 1e-5
    pt = kit["enc"].encode_complex_vector(ctx, kit["y"], SCALE)
    mp = ph.rescale_to_next(ctx, ph.multiply_plain(ctx, kit["cx"], pt))
    assert np.max(np.abs(_dec(kit, mp) - kit["x"] * kit["y"])) < 1e-5


def test_rotations_conjugation_and_hoisting(kit):
    ctx = kit["ctx"]
    for s in kit["steps"]:
        got = _dec(kit, ph.rotate(ctx, kit["cx"], s, kit["glk"]))
        assert np.max(np.abs(got - np.roll(kit["x"], -s))) < 1e-3, s
    got = _dec(kit, ph.rotate(ctx, kit["cx"], 7, kit["glk"]))  # NAF chain 8 - 1
    assert np.max(np.abs(got - np.roll(kit["x"], -7))) < 1e-3
    conj = _dec(kit, ph.apply_galois(ctx, kit["cx"], 2 * N - 1, kit["glk"]))
    assert np.max(np.abs(conj - np.conj(kit["x"]))) < 1e-3
    outs = ph.hoist_rotations(ctx, kit["cx"], kit["glk"], [1, 2, 8])
    for s, o in zip([1, 2, 8], outs):
        assert np.max(np.abs(_dec(kit, o) - np.roll(kit["x"], -s))) < 1e-3
    low = ph.mod_switch_to(ctx, kit["cx"], 4)  # two limbs left: one digit only
    assert np.max(np.abs(_dec(kit, ph.rotate(ctx, low, 2, kit["glk"])) - np.roll(kit["x"], -2))) < 1e-3


def test_sparse_secret_and_key_serialisation(kit):
    ctx, enc = kit["ctx"], kit["enc"]
    sk = ph.secret_key(ctx, seed=5)
    sk.generate_sparse(ctx, 192)
    assert int(np.count_nonzero(sk.coeffs)) == 192 and set(np.unique(sk.coeffs)) <= {-1, 0, 1}
    ct = sk.encrypt_symmetric(ctx, enc.encode_complex_vector(ctx, kit["x"], SCALE))
    buf = io.BytesIO()
    sk.save(buf)
    assert len(buf.getvalue()) == 24 + ctx.size_QP * N * 8
    sk2 = ph.secret_key().load(io.BytesIO(buf.getvalue()))
    assert np.max(np.abs(enc.decode_complex_vector(ctx, sk2.decrypt(ctx, ct)) - kit["x"])) < 1e-7
    pk = sk.gen_publickey(ctx)
    pb = io.BytesIO()
    pk.save(pb)
    assert ph.public_key().load(io.BytesIO(pb.getvalue())).pk.coeff_modulus_size() == ctx.size_QP


def test_bsgs_matrix_vector_product(kit):
    ctx, enc, sk = kit["ctx"], kit["enc"], kit["sk"]
    d, M, G = 16, 4, 4
    rng = np.random.default_rng(11)
    W = rng.normal(0, 0.5, (d, d))
    v = rng.normal(0, 1, d)
    slots = enc.slot_count()
    xv = np.tile(v, slots // d)
    cx = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, xv, SCALE))
    diags = []
    for g in range(G):
        for b in range(M):
            k = g * M + b
            diag = np.array([W[i, (i + k) % d] for i in range(d)])
            diag = np.roll(np.tile(diag, slots // d), g * M)  # pre-rotated by -g*M (src/bsgs.cu:131-176)
            pt = enc.encode_double_vector(ctx, diag, SCALE)
            pt0 = pt.data[:1].clone()
            ph._native.check(ph._native.LIB.b2_ntt_inverse(ctx._h, pt0.data_ptr(), 1, 0, torch.cuda.current_stream().cuda_stream))
            c = pt0.cpu().numpy().view(np.uint64)[0].astype(object)
            q0 = int(ctx.primes[0])
            c = np.where(c >= (q0 + 1) // 2, c - q0, c)
            diags.append(ph.single_chain_plaintext(np.array([int(t) for t in c], dtype=np.int64), SCALE))
    y = ph.bsgs_matmul_preencoded(ctx, kit["glk"], cx, ph.bsgs_diagonals(diags, d, M, G))
    got = enc.decode_double_vector(ctx, sk.decrypt(ctx, y))[:d]
    assert np.max(np.abs(got - W @ v)) < 1e-3
    assert y.chain_index() == 2


def test_interchange_with_the_reference_library(tmp_path):
    """Both directions through save()/load() bytes, on this GPU: the reference's secret key and
    ciphertext decrypt and decode here, and what this library encrypts decrypts in the reference.
    Needs oracle/_ref/ref_harness (the reference compiled from its own sources)."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    harness = os.path.join(root, "oracle", "_ref", "ref_harness")
    if not os.path.exists(harness):
        pytest.skip("reference harness not built")
    n, bits, special = 1 << 13, [60, 40, 40, 40, 60, 60], 2
    args = [harness, "--logn", "13", "--bits", ",".join(map(str, bits)), "--special", str(special), "--steps", "1"]
    subprocess.run(args + ["--interop-write", str(tmp_path)], check=True, capture_output=True, timeout=300)
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(n)
    parms.set_coeff_modulus(ph.create_coeff_modulus(n, bits))
    parms.set_special_modulus_size(special)
    parms.set_galois_elts([ph.get_elt_from_step(1, n)])
    ctx = ph.context(parms)
    enc = ph.ckks_encoder(ctx)
    j = np.arange(enc.slot_count(), dtype=np.float64)
    z = np.cos(j) + 0.5j * np.sin(2 * j)
    sk = ph.secret_key().load(open(tmp_path / "ref_sk.bin", "rb"))
    ct = ph.ciphertext().load(open(tmp_path / "ref_ct.bin", "rb"))
    assert ct.chain_index() == 1 and ct.scale() == SCALE
    assert np.max(np.abs(enc.decode_complex_vector(ctx, sk.decrypt(ctx, ct)) - z)) < 1e-6
    # the reference's relinearisation key after its mod_drop_to_inplace(3): one digit of two; it relinearises here at chain
    # index 3 (two limbs, one digit), and is refused a level up where two digits are needed
    rlk = ph.relin_key().load(open(tmp_path / "ref_rlk_trunc.bin", "rb"))
    assert rlk.dnum() == 1
    low = ph.mod_switch_to(ctx, ct, 3)
    sq = ph.multiply_and_relin(ctx, low, low, rlk)
    got = enc.decode_complex_vector(ctx, sk.decrypt(ctx, sq))
    assert np.max(np.abs(got - z * z)) < 1e-4
    with pytest.raises(ValueError):
        ph.multiply_and_relin(ctx, ct, ct, rlk)
    mine = ph.secret_key(ctx, seed=99)
    with open(tmp_path / "b2_sk.bin", "wb") as f:
        mine.save(f)
    my_ct = mine.encrypt_symmetric(ctx, enc.encode_complex_vector(ctx, z, SCALE))
    with open(tmp_path / "b2_ct.bin", "wb") as f:
        my_ct.save(f)
    res = subprocess.run(args + ["--interop-read", str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("interop-plain:")][0]
    from oracle_lib import limb_hashes
    want = limb_hashes(mine.decrypt(ctx, my_ct).data.cpu().numpy().view(np.uint64), n)
    assert line.split()[1:] == want, "the reference decrypts this library's bytes to a different plaintext"
    assert np.max(np.abs(enc.decode_complex_vector(ctx, mine.decrypt(ctx, my_ct)) - z)) < 1e-6


def test_asymmetric_encryption_round_trip(kit):
    ctx, enc, sk = kit["ctx"], kit["enc"], kit["sk"]
    pk = sk.gen_publickey(ctx)
    v = kit["x"]
    for chain in (1, 3):
        ct = pk.encrypt_asymmetric(ctx, enc.encode_complex_vector(ctx, v, SCALE, chain), seed=chain)
        assert ct.chain_index() == chain and ct.coeff_modulus_size() == ctx.limbs_at(chain)
        assert np.max(np.abs(_dec(kit, ct) - v)) < 1e-6
    prod = ph.rescale_to_next(ctx, ph.multiply_and_relin(ctx, ct, ct, kit["rlk"]))
    assert np.max(np.abs(_dec(kit, prod) - v * v)) < 1e-4


def test_pre_encoded_bsgs_matches_numpy(kit):
    ctx, enc, sk = kit["ctx"], kit["enc"], kit["sk"]
    d_pad, M = 16, 4
    rng = np.random.default_rng(4)
    W = rng.normal(0, 0.5, (12, 10))
    x = np.zeros(d_pad)
    x[:10] = rng.normal(size=10)
    diags = ph.pre_encode_bsgs_diagonals(ctx, enc, W.ravel(), 12, 10, d_pad, M, SCALE)
    assert (diags.d_pad, diags.baby_steps, diags.giant_steps, len(diags.diagonals)) == (16, 4, 4, 16)
    ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, np.tile(x, enc.slot_count() // d_pad), SCALE, 1))
    y = ph.bsgs_matmul_preencoded(ctx, kit["glk"], ct, diags)
    got = enc.decode_double_vector(ctx, sk.decrypt(ctx, y))[:12]
    assert np.max(np.abs(got - W @ x[:10])) < 2e-5       # python/llm_project/blocks/bsgs_test.py:84-89
    with pytest.raises(ValueError):
        ph.pre_encode_bsgs_diagonals(ctx, enc, W.ravel(), 12, 10, 12, 4, SCALE)
    with pytest.raises(ValueError):
        ph.pre_encode_bsgs_diagonals(ctx, enc, W.ravel(), 12, 11, 16, 4, SCALE)


def test_remaining_surface_names(kit):
    ctx, enc, sk = kit["ctx"], kit["enc"], kit["sk"]
    x = kit["x"]
    # hoisting = sum of the rotations
    got = _dec(kit, ph.hoisting(ctx, kit["cx"], kit["glk"], [1, 2, 4]))
    assert np.max(np.abs(got - (np.roll(x, -1) + np.roll(x, -2) + np.roll(x, -4)))) < 1e-5
    # keys for a subset of the elements, the rest served by a fallback
    idx = [ctx.galois_elts.index(ph.get_elt_from_step(s, N)) for s in (1, 2)]
    some = sk.create_galois_keys_per_level(ctx, idx, [1, 1])
    assert np.max(np.abs(_dec(kit, ph.rotate(ctx, kit["cx"], 2, some)) - np.roll(x, -2))) < 1e-6
    with pytest.raises(ValueError):
        ph.rotate(ctx, kit["cx"], 4, some)
    some.set_fallback(ctx.galois_elts.index(ph.get_elt_from_step(4, N)), kit["glk"].get_relin_keys(ctx.galois_elts.index(ph.get_elt_from_step(4, N))))
    assert np.max(np.abs(_dec(kit, ph.rotate(ctx, kit["cx"], 4, some)) - np.roll(x, -4))) < 1e-6
    with pytest.raises(ValueError):
        sk.create_galois_keys_per_level(ctx, idx, [1])
    # single-chain encoding of a slot vector expands to the plaintext the encoder makes
    scp = ph.encode_single_chain_plaintext(ctx, enc, x, SCALE)
    full = ph.expand_single_chain_to_full(ctx, scp, 2)
    assert torch.equal(full.data, enc.encode_complex_vector(ctx, x, SCALE, 2).data)


def test_resident_bsgs_product():
    """diagonals resident in HBM, hoisted babies, giants with one ModDown per stream: same product as numpy"""
    from pyPhantom.linalg import resident_bsgs
    n_ring, d_pad, M = 1 << 12, 16, 4
    steps = [1, 2, 3, 4, 8, 12]
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(n_ring)
    parms.set_coeff_modulus(ph.create_coeff_modulus(n_ring, [60, 40, 40, 40, 60, 60]))
    parms.set_special_modulus_size(2)
    parms.set_galois_elts(ph.get_elts_from_steps(steps, n_ring))
    ctx = ph.context(parms)
    sk = ph.secret_key(ctx, seed=5)
    enc = ph.ckks_encoder(ctx)
    glk = sk.create_galois_keys(ctx)
    rng = np.random.default_rng(6)
    W = rng.normal(0, 0.5, (d_pad, d_pad))
    v = rng.normal(size=d_pad)
    diags = ph.pre_encode_bsgs_diagonals(ctx, enc, W.ravel(), d_pad, d_pad, d_pad, M, SCALE)
    x = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, np.tile(v, enc.slot_count() // d_pad), SCALE, 1))
    op = resident_bsgs(ctx, glk, diags, 1)
    for _ in range(2):   # the buffers of the operator are reused from call to call
        y = op.apply(x)
        assert y.chain_index() == 2 and y.scale() == SCALE
        got = enc.decode_double_vector(ctx, sk.decrypt(ctx, y))[:d_pad]
        assert np.max(np.abs(got - W @ v)) < 2e-5
    ref = enc.decode_double_vector(ctx, sk.decrypt(ctx, ph.bsgs_matmul_preencoded(ctx, sk.create_galois_keys(ctx), x, diags)))[:d_pad]
    assert np.max(np.abs(got - ref)) < 1e-5
    with pytest.raises(ValueError):
        op.apply(ph.mod_switch_to_next(ctx, x))


def test_flow_of_the_ckks_example():
    """the calls of python/examples/ckks.py in its order: asymmetric encryption, square, rescale, summed hoisted
    rotations, add; checked against the same computation on the plain vector"""
    n_ring = 1 << 14
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(n_ring)
    parms.set_coeff_modulus(ph.create_coeff_modulus(n_ring, [60, 40, 40, 60]))
    parms.set_special_modulus_size(1)
    steps = [1, 2, 3, 4, 5, 6, 7]
    parms.set_galois_elts(ph.get_elts_from_steps(steps, n_ring))
    ctx = ph.context(parms)
    sk = ph.secret_key(ctx)
    pk, rlk, glk = sk.gen_publickey(ctx), sk.gen_relinkey(ctx), sk.create_galois_keys(ctx)
    enc = ph.ckks_encoder(ctx)
    msg = np.zeros(enc.slot_count())
    msg[:8] = np.arange(1.0, 9.0)
    ct = pk.encrypt_asymmetric(ctx, enc.encode_double_vector(ctx, list(msg), 2.0 ** 40, chain_index=1))
    ct = ph.rescale_to_next(ctx, ph.multiply_and_relin(ctx, ct, ct, rlk))
    ct = ph.add(ctx, ct, ph.hoisting(ctx, ct, glk, steps))
    got = enc.decode_double_vector(ctx, sk.decrypt(ctx, ct))
    sq = msg * msg
    want = sq + sum(np.roll(sq, -k) for k in steps)
    assert np.max(np.abs(got - want)) < 1e-3


def test_complex_folded_bsgs(kit):
    """row fold: one product gives rows 0..h-1 in the real part and rows h..2h-1 in the imaginary part"""
    ctx, enc, sk = kit["ctx"], kit["enc"], kit["sk"]
    d_pad, M = 16, 4
    rng = np.random.default_rng(12)
    W = rng.normal(0, 0.5, (20, 12))
    v = np.zeros(d_pad)
    v[:12] = rng.normal(size=12)
    diags = ph.pre_encode_bsgs_diagonals_complex(ctx, enc, W.ravel(), 20, 12, d_pad, M, SCALE, ph.complex_fold_mode.Rows)
    ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, np.tile(v, enc.slot_count() // d_pad), SCALE, 1))
    got = enc.decode_complex_vector(ctx, sk.decrypt(ctx, ph.bsgs_matmul_preencoded_complex(ctx, kit["glk"], ct, diags)))[:10]
    want = W @ v[:12]
    assert np.max(np.abs(got.real - want[:10])) < 2e-5 and np.max(np.abs(got.imag - want[10:])) < 2e-5
    cols = ph.pre_encode_bsgs_diagonals_complex(ctx, enc, W.ravel(), 20, 12, 32, M, SCALE, ph.complex_fold_mode.ColsConj)
    assert len(cols.inner.diagonals) == 32
    with pytest.raises(ValueError):
        ph.pre_encode_bsgs_diagonals_complex(ctx, enc, W.ravel(), 20, 12, 8, M, SCALE, ph.complex_fold_mode.Rows)


def test_inner_sum_replicate_and_polynomial(kit):
    ctx, enc, sk = kit["ctx"], kit["enc"], kit["sk"]
    n = enc.slot_count()
    x = kit["x"].real
    cx = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, x, SCALE, 1))
    got = enc.decode_double_vector(ctx, sk.decrypt(ctx, ph.inner_sum(ctx, kit["glk"], cx, 8)))
    want = sum(np.roll(x, -k) for k in range(8))
    assert np.max(np.abs(got - want)) < 1e-5
    with pytest.raises(ValueError):
        ph.inner_sum(ctx, kit["glk"], cx, 6)
    # degree 7 and degree 3 on [-1, 1]; the result sits where the reference's schedule ends
    for coeffs in ([0.5, -1.0, 0.25, 2.0, -0.75, 0.1, 0.3, -0.2], [1.0, 0.0, -0.5, 0.125]):
        y = ph.eval_polynomial(ctx, enc, kit["rlk"], cx, coeffs)
        d = len(coeffs) - 1
        m = int(np.ceil(np.sqrt(d + 1)))
        assert y.chain_index() == 1 + m + (d + m) // m - 2 and y.scale() == SCALE
        got = enc.decode_double_vector(ctx, sk.decrypt(ctx, y))
        assert np.max(np.abs(got - np.polynomial.polynomial.polyval(x, coeffs))) < 1e-4


def test_level_truncated_keys(kit, tmp_path):
    """Keys with only the digits a level needs (src/secretkey.cu:301-352, 400-472, 726-775): 5 Q limbs in digits of 2 give
    3 digits at the top; a ciphertext with 2 limbs needs one. A truncated key switches that level like the full key does
    in meaning (other randomness: compare decryptions), refuses levels that need more digits, survives save / load, and
    serves as a fallback of a Galois-key bundle."""
    ctx, sk, enc = kit["ctx"], kit["sk"], kit["enc"]
    assert ctx.beta(ctx.size_Q) == 3
    low_chain = ctx.size_Q - 2 + 1                       # chain index whose ciphertexts have 2 limbs
    x = kit["x"]
    ct_low = sk.encrypt_symmetric(ctx, enc.encode_complex_vector(ctx, x, SCALE, low_chain))
    assert ct_low.coeff_modulus_size() == 2
    full = sk.gen_relinkey(ctx)
    assert full.dnum() == 3
    dropped = sk.gen_relinkey(ctx)
    dropped.mod_drop_to_inplace(ctx, low_chain)
    assert dropped.dnum() == 1 and dropped.device_bytes() * 3 == full.device_bytes()
    dropped.mod_drop_to_inplace(ctx, low_chain)           # already there: nothing happens
    assert dropped.dnum() == 1
    with pytest.raises(RuntimeError, match="more dnum entries"):
        dropped.mod_drop_to_inplace(ctx, 1)
    with pytest.raises(ValueError):
        dropped.mod_drop_to_inplace(ctx, 0)
    sq = ph.rescale_to_next(ctx, ph.multiply_and_relin(ctx, ct_low, ct_low, dropped))
    assert np.max(np.abs(_dec(kit, sq) - x * x)) < 1e-4
    with pytest.raises(ValueError, match="fewer digits"):
        ph.multiply_and_relin(ctx, kit["cx"], kit["cx"], dropped)   # 5 limbs need all three digits
    # generated at a level: the same number of digits, never more
    idx = ctx.galois_elts.index(ph.get_elt_from_step(1, N))
    one = sk.create_one_galois_key(ctx, idx, low_chain)
    assert one.dnum() == 1 and sk.create_one_galois_key(ctx, idx).dnum() == 3
    want = np.roll(x, -1)
    assert np.max(np.abs(_dec(kit, ph.rotate_with_key(ctx, ct_low, 1, one)) - want)) < 1e-6
    per_level = sk.create_galois_keys_per_level(ctx, [idx], [low_chain])
    assert per_level.get_relin_keys(idx).dnum() == 1 and per_level.resolve(idx + 1 if idx + 1 < len(ctx.galois_elts) else 0) is None
    assert np.max(np.abs(_dec(kit, ph.rotate(ctx, ct_low, 1, per_level)) - want)) < 1e-6
    with pytest.raises(ValueError):
        sk.create_galois_keys_per_level(ctx, [idx], [low_chain, 1])
    # bytes: a truncated key is its first digits, in the reference's layout
    with open(tmp_path / "k.bin", "wb") as f:
        one.save(f)
    back = ph.relin_key().load(open(tmp_path / "k.bin", "rb"))
    assert back.dnum() == 1 and torch.equal(back.public_keys[0].data, one.public_keys[0].data)
    bundle = ph.galois_key.from_keys([ph.relin_key() for _ in ctx.galois_elts])
    bundle.set_fallback(idx, back)
    assert np.max(np.abs(_dec(kit, ph.rotate(ctx, ct_low, 1, bundle)) - want)) < 1e-6
