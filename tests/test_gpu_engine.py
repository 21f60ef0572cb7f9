"""ckks_engine facade (test/ckks_engine_test.cu is the model: round trip, multiply + rescale, deplete + bootstrap)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

import pyPhantom as ph


@pytest.fixture(scope="module")
def engine():
    cfg = ph.ckks_engine_config()
    cfg.log_n = 12                 # the reference pins 16; the facade is the same at any ring size
    cfg.num_scale_levels = 5       # size_Q = 21 = 3 * 7
    cfg.num_special_primes = 7
    cfg.build_two_scale_arrays = True
    return ph.ckks_engine(cfg)


def test_levels_and_round_trip(engine):
    e = engine
    assert e.slot_count() == 2048 and e.max_user_level() == 4 and e.user_scale() == 2.0 ** 40
    assert e.user_level_chain_index(0) == 16 and e.user_level_chain_index(4) == 20
    with pytest.raises(ValueError):
        e.user_level_chain_index(5)
    rng = np.random.default_rng(1)
    v = rng.uniform(-0.5, 0.5, e.slot_count()) + 1j * rng.uniform(-0.5, 0.5, e.slot_count())
    ct = e.encrypt(e.encode(v))
    assert e.user_level(ct) == 0
    assert np.max(np.abs(np.array(e.decrypt_decode(ct)) - v)) < 1e-7          # test/ckks_engine_test.cu:56
    sq = e.encrypt(e.encode(v))
    e.mul_and_relin_inplace(sq, ct)
    e.rescale_inplace(sq)
    assert e.user_level(sq) == 1
    assert np.max(np.abs(np.array(e.decrypt_decode(sq)) - v * v)) < 1e-5      # :96
    e.rotate_inplace(ct, 1)
    assert np.max(np.abs(np.array(e.decrypt_decode(ct)) - np.roll(v, -1))) < 1e-6
    e.rotate_inplace(ct, -2)
    assert np.max(np.abs(np.array(e.decrypt_decode(ct)) - np.roll(v, 1))) < 1e-6
    assert e.scale_array_size() == e.context().total_parm_size()
    assert e.ckks_scale_at(0) == 2.0 ** 80 and 0 < e.ckks_rescaled_scale_at(1) < e.ckks_scale_at(1)


def test_deplete_and_bootstrap(engine):
    e = engine
    rng = np.random.default_rng(2)
    v = rng.uniform(-0.4, 0.4, e.slot_count())
    ct = e.encrypt(e.encode(v))
    want = v.copy()
    for _ in range(e.max_user_level()):            # square down to the last user level
        e.mul_and_relin_inplace(ct, ct)
        e.rescale_inplace(ct)
        ct.set_scale(e.user_scale())
        want = want * want
    assert e.user_level(ct) == e.max_user_level()
    with pytest.raises(RuntimeError):
        e.rescale_inplace(ct)
    e.bootstrap_inplace(ct)
    assert e.user_level(ct) == 0 and ct.scale() == e.user_scale()
    assert np.max(np.abs(np.array(e.decrypt_decode(ct)).real - want)) < 1e-3   # test/ckks_engine_test.cu:182
    e.mul_and_relin_inplace(ct, ct)                # and the refreshed ciphertext computes
    e.rescale_inplace(ct)
    assert np.max(np.abs(np.array(e.decrypt_decode(ct)).real - want * want)) < 1e-3


def test_config_errors():
    cfg = ph.ckks_engine_config()
    cfg.log_n, cfg.num_scale_levels, cfg.num_special_primes = 12, 5, 4   # 21 limbs not divisible by 4
    with pytest.raises(ValueError):
        ph.ckks_engine(cfg)
    cfg.num_special_primes, cfg.use_bootstrap_to_17_levels = 7, True     # 5 + 14 limbs not divisible by 7
    with pytest.raises(ValueError):
        ph.ckks_engine(cfg)
    cfg.use_bootstrap_to_17_levels, cfg.num_scale_levels = False, 1
    with pytest.raises(ValueError):
        ph.ckks_engine(cfg)


def test_second_chain_layout_has_no_bootstrap():
    """use_bootstrap_to_17_levels (src/ckks_engine.cu:99-118, 171-214, 570-578): 40 x NSL | 29 | 54 x 12 | 42 | specials;
    user level 0 sits 13 primes below the top; encode / encrypt / decrypt work, bootstrap_inplace refuses"""
    cfg = ph.ckks_engine_config()
    cfg.log_n, cfg.num_scale_levels, cfg.num_special_primes = 12, 6, 5   # 6 + 14 = 20 limbs = 4 x 5
    cfg.use_bootstrap_to_17_levels, cfg.build_two_scale_arrays = True, True
    e = ph.ckks_engine(cfg)
    ctx = e.context()
    bits = [int(q).bit_length() for q in ctx.primes]
    assert bits == [40] * 6 + [29] + [54] * 12 + [42] + [60] * 5
    assert e.user_level_chain_index(0) == ctx.get_first_index() + 13 and e.max_user_level() == 5
    assert e.scale_array_size() == ctx.total_parm_size()
    v = np.random.default_rng(3).uniform(-1, 1, e.slot_count())
    ct = e.encrypt(e.encode(v, 2))
    assert e.user_level(ct) == 2
    assert np.max(np.abs(np.array(e.decrypt_decode(ct)).real - v)) < 1e-6
    with pytest.raises(RuntimeError, match="does not have a bootstrap"):
        e.bootstrap_inplace(ct)
