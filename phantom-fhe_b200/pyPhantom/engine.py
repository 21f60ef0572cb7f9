"""ckks_engine: the facade the reference's applications construct (python/src/binding.cu:338-385;
include/ckks_engine.h, src/ckks_engine.cu): one fixed modulus chain with its context, encoder, keys and
bootstrap key, and the "user level" bookkeeping on top of chain indices.

Chain (src/ckks_engine.cu:119-131):  58 | 40 x num_scale_levels | 58 x 3 | 58 x 9 | 29 x 3 | 58 x num_special_primes.
User level u lives at chain index freshest + u, freshest = first + 15; the level with q0 alone is internal.
The reference pins log_n to 16; smaller rings are accepted here so that the facade can be tested quickly.
"""
import numpy as np

from . import (add, ckks_encoder, context, create_coeff_modulus, galois_key, mod_switch_to_inplace, multiply_and_relin,
               multiply_plain, params, relin_key, rescale_to_next, rotate, scheme_type, secret_key, sub)
from . import boot


class ckks_engine_config:
    def __init__(self):
        self.log_n = 16
        self.user_scale = 2.0 ** 40
        self.num_scale_levels = 14
        self.sparse_hw = 128
        self.num_special_primes = 6
        self.include_user_rotations = True
        self.user_rotation_steps = []
        self.user_rotation_target_chain_indices = []
        self.split_scale_down = False
        self.build_two_scale_arrays = False
        self.use_bootstrap_to_17_levels = False


class ckks_engine:
    def __init__(self, config=None):
        cfg = self._cfg = config if config is not None else ckks_engine_config()
        if not 12 <= cfg.log_n <= 16:
            raise ValueError("CKKSEngine: log_n must be in [12, 16]")
        if cfg.num_scale_levels < 2:
            raise ValueError("CKKSEngine: num_scale_levels must be >= 2")
        if cfg.num_special_primes < 1:
            raise ValueError("CKKSEngine: num_special_primes must be >= 1")
        if cfg.user_rotation_target_chain_indices and len(cfg.user_rotation_target_chain_indices) != len(cfg.user_rotation_steps):
            raise ValueError("CKKSEngine: user_rotation_target_chain_indices size must match user_rotation_steps size")
        deep = bool(cfg.use_bootstrap_to_17_levels)
        size_q = cfg.num_scale_levels + 14 if deep else 1 + cfg.num_scale_levels + 3 + 9 + 3
        if size_q % cfg.num_special_primes != 0:
            raise ValueError("CKKSEngine: size_Q must be divisible by num_special_primes "
                             "(required by the hybrid KSK decomposition).")
        N = 1 << cfg.log_n
        if deep:
            # src/ckks_engine.cu:99-118: 40 x NSL (the first is the message prime) | 29 | 54 x 12 | 42 | 60 x NSP
            bits = [40] * cfg.num_scale_levels + [29] + [54] * 12 + [42] + [60] * cfg.num_special_primes
        else:
            bits = [58] + [40] * cfg.num_scale_levels + [58] * 3 + [58] * 9 + [29] * 3 + [58] * cfg.num_special_primes
        parms = params(scheme_type.ckks)
        parms.set_poly_modulus_degree(N)
        parms.set_special_modulus_size(cfg.num_special_primes)
        parms.set_coeff_modulus(create_coeff_modulus(N, bits))
        user_steps = list(cfg.user_rotation_steps) or ([1, -1, 2, -2] if cfg.include_user_rotations else [])
        boot_elts = boot.bootstrap_required_galois_elts(cfg.log_n)
        user_elts = [boot._elt(s, N) for s in user_steps]
        elts = []
        for e in boot_elts[:-1] + user_elts + [2 * N - 1]:
            if e not in elts:
                elts.append(e)
        parms.set_galois_elts(elts)
        self._ctx = context(parms)
        self._sk = secret_key(self._ctx)
        self._enc = ckks_encoder(self._ctx)
        self._scale, self._rescaled = [], []
        if deep:
            # src/ckks_engine.cu:171-214: on this chain the reference builds no bootstrap, relinearisation or rotation
            # keys: encode / encrypt / decrypt and the scale arrays only, and bootstrap_inplace refuses
            self._bk, self._glk = None, galois_key.from_keys([relin_key() for _ in elts])
            self._freshest = self._ctx.get_first_index() + 13
            self._bottom = self._ctx.total_parm_size() - 1
            if self._freshest + cfg.num_scale_levels != self._bottom:
                raise RuntimeError("CKKSEngine: BootstrapTo17Levels chain mismatch: freshest + num_scale_levels != bottom.")
            if cfg.build_two_scale_arrays:
                self._build_scale_arrays()
            return
        self._bk = boot.create_bootstrap_key(self._ctx, self._enc, self._sk, cfg.sparse_hw, 9, cfg.user_scale, cfg.split_scale_down)
        # user rotation keys: steps the bootstrap already owns are shared (src/ckks_engine.cu:268-360 registers them as
        # non-owning fallbacks), the rest are generated
        n = N // 2
        self._glk = galois_key.from_keys([relin_key() for _ in elts])
        targets = list(cfg.user_rotation_target_chain_indices) or [0] * len(user_steps)
        for s, e, target in zip(user_steps, user_elts, targets):
            shared = self._bk.rot.get(s % n)
            if shared is not None:
                self._glk.set_fallback(elts.index(e), shared)
            else:
                # generated with the digits its target chain index needs (src/ckks_engine.cu:300-352; 0: every digit)
                self._glk.relin_keys[elts.index(e)] = boot._key_for_elt(self._sk, self._ctx, e, self._ctx.limbs_at(target) if target else 0)
        self._glk.set_fallback(elts.index(2 * N - 1), self._bk.conj)
        self._freshest = self._ctx.get_first_index() + boot.BOOT_LEVELS
        self._bottom = self._ctx.total_parm_size() - 1
        if self._freshest + cfg.num_scale_levels != self._bottom:
            raise RuntimeError("CKKSEngine: chain layout mismatch")
        if cfg.build_two_scale_arrays:
            self._build_scale_arrays()

    def _build_scale_arrays(self):
        """src/ckks_engine.cu:437-464: the scale a product has at each chain index and what is left after its rescale"""
        ctx = self._ctx
        cur = np.longdouble(self._cfg.user_scale) ** 2
        for idx in range(ctx.total_parm_size()):
            q_drop = np.longdouble(int(ctx.primes[ctx.limbs_at(idx) - 1]))
            self._scale.append(cur)
            self._rescaled.append(cur / q_drop)
            cur = self._rescaled[-1] ** 2

    # ---- the bound surface -----------------------------------------------------------------------------
    def slot_count(self):
        return self._enc.slot_count()

    def user_scale(self):
        return self._cfg.user_scale

    def max_user_level(self):
        return self._cfg.num_scale_levels - 1

    def user_level(self, ct):
        ci = ct.chain_index()
        if ci < self._freshest or ci > self._bottom - 1:
            raise ValueError("CKKSEngine::user_level: ciphertext chain_index is outside the user-scale segment")
        return ci - self._freshest

    def user_level_chain_index(self, user_level):
        if not 0 <= user_level < self._cfg.num_scale_levels:
            raise ValueError("CKKSEngine::user_level_chain_index: user_level out of range")
        return self._freshest + user_level

    def encode(self, values, user_level=0):
        if not 0 <= user_level < self._cfg.num_scale_levels:
            raise ValueError("CKKSEngine::encode: user_level out of range")
        return self._enc.encode_complex_vector(self._ctx, values, self._cfg.user_scale, self._freshest + user_level)

    def encrypt(self, pt):
        return self._sk.encrypt_symmetric(self._ctx, pt)

    def decrypt_decode(self, ct):
        return list(self._enc.decode_complex_vector(self._ctx, self._sk.decrypt(self._ctx, ct)))

    def _assign(self, dst, src):
        dst.__dict__.update(src.__dict__)

    def add_inplace(self, dst, src):
        self._assign(dst, add(self._ctx, dst, src))

    def sub_inplace(self, dst, src):
        self._assign(dst, sub(self._ctx, dst, src))

    def mul_and_relin_inplace(self, dst, src):
        self._assign(dst, multiply_and_relin(self._ctx, dst, src, self.relin_key()))

    def mul_plain_inplace(self, dst, pt):
        self._assign(dst, multiply_plain(self._ctx, dst, pt))

    def rescale_inplace(self, ct):
        if ct.chain_index() >= self._bottom - 1:
            raise RuntimeError("CKKSEngine::rescale_inplace: ciphertext is already at max user_level (pre_boot_index); "
                               "call bootstrap_inplace next.")
        self._assign(ct, rescale_to_next(self._ctx, ct))

    def rotate_inplace(self, ct, step):
        self._assign(ct, rotate(self._ctx, ct, step, self._glk))

    def bootstrap_inplace(self, ct):
        """src/ckks_engine.cu:557-603: any user level in, user level 0 out, scale snapped to user_scale"""
        if self._cfg.use_bootstrap_to_17_levels:
            raise RuntimeError("CKKSEngine::bootstrap_inplace: use_bootstrap_to_17_levels chain does not have a bootstrap "
                               "algorithm yet. For now the new chain supports encode/encrypt/decrypt only.")
        self.user_level(ct)
        if ct.chain_index() != self._bottom - 1:
            mod_switch_to_inplace(self._ctx, ct, self._bottom - 1)
        ct.set_scale(self._cfg.user_scale)
        out = boot.bootstrap(self._ctx, self._enc, ct, self._bk, self._cfg.user_scale, self._cfg.split_scale_down)
        if out.chain_index() != self._freshest + (1 if self._cfg.split_scale_down else 0):
            raise RuntimeError("CKKSEngine::bootstrap_inplace: post-bootstrap chain_index != expected (freshest"
                               + ("+1)" if self._cfg.split_scale_down else ")"))
        out.set_scale(self._cfg.user_scale)
        self._assign(ct, out)

    def context(self):
        return self._ctx

    def encoder(self):
        return self._enc

    def secret_key(self):
        return self._sk

    def relin_key(self):
        return self._bk.relin if self._bk is not None else relin_key()

    def galois_key(self):
        return self._glk

    def scale_array_size(self):
        return len(self._rescaled)

    def ckks_scale_at(self, chain_index):
        return float(self._scale[chain_index]) if chain_index < len(self._scale) else 0.0

    def ckks_rescaled_scale_at(self, chain_index):
        return float(self._rescaled[chain_index]) if chain_index < len(self._rescaled) else 0.0
