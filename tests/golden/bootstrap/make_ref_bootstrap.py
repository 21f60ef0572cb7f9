"""Regenerates tests/golden/bootstrap/ref_bootstrap_n16.json: the UNMODIFIED reference's bootstrap run on this GPU through
oracle/_ref/ref_harness (the chain and inputs of its own round-trip test, test/bootstrap_test.cu:517-662), its refreshed
ciphertext decrypted and decoded by this library (the reference's own decode is broken in this toolchain: its multi-word
add / subtract keep the carry flag across separate asm statements, include/uintmath.cuh:326-361), and this library's
bootstrap on the same chain, message and secret weight beside it.
    usage (GPU box, reference harness built):  python tests/golden/bootstrap/make_ref_bootstrap.py [OUT.json]"""
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.join(ROOT, "phantom-fhe_b200"))
import pyPhantom as ph  # noqa: E402

LOG_N, ALPHA, SCALE = 16, 4, 2.0 ** 40
BITS = [58] + [40] * 4 + [58] * 12 + [29] * 3 + [58] * ALPHA


def context():
    n = 1 << LOG_N
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(n)
    parms.set_special_modulus_size(ALPHA)
    parms.set_coeff_modulus(ph.create_coeff_modulus(n, BITS))
    parms.set_galois_elts(ph.bootstrap_required_galois_elts(LOG_N, [5, 5, 5]))
    return ph.context(parms)


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_bootstrap_n16.json")
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    ctx = context()
    enc = ph.ckks_encoder(ctx)
    rec = {"log_n": LOG_N, "chain_bits": "58|40x4|58x12|29x3|P 58x4", "scale_log2": 40, "slots": 1 << (LOG_N - 1),
           "message": "real, uniform in (-0.5, 0.5), mt19937_64(0xB007B007)", "gpu": torch.cuda.get_device_name(0), "cases": {}}
    for secret, flag in (("sparse128", "0"), ("dense", "1")):
        with tempfile.TemporaryDirectory() as tmp:
            r = subprocess.run([harness, "--bootstrap", tmp, "--boot-dense", flag], capture_output=True, text=True, timeout=900)
            line = [ln for ln in r.stdout.splitlines() if ln.startswith("{\"reference_bootstrap\"")]
            if r.returncode != 0 or not line:
                raise SystemExit("harness failed: " + r.stdout[-500:] + r.stderr[-500:])
            ref = json.loads(line[0])["reference_bootstrap"]
            sk = ph.secret_key().load(open(os.path.join(tmp, "boot_sk.bin"), "rb"))
            ct = ph.ciphertext().load(open(os.path.join(tmp, "boot_ct.bin"), "rb"))
            msg = np.fromfile(os.path.join(tmp, "boot_msg.bin"), dtype=np.float64)
        err = np.abs(enc.decode_double_vector(ctx, sk.decrypt(ctx, ct)) - msg)
        case = {"reference": {"ms": ref["ms_median"], "ms_min": ref["ms_min"], "keygen_s": ref["keygen_s"], "limbs_out": ref["out_limbs"],
                              "max_err": float(err.max()), "mean_err": float(err.mean()), "log2_max_err": math.log2(float(err.max())),
                              "decoded_by": "this library (decrypt + decode of the reference's saved ciphertext with its saved secret)",
                              "its_own_decode_max_err": ref["own_decode_max_err"]}}
        # this library on the same message, with the reference's secret key (so the same weight and values)
        t0 = time.perf_counter()
        bk = ph.create_bootstrap_key(ctx, enc, sk, sparse_hamming_weight=128, eval_mod_levels=9, user_scale=SCALE)
        torch.cuda.synchronize()
        keygen_s = time.perf_counter() - t0
        mine = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, msg, SCALE, chain_index=1))
        ph.mod_switch_to_inplace(ctx, mine, ctx.total_parm_size() - 2)
        for _ in range(3):
            out = ph.bootstrap(ctx, enc, mine, bk, SCALE)
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = ph.bootstrap(ctx, enc, mine, bk, SCALE)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        e2 = np.abs(enc.decode_double_vector(ctx, sk.decrypt(ctx, out)) - msg)
        case["this_library"] = {"ms": float(np.median(times)), "keygen_s": keygen_s, "limbs_out": out.coeff_modulus_size(),
                                "max_err": float(e2.max()), "mean_err": float(e2.mean()), "log2_max_err": math.log2(float(e2.max()))}
        rec["cases"][secret] = case
        del bk
        torch.cuda.empty_cache()
        print(secret, json.dumps(case))
    json.dump(rec, open(out_path, "w"), indent=1)
    print("wrote", out_path)


if __name__ == "__main__":
    main()
