#!/usr/bin/env python
"""bench.py - KeySwitch/s of CKKS hybrid key switching at N = 2^16, L = 24, dnum = 3 on B200.

Workload (the configuration the headline metric is quoted on): 24 Q limbs (one 60-bit prime and 23
primes of 40 bits), 8 special primes of 60 bits, alpha = 8, 3 digits; ciphertext and evaluation-key
limbs uniform in [0, q_i) from a seeded generator (synthetic; the path is integer-only).
A step = one batch of BATCH (default 64) key switches on distinct ciphertexts cycling over KEYS
distinct evaluation keys, so one step touches several GB, far more than the 126 MB L2 (that is this
file's answer to the L2-flush rule: inputs larger than L2).

  value : KeySwitch/s over all ranks, inputs resident in HBM, device time (CUDA events, max over ranks)
  e2e   : the same metric through the reference-facing Python call (pyPhantom.relinearize, the
          pybind11 surface of the reference) with HOST buffers: every key switch copies its
          3-polynomial ciphertext in from pinned memory and its 2-polynomial result back out
  roofline : the WHOLE key switch against the HBM roofline: 312 limbs = 163.6 MB of compulsory traffic
          (c2, key digits, ciphertext in and out) over the measured time per key switch
  roofline_issue : the same time against the instruction-issue roofline (warp instructions per key
          switch from the committed ncu capture over 148 SMs x 4 schedulers x the sampled SM clock)
  kernels : per kernel, timed live with CUDA events on its own stream: algorithmic bytes beside the DRAM
          bytes ncu saw, and what actually bounds it
  cpu_baseline : the CPU restatement (oracle/) timed on this box's cores on a bounded sample

Multi-GPU: one process per GPU (torchrun); the path shards by independent ciphertexts, every rank
runs its own batch with its own copy of the keys, no data-path collective ("weak" scaling).
`--impl reference` times the reference's algorithm on the host cores: the reference has no CPU
implementation of this path (its src/host only builds tables), so the arm runs the CPU
restatement under oracle/ with every host thread.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "phantom-fhe_b200"))

LOGN, N = 16, 1 << 16
BITS = [60] + [40] * 23 + [60] * 8
SPECIAL, LEVEL = 8, 24
BETA = 3
LIMB_BYTES = 8 * N
# algorithmic bytes of one key switch: c2 + evk + ct in + ct out = 5l + 2*beta*(l+alpha) limbs
KS_LIMBS = 5 * LEVEL + 2 * BETA * (LEVEL + SPECIAL)
KS_BYTES = KS_LIMBS * LIMB_BYTES
WORKLOAD = "hybrid_keyswitch_N65536_L24_dnum3_alpha8"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """samples nvidia-smi clocks and throttle reasons; start() early (the tool needs about a second to
    come up), then mark() the timed region; only samples taken inside it are summarised"""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.lines, self.proc, self.t0, self.t1 = gpu_index, [], None, None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc:
            time.sleep(0.12)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        inside = [ln for (t, ln) in self.lines if self.t0 is not None and self.t0 <= t <= self.t1 + 0.1]
        used = inside or [ln for (_, ln) in self.lines]
        sm, mx, reasons = [], 0.0, set()
        for ln in used:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm), "window": "timed region" if inside else "whole run (timed region shorter than the sampling period)"}


def bind_to_gpu_numa_node(torch, local_rank):
    """Pinned host buffers are placed by first touch: running this rank's threads on the cores of the NUMA node its GPU
    hangs off keeps the e2e arm's staging memory on that node, so that eight ranks do not all copy through one socket's
    memory controller. Returns what was done, for the line; does nothing where the node is not exposed (-1)."""
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bus = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return {"node": None, "why": "the GPU's NUMA node is not exposed"}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return {"node": node, "why": "none of the node's cores is in this process's affinity mask"}
        os.sched_setaffinity(0, cpus)
        return {"node": node, "cores": len(cpus)}
    except (OSError, ValueError, AttributeError) as e:
        return {"node": None, "why": str(e)[:120]}


def config_dict(args, world):
    """what both arms report as `config`: the workload and how a step is made of it"""
    S = max(1, min(args.streams, args.batch))
    return {"workload": WORKLOAD, "batch_per_step_per_gpu": args.batch, "distinct_keys": args.keys, "streams": S,
            "launch": ("b2_keyswitch_batch: one call per key over its %d ciphertexts" % (-(-args.batch // args.keys))) if args.launch == "batched"
            else "b2_keyswitch: one call per ciphertext",
            "l2": "inputs larger than L2 (a step touches %.1f GB)" % (args.batch * 3 * LEVEL * LIMB_BYTES / 1e9 + args.keys * 0.1),
            "parallelism": f"dp{world}"}


def run_reference_arm(args, rank, world, out_stream):
    """the reference's algorithm on the host cores (CPU restatement, every core this process may use, whatever
    OMP_NUM_THREADS the launcher exported); rank 0 only. A step of this arm is ONE key switch of the workload (a bounded
    sample of the batch the GPU arm runs per step): the value is key switches per second either way."""
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Oracle, create_coeff_modulus, use_all_cores
    cores = use_all_cores()
    primes = create_coeff_modulus(N, BITS)
    o = Oracle(N, primes, SPECIAL)
    key = o.synth_key(BETA, 2, 10)
    c2 = o.fill(1, primes[:LEVEL], 2, 3)[0]
    ct = o.synth_ct(LEVEL, 2, 1)
    for _ in range(args.warmup):
        o.keyswitch(LEVEL, c2, key, ct)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.keyswitch(LEVEL, c2, key, ct)
    dt = time.perf_counter() - t0
    v = args.steps / dt
    line = {"impl": "reference", "metric": "KeySwitch/s", "value": v, "unit": "KeySwitch/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": config_dict(args, world),
            "cpu_baseline": {"value": v, "unit": "KeySwitch/s", "cores": cores, "kind": "port",
                             "sample": f"{args.steps} key switches of the workload, one per step (a bounded sample of the batch)"},
            "e2e": {"value": v, "unit": "KeySwitch/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference has no CPU implementation of this path; this is the CPU restatement in oracle/"}
    print(json.dumps(line), file=out_stream, flush=True)


def cpu_baseline_sample(budget_s=12.0):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Oracle, create_coeff_modulus, use_all_cores
    cores = use_all_cores()
    primes = create_coeff_modulus(N, BITS)
    o = Oracle(N, primes, SPECIAL)
    key = o.synth_key(BETA, 2, 10)
    c2 = o.fill(1, primes[:LEVEL], 2, 3)[0]
    ct = o.synth_ct(LEVEL, 2, 1)
    o.keyswitch(LEVEL, c2, key, ct)
    n, t0 = 0, time.perf_counter()
    while True:
        o.keyswitch(LEVEL, c2, key, ct)
        n += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or n >= 64:
            break
    return {"value": n / dt, "unit": "KeySwitch/s", "cores": cores, "kind": "port",
            "sample": f"{n} key switches of the same workload in {dt:.1f} s"}


# algorithmic limbs moved per launch class inside ONE key switch at this workload
# (a two-pass transform moves 2 limb-passes per limb algorithmically, so each pass is credited one)
def kernel_alg_bytes_per_keyswitch():
    l, a, b, lP = LEVEL, SPECIAL, BETA, LEVEL + SPECIAL
    up_ntt = b * lP - l
    alg = {
        "ntt_inv_cluster": 2 * (l + 2 * a) * LIMB_BYTES,
        "ntt_fwd_cluster": 2 * (up_ntt + 2 * l) * LIMB_BYTES,
        "ntt_inv_rows": (l + 2 * a) * LIMB_BYTES,
        "ntt_inv_cols": (l + 2 * a) * LIMB_BYTES,
        "ntt_fwd_cols": (up_ntt + 2 * l) * LIMB_BYTES,
        "ntt_fwd_rows": (up_ntt + 2 * l) * LIMB_BYTES,
        "bconv": ((l + l + b * lP) + (2 * a + 2 * l)) * LIMB_BYTES,
        "ks_inner_prod": (b * lP + 2 * b * lP + 2 * lP) * LIMB_BYTES,
    }
    if os.environ.get("B2_KS_FUSED_IP", "1")[:1] != "0":
        # the Q limbs on FP64 primes (all but the leading 60-bit one) take their inner product inside ModUp's last pass:
        # per such limb (b - 1) unfinished digits + the input's own limb + 2 b key limbs + read and write of both ct limbs
        wide = sum(1 for x in BITS[:l] if x > 41)
        nf, rest = l - wide, wide + a
        alg["ntt_fwd_rows"] = (b * rest - wide + 2 * l) * LIMB_BYTES
        alg["ks_inner_prod"] = (b * rest + 2 * b * rest + 2 * rest) * LIMB_BYTES
        alg["ntt_fwd_rows_mac"] = ((b - 1) * nf + nf + 2 * b * nf + 4 * nf) * LIMB_BYTES
    return alg


def ntt_section(ph, ctx, torch, LIB, check, N, n_limbs, reps=20):
    """forward and inverse transforms over n_limbs limbs, cycling through 16 buffers (268 MB at 32 limbs: larger than L2)"""
    bufs = torch.randint(0, 1 << 30, (16, n_limbs, N), dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream()
    out = {}
    for name, fn in (("forward", LIB.b2_ntt_forward), ("inverse", LIB.b2_ntt_inverse)):
        for i in range(16):
            check(fn(ctx._h, bufs[i].data_ptr(), n_limbs, 0, st.cuda_stream))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(st)
        for r in range(reps):
            for i in range(16):
                check(fn(ctx._h, bufs[i].data_ptr(), n_limbs, 0, st.cuda_stream))
        e1.record(st)
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / 1e3
        per_s = reps * 16 * n_limbs / sec
        # the same calls dealt over four streams (independent buffers), as a batch of ciphertexts would issue them
        side = [torch.cuda.Stream() for _ in range(4)]
        for sd in side:
            sd.wait_stream(st)
        torch.cuda.synchronize()
        e0.record(st)
        for sd in side:
            sd.wait_stream(st)
        for r in range(reps):
            for i in range(16):
                check(fn(ctx._h, bufs[i].data_ptr(), n_limbs, 0, side[i % 4].cuda_stream))
        for sd in side:
            st.wait_stream(sd)
        e1.record(st)
        torch.cuda.synchronize()
        per_s4 = reps * 16 * n_limbs / (e0.elapsed_time(e1) / 1e3)
        out[name] = {"limb_transforms_per_s": per_s4, "alg_gbs": per_s4 * 2 * 8 * N / 1e9, "streams": 4,
                     "one_stream_limb_transforms_per_s": per_s}
    return {"N": N, "limbs_per_call": n_limbs, **out}


def bootstrap_section(ph, torch, np):
    """one CKKS bootstrap at N = 2^16 on a 24-limb chain (dnum 3), sparse ternary secret of weight 192,
    2^15 slots uniform in [-1, 1] scaled into |m| <= 0.5; decryption error against the message"""
    import math
    log_n, alpha = 16, 8
    n_ring = 1 << log_n
    bits = [58] + [40] * 8 + [58] * 12 + [29] * 3 + [58] * alpha
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(n_ring)
    parms.set_special_modulus_size(alpha)
    parms.set_coeff_modulus(ph.create_coeff_modulus(n_ring, bits))
    parms.set_galois_elts(ph.bootstrap_required_galois_elts(log_n, [5, 5, 5]))
    ctx = ph.context(parms)
    sk = ph.secret_key(ctx, seed=5)
    sk.generate_sparse(ctx, 192)
    enc = ph.ckks_encoder(ctx)
    t0 = time.perf_counter()
    bk = ph.create_bootstrap_key(ctx, enc, sk, sparse_hamming_weight=128, eval_mod_levels=9, user_scale=2.0 ** 40)
    torch.cuda.synchronize()
    keygen_s = time.perf_counter() - t0
    msg = 0.5 * np.random.default_rng(5).uniform(-1.0, 1.0, n_ring // 2)
    ct = sk.encrypt_symmetric(ctx, enc.encode_double_vector(ctx, msg, 2.0 ** 40, chain_index=1))
    ph.mod_switch_to_inplace(ctx, ct, ctx.total_parm_size() - 2)
    launches0 = int(ph._native.LIB.b2_launch_count())
    ph._native.check(ph._native.LIB.b2_profile_start(ctx._h))
    out = ph.bootstrap(ctx, enc, ct, bk, 2.0 ** 40)   # eager: every kernel is launched from the host, counted and timed
    names = ctypes.create_string_buffer(8192)
    tot, cnt, n_out = (ctypes.c_float * 128)(), (ctypes.c_uint32 * 128)(), ctypes.c_size_t()
    ph._native.check(ph._native.LIB.b2_profile_stop(ctx._h, names, 8192, tot, cnt, 128, ctypes.byref(n_out)))
    launches = int(ph._native.LIB.b2_launch_count()) - launches0
    nm = names.value.decode().strip(";").split(";")
    # summed device time per kernel name with every launch timed on its own stream (they overlap across the pipeline's
    # streams, so the sum is well above the wall time of one bootstrap: read the shares)
    kernel_ms = {nm[i]: {"launches": int(cnt[i]), "ms": round(float(tot[i]), 3)} for i in range(n_out.value)}
    for _ in range(3):                                  # the second call captures the CUDA graph, later ones replay it
        out = ph.bootstrap(ctx, enc, ct, bk, 2.0 ** 40)
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = ph.bootstrap(ctx, enc, ct, bk, 2.0 ** 40)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    err = np.abs(enc.decode_double_vector(ctx, sk.decrypt(ctx, out)) - msg)
    return {"ms": float(np.median(times)), "ms_min": float(min(times)), "kernels_per_bootstrap": launches, "mode": "CUDA graph replay",
            "log2_max_err": math.log2(float(err.max())), "max_err": float(err.max()), "mean_err": float(err.mean()),
            "limbs_in": 2, "limbs_out": out.coeff_modulus_size(), "usable_levels_out": out.coeff_modulus_size() - 1, "chain_bits": "58|40x8|58x12|29x3|P 58x8",
            "secret_hamming_weight": 192, "keygen_s": keygen_s,
            "key_bytes": int(bk.key_bytes), "key_bytes_what": "rotation keys (each with only the digits its shallowest use needs), conjugation and relinearisation key",
            "kernels_eager": kernel_ms}


def compositions_section(ph, ctx, torch, np, synth, primes, keys, N, level, reps=20):
    """the evaluator calls built on the key switch, at the bench level (24 limbs), through the pyPhantom surface:
    one stream (latency; the reference's own kernels, timed in the same run, are under `reference_gpu`) and a batch
    of 8 over 4 streams (throughput)"""
    from pyPhantom import _native
    def ct_of(buf, n_poly=2):
        c = ph.ciphertext()
        c._chain_index, c._size, c._N, c._limbs = 1, n_poly, N, level
        c.data = torch.from_numpy(synth.poly(N, primes[:level], n_poly, 77, buf).view(np.int64)).cuda()
        return c
    cts = [ct_of(300 + i) for i in range(8)]
    rlk = keys[0]
    glk = ph.galois_key.from_keys([keys[i % len(keys)] for i in range(len(ctx.galois_elts))])
    steps = [s for s in (1, 2, 3) if ph.get_elt_from_step(s, N) in ctx.galois_elts]
    ops = {
        "multiply_and_relin": lambda c: ph.multiply_and_relin(ctx, c, c, rlk),
        "multiply_and_relin_rescale": lambda c: ph.rescale_to_next(ctx, ph.multiply_and_relin(ctx, c, c, rlk)),
        "rescale": lambda c: ph.rescale_to_next(ctx, c),
    }
    if steps:
        ops["rotate"] = lambda c: ph.rotate(ctx, c, steps[0], glk)
        ops["hoist_rotations_x%d" % len(steps)] = lambda c: ph.hoist_rotations(ctx, c, glk, steps)
    out = {}
    main = torch.cuda.current_stream()
    side = [torch.cuda.Stream() for _ in range(4)]
    for name, fn in ops.items():
        for _ in range(3):
            fn(cts[0])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for r in range(reps):
            fn(cts[r % 8])
        e1.record()
        torch.cuda.synchronize()
        one = 1e3 * e0.elapsed_time(e1) / reps

        def batch8(n):
            for sd in side:
                sd.wait_stream(main)
            for r in range(n):
                for b in range(8):
                    with torch.cuda.stream(side[b % 4]):
                        fn(cts[b])
            for sd in side:
                main.wait_stream(sd)

        batch8(2)  # the side streams' allocator pools grow on first use: not part of the measurement
        torch.cuda.synchronize()
        e0.record()
        batch8(reps)
        e1.record()
        torch.cuda.synchronize()
        out[name] = {"us_one_stream": one, "per_s_batch8_streams4": 8 * reps / (e0.elapsed_time(e1) / 1e3)}
    return out


def bsgs_section(ph, torch, np, synth):
    """plaintext 4096 x 4096 matrix times ciphertext by the diagonal method: N = 2^16, 16 limbs at input, baby step 64,
    giant step 64, synthetic diagonals and keys (8 distinct keys cycled over the 126 rotation steps).
    reference_driver: pyPhantom.bsgs_matmul_preencoded, the reference's algorithm (host-resident int64 diagonals expanded
    per giant, chained babies, Horner giants; limb-identical to the reference, tests/golden/full).
    resident: pyPhantom.linalg.resident_bsgs (expanded diagonals resident in HBM, hoisted babies, giants sharing a ModDown)."""
    from pyPhantom.linalg import resident_bsgs
    n_ring, level, M, G = 1 << 16, 16, 64, 64
    steps = list(range(1, M)) + [g * M for g in range(1, G)]
    mods = ph.create_coeff_modulus(n_ring, [60] + [40] * 23 + [60] * 8)
    primes = [m.value() for m in mods]
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(n_ring)
    parms.set_coeff_modulus(mods)
    parms.set_special_modulus_size(8)
    parms.set_galois_elts(ph.get_elts_from_steps(steps, n_ring))
    ctx = ph.context(parms)
    chain = ctx.size_Q - level + 1
    beta = ctx.beta(level)
    keys = [ph.relin_key.from_numpy(ctx, [synth.poly(n_ring, primes, 2, 91, 10 + 8 * k + d) for d in range(beta)]) for k in range(8)]
    glk = ph.galois_key.from_keys([keys[i % 8] for i in range(len(ctx.galois_elts))])
    x = ph.ciphertext()
    x._chain_index, x._size, x._N, x._limbs, x._scale = chain, 2, n_ring, level, 2.0 ** 40
    x.data = torch.from_numpy(synth.poly(n_ring, primes[:level], 2, 91, 1).view(np.int64)).cuda()
    rng = np.random.default_rng(91)
    base = [ph.single_chain_plaintext(rng.integers(-(1 << 39), 1 << 39, n_ring, dtype=np.int64), 2.0 ** 40) for _ in range(64)]
    diags = ph.bsgs_diagonals([base[d % 64] for d in range(M * G)], M * G, M, G)

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ref_driver_ms = timed(lambda: ph.bsgs_matmul_preencoded(ctx, glk, x, diags), 2)
    t0 = time.perf_counter()
    op = resident_bsgs(ctx, glk, diags, chain)
    setup_s = time.perf_counter() - t0
    resident_ms = timed(lambda: op.apply(x), 5)
    ref_ms = None
    try:
        ref_ms = json.load(open(os.path.join(ROOT, "tests", "golden", "full", "n16_l16_bsgs_m64g64.json")))["times_us"]["bsgs_us"] / 1e3
    except (OSError, KeyError, ValueError):
        pass
    return {"workload": "4096x4096 plaintext matrix x ciphertext, N=65536, 16 limbs, M=G=64", "resident_ms": resident_ms,
            "resident_setup_s": setup_s, "resident_hbm_gb": op.pts.numel() * 8 / 1e9, "reference_driver_ms": ref_driver_ms,
            "reference_ms_same_gpu": ref_ms, "reference_source": "tests/golden/full/n16_l16_bsgs_m64g64.json times_us.bsgs_us"}


def hmult_section(torch, dist, ctx, LIB, check, _native, dev_ct3, key_tabs, world, streams_n, reps=5, batched=True):
    """BASELINE config 3: HMult + relinearise + rescale on 64 independent ciphertext pairs at 24 limbs, sharded data-parallel
    (64 / world pairs per rank, no collective), resident, spread over the same number of streams as the headline batch.
    Algorithmic bytes per pair: 4l + 2 beta (l + alpha) + 2 (l - 1) = 334 limbs = 175.1 MB."""
    pairs = max(1, 64 // world)
    B = len(dev_ct3)
    S = max(1, min(streams_n, pairs))
    main = torch.cuda.current_stream()
    side = [torch.cuda.Stream() for _ in range(S)] if S > 1 else [main]
    prod = [torch.empty(2, LEVEL, N, dtype=torch.int64, device="cuda") for _ in range(S)]
    outs = [torch.empty(2, LEVEL - 1, N, dtype=torch.int64, device="cuda") for _ in range(S)]
    ws_m = [ctx.workspace(_native.OP_MUL_RELIN, LEVEL) for _ in range(S)]
    ws_r = [ctx.workspace(_native.OP_RESCALE, LEVEL) for _ in range(S)]

    if batched:
        # the pairs of one key in one b2_multiply_relin_rescale_batch call (operands a = (c0, c1) of ciphertext p, b = those of
        # ciphertext p + 1, gathered once outside the timed region); the keys' groups on their own streams
        K = len(key_tabs)
        groups = []
        for k in range(K):
            idx = list(range(k, pairs, K))
            if idx:
                a = torch.stack([dev_ct3[p % B][:2] for p in idx]).contiguous()
                b = torch.stack([dev_ct3[(p + 1) % B][:2] for p in idx]).contiguous()
                out = torch.empty(len(idx), 2, LEVEL - 1, N, dtype=torch.int64, device="cuda")
                nbytes = int(LIB.b2_multiply_relin_batch_workspace_bytes(ctx._h, LEVEL, len(idx)))
                groups.append((k, a, b, out, torch.empty(nbytes // 8, dtype=torch.int64, device="cuda"), nbytes))
        S = max(1, min(streams_n, len(groups)))
        side = side[:S]

    def run_batched():
        for sd in side:
            sd.wait_stream(main)
        for i, (k, a, b, out, ws, nbytes) in enumerate(groups):
            check(LIB.b2_multiply_relin_rescale_batch(ctx._h, LEVEL, a.shape[0], a.data_ptr(), 2 * LEVEL, b.data_ptr(), 2 * LEVEL, key_tabs[k].ctypes.data,
                                                      BETA, out.data_ptr(), 2 * (LEVEL - 1), 1, ws.data_ptr(), nbytes, side[i % S].cuda_stream))
        for sd in side:
            main.wait_stream(sd)

    def run():
        if batched:
            return run_batched()
        for sd in side:
            sd.wait_stream(main)
        for p in range(pairs):
            i = p % S
            a, b = dev_ct3[p % B], dev_ct3[(p + 1) % B]
            st = side[i].cuda_stream
            check(LIB.b2_multiply_and_relin(ctx._h, LEVEL, a.data_ptr(), b.data_ptr(), key_tabs[p % len(key_tabs)].ctypes.data, BETA,
                                            prod[i].data_ptr(), ws_m[i][0].data_ptr(), ws_m[i][1], st))
            check(LIB.b2_rescale(ctx._h, LEVEL, 2, prod[i].data_ptr(), outs[i].data_ptr(), ws_r[i][0].data_ptr(), ws_r[i][1], st))
        for sd in side:
            main.wait_stream(sd)

    run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    for _ in range(reps):
        run()
    e1.record(main)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    per_s = world * pairs * reps / (ms / 1e3)
    limbs = 4 * LEVEL + 2 * BETA * (LEVEL + SPECIAL) + 2 * (LEVEL - 1)
    peak, peak_kind = peaks()
    return {"workload": "64 ciphertext pairs, HMult + relinearise + rescale, N=65536, 24 limbs, dnum 3", "pairs_per_gpu": pairs, "streams": S,
            "launch": "b2_multiply_relin_rescale_batch: one call per key" if batched else "b2_multiply_and_relin + b2_rescale per pair",
            "pairs_per_s": per_s, "us_per_pair_per_gpu": 1e3 * ms / (pairs * reps), "alg_bytes_per_pair": limbs * LIMB_BYTES,
            "hbm_frac": per_s / world * limbs * LIMB_BYTES / 1e9 / peak, "peak_kind": peak_kind, "reps": reps}


def reference_gpu_section():
    """the unmodified reference's own kernels on this GPU, measured in this run through oracle/_ref/ref_harness (built from the
    reference's sources where a checkout was present; None when it is absent): the key switch and its callers on one stream,
    and the key switch from four host threads (the reference runs on per-thread default streams)"""
    h = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    if not os.path.exists(h):
        return None
    import tempfile
    bits = ",".join(str(b) for b in BITS)
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "ref.json")
        cmd = [h, "--logn", str(LOGN), "--bits", bits, "--special", str(SPECIAL), "--level", str(LEVEL), "--seed", "2", "--steps", "1,2,-1",
               "--time", "40", "--threads", "4", "--out", out]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
            if r.returncode != 0:
                return {"error": (r.stderr or r.stdout)[-300:]}
            t = json.load(open(out))["times_us"]
        except (OSError, subprocess.SubprocessError, ValueError, KeyError) as e:
            return {"error": str(e)[:300]}
    res = {"keyswitch_us": t.get("keyswitch_us"), "multiply_and_relin_us": t.get("mul_relin_us"), "multiply_and_relin_rescale_us": t.get("mul_relin_rescale_us"),
           "rotate_us": t.get("rotate_us"), "hoist_rotations_x3_us": t.get("hoist_rotations_us"), "ntt_fwd_32_limbs_us": t.get("ntt_fwd_us"),
           "modup_us": t.get("modup_us"), "inner_prod_us": t.get("inner_prod_us"), "moddown_x2_us": t.get("moddown_x2_us"),
           "source": "oracle/_ref/ref_harness --time 40 --threads 4, run inside this bench"}
    if t.get("keyswitch_mt_us"):
        res["keyswitch_per_s_4_threads"] = 4e6 / t["keyswitch_mt_us"]
    return res


def _claim_stdout():
    """stdout carries the one JSON line and nothing else: libraries that write to file descriptor 1 on their own (NCCL's
    version banner does) are pointed at stderr, and the line goes out through a private copy of the original descriptor"""
    sys.stdout.flush()
    keep = os.dup(1)
    os.dup2(2, 1)
    return os.fdopen(keep, "w")


def main():
    out_stream = _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64, help="key switches per step per GPU")
    ap.add_argument("--keys", type=int, default=4, help="distinct evaluation keys cycled over")
    ap.add_argument("--streams", type=int, default=4, help="CUDA streams the batch of independent key switches is spread over")
    ap.add_argument("--launch", default="batched", choices=["batched", "single"],
                    help="batched: the ciphertexts of one key go through b2_keyswitch_batch in one call; single: one b2_keyswitch call each")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer arm (used for ncu captures)")
    ap.add_argument("--e2e-streams", type=int, default=4, help="streams of the host-buffer arm (copy in, key switch, copy out per stream)")
    ap.add_argument("--no-extras", action="store_true", help="skip the NTT and bootstrap sections of the line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world, out_stream)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import pyPhantom as ph
    from pyPhantom import _native
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import synth  # the seeded generator of synthetic limbs the tests use
    from pyPhantom._native import LIB, check

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # ---- context, keys and ciphertexts ---------------------------------------------------------
    mods = ph.create_coeff_modulus(N, BITS)
    primes = [m.value() for m in mods]
    parms = ph.params(ph.scheme_type.ckks)
    parms.set_poly_modulus_degree(N)
    parms.set_coeff_modulus(mods)
    parms.set_special_modulus_size(SPECIAL)
    parms.set_galois_elts([2 * N - 1] + ph.get_elts_from_steps([1, 2, 3], N))
    ctx = ph.context(parms)
    B, K = args.batch, args.keys
    seed = 1000 + rank
    keys = [ph.relin_key.from_numpy(ctx, [synth.poly(N, primes, 2, seed, 10 + 8 * k + d) for d in range(BETA)])
            for k in range(K)]
    key_tabs = [k.pointer_table() for k in keys]
    # ciphertexts (c0, c1, c2): limb j uniform in [0, q_j), drawn on the device (64 of them from the host generator would
    # take half a minute); the e2e arm copies them out to pinned host buffers once, before its timed region
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    # Ciphertext b is switched with key b % K: the ciphertexts of one key sit in one tensor [B / K][3][limbs][N], so that the
    # batched entry point can take them in one call.
    per_key = [len(range(k, B, K)) for k in range(K)]
    dev_groups = [torch.stack([torch.randint(0, int(q), (n, 3, N), dtype=torch.int64, device="cuda", generator=gen) for q in primes[:LEVEL]], dim=2)
                  if n else None for n in per_key]
    dev_ct3 = [dev_groups[b % K][b // K] for b in range(B)]
    # pinned staging: at most 32 ciphertexts' worth per rank (2 GB in, 1.3 GB out; eight ranks share one host), reused in stream
    # order: ciphertext b travels through buffers b % n_host, and 32 is a multiple of the stream and key counts, so ciphertexts
    # that share a buffer also share the stream and the key
    lcm = int(np.lcm(max(1, args.e2e_streams), max(1, args.keys)))
    n_host = 0 if args.no_e2e else (B if B <= 32 else max(lcm, 32 // lcm * lcm))
    affinity = os.sched_getaffinity(0)
    numa = None if args.no_e2e else bind_to_gpu_numa_node(torch, local_rank)
    host_ct3 = [torch.empty(3, LEVEL, N, dtype=torch.int64).pin_memory() for _ in range(n_host)]
    for h, d in zip(host_ct3, dev_ct3):
        h.copy_(d)
    host_out = [torch.empty(2, LEVEL, N, dtype=torch.int64).pin_memory() for _ in range(n_host)]
    for h in host_out:
        h.zero_()  # first touch while still bound to the GPU's node
    os.sched_setaffinity(0, affinity)
    S = max(1, min(args.streams, B))
    wss = [ctx.workspace(_native.OP_KEYSWITCH, LEVEL) for _ in range(S)]
    batched = args.launch == "batched"
    if batched:
        ks_wsb = [ph.keyswitch_batch_workspace(ctx, LEVEL, max(per_key)) for _ in range(min(S, K))]
    stream = torch.cuda.current_stream()
    side = [torch.cuda.Stream() for _ in range(S)] if S > 1 else [stream]
    fork, joins = torch.cuda.Event(), [torch.cuda.Event() for _ in range(S)]

    def step_batched():
        # the ciphertexts that share a key go through b2_keyswitch_batch in one call (every kernel one launch over them);
        # the keys' groups are spread over the streams
        L = len(ks_wsb)
        if L > 1:
            fork.record(stream)
        for i in range(L):
            st = side[i] if L > 1 else stream
            if L > 1:
                st.wait_event(fork)
            for k in range(i, K, L):
                g = dev_groups[k]
                if g is None:
                    continue
                check(LIB.b2_keyswitch_batch(ctx._h, LEVEL, g.shape[0], g[0, 2].data_ptr(), 3 * LEVEL, key_tabs[k].ctypes.data, BETA,
                                             g.data_ptr(), 3 * LEVEL, ks_wsb[i].data_ptr(), ks_wsb[i].numel() * 8, st.cuda_stream))
            if L > 1:
                joins[i].record(st)
                stream.wait_event(joins[i])

    def step_resident():
        # the batch's key switches are independent: spread them over S streams (each with its own
        # scratch) so that one ciphertext's memory phases overlap another's arithmetic
        if batched:
            return step_batched()
        if S > 1:
            fork.record(stream)
        for i, st in enumerate(side):
            if S > 1:
                st.wait_event(fork)
            ws, ws_bytes = wss[i]
            for b in range(i, B, S):
                t = dev_ct3[b]
                check(LIB.b2_keyswitch(ctx._h, LEVEL, t[2].data_ptr(), key_tabs[b % K].ctypes.data, BETA, t.data_ptr(),
                                       ws.data_ptr(), ws_bytes, st.cuda_stream))
            if S > 1:
                joins[i].record(st)
                stream.wait_event(joins[i])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- value: inputs resident --------------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step_resident()
    barrier()
    sampler.mark_begin()
    launches0 = int(LIB.b2_launch_count())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step_resident()
    e1.record(stream)
    barrier()
    sampler.mark_end()
    ms = e0.elapsed_time(e1)
    launches = int(LIB.b2_launch_count()) - launches0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * B * args.steps / (ms / 1e3)

    # ---- e2e: host buffers through the pyPhantom surface, copies inside the timed region -----------
    streams = [torch.cuda.Stream() for _ in range(args.e2e_streams)]
    stage = [torch.empty(3, LEVEL, N, dtype=torch.int64, device="cuda") for _ in streams]

    def step_e2e():
        for b in range(B):
            st = streams[b % len(streams)]
            with torch.cuda.stream(st):
                buf = stage[b % len(streams)]
                buf.copy_(host_ct3[b % n_host], non_blocking=True)
                ct = ph.ciphertext()
                ct._chain_index, ct._size, ct._N, ct._limbs, ct.data = 1, 3, N, LEVEL, buf
                res = ph.relinearize(ctx, ct, keys[b % K])
                host_out[b % n_host].copy_(res.data, non_blocking=True)

    def drain_e2e():
        for st in streams:
            st.synchronize()

    # The steps are issued back to back, as a service with requests queued would issue them: ciphertext b always
    # travels on stream b % streams, so its staging buffer and its host result are reused in stream order, and the
    # copy engines never idle between steps. One drain ends the timed region.
    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 10))
    for _ in range(0 if args.no_e2e else 2):
        step_e2e()
    drain_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    drain_e2e()
    barrier()
    e2e_s = max(time.perf_counter() - t0, 1e-9)
    if e2e_steps:
        # what came back over PCIe is what the same call gives with nothing else in flight
        ct = ph.ciphertext()
        ct._chain_index, ct._size, ct._N, ct._limbs, ct.data = 1, 3, N, LEVEL, host_ct3[(B - 1) % n_host].cuda()
        alone = ph.relinearize(ctx, ct, keys[(B - 1) % K]).data.cpu()
        if not torch.equal(alone, host_out[(B - 1) % n_host]):
            raise RuntimeError("e2e: the pipelined result differs from the same key switch run alone")
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * B * e2e_steps / e2e_s

    # ---- what the link itself gives for this call's traffic: bare pinned copies, both directions at once ----------
    pcie = None
    if e2e_steps and world == 1 and not args.no_extras:
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        d_res = [torch.empty(2, LEVEL, N, dtype=torch.int64, device="cuda") for _ in range(2)]

        def copies(reps):
            for i in range(reps):
                with torch.cuda.stream(s_in):
                    stage[i % len(stage)].copy_(host_ct3[i % n_host], non_blocking=True)
                with torch.cuda.stream(s_out):
                    host_out[i % n_host].copy_(d_res[i % 2], non_blocking=True)
            s_in.synchronize()
            s_out.synchronize()

        copies(8)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        copies(40)
        dt = time.perf_counter() - t0
        pcie = {"h2d_gbs": 40 * 3 * LEVEL * LIMB_BYTES / dt / 1e9, "d2h_gbs": 40 * 2 * LEVEL * LIMB_BYTES / dt / 1e9,
                "keyswitch_per_s_ceiling": 40 / dt, "what": "bare pinned copies of one call's input and result, both directions at once"}

    # ---- N > 1: key switches with their RNS limbs spread over the ranks (NCCL all-gathers between the phases) ---------
    limb_sharded = None
    if world > 1:
        from pyPhantom.parallel import BatchedLimbShardedKeySwitch
        sh = BatchedLimbShardedKeySwitch(ctx)
        ws_sh, _ = sh.workspace(LEVEL)
        # one ciphertext spread over the ranks: every rank holds the SAME key and ciphertexts here (the data-parallel arm above
        # gives each rank its own), drawn from a seed common to all ranks
        key_sh = ph.relin_key.from_numpy(ctx, [synth.poly(N, primes, 2, 999, 10 + d) for d in range(BETA)])
        key_sh_tab = key_sh.pointer_table()
        gen_sh = torch.Generator(device="cuda")
        gen_sh.manual_seed(999)
        n_sh_ct = max(1, min(B, 32))
        sh_ct3 = [torch.stack([torch.randint(0, int(q), (3, N), dtype=torch.int64, device="cuda", generator=gen_sh) for q in primes[:LEVEL]], dim=1)
                  for _ in range(n_sh_ct)]
        c2_sh, ct_sh = sh_ct3[0][2], sh_ct3[0][:2].clone()
        # what the sharded ranks produce is what one GPU's b2_keyswitch produces: gather the limbs and compare (every rank)
        want = sh_ct3[0][:2].clone()
        ws1, ws1_bytes = wss[0]
        check(LIB.b2_keyswitch(ctx._h, LEVEL, c2_sh.data_ptr(), key_sh_tab.ctypes.data, BETA, want.data_ptr(), ws1.data_ptr(), ws1_bytes,
                               stream.cuda_stream))
        sh.keyswitch(LEVEL, c2_sh, key_sh, ct_sh, ws_sh)
        sh.allgather_ct(LEVEL, ct_sh)
        ok = torch.equal(ct_sh, want)
        for _ in range(3):
            sh.keyswitch(LEVEL, c2_sh, key_sh, ct_sh, ws_sh)
        barrier()
        n_sh = max(10, min(args.steps, 50))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for _ in range(n_sh):
            sh.keyswitch(LEVEL, c2_sh, key_sh, ct_sh, ws_sh)
        s1.record(stream)
        barrier()
        t = torch.tensor([s0.elapsed_time(s1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us_one = 1e3 * float(t.item()) / n_sh
        # throughput: batches of LB ciphertexts, NB batches in flight on two lanes (own stream and communicator each)
        n_lanes = max(1, int(os.environ.get("B2_SHARD_LANES", "4")))
        LB = max(1, min(int(os.environ.get("B2_SHARD_BATCH", "32")), 32))
        NB = max(4, 2 * n_lanes)
        lanes = sh.make_lanes(n_lanes)
        # four or more workspaces: the staggered pipeline keeps three batches in flight. Peer-writable ones where the ranks can
        # map one another's memory (the exchanges are then copy-engine pushes, B2_SHARD_EXCHANGE=nccl keeps the all-gathers)
        n_ws = max(4, n_lanes)
        # (measured on B200s: pushes win at 2 and 4 ranks, 10380 vs 9680 and 19250 vs 16810 KeySwitch/s; at 8 ranks seven DMA
        # copies per exchange reach 420 GB/s where the all-gather reaches 590, 18520 vs 21900: B2_SHARD_EXCHANGE=peer|nccl overrides)
        xmode = os.environ.get("B2_SHARD_EXCHANGE", "peer" if world <= 4 else "nccl")
        wsb = None if xmode == "nccl" else sh.peer_workspaces(LEVEL, LB, n_ws)
        exchange_kind = "peer copies (DMA) + one-word all-reduce" if wsb is not None else "NCCL all-gather"
        if wsb is None:
            wsb = [sh.batch_workspace(LEVEL, LB)[0] for _ in range(n_ws)]
        batches = [(torch.stack([sh_ct3[(i * LB + b) % n_sh_ct][2] for b in range(LB)]),
                    torch.stack([sh_ct3[(i * LB + b) % n_sh_ct][:2] for b in range(LB)])) for i in range(NB)]
        want_b = batches[0][1][0].clone()
        check(LIB.b2_keyswitch(ctx._h, LEVEL, batches[0][0][0].data_ptr(), key_sh_tab.ctypes.data, BETA, want_b.data_ptr(), ws1.data_ptr(), ws1_bytes,
                               stream.cuda_stream))
        sh.pipeline(LEVEL, batches, key_sh, lanes, wsb)
        got_b = batches[0][1][0].clone()
        sh.allgather_ct(LEVEL, got_b)
        ok = ok and torch.equal(got_b, want_b)
        flag = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) != 1:
            raise RuntimeError("limb-sharded key switch differs from the one-GPU key switch")
        for _ in range(2):
            sh.pipeline(LEVEL, batches, key_sh, lanes, wsb)
        barrier()
        n_pb = max(5, min(args.steps, 20))
        s0.record(stream)
        for _ in range(n_pb):
            sh.pipeline(LEVEL, batches, key_sh, lanes, wsb)
        s1.record(stream)
        barrier()
        t = torch.tensor([s0.elapsed_time(s1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us_b = 1e3 * float(t.item()) / (n_pb * NB * LB)
        # the same batches with the exchanges alone (no kernels): what the collectives cost by themselves
        def exchanges():
            st, grp = lanes[0]
            st.wait_stream(stream)
            with torch.cuda.stream(st):
                for i in range(NB):
                    sh.exchange(LEVEL, LB, wsb[i % len(wsb)], 0, grp)
                    sh.exchange(LEVEL, LB, wsb[i % len(wsb)], 1, grp)
            stream.wait_stream(st)
        exchanges()
        barrier()
        s0.record(stream)
        for _ in range(n_pb):
            exchanges()
        s1.record(stream)
        barrier()
        t = torch.tensor([s0.elapsed_time(s1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us_x = 1e3 * float(t.item()) / (n_pb * NB * LB)
        # and the kernels alone (the three phases without the exchanges between them: results are not used): with both in
        # hand one reads how much of the shorter one the lanes hide
        def kernels_only():
            for i in range(NB):
                st, _ = lanes[i % n_lanes]
                st.wait_stream(stream)
                with torch.cuda.stream(st):
                    c2_b, ct_b = batches[i]
                    w = wsb[i % len(wsb)]
                    for ph_i in (0, 1, 2):
                        sh.phase_batch(LEVEL, ph_i, LB, c2_b, key_sh_tab, ct_b, w, w.numel() * 8)
            for st, _ in lanes:
                stream.wait_stream(st)
        kernels_only()
        barrier()
        s0.record(stream)
        for _ in range(n_pb):
            kernels_only()
        s1.record(stream)
        barrier()
        t = torch.tensor([s0.elapsed_time(s1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us_k = 1e3 * float(t.item()) / (n_pb * NB * LB)
        rx = int((LEVEL + 2 * SPECIAL) * LIMB_BYTES * (1 - 1 / world))
        limb_sharded = {"verified": True, "ranks": world, "keyswitch_per_s": 1e6 / us_b, "us_per_keyswitch": us_b,
                        "batch_per_lane": LB, "batches_in_flight": NB, "lanes": n_lanes, "exchange": exchange_kind,
                        "one_ciphertext_latency_us": us_one,
                        "nvlink_bytes_received_per_gpu_per_keyswitch": rx,
                        "nvlink_gbs_per_gpu": rx / (us_b * 1e-6) / 1e9, "nvlink_frac_of_900": rx / (us_b * 1e-6) / 1e9 / 900.0,
                        "kernels_alone_us_per_keyswitch": us_k, "collectives_alone_us_per_keyswitch": us_x, "collectives_share": us_x / us_b,
                        "note": "every ciphertext's limbs are spread over all ranks (the weak-scaling value above is data parallel)"}
        barrier()
        for w in wsb:
            if hasattr(w, "close"):
                w.close()

    # ---- per-kernel timing (live, CUDA events on the launching stream) and roofline -------------
    roofline, roofline_issue, kernels = None, None, None
    if rank == 0:
        # one stream here: a kernel's event pair must time that kernel alone, not a mix of streams
        check(LIB.b2_profile_start(ctx._h))
        prof_steps = 2
        ws0, ws0_bytes = wss[0]
        PB = min(B, 8)
        if batched:
            # the timed region's own call, on one stream: one key's ciphertexts per launch
            g = dev_groups[0]
            PB = int(g.shape[0])
            for _ in range(prof_steps):
                check(LIB.b2_keyswitch_batch(ctx._h, LEVEL, PB, g[0, 2].data_ptr(), 3 * LEVEL, key_tabs[0].ctypes.data, BETA, g.data_ptr(),
                                             3 * LEVEL, ks_wsb[0].data_ptr(), ks_wsb[0].numel() * 8, stream.cuda_stream))
        for _ in range(0 if batched else prof_steps):
            for b in range(PB):
                t = dev_ct3[b]
                check(LIB.b2_keyswitch(ctx._h, LEVEL, t[2].data_ptr(), key_tabs[b % K].ctypes.data, BETA, t.data_ptr(),
                                       ws0.data_ptr(), ws0_bytes, stream.cuda_stream))
        names = ctypes.create_string_buffer(4096)
        tot = (ctypes.c_float * 64)()
        cnt = (ctypes.c_uint32 * 64)()
        n_out = ctypes.c_size_t()
        check(LIB.b2_profile_stop(ctx._h, names, 4096, tot, cnt, 64, ctypes.byref(n_out)))
        nm = names.value.decode().strip(";").split(";")
        alg = kernel_alg_bytes_per_keyswitch()
        n_ks = prof_steps * PB
        total_ms = sum(tot[i] for i in range(n_out.value))
        # what ncu saw for the same kernels (committed summary of one capture; cold caches, one stream)
        ncu = {}
        tp = os.path.join(ROOT, "profiles", "ncu_traffic.json")
        if os.path.exists(tp):
            ncu = json.load(open(tp))
        kernels = {}
        for i in range(n_out.value):
            per_ks_ms = tot[i] / n_ks
            gbs = alg.get(nm[i], 0) / (per_ks_ms * 1e-3) / 1e9 if per_ks_ms > 0 else 0.0
            rec = ncu.get(nm[i], {})
            kernels[nm[i]] = {"launches_per_keyswitch": cnt[i] / n_ks, "us_per_keyswitch": 1e3 * per_ks_ms,
                              "share": tot[i] / total_ms, "alg_bytes_per_keyswitch": alg.get(nm[i]), "alg_gbs": gbs,
                              "dram_bytes_per_keyswitch": rec.get("dram_bytes_per_keyswitch"),
                              "warp_instructions_per_keyswitch": rec.get("warp_instructions_per_keyswitch"),
                              "bound": rec.get("bound")}
        peak, peak_kind = peaks()
        ks_us = 1e3 * ms / (B * args.steps)
        dram = [k.get("dram_bytes_per_keyswitch") for k in kernels.values()]
        roofline = {"what": "one hybrid key switch (all its kernels)", "bound": "hbm", "alg_bytes": KS_BYTES, "us_per_keyswitch": ks_us,
                    "achieved": KS_BYTES / (ks_us * 1e-6) / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": KS_BYTES / (ks_us * 1e-6) / 1e9 / peak, "peak_kind": peak_kind,
                    "traffic": sum(dram) if dram and all(d is not None for d in dram) else None,
                    "traffic_note": "sum over the key switch's kernels of dram read + write bytes, each kernel captured with cold caches (upper bound)"}
        instr = [k.get("warp_instructions_per_keyswitch") for k in kernels.values()]
        if instr and all(v is not None for v in instr) and clocks and clocks.get("sm_mhz"):
            slots = 148 * 4 * clocks["sm_mhz"] * 1e6
            roofline_issue = {"bound": "issue", "warp_instructions_per_keyswitch": sum(instr), "issue_slots_per_s": slots,
                              "achieved": sum(instr) / (ks_us * 1e-6), "frac": sum(instr) / (ks_us * 1e-6) / slots, "unit": "warp instructions/s",
                              "floor_us_per_keyswitch": 1e6 * sum(instr) / slots}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_sample()

    hmult = None
    if not args.no_extras:
        hmult = hmult_section(torch, dist, ctx, LIB, check, _native, dev_ct3, key_tabs, world, S, batched=batched)
    reference_gpu = None
    ntt, bootstrap, compositions, bsgs = None, None, None, None
    if rank == 0 and world == 1 and not args.no_extras:
        reference_gpu = reference_gpu_section()
        ntt = ntt_section(ph, ctx, torch, LIB, check, N, len(primes))
        compositions = compositions_section(ph, ctx, torch, np, synth, primes, keys, N, LEVEL)
        del dev_ct3, dev_groups, keys, stage
        if batched:
            del ks_wsb
        torch.cuda.empty_cache()
        bsgs = bsgs_section(ph, torch, np, synth)
        torch.cuda.empty_cache()
        bootstrap = bootstrap_section(ph, torch, np)

    if rank == 0:
        line = {
            "metric": "KeySwitch/s", "value": value, "unit": "KeySwitch/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": config_dict(args, world),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "KeySwitch/s", "h2d_bytes_per_step": B * 3 * LEVEL * LIMB_BYTES,
                    "d2h_bytes_per_step": B * 2 * LEVEL * LIMB_BYTES, "api": "pyPhantom.relinearize", "steps": e2e_steps, "streams": len(streams), "pcie": pcie, "numa": numa},
            "gpu_launches": launches,
            "device_status": ctx.device_status(),
            "roofline": roofline,
            "roofline_issue": roofline_issue,
            "kernels": kernels,
            "cpu_baseline": cpu,
            "reference_gpu": reference_gpu,
            "hmult_batch64": hmult,
            "ntt": ntt,
            "compositions": compositions,
            "bsgs_matvec": bsgs,
            "bootstrap": bootstrap,
            "limb_sharded": limb_sharded,
        }
        print(json.dumps(line), file=out_stream, flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
