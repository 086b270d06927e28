#!/usr/bin/env python
"""Benchmark of the CKKS runtime on B200.

Default workload (the configuration the headline metric is quoted on):
encrypted ResNet-20 inference, the program the ANT-ACE
compiler emitted for resnet20_cifar10 (N = 2^16, 34 RNS limbs of 51/46 bits,
dnum = 3, 19 bootstraps), linked unchanged against this runtime
(ace_compiler_b200/programs/build_programs.sh builds it where the reference
checkout is present).  One step = one image: a seeded uniform[-1,1] 3x32x32
tensor is encoded and encrypted, Main_graph runs, the logits are decrypted.
Weights are a synthetic data file of seeded N(0, sigma) values in the
compiler's format; the encoded weight plaintexts stay resident in HBM (the
runtime's plaintext cache), so a step does not re-encode them.  Main_graph
issues the same kernels on the same device blocks for every image, so the
second warm-up image is captured as one CUDA graph and the timed images launch
that graph on their own freshly encrypted input (Fhert_replay_mode;
--no-replay launches every kernel from the host as a plain driver would; the
line reports both).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--workload resnet20|primitives|bootstrap|resnet32_cifar100]
                  [--levels 4,12,24,36]

`value` is images/s over the device time of Main_graph with the encrypted
input resident in HBM; `e2e` is images/s over the whole step from the host
tensor to the host logits.  `--workload primitives` runs the configs[1] sweep
at L = 36 instead (16 rotations + 16 HMult+relinearise+rescale per step), which
is also what runs when the compiled program is not available.
`--workload bootstrap` times one full bootstrap of a 32768-slot ciphertext at
N = 2^16, L = 36; `--workload resnet32_cifar100` runs that compiled program the
way the default workload runs ResNet-20.  `--impl reference` times the
unmodified reference CPU runtime (oracle/_ref) on the host cores: samples of the
workload's operation classes (rotations and products at three levels, weight
encodes, per-limb vector calls, rescales, one bootstrap), extrapolated to whole
images with the program's operation counts; also on the reference's OpenMP build.
"""
import argparse
import ctypes as C
import json
import multiprocessing as mp
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DEGREE, LEVELS, DNUM, Q0_BITS, SF_BITS = 65536, 36, 3, 60, 56
ROTATIONS = tuple(1 << i for i in range(16))
OPS_PER_STEP = 2 * len(ROTATIONS)
LIMB_BYTES = DEGREE * 8
METRIC = "CKKS primitive ops/s (Rotate and HMult+relin+rescale, N=2^16, L=36, dnum=3)"
WORKLOAD = ("configs[1] primitive sweep at L=36: per step 16 Rotate(k=2^0..2^15) + "
            "16 HMult+relinearise+rescale on seeded uniform ciphertexts")

# the compiled ResNet-20 program and the counts the CPU extrapolation uses
# (rotations and relinearised products executed per image, from the loop nests
# of the generated file)
PROGRAM = "resnet20_cifar10"
PROGRAM_DIR = os.path.join(ROOT, "ace_compiler_b200", "programs", "_ref")
PROGRAM_SO = os.path.join(PROGRAM_DIR, PROGRAM + ".so")
# other compiled programs that run through the same path: name -> (file, weight
# entries to provide, logits, metric, workload text)
OTHER_PROGRAMS = {
    "resnet32_cifar100": ("resnet32_cifar100", 16000, 100,
                          "ResNet-32 (CIFAR-100 head) CKKS inference images/s",
                          "compiler-emitted resnet32_cifar100 program, N=2^16, 34 limbs (q0 51 "
                          "bits, scale 46 bits), dnum=3, 31 bootstraps; one seeded uniform[-1,1] "
                          "3x32x32 image per step; synthetic seeded weights"),
}
R20_LEVELS, R20_Q0, R20_SF, R20_K = 34, 51, 46, 10
R20_ROTATIONS, R20_RELINS, R20_BOOTSTRAPS, R20_WEIGHTS = 1814, 513, 19, 6044
R20_METRIC = "ResNet-20 CKKS inference images/s (s/image = 1/value at 1 GPU)"
R20_WORKLOAD = ("configs[0]: compiler-emitted resnet20_cifar10 program, N=2^16, 34 limbs "
                "(q0 51 bits, scale 46 bits), dnum=3, 19 bootstraps; one seeded uniform[-1,1] "
                "3x32x32 image per step; synthetic seeded weights")


class c_stdout_to_stderr:
    """The runtime libraries print their parameter line with C stdio; the one
    JSON line must stay alone on stdout."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def __exit__(self, *exc):
        C.CDLL(None).fflush(None)
        os.dup2(self.saved, 1)
        os.close(self.saved)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while running: one NVML session (the
    library nvidia-smi reads from), nvidia-smi itself as the fallback."""

    def __init__(self, index):
        self.index = index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period = float(os.environ.get("BENCH_CLOCK_PERIOD_S", "0.2"))
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def _run_nvml(self):
        # one NVML session for the whole run: starting nvidia-smi again and again
        # attaches to the driver every time and disturbs the launching thread
        import pynvml
        pynvml.nvmlInit()
        try:
            try:
                import torch
                prop = torch.cuda.get_device_properties(self.index)
                bus = "%08x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
                h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            bits = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                    0x4: "sw_power_cap"}
            while not self._stop.is_set():
                self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                try:
                    mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in bits.items():
                    if mask & bit:
                        self.reasons.add(name)
                self._stop.wait(self.period)
        finally:
            pynvml.nvmlShutdown()

    def _run_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                f = [x.strip() for x in out.stdout.strip().split(",")]
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
                for n, v in zip(names, f[2:]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(1.0)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------

def synthetic_keys(gpu, rng):
    """Rotation / relinearisation keys of seeded uniform residues (the cost of a
    key switch does not depend on the key values)."""
    total = gpu.L + gpu.K
    for is_rot, idx in [(False, 0)] + [(True, r) for r in ROTATIONS]:
        for part in range(gpu.dnum):
            for which in (0, 1):
                data = np.stack([rng.integers(0, p, gpu.N, dtype=np.int64) for p in gpu.primes])
                assert data.shape[0] == total
                gpu.import_switch_key(is_rot, idx, part, which, data)


def run_primitives(args):
    import torch

    import ace_compiler_b200 as rt

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        with c_stdout_to_stderr():  # NCCL prints its version line when the communicator is made
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()

    with c_stdout_to_stderr():
        gpu = rt.Runtime(DEGREE, LEVELS, Q0_BITS, SF_BITS, DNUM, rot_idxs=ROTATIONS)
    lib = gpu.lib
    rng = np.random.default_rng(1000 + rank)
    synthetic_keys(gpu, rng)
    stream = torch.cuda.ExternalStream(lib.Fhert_stream(), device=torch.device("cuda", local))

    def host_ct():
        t = torch.empty((2, LEVELS, DEGREE), dtype=torch.int64).pin_memory()
        a = t.numpy()
        for i, p in enumerate(gpu.primes[:LEVELS]):
            a[0, i] = rng.integers(0, p, DEGREE, dtype=np.int64)
            a[1, i] = rng.integers(0, p, DEGREE, dtype=np.int64)
        return t, a

    keep_a, ha = host_ct()
    keep_b, hb = host_ct()
    keep_o = torch.empty((2, LEVELS, DEGREE), dtype=torch.int64).pin_memory()
    ho = keep_o.numpy()
    ct_a, ct_b = gpu.new_ciph(ha[0], ha[1]), gpu.new_ciph(hb[0], hb[1])
    out, prod, res = rt.CIPHERTEXT(), rt.CIPHERTEXT(), rt.CIPHERTEXT()

    def step_resident():
        for r in ROTATIONS:
            lib.Rotate_ciph(C.byref(out), C.byref(ct_a), r)
        for _ in ROTATIONS:
            lib.Mul_ciph(C.byref(prod), C.byref(ct_a), C.byref(ct_b))
            lib.Rescale_ciph(C.byref(res), C.byref(prod))

    def up(ct, h):
        lib.Fhert_upload(C.pointer(ct._c0_poly), 0, LEVELS, h[0].ctypes.data_as(C.c_void_p))
        lib.Fhert_upload(C.pointer(ct._c1_poly), 0, LEVELS, h[1].ctypes.data_as(C.c_void_p))

    def down(ct, levels):
        lib.Fhert_download(C.pointer(ct._c0_poly), 0, levels, ho[0].ctypes.data_as(C.c_void_p))
        lib.Fhert_download(C.pointer(ct._c1_poly), 0, levels, ho[1].ctypes.data_as(C.c_void_p))

    def step_e2e():
        for r in ROTATIONS:
            up(ct_a, ha)
            lib.Rotate_ciph(C.byref(out), C.byref(ct_a), r)
            down(out, LEVELS)
        for _ in ROTATIONS:
            up(ct_a, ha)
            up(ct_b, hb)
            lib.Mul_ciph(C.byref(prod), C.byref(ct_a), C.byref(ct_b))
            lib.Rescale_ciph(C.byref(res), C.byref(prod))
            down(res, LEVELS - 1)

    h2d = len(ROTATIONS) * 2 * LEVELS * LIMB_BYTES + len(ROTATIONS) * 4 * LEVELS * LIMB_BYTES
    d2h = len(ROTATIONS) * 2 * LEVELS * LIMB_BYTES + len(ROTATIONS) * 2 * (LEVELS - 1) * LIMB_BYTES

    def barrier():
        lib.Fhert_sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        from ace_compiler_b200 import parallel
        return parallel.slowest_rank([e0.elapsed_time(e1)], device="cuda")[0]

    for _ in range(args.warmup):
        step_resident()
    launches0 = lib.Fhert_kernel_launches()
    with ClockSampler(local) as clocks:
        ms = timed(step_resident, args.steps)
    launches = lib.Fhert_kernel_launches() - launches0
    value = OPS_PER_STEP * args.steps * world / (ms * 1e-3)

    step_e2e()
    ms_e2e = timed(step_e2e, max(1, args.steps // 2))
    e2e_value = OPS_PER_STEP * max(1, args.steps // 2) * world / (ms_e2e * 1e-3)

    # separate figures per op kind, and the per-kernel breakdown of one step
    def rot_only():
        for r in ROTATIONS:
            lib.Rotate_ciph(C.byref(out), C.byref(ct_a), r)

    def mul_only():
        for _ in ROTATIONS:
            lib.Mul_ciph(C.byref(prod), C.byref(ct_a), C.byref(ct_b))
            lib.Rescale_ciph(C.byref(res), C.byref(prod))

    ms_rot = timed(rot_only, 2) / 2
    ms_mul = timed(mul_only, 2) / 2

    # the same two primitives and the transforms at lower ciphertext levels of
    # the same 36-limb context (digits stay 12 limbs wide: beta = ceil(l / 12))
    per_level = {}
    peak_gbs = peaks()[0]
    for lv in args.levels:
        if lv > LEVELS:
            continue
        ca, cb = gpu.new_ciph(ha[0][:lv], ha[1][:lv]), gpu.new_ciph(hb[0][:lv], hb[1][:lv])
        pa = gpu.new_poly(lv, data=ha[0][:lv])

        def rot_lv():
            for r in ROTATIONS:
                lib.Rotate_ciph(C.byref(out), C.byref(ca), r)

        def mul_lv():
            for _ in ROTATIONS:
                lib.Mul_ciph(C.byref(prod), C.byref(ca), C.byref(cb))
                lib.Rescale_ciph(C.byref(res), C.byref(prod))

        def ntt_lv():
            for _ in ROTATIONS:
                lib.Conv_ntt2poly_inplace(pa)
                lib.Conv_poly2ntt_inplace(pa)

        rot_lv(); mul_lv(); ntt_lv()
        t_rot, t_mul, t_ntt = timed(rot_lv, 2) / 2, timed(mul_lv, 2) / 2, timed(ntt_lv, 2) / 2
        beta = -(-lv // gpu.alpha)
        ks_b = (3 * lv + 2 * beta * (lv + gpu.K)) * LIMB_BYTES
        k = len(ROTATIONS)
        rot_gbs = (ks_b + 7 * lv * LIMB_BYTES) * k / (t_rot * 1e-3) / 1e9
        mul_gbs = (7 * lv * LIMB_BYTES + ks_b + 6 * lv * LIMB_BYTES
                   + 2 * (2 * lv - 1) * LIMB_BYTES) * k / (t_mul * 1e-3) / 1e9
        ntt_gbs = 2 * 2 * lv * LIMB_BYTES * k / (t_ntt * 1e-3) / 1e9
        per_level[f"L={lv}"] = {
            "rotate_ops_s": round(k / (t_rot * 1e-3), 1), "rotate_GBs": round(rot_gbs, 1),
            "rotate_frac": round(rot_gbs / peak_gbs, 4),
            "hmult_relin_rescale_ops_s": round(k / (t_mul * 1e-3), 1),
            "hmult_GBs": round(mul_gbs, 1), "hmult_frac": round(mul_gbs / peak_gbs, 4),
            "ntt_plus_intt_limbs_s": round(2 * lv * k / (t_ntt * 1e-3), 1),
            "ntt_GBs": round(ntt_gbs, 1), "ntt_frac": round(ntt_gbs / peak_gbs, 4)}
        gpu.free_ciph(ca)
        gpu.free_ciph(cb)
        gpu.free(pa)
    with gpu.profile() as prof:
        step_resident()
    kernels = prof.kernels

    line = None
    if rank == 0:
        peak, peak_kind = peaks()
        # dominant kernel by device time; NTT passes are reported as the pair that
        # makes one transform (strided + contiguous), 2 limb passes each
        groups = {
            "ntt (strided+contig passes)": ["ntt_strided", "ntt_contig"],
            "intt (contig+strided passes)": ["intt_contig", "intt_strided"],
        }
        rows = {}
        for name, (cnt, limbs, t) in kernels.items():
            rows[name] = {"launches": cnt, "limbs": limbs, "ms": t}
        total_ms = sum(v["ms"] for v in rows.values())
        fwd = [rows[k] for k in groups["ntt (strided+contig passes)"] if k in rows]
        fwd_ms = sum(r["ms"] for r in fwd)
        fwd_limbs = fwd[0]["limbs"] if fwd else 0
        fwd_launch_pairs = fwd[0]["launches"] if fwd else 1
        # algorithmic bytes of one forward NTT = 2 * 512 KiB per limb
        alg_bytes = 2.0 * LIMB_BYTES * fwd_limbs
        achieved = alg_bytes / (fwd_ms * 1e-3) / 1e9 if fwd_ms else 0.0
        roofline = {
            "bound": "hbm", "kernel": "ntt (strided+contig passes)",
            "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4), "peak_kind": peak_kind,
            "traffic": None,
            "alg_bytes_per_launch_pair": alg_bytes / max(1, fwd_launch_pairs),
            "avg_ms_per_launch_pair": fwd_ms / max(1, fwd_launch_pairs),
            "share_of_step": round(fwd_ms / total_ms, 4) if total_ms else None,
        }
        # hybrid key switch: (3l + 2*beta*(l+K)) limbs of algorithmic traffic
        ks_bytes = (3 * LEVELS + 2 * DNUM * (LEVELS + gpu.K)) * LIMB_BYTES
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "ops/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "ring_degree": DEGREE, "levels": LEVELS,
                       "dnum": DNUM, "special_primes": gpu.K, "ops_per_step": OPS_PER_STEP,
                       "l2": "inputs_larger_than_l2 (17 keys x 144 MiB cycled every step)",
                       "parallelism": f"replicas x{world}, no communication"},
            "e2e": {"value": round(e2e_value, 2), "unit": "ops/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": roofline,
            "breakdown": {
                "rotate_ops_s": round(len(ROTATIONS) / (ms_rot * 1e-3), 2),
                "hmult_relin_rescale_ops_s": round(len(ROTATIONS) / (ms_mul * 1e-3), 2),
                "rotate_keyswitch_alg_GBs": round(
                    ks_bytes * len(ROTATIONS) / (ms_rot * 1e-3) / 1e9, 1),
                "per_level": per_level,
                "kernels_one_step": {k: {"launches": v["launches"], "limbs": v["limbs"],
                                         "ms": round(v["ms"], 3)} for k, v in rows.items()},
            },
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample("primitives")
    for c in (ct_a, ct_b, out, prod, res):
        gpu.free_ciph(c)
    gpu.close()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


# ---------------------------------------------------------------------------
# our arm, default workload: the compiled ResNet-20 program
# ---------------------------------------------------------------------------

def key_switch_roofline(lib, rt, stream, levels, rot_idx, peak):
    """Device time of the library's whole hybrid key switch (Rotate_ciph: ModUp of
    all digits, key inner product, ModDown, automorphism) at the given ciphertext
    levels of the current context, against its algorithmic bytes
    (3l + 2*beta*(l+K)) * W, beta = ceil(l / alpha)."""
    import torch
    n, K, alpha = lib.Degree(), lib.Get_p_cnt(), lib.Get_part_size()
    out = {}
    for level in levels:
        ct, res = rt.CIPHERTEXT(), rt.CIPHERTEXT()
        for poly in (ct._c0_poly, ct._c1_poly):
            lib.Alloc_poly_data(C.byref(poly), n, level, 0)  # zero residues: time does not depend on values
            poly._is_ntt = True
        ct._slots, ct._scaling_factor, ct._sf_degree = n // 2, lib.Get_default_sc(), 1
        for _ in range(3):
            lib.Rotate_ciph(C.byref(res), C.byref(ct), rot_idx)
        lib.Fhert_sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 16
        e0.record(stream)
        for _ in range(reps):
            lib.Rotate_ciph(C.byref(res), C.byref(ct), rot_idx)
        e1.record(stream)
        lib.Fhert_sync()
        ms = e0.elapsed_time(e1) / reps
        beta = -(-level // alpha)
        alg = (3 * level + 2 * beta * (level + K)) * n * 8
        gbs = alg / (ms * 1e-3) / 1e9
        out[f"level {level}"] = {"ms": round(ms, 4), "alg_MB": round(alg / 1e6, 1),
                                 "GB/s": round(gbs, 1), "frac": round(gbs / peak, 4)}
        lib.Free_ciph_poly(C.byref(ct), 1)
        lib.Free_ciph_poly(C.byref(res), 1)
    return out


def run_resnet20(args):
    import torch

    if args.workload in OTHER_PROGRAMS:
        program, weight_entries, n_logits, metric, workload_text = OTHER_PROGRAMS[args.workload]
    else:
        program, weight_entries, n_logits = PROGRAM, R20_WEIGHTS + 56, 10
        metric, workload_text = R20_METRIC, R20_WORKLOAD
    program_so = os.path.join(PROGRAM_DIR, program + ".so")

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        with c_stdout_to_stderr():  # NCCL prints its version line when the communicator is made
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()

    from ace_compiler_b200.msgfile import write_synthetic_msg_file
    weights = f"/tmp/fhert_{program}_{os.getpid()}.msg"
    write_synthetic_msg_file(weights, weight_entries, sigma=0.02, seed=7)
    os.environ["FHERT_DATA_FILE"] = weights
    os.environ["FHERT_PT_CACHE_MB"] = str(args.cache_mb)
    os.environ["FHERT_RT_STAT"] = "0"
    # the program's hooks (Get_context_params, Main_graph ...) must come first
    # in the global symbol scope, before the library's weak defaults
    C.CDLL(program_so, mode=C.RTLD_GLOBAL)
    import ace_compiler_b200 as rt
    lib = rt.load()
    libc = C.CDLL(None)
    libc.free.argtypes = [C.c_void_p]

    t0 = time.perf_counter()
    with c_stdout_to_stderr():
        lib.Prepare_context()
    lib.Fhert_sync()
    setup_s = time.perf_counter() - t0
    stream = torch.cuda.ExternalStream(lib.Fhert_stream(), device=torch.device("cuda", local))
    rng = np.random.default_rng(2000 + rank)

    pin_words = (C.c_uint32 * 16)(*[(7 * 2654435761 + 40503 * k) & 0xffffffff for k in range(16)])
    pin_vals = np.ascontiguousarray(np.random.default_rng(99).uniform(-1.0, 1.0, 3 * 32 * 32))

    def one_image(events=None, pinned=False):
        if pinned:  # the same input under the same encryption randomness: results must repeat bit for bit
            lib.Fhert_seed(pin_words, 0, 1700000000000007 + rank)
            vals = pin_vals
        else:
            vals = np.ascontiguousarray(rng.uniform(-1.0, 1.0, 3 * 32 * 32))
        t = lib.Alloc_tensor(1, 3, 32, 32, vals.ctypes.data_as(C.POINTER(C.c_double)))
        lib.Prepare_input(t, b"input")
        lib.Free_tensor(t)
        if events is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        lib.Run_main_graph()
        if events is not None:
            e1.record(stream)
            events.append((e0, e1))
        out = lib.Handle_output(b"output")
        logits = [out[i] for i in range(n_logits)]
        libc.free(C.cast(out, C.c_void_p))
        return logits

    def barrier():
        lib.Fhert_sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def transfer():
        a, b = C.c_uint64(), C.c_uint64()
        lib.Fhert_transfer_bytes(C.byref(a), C.byref(b))
        return a.value, b.value

    # Replay: the first image runs as usual (it fills the plaintext cache), the
    # second one captures the launches of Main_graph into one CUDA graph, the
    # following ones launch that graph on their own encrypted input
    replay = not args.no_replay
    if replay:
        lib.Fhert_replay_mode(1)
    # the first (directly launched) and the last warm-up image (a replay) are the same
    # pinned image: the replayed graph has to reproduce the direct launches bit for bit
    warm = max(3 if replay else 1, args.warmup)
    first_logits = one_image(pinned=True)
    for _ in range(warm - 2):
        one_image()
    replay_checked = None
    if warm >= 2:
        again = one_image(pinned=True)
        if replay and lib.Fhert_replay_state(None, 0, None) == 2:
            replay_checked = again == first_logits
            if not replay_checked:  # never report numbers of a graph that computes something else
                print("replayed run differs from the direct run: replay switched off", file=sys.stderr)
                lib.Fhert_replay_mode(0)
                replay = False
    barrier()
    launches0, (h2d0, d2h0) = lib.Fhert_kernel_launches(), transfer()
    events = []
    E0, E1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cpu0 = time.process_time()
    with ClockSampler(local) as clocks:
        E0.record(stream)
        for _ in range(args.steps):
            logits = one_image(events)
        E1.record(stream)
        barrier()
    host_cpu_s = (time.process_time() - cpu0) / args.steps
    ms_total = E0.elapsed_time(E1)
    image_ms = [round(a.elapsed_time(b), 1) for a, b in events]
    ms_graph = sum(a.elapsed_time(b) for a, b in events)
    launches = lib.Fhert_kernel_launches() - launches0
    h2d1, d2h1 = transfer()
    from ace_compiler_b200 import parallel
    ms_total, ms_graph = parallel.slowest_rank([ms_total, ms_graph], device="cuda")
    value = parallel.job_throughput(args.steps, world, ms_graph)
    e2e_value = parallel.job_throughput(args.steps, world, ms_total)

    # how the timed images were launched, and the same program launched kernel by
    # kernel from the host (outside the timed region)
    why, served = C.create_string_buffer(256), C.c_uint64()
    replay_state = lib.Fhert_replay_state(why, len(why), C.byref(served))
    graph_shape = None
    if replay_state == 2:
        g5 = [C.c_uint64() for _ in range(5)]
        lib.Fhert_replay_graph(*[C.byref(x) for x in g5])
        graph_shape = dict(zip(("launches", "described_launch_groups", "dependences",
                                "undescribed_barriers", "longest_chain"), (x.value for x in g5)))
        main_graph_text = (f"captured once as one CUDA graph of {launches // args.steps} kernel launches "
                           f"(second warm-up image), replayed for every timed image "
                           f"({served.value} replays so far); the input ciphertext is new every image")
    elif replay:
        main_graph_text = "launched kernel by kernel from the host; replay went off: " + why.value.decode()
    elif replay_checked is False:
        main_graph_text = ("launched kernel by kernel from the host: the replayed run differed from the "
                           "direct run of the same pinned image, replay was switched off")
    else:
        main_graph_text = "launched kernel by kernel from the host (--no-replay)"
    lib.Fhert_replay_mode(0)
    direct = []
    cpu1 = time.process_time()
    for _ in range(2):
        one_image(direct)
    barrier()
    direct_cpu_s = (time.process_time() - cpu1) / 2
    image_ms_direct = [round(a.elapsed_time(b), 1) for a, b in direct]

    # the same program with every weight plaintext encoded afresh on the device
    # for every image, as the CPU runtime does (outside the timed region)
    lib.Fhert_pt_cache_bypass(1)
    uncached = []
    one_image()
    for _ in range(2):
        one_image(uncached)
    barrier()
    ms_uncached = sum(a.elapsed_time(b) for a, b in uncached) / len(uncached)
    # and the same replayed: the capture snapshots the weight messages in pinned
    # memory, every replay copies and encodes all of them again
    ms_uncached_replayed, uncached_state = None, ""
    if replay:
        lib.Fhert_replay_mode(1)
        one_image()   # launched directly
        one_image()   # captured
        replayed_uncached = []
        for _ in range(2):
            one_image(replayed_uncached)
        barrier()
        if lib.Fhert_replay_state(why, len(why), C.byref(served)) == 2:
            ms_uncached_replayed = sum(a.elapsed_time(b) for a, b in replayed_uncached) / 2
        else:
            uncached_state = why.value.decode()
        lib.Fhert_replay_mode(0)
    lib.Fhert_pt_cache_bypass(0)

    # per-kernel device times of one more image (outside the timed region)
    buf = C.create_string_buffer(1 << 16)
    lib.Fhert_profile_begin()
    one_image()
    used = lib.Fhert_profile_end(buf, len(buf))
    rows = {}
    for ln in buf.raw[:used].decode().splitlines():
        name, cnt, limbs, ms = ln.split()
        rows[name] = {"launches": int(cnt), "limbs": int(limbs), "ms": float(ms)}
    # BENCH_PROFILE_IMAGES=k: k more profiled images, kernel-time sum against the
    # image's own device time, to tell a slow GPU from a starved one (stderr)
    for k in range(int(os.environ.get("BENCH_PROFILE_IMAGES", "0"))):
        ev = []
        lib.Fhert_profile_begin()
        one_image(ev)
        n_used = lib.Fhert_profile_end(buf, len(buf))
        barrier()
        ksum = sum(float(ln.split()[3]) for ln in buf.raw[:n_used].decode().splitlines())
        print(f"profiled image {k}: kernels {ksum:.1f} ms, image {ev[0][0].elapsed_time(ev[0][1]):.1f} ms",
              file=sys.stderr)
    stats = [C.c_size_t() for _ in range(4)]
    lib.Fhert_pt_cache_stats(*[C.byref(x) for x in stats])
    # the library's own key switch at levels the program works at (its rotation keys
    # are those of the program; -4096 is one of the replication rotations)
    ks = key_switch_roofline(lib, rt, stream, R20_SAMPLE_LEVELS + (R20_LEVELS,), -4096, peaks()[0])

    if rank == 0:
        peak, peak_kind = peaks()
        total_ms = sum(v["ms"] for v in rows.values()) or 1.0

        def group(names, bytes_per_limb):
            sel = [rows[k] for k in names if k in rows]
            if not sel:
                return None
            ms = sum(r["ms"] for r in sel)
            limbs, launches_ = sel[0]["limbs"], sel[0]["launches"]
            gbs = bytes_per_limb * limbs / (ms * 1e-3) / 1e9
            return {"ms": ms, "limbs": limbs, "launches": launches_, "gbs": gbs,
                    "bytes_per_limb": bytes_per_limb}
        # algorithmic bytes per limb: one transform reads and writes a limb
        # (2 x 512 KiB); a recorded element-wise limb operation reads two and
        # writes one (3 x 512 KiB)
        groups = {
            "ntt (strided+contig passes)": group(["ntt_strided", "ntt_contig"], 2 * LIMB_BYTES),
            "intt (contig+strided passes)": group(["intt_contig", "intt_strided"], 2 * LIMB_BYTES),
            "hw_batch (recorded per-limb add/mul/rotate)": group(["hw_batch"], 3 * LIMB_BYTES),
        }
        groups = {k: v for k, v in groups.items() if v}
        top = max(groups, key=lambda k: groups[k]["ms"])
        g = groups[top]
        roofline = {
            "bound": "hbm", "kernel": top, "achieved": round(g["gbs"], 1), "peak": peak,
            "unit": "GB/s", "frac": round(g["gbs"] / peak, 4), "peak_kind": peak_kind,
            "traffic": (round(NTT_DRAM_BYTES_PER_LIMB_CAPTURED * g["limbs"] / max(1, g["launches"]))
                        if top.startswith("ntt") else None),
            "traffic_source": "profiler capture of the transform pair at 48 limbs, scaled by "
                              "the limbs per launch of this run (not measured by this run)",
            "alg_bytes_per_launch": g["bytes_per_limb"] * g["limbs"] / max(1, g["launches"]),
            "avg_ms_per_launch": g["ms"] / max(1, g["launches"]),
            "share_of_image": round(g["ms"] / total_ms, 4),
            "others": {k: {"GB/s": round(v["gbs"], 1), "frac": round(v["gbs"] / peak, 4),
                           "share_of_image": round(v["ms"] / total_ms, 4)}
                       for k, v in groups.items() if k != top},
        }
        roofline["others"]["hybrid key switch (Rotate_ciph, timed alone after the images)"] = ks
        line = {
            "metric": metric, "value": round(value, 4), "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_graph / args.steps, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic",
            "config": {"workload": workload_text, "ring_degree": DEGREE, "levels": R20_LEVELS,
                       "dnum": DNUM, "special_primes": R20_K,
                       "s_per_image": round(ms_graph / args.steps / 1e3, 4),
                       "published_cpu_s_per_image": "1453.96 (one CPU thread, 60/56-bit primes; "
                                                    "not this program's 51/46-bit parameters, "
                                                    "so vs_baseline stays null)",
                       "setup_s": round(setup_s, 1),
                       "image_ms_this_rank": image_ms,
                       "main_graph": main_graph_text,
                       "replay_equals_direct_launch_on_a_pinned_image": replay_checked,
                       "captured_graph": graph_shape,
                       "image_ms_launched_from_the_host": image_ms_direct,
                       "host_cpu_s_per_image_launched_from_the_host": round(direct_cpu_s, 3),
                       "s_per_image_weights_encoded_every_image": round(
                           (ms_uncached_replayed or ms_uncached) / 1e3, 3),
                       "s_per_image_weights_encoded_every_image_launched_from_the_host": round(
                           ms_uncached / 1e3, 3),
                       **({"weights_encoded_every_image_not_replayed_because": uncached_state}
                          if uncached_state else {}),
                       "host_cpu_s_per_image": round(host_cpu_s, 3),
                       "weight_plaintexts_resident": {"entries": stats[0].value,
                                                      "GiB": round(stats[1].value / 2 ** 30, 2)},
                       "l2": "inputs_larger_than_l2 (keys and cached plaintexts, tens of GiB, "
                             "are streamed once per image)",
                       "parallelism": f"independent images, one per GPU x{world}, "
                                      "no communication"},
            "e2e": {"value": round(e2e_value, 4), "unit": "images/s",
                    "h2d_bytes_per_step": (h2d1 - h2d0) // args.steps,
                    "d2h_bytes_per_step": (d2h1 - d2h0) // args.steps},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": roofline,
            "breakdown": {
                "device_ms_one_image_by_kernel": {k: {"launches": v["launches"],
                                                       "limbs": v["limbs"],
                                                       "ms": round(v["ms"], 2)}
                                                  for k, v in sorted(rows.items(),
                                                                     key=lambda kv: -kv[1]["ms"])},
                "logits_last_image": [round(x, 6) for x in logits],
            },
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample("resnet20")
            if args.workload in OTHER_PROGRAMS:
                line["cpu_baseline"]["sample"] += (" (operation counts of the ResNet-20 program; "
                                                   "this program executes about 1.6x as many)")
    with c_stdout_to_stderr():
        lib.Finalize_context()
    try:
        os.remove(weights)
    except OSError:
        pass
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))



# ---------------------------------------------------------------------------
# our arm: one full bootstrap (CoeffToSlot / EvalMod / SlotToCoeff), 32768 slots
# ---------------------------------------------------------------------------

BTS_LEVELS = 36
BTS_METRIC = "CKKS bootstraps/s (N=2^16, 32768 slots, 60/56-bit primes, L=36, dnum=3)"
BTS_WORKLOAD = ("full bootstrapping of one ciphertext at N=2^16 with 32768 slots holding seeded "
                "uniform[-1,1] values: raise, CoeffToSlot, EvalMod, SlotToCoeff (hoisted rotations)")


def run_bootstrap(args):
    import torch

    import ace_compiler_b200 as rt

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        with c_stdout_to_stderr():  # NCCL prints its version line when the communicator is made
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
    os.environ["RTLIB_DISABLE_BOOTSTRAP_PRECOM"] = "0"
    t0 = time.perf_counter()
    with c_stdout_to_stderr():
        gpu = rt.Runtime(DEGREE, BTS_LEVELS, Q0_BITS, SF_BITS, DNUM, keygen=True,
                         seed=np.arange(16, dtype=np.uint32) + 11 + rank)
    lib = gpu.lib
    lib.Fhert_sync()
    setup_s = time.perf_counter() - t0
    stream = torch.cuda.ExternalStream(lib.Fhert_stream(), device=torch.device("cuda", local))
    rng = np.random.default_rng(3000 + rank)
    values = rng.uniform(-1, 1, DEGREE // 2) + 0j
    keep = torch.from_numpy(values.view(np.float64).copy()).pin_memory()
    host_vals = keep.numpy().view(np.complex128)
    level_in = 2

    def fresh():
        pt = gpu.encode(host_vals, 1, level_in)
        ct = gpu.encrypt(pt)
        lib.Free_plain_data(C.byref(pt))
        return ct

    def barrier():
        lib.Fhert_sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    ct = fresh()
    res = rt.CIPHERTEXT()
    for _ in range(max(1, args.warmup)):
        lib.Bootstrap(C.byref(res), C.byref(ct), 0)
    barrier()
    launches0 = lib.Fhert_kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record(stream)
        for _ in range(args.steps):
            lib.Bootstrap(C.byref(res), C.byref(ct), 0)
        e1.record(stream)
        barrier()
    launches = lib.Fhert_kernel_launches() - launches0
    from ace_compiler_b200 import parallel
    ms = parallel.slowest_rank([e0.elapsed_time(e1)], device="cuda")[0]
    value = parallel.job_throughput(args.steps, world, ms)
    # end to end: slot values on the host -> encode + encrypt -> bootstrap -> decrypt + decode
    barrier()
    t0 = time.perf_counter()
    reps = max(1, args.steps // 2)
    for _ in range(reps):
        c2 = fresh()
        lib.Bootstrap(C.byref(res), C.byref(c2), 0)
        back = gpu.decrypt_decode(res)
        gpu.free_ciph(c2)
    barrier()
    e2e_ms = parallel.slowest_rank([(time.perf_counter() - t0) * 1e3], device="cuda")[0]
    err = float(np.max(np.abs(back.real - values.real)))
    with gpu.profile() as prof:
        lib.Bootstrap(C.byref(res), C.byref(ct), 0)
    out_level = res._c0_poly._num_primes
    if rank == 0:
        peak, peak_kind = peaks()
        rows = {k: {"launches": v[0], "limbs": v[1], "ms": round(v[2], 3)}
                for k, v in sorted(prof.kernels.items(), key=lambda kv: -kv[1][2])}
        total = sum(v["ms"] for v in rows.values()) or 1.0

        def fam(names):
            sel = [rows[k] for k in names if k in rows]
            t = sum(r["ms"] for r in sel)
            return (2 * LIMB_BYTES * sel[0]["limbs"] / (t * 1e-3) / 1e9, t) if sel and t else (0.0, 0.0)
        ntt_gbs, ntt_ms = fam(["ntt_strided", "ntt_contig"])
        intt_gbs, intt_ms = fam(["intt_contig", "intt_strided"])
        ip = rows.get("inner_product")
        line = {
            "metric": BTS_METRIC, "value": round(value, 4), "unit": "bootstraps/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic",
            "config": {"workload": BTS_WORKLOAD, "ring_degree": DEGREE, "levels": BTS_LEVELS,
                       "special_primes": gpu.K, "dnum": DNUM, "input_level": level_in,
                       "output_level": int(out_level), "setup_s": round(setup_s, 1),
                       "max_abs_error_of_refreshed_slots": err,
                       "l2": "inputs_larger_than_l2 (64 rotation keys of 144 MiB and the "
                             "transform plaintexts are streamed every bootstrap)",
                       "parallelism": f"replicas x{world}, no communication"},
            "e2e": {"value": round(reps * world / (e2e_ms * 1e-3), 4), "unit": "bootstraps/s",
                    "h2d_bytes_per_step": int(values.nbytes), "d2h_bytes_per_step": int(values.nbytes)},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "kernel": "ntt (strided+contig passes)",
                         "achieved": round(ntt_gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(ntt_gbs / peak, 4), "peak_kind": peak_kind, "traffic": None,
                         "share_of_bootstrap": round(ntt_ms / total, 4),
                         "others": {"intt (contig+strided passes)": {
                             "GB/s": round(intt_gbs, 1), "frac": round(intt_gbs / peak, 4),
                             "share_of_bootstrap": round(intt_ms / total, 4)}}},
            "breakdown": {"device_ms_one_bootstrap_by_kernel": rows,
                          "kernel_time_sum_ms": round(total, 2)},
        }
        if ip:
            line["roofline"]["others"]["inner_product"] = {"share_of_bootstrap": round(ip["ms"] / total, 4)}
    gpu.free_ciph(ct)
    gpu.free_ciph(res)
    gpu.close()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))

# ---------------------------------------------------------------------------
# reference arm / CPU baseline: the unmodified reference runtime on host cores
# ---------------------------------------------------------------------------

# DRAM bytes (read + write) per limb of a forward transform pair, from a profiler
# capture of the two kernels on 48 limbs with cold caches (25.4 MB strided + 77.1 MB
# contiguous per launch pair, twiddles included); this run does not measure DRAM
# traffic itself
NTT_DRAM_BYTES_PER_LIMB_CAPTURED = (25.4e6 + 77.1e6) / 48

# What one image of the compiled ResNet-20 program executes, by operation class
# (static analysis of the loop nests of the generated file): the CPU figures are
# the measured cost of each class times these counts.
R20_SAMPLE_LEVELS = (4, 10, 18)   # the program works between 2 and 19 limbs after a bootstrap
R20_BOOTSTRAP_LEVEL_AFTER = 16    # the program asks for 15..18
R20_HW_LIMB_CALLS = 1_400_000     # Hw_modadd / Hw_modmul / Hw_rotate calls, one limb each
R20_RESCALES = 3112               # polynomial rescales


def _ref_lib_path(omp):
    name = "libFHErt_ant_ref_omp.so" if omp else "libFHErt_ant_ref.so"
    return os.path.join(ROOT, "oracle", "_ref", name)


def _ref_worker(seed, steps, warmup, q, workload, omp, bootstrap):
    """One process = one reference context.  Times `steps` samples of the
    workload's operation classes and sends the per-class seconds back."""
    os.dup2(2, 1)  # the library's parameter line goes to stderr
    from tests import ref_runtime as rr
    rr.REF_LIB = _ref_lib_path(omp)
    if bootstrap:
        os.environ["RTLIB_DISABLE_BOOTSTRAP_PRECOM"] = "0"
    if workload == "resnet20":
        levels, q0, sf, op_levels = R20_LEVELS, R20_Q0, R20_SF, R20_SAMPLE_LEVELS
    else:
        levels, q0, sf, op_levels = LEVELS, Q0_BITS, SF_BITS, (LEVELS,)
    t0 = time.perf_counter()
    ref = rr.RefRuntime(DEGREE, levels, q0, sf, DNUM, rot_idxs=(1,), seed=np.arange(16) + seed)
    setup_s = time.perf_counter() - t0
    rng = np.random.default_rng(seed)
    q.put("ready")
    out = {"setup_s": setup_s, "rot": {}, "mul": {}, "encode": [], "hw": [], "rescale": [],
           "bootstrap": None, "step": []}
    if bootstrap:
        lib = ref.lib
        lib.Ref_bootstrap.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32,
                                      C.c_void_p, C.c_void_p]
        lib.Ref_bootstrap.restype = C.c_size_t
        vals = rng.uniform(-1, 1, DEGREE // 2) + 0j
        c0, c1 = ref.encrypt(ref.encode(vals, 1, 2))
        o0, o1 = np.zeros((ref.L, DEGREE), np.int64), np.zeros((ref.L, DEGREE), np.int64)
        t = time.perf_counter()
        lib.Ref_bootstrap(rr._p(c0), rr._p(c1), 2, DEGREE // 2, R20_BOOTSTRAP_LEVEL_AFTER,
                          rr._p(o0), rr._p(o1))
        out["bootstrap"] = time.perf_counter() - t
        q.put(out)
        return
    cts = {lv: (rr.uniform_limbs(rng, ref.primes[:lv], DEGREE),
                rr.uniform_limbs(rng, ref.primes[:lv], DEGREE)) for lv in op_levels}
    vals = rng.uniform(-1, 1, DEGREE // 4) + 0j
    for it in range(warmup + steps):
        rec = it >= warmup
        s0 = time.perf_counter()
        for lv in op_levels:
            c0, c1 = cts[lv]
            t0 = time.perf_counter()
            ref.rotate(c0, c1, 1)
            t1 = time.perf_counter()
            ref.mul_relin_rescale(c0, c1, c1, c0)
            t2 = time.perf_counter()
            if rec:
                out["rot"].setdefault(lv, []).append(t1 - t0)
                out["mul"].setdefault(lv, []).append(t2 - t1)
        if workload == "resnet20":
            mid = op_levels[len(op_levels) // 2]
            t0 = time.perf_counter()
            ref.encode(vals, 1, mid)            # one weight plaintext (Pt_from_msg)
            t1 = time.perf_counter()
            a, b = cts[mid][0][0], cts[mid][1][0]
            for _ in range(4):
                ref.hw("Hw_modmul", a, b, 0)
                ref.hw("Hw_modadd", a, b, 0)
            t2 = time.perf_counter()
            ref.rescale(cts[mid][0])
            t3 = time.perf_counter()
            if rec:
                out["encode"].append(t1 - t0)
                out["hw"].append((t2 - t1) / 8)
                out["rescale"].append(t3 - t2)
        if rec:
            out["step"].append(time.perf_counter() - s0)
    q.put(out)


def run_reference_workers(workers, steps, warmup, workload, omp=False, bootstrap=False):
    """`workers` processes, each with its own reference context, time `steps`
    samples; with `bootstrap` one more process times one bootstrap at the
    program's parameters meanwhile.  Returns the wall time of the samples and
    the per-class mean seconds."""
    if not os.path.exists(_ref_lib_path(omp)):
        return None
    ctx = mp.get_context("spawn")
    qs, ps = [], []
    for w in range(workers):
        q = ctx.Queue()
        p = ctx.Process(target=_ref_worker, args=(100 + w, steps, warmup, q, workload, omp, False))
        p.start()
        qs.append(q)
        ps.append(p)
    bq = bp = None
    if bootstrap:
        bq = ctx.Queue()
        bp = ctx.Process(target=_ref_worker, args=(99, 1, 0, bq, workload, omp, True))
        bp.start()
    for q in qs:
        q.get()
    t0 = time.perf_counter()
    per = [q.get() for q in qs]
    wall = time.perf_counter() - t0
    for p in ps:
        p.join()
    t_bts = None
    if bootstrap:
        bq.get()
        t_bts = bq.get()["bootstrap"]
        bp.join()

    def mean(key):
        vals = [v for r in per for v in r[key]]
        return float(np.mean(vals)) if vals else None

    levels = sorted(per[0]["rot"])
    fig = {"wall_s": wall, "workers": workers, "steps": steps,
           "rot": {lv: float(np.mean([np.mean(r["rot"][lv]) for r in per])) for lv in levels},
           "mul": {lv: float(np.mean([np.mean(r["mul"][lv]) for r in per])) for lv in levels},
           "encode": mean("encode"), "hw": mean("hw"), "rescale": mean("rescale"),
           "step": mean("step"), "bootstrap": t_bts}
    return fig


def _r20_image_seconds(fig):
    """Seconds of one ResNet-20 image on one core from the measured class costs;
    returns (seconds, breakdown, classes left out)."""
    rot = float(np.mean(list(fig["rot"].values())))
    mul = float(np.mean(list(fig["mul"].values())))
    parts = {"rotations": R20_ROTATIONS * rot, "relinearised_products": R20_RELINS * mul,
             "weight_encodes": R20_WEIGHTS * fig["encode"],
             "per_limb_vector_calls": R20_HW_LIMB_CALLS * fig["hw"],
             "rescales": R20_RESCALES * fig["rescale"]}
    missing = []
    if fig["bootstrap"] is not None:
        parts["bootstraps"] = R20_BOOTSTRAPS * fig["bootstrap"]
    else:
        missing.append("bootstraps (19 per image, not timed in this short sample)")
    return sum(parts.values()), {k: round(v, 1) for k, v in parts.items()}, missing


def _reference_summary(fig, workload, omp):
    workers, steps = fig["workers"], fig["steps"]
    lib = "OpenMP build of the reference library" if omp else "reference library"
    if workload == "resnet20":
        s_image, parts, missing = _r20_image_seconds(fig)
        value, unit = workers / s_image, "images/s"
        per_level = ", ".join(f"level {lv}: rotate {fig['rot'][lv]:.3f} s, product {fig['mul'][lv]:.3f} s"
                              for lv in sorted(fig["rot"]))
        sample = (f"{workers} process(es) x {steps} step(s) on the {lib}; one step = 1 Rotate + 1 "
                  f"HMult+relin+rescale at each of levels {list(sorted(fig['rot']))} of {R20_LEVELS} "
                  f"(N=2^16, dnum=3), 1 weight encode, 8 per-limb vector calls, 1 rescale; measured: "
                  f"{per_level}; encode {fig['encode']:.4f} s; vector call {fig['hw'] * 1e3:.3f} ms; "
                  f"rescale {fig['rescale']:.3f} s"
                  + (f"; one bootstrap (level_after {R20_BOOTSTRAP_LEVEL_AFTER}) {fig['bootstrap']:.1f} s"
                     if fig["bootstrap"] is not None else "")
                  + f"; extrapolated image = counts x class cost = {s_image:.0f} s per process {parts}"
                  + (f"; left out: {missing}" if missing else ""))
        extra = {"extrapolated": True, "s_per_image_one_core": round(s_image, 1),
                 "image_breakdown_s": parts}
    else:
        lv = max(fig["rot"])
        t_rot, t_mul = fig["rot"][lv], fig["mul"][lv]
        value, unit = 2 * steps * workers / fig["wall_s"], "ops/s"
        sample = (f"{workers} process(es) x {steps} step(s) of 1 Rotate(k=1) + 1 "
                  f"HMult+relin+rescale at N=2^16, L={lv}, dnum=3 on the {lib} "
                  f"({t_rot + t_mul:.2f} s each)")
        extra = {"extrapolated": False}
    return value, unit, sample, fig["step"] * 1e3, extra


def cpu_baseline_sample(workload="primitives"):
    """Rank 0, N=1 only: a bounded sample (tens of seconds of CPU work) of the
    workload's operation classes on one host core."""
    fig = run_reference_workers(1, 1, 0, workload)
    unit = "images/s" if workload == "resnet20" else "ops/s"
    if fig is None:
        return {"value": None, "unit": unit, "cores": 0, "kind": "reference",
                "sample": "reference runtime library not built"}
    value, unit, sample, _, extra = _reference_summary(fig, workload, False)
    out = {"value": round(value, 6), "unit": unit, "cores": 1, "kind": "reference",
           "sample": sample}
    out.update(extra)
    return out


def cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for ln in f:
                if ln.startswith("model name"):
                    return ln.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def run_reference(args):
    if int(os.environ.get("RANK", 0)) != 0:
        return
    cores = os.cpu_count() or 1
    r20 = args.workload == "resnet20"
    # every worker holds its own context, keys and buffers (about 1.2 GB); with
    # the ResNet workload one more process times a bootstrap (about 12 GB)
    workers = max(1, min(cores - (1 if r20 else 0), 32))
    fig = run_reference_workers(workers, max(1, args.steps), min(1, args.warmup), args.workload,
                                bootstrap=r20)
    if fig is None:
        print(json.dumps({"impl": "reference", "unavailable":
                          "oracle/_ref/libFHErt_ant_ref.so not built on this box"}))
        return
    value, unit, sample, ms_step, extra = _reference_summary(fig, args.workload, False)
    baseline = {"value": round(value, 6), "unit": unit, "cores": workers, "kind": "reference",
                "sample": sample, "cpu": cpu_model(), "nproc": cores}
    baseline.update(extra)
    # the reference's OpenMP build (its BUILD_WITH_OPENMP option), one process
    # with all host threads, on the same sample
    omp_threads = str(cores)
    os.environ["OMP_NUM_THREADS"] = omp_threads
    omp = run_reference_workers(1, 1, 0, args.workload, omp=True)
    if omp is not None:
        ov, ou, osample, _, oextra = _reference_summary(omp, args.workload, True)
        baseline["openmp"] = {"value": round(ov, 6), "unit": ou, "OMP_NUM_THREADS": int(omp_threads),
                              "sample": osample}
        baseline["openmp"].update(oextra)
    else:
        baseline["openmp"] = {"unavailable": "oracle/_ref/libFHErt_ant_ref_omp.so not built "
                                             "(oracle/build_ref.sh with OMP=1)"}
    line = {
        "impl": "reference", "metric": R20_METRIC if r20 else METRIC, "value": round(value, 6),
        "unit": unit, "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
        "data": "synthetic",
        "config": {"workload": R20_WORKLOAD if r20 else WORKLOAD, "ring_degree": DEGREE,
                   "levels": R20_LEVELS if r20 else LEVELS, "dnum": DNUM,
                   "step": "one timed step = one sample of the workload's operation classes "
                           "(ms_per_step is its measured wall time); value extrapolates the "
                           "sample to whole images with the program's operation counts"},
        "cpu_baseline": baseline,
        "e2e": {"value": round(value, 6), "unit": unit, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-replay", action="store_true",
                    help="compiled programs: launch every image's kernels from the host instead of "
                         "replaying the captured Main_graph")
    ap.add_argument("--cache-mb", type=int, default=120000,
                    help="HBM budget of the weight-plaintext cache (resnet20 workload)")
    ap.add_argument("--workload", default="auto",
                    choices=["auto", "resnet20", "primitives", "bootstrap"] + sorted(OTHER_PROGRAMS))
    ap.add_argument("--levels", default="4,12,24,36",
                    help="ciphertext levels of the per-level figures (primitives workload)")
    args = ap.parse_args()
    args.levels = [int(x) for x in args.levels.split(",") if x]
    if args.workload == "auto":
        args.workload = "resnet20" if os.path.exists(PROGRAM_SO) else "primitives"
    program_so = PROGRAM_SO
    if args.workload in OTHER_PROGRAMS:
        program_so = os.path.join(PROGRAM_DIR, OTHER_PROGRAMS[args.workload][0] + ".so")
    if (args.workload == "resnet20" or args.workload in OTHER_PROGRAMS) and not os.path.exists(program_so):
        sys.exit(f"{program_so} is missing: run ace_compiler_b200/programs/build_programs.sh "
                 "where the reference checkout is present")
    if args.impl == "reference":
        if args.workload in OTHER_PROGRAMS or args.workload == "bootstrap":
            args.workload = "resnet20" if args.workload in OTHER_PROGRAMS else "primitives"
        run_reference(args)
    elif args.workload == "resnet20" or args.workload in OTHER_PROGRAMS:
        run_resnet20(args)
    elif args.workload == "bootstrap":
        run_bootstrap(args)
    else:
        run_primitives(args)


if __name__ == "__main__":
    main()
