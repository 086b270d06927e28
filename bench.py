#!/usr/bin/env python
"""Benchmark of the CKKS runtime on B200.

Default workload (BASELINE.json configs[0], the configuration the headline
metric is quoted on): encrypted ResNet-20 inference, the program the ANT-ACE
compiler emitted for resnet20_cifar10 (N = 2^16, 34 RNS limbs of 51/46 bits,
dnum = 3, 19 bootstraps), linked unchanged against this runtime
(ace_compiler_b200/programs/build_programs.sh builds it where the reference
checkout is present).  One step = one image: a seeded uniform[-1,1] 3x32x32
tensor is encoded and encrypted, Main_graph runs, the logits are decrypted.
Weights are a synthetic data file of seeded N(0, sigma) values in the
compiler's format; the encoded weight plaintexts stay resident in HBM (the
runtime's plaintext cache), so a step does not re-encode them.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--workload resnet20|primitives]

`value` is images/s over the device time of Main_graph with the encrypted
input resident in HBM; `e2e` is images/s over the whole step from the host
tensor to the host logits.  `--workload primitives` runs the configs[1] sweep
at L = 36 instead (16 rotations + 16 HMult+relinearise+rescale per step), which
is also what runs when the compiled program is not available.
`--impl reference` times the unmodified reference CPU runtime (oracle/_ref) on
the host cores.
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
PROGRAM_SO = os.path.join(ROOT, "ace_compiler_b200", "programs", "_ref", PROGRAM + ".so")
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

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

def run_resnet20(args):
    import torch

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from ace_compiler_b200.msgfile import write_synthetic_msg_file
    weights = f"/tmp/fhert_{PROGRAM}_{os.getpid()}.msg"
    write_synthetic_msg_file(weights, R20_WEIGHTS + 56, sigma=0.02, seed=7)
    os.environ["FHERT_DATA_FILE"] = weights
    os.environ["FHERT_PT_CACHE_MB"] = str(args.cache_mb)
    os.environ["FHERT_RT_STAT"] = "0"
    # the program's hooks (Get_context_params, Main_graph ...) must come first
    # in the global symbol scope, before the library's weak defaults
    C.CDLL(PROGRAM_SO, mode=C.RTLD_GLOBAL)
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

    def one_image(events=None):
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
        logits = [out[i] for i in range(10)]
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

    for _ in range(max(1, args.warmup)):  # the first image also fills the plaintext cache
        one_image()
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

    # the same program with every weight plaintext encoded afresh on the device
    # for every image, as the CPU runtime does (outside the timed region)
    lib.Fhert_pt_cache_bypass(1)
    uncached = []
    one_image()
    for _ in range(2):
        one_image(uncached)
    barrier()
    lib.Fhert_pt_cache_bypass(0)
    ms_uncached = sum(a.elapsed_time(b) for a, b in uncached) / len(uncached)

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
            # DRAM bytes per launch: read + write per limb of the forward transform
            # pair measured by ncu at 48 limbs (profiles/ntt_forward_48limbs_N65536.md:
            # 25.4 MB + 77.3 MB per 48-limb launch pair), scaled by the limbs per launch
            "traffic": (round(NTT_DRAM_BYTES_PER_LIMB * g["limbs"] / max(1, g["launches"]))
                        if top.startswith("ntt") else None),
            "alg_bytes_per_launch": g["bytes_per_limb"] * g["limbs"] / max(1, g["launches"]),
            "avg_ms_per_launch": g["ms"] / max(1, g["launches"]),
            "share_of_image": round(g["ms"] / total_ms, 4),
            "others": {k: {"GB/s": round(v["gbs"], 1), "frac": round(v["gbs"] / peak, 4),
                           "share_of_image": round(v["ms"] / total_ms, 4)}
                       for k, v in groups.items() if k != top},
        }
        line = {
            "metric": R20_METRIC, "value": round(value, 4), "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_graph / args.steps, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic",
            "config": {"workload": R20_WORKLOAD, "ring_degree": DEGREE, "levels": R20_LEVELS,
                       "dnum": DNUM, "special_primes": R20_K,
                       "s_per_image": round(ms_graph / args.steps / 1e3, 4),
                       "published_cpu_s_per_image": "1453.96 (one CPU thread, 60/56-bit primes; "
                                                    "not this program's 51/46-bit parameters, "
                                                    "so vs_baseline stays null)",
                       "setup_s": round(setup_s, 1),
                       "image_ms_this_rank": image_ms,
                       "s_per_image_weights_encoded_every_image": round(ms_uncached / 1e3, 3),
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
# reference arm / CPU baseline: the unmodified reference runtime on host cores
# ---------------------------------------------------------------------------

NTT_DRAM_BYTES_PER_LIMB = (25.4e6 + 77.3e6) / 48

R20_SAMPLE_LEVEL = 10  # between the 19 limbs after a bootstrap and the 2 before the next


def _ref_worker(seed, steps, warmup, q, workload):
    os.dup2(2, 1)  # the library's parameter line goes to stderr
    from tests import ref_runtime as rr
    if workload == "resnet20":
        levels, q0, sf, op_level = R20_LEVELS, R20_Q0, R20_SF, R20_SAMPLE_LEVEL
    else:
        levels, q0, sf, op_level = LEVELS, Q0_BITS, SF_BITS, LEVELS
    ref = rr.RefRuntime(DEGREE, levels, q0, sf, DNUM, rot_idxs=(1,), seed=np.arange(16) + seed)
    rng = np.random.default_rng(seed)
    c0 = rr.uniform_limbs(rng, ref.primes[:op_level], DEGREE)
    c1 = rr.uniform_limbs(rng, ref.primes[:op_level], DEGREE)
    q.put("ready")
    rot, mul = [], []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        ref.rotate(c0, c1, 1)
        t1 = time.perf_counter()
        ref.mul_relin_rescale(c0, c1, c1, c0)
        t2 = time.perf_counter()
        if it >= warmup:
            rot.append(t1 - t0)
            mul.append(t2 - t1)
    q.put((rot, mul))


def run_reference_workers(workers, steps, warmup, workload):
    """Each worker process owns a reference context and runs `steps` samples of
    one Rotate plus one HMult+relin+rescale; returns the wall time of the
    samples and the mean seconds per rotation and per product."""
    from tests import ref_runtime as rr
    if not rr.available():
        return None
    ctx = mp.get_context("spawn")
    qs, ps = [], []
    for w in range(workers):
        q = ctx.Queue()
        p = ctx.Process(target=_ref_worker, args=(100 + w, steps, warmup, q, workload))
        p.start()
        qs.append(q)
        ps.append(p)
    for q in qs:
        q.get()
    t0 = time.perf_counter()
    per = [q.get() for q in qs]
    wall = time.perf_counter() - t0
    for p in ps:
        p.join()
    t_rot = float(np.mean([np.mean(r) for r, _ in per]))
    t_mul = float(np.mean([np.mean(m) for _, m in per]))
    return wall, t_rot, t_mul


def _reference_figures(workers, steps, warmup, workload):
    res = run_reference_workers(workers, steps, warmup, workload)
    if res is None:
        return None
    wall, t_rot, t_mul = res
    if workload == "resnet20":
        # the rotations and relinearised products of one image at the sampled
        # cost; bootstraps, encodes and element-wise work are left out, which
        # flatters the CPU figure
        s_image = R20_ROTATIONS * t_rot + R20_RELINS * t_mul
        value, unit = workers / s_image, "images/s"
        sample = (f"{workers} process(es) x {steps} sample(s) of 1 Rotate + 1 HMult+relin+rescale at "
                  f"N=2^16, level {R20_SAMPLE_LEVEL} of {R20_LEVELS}, dnum=3 on the reference "
                  f"library ({t_rot:.3f} s and {t_mul:.3f} s each); one image = "
                  f"{R20_ROTATIONS} rotations + {R20_RELINS} products = {s_image:.0f} s per process, "
                  "bootstraps / encodes / element-wise work not counted")
        ms_step = s_image * 1e3
    else:
        value, unit = 2 * steps * workers / wall, "ops/s"
        sample = (f"{workers} process(es) x {steps} sample(s) of 1 Rotate(k=1) + 1 "
                  f"HMult+relin+rescale at N=2^16, L=36, dnum=3 ({t_rot + t_mul:.2f} s each)")
        ms_step = (t_rot + t_mul) * 1e3 * OPS_PER_STEP / 2
    return value, unit, sample, ms_step


def cpu_baseline_sample(workload="primitives"):
    fig = _reference_figures(1, 1, 0, workload)
    unit = "images/s" if workload == "resnet20" else "ops/s"
    if fig is None:
        return {"value": None, "unit": unit, "cores": 0, "kind": "reference",
                "sample": "reference runtime library not built"}
    value, unit, sample, _ = fig
    return {"value": round(value, 6), "unit": unit, "cores": 1, "kind": "reference",
            "sample": sample}


def run_reference(args):
    if int(os.environ.get("RANK", 0)) != 0:
        return
    cores = os.cpu_count() or 1
    # every worker holds its own context, keys and buffers (about 1.2 GB)
    workers = max(1, min(cores, 32))
    fig = _reference_figures(workers, max(1, args.steps), min(1, args.warmup), args.workload)
    if fig is None:
        print(json.dumps({"impl": "reference", "unavailable":
                          "oracle/_ref/libFHErt_ant_ref.so not built on this box"}))
        return
    value, unit, sample, ms_step = fig
    r20 = args.workload == "resnet20"
    line = {
        "impl": "reference", "metric": R20_METRIC if r20 else METRIC, "value": round(value, 6),
        "unit": unit, "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
        "data": "synthetic",
        "config": {"workload": R20_WORKLOAD if r20 else WORKLOAD, "ring_degree": DEGREE,
                   "levels": R20_LEVELS if r20 else LEVELS, "dnum": DNUM},
        "cpu_baseline": {"value": round(value, 6), "unit": unit, "cores": workers,
                         "kind": "reference", "sample": sample},
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
    ap.add_argument("--cache-mb", type=int, default=120000,
                    help="HBM budget of the weight-plaintext cache (resnet20 workload)")
    ap.add_argument("--workload", default="auto", choices=["auto", "resnet20", "primitives"])
    args = ap.parse_args()
    if args.workload == "auto":
        args.workload = "resnet20" if os.path.exists(PROGRAM_SO) else "primitives"
    if args.workload == "resnet20" and not os.path.exists(PROGRAM_SO):
        sys.exit(f"{PROGRAM_SO} is missing: run ace_compiler_b200/programs/build_programs.sh "
                 "where the reference checkout is present")
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "resnet20":
        run_resnet20(args)
    else:
        run_primitives(args)


if __name__ == "__main__":
    main()
