#!/usr/bin/env python
"""Benchmark of the CKKS runtime hot path on B200.

Workload (BASELINE.json configs[1], the primitive sweep at its largest level):
N = 2^16, L = 36 sixty/fifty-six-bit RNS primes, dnum = 3 (K = 12 special
primes).  One step = 16 rotations (k = 1, 2, 4, .., 2^15, each with its own
rotation key) + 16 HMult+relinearise+rescale on ciphertexts of seeded uniform
residues.  Every op is a full hybrid key switch (ModUp, key inner product,
ModDown) plus its element-wise / automorphism / rescale work.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

`value` times the ops with inputs resident in HBM; `e2e` times the same ops
through the C ABI with host buffers (pinned), i.e. with the upload of every
input ciphertext and the download of every result inside the timed region.
`--impl reference` times the unmodified reference CPU runtime (oracle/_ref) on
the host cores, one independent ciphertext stream per worker process.
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


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while running."""

    def __init__(self, index):
        self.index = index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
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
            self._stop.wait(0.2)

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


def run_ours(args):
    import torch

    import ace_compiler_b200 as rt

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

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
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

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
            line["cpu_baseline"] = cpu_baseline_sample()
    for c in (ct_a, ct_b, out, prod, res):
        gpu.free_ciph(c)
    gpu.close()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


# ---------------------------------------------------------------------------
# reference arm / CPU baseline: the unmodified reference runtime on host cores
# ---------------------------------------------------------------------------

def _ref_worker(seed, steps, warmup, q):
    from tests import ref_runtime as rr
    ref = rr.RefRuntime(DEGREE, LEVELS, Q0_BITS, SF_BITS, DNUM, rot_idxs=(1,),
                        seed=np.arange(16) + seed)
    rng = np.random.default_rng(seed)
    c0 = rr.uniform_limbs(rng, ref.primes[:LEVELS], DEGREE)
    c1 = rr.uniform_limbs(rng, ref.primes[:LEVELS], DEGREE)
    q.put("ready")
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        ref.rotate(c0, c1, 1)
        ref.mul_relin_rescale(c0, c1, c1, c0)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    q.put(times)


def run_reference_workers(workers, steps, warmup):
    """Each worker owns a context and runs `steps` samples of one Rotate plus one
    HMult+relin+rescale at L=36; returns aggregate ops/s and seconds per sample."""
    from tests import ref_runtime as rr
    if not rr.available():
        return None
    ctx = mp.get_context("spawn")
    qs, ps = [], []
    for w in range(workers):
        q = ctx.Queue()
        p = ctx.Process(target=_ref_worker, args=(100 + w, steps, warmup, q))
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
    ops = 2 * steps * workers
    return ops / wall, float(np.mean([np.mean(t) for t in per]))


def cpu_baseline_sample():
    res = run_reference_workers(1, 1, 0)
    if res is None:
        return {"value": None, "unit": "ops/s", "cores": 0, "kind": "reference",
                "sample": "reference runtime library not built"}
    ops_s, sec = res
    return {"value": round(ops_s, 4), "unit": "ops/s", "cores": 1, "kind": "reference",
            "sample": "1 Rotate(k=1) + 1 HMult+relin+rescale at N=2^16, L=36, dnum=3 on one "
                      f"host thread ({sec:.2f} s)"}


def run_reference(args):
    if int(os.environ.get("RANK", 0)) != 0:
        return
    cores = os.cpu_count() or 1
    # every worker holds its own context, keys and buffers (about 1.2 GB)
    workers = max(1, min(cores, 32))
    res = run_reference_workers(workers, max(1, args.steps), min(1, args.warmup))
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable":
                          "oracle/_ref/libFHErt_ant_ref.so not built on this box"}))
        return
    ops_s, sec = res
    sample = (f"{workers} worker processes x {max(1, args.steps)} samples of 1 Rotate(k=1) + 1 "
              "HMult+relin+rescale at N=2^16, L=36, dnum=3")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(ops_s, 4), "unit": "ops/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(sec * 1e3 * OPS_PER_STEP / 2, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "ring_degree": DEGREE, "levels": LEVELS,
                   "dnum": DNUM},
        "cpu_baseline": {"value": round(ops_s, 4), "unit": "ops/s", "cores": workers,
                         "kind": "reference", "sample": sample},
        "e2e": {"value": round(ops_s, 4), "unit": "ops/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
