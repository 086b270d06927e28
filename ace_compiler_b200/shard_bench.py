"""Latency of one rotation with the ciphertext's limbs sharded over the GPUs
of a node (single-ciphertext latency mode), next to the same rotation on one
GPU.  Launch with

  python -m torch.distributed.run --nnodes=1 --nproc-per-node G \\
      --master-addr 127.0.0.1 --master-port P -m ace_compiler_b200.shard_bench

Workload: N = 2^16, L limbs (default 36), dnum = 3, seeded uniform residues and
a seeded uniform rotation key (the cost of a key switch does not depend on the
key values); every rank builds the same key and ciphertext from the same seed.
Rank 0 prints one JSON line.
"""
import argparse
import ctypes as C
import json
import os

import numpy as np


def main():
    import torch
    import torch.distributed as dist

    import ace_compiler_b200 as rt
    from ace_compiler_b200 import parallel, sharded

    ap = argparse.ArgumentParser()
    ap.add_argument("--levels", type=int, default=36)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = parallel.rank_world()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    n, levels, rot_idx = 65536, args.levels, 1
    os.dup2(2, 1) if rank else None
    gpu = rt.Runtime(n, levels, 60, 56, 3, rot_idxs=(rot_idx,))
    lib = gpu.lib
    rng = np.random.default_rng(4242)
    for part in range(gpu.dnum):
        for which in (0, 1):
            data = np.stack([rng.integers(0, p, n, dtype=np.int64) for p in gpu.primes])
            gpu.import_switch_key(True, rot_idx, part, which, data)
    c0 = np.stack([rng.integers(0, p, n, dtype=np.int64) for p in gpu.primes[:levels]])
    c1 = np.stack([rng.integers(0, p, n, dtype=np.int64) for p in gpu.primes[:levels]])
    ct = gpu.new_ciph(c0, c1)
    out = gpu.new_ciph(np.zeros_like(c0), np.zeros_like(c1))
    whole = rt.CIPHERTEXT()
    stream = torch.cuda.ExternalStream(lib.Fhert_stream(), device=torch.device("cuda", local))
    rot = sharded.ShardedRotator(gpu, levels, rank, world)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        lib.Fhert_sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.iters):
            fn()
        e1.record(stream)
        lib.Fhert_sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return parallel.slowest_rank([e0.elapsed_time(e1)], device="cuda")[0] / args.iters

    ms_one = timed(lambda: lib.Rotate_ciph(C.byref(whole), C.byref(ct), rot_idx))
    ms_sharded = timed(lambda: rot.rotate(ct._c0_poly._data, ct._c1_poly._data, rot_idx,
                                          out._c0_poly._data, out._c1_poly._data))
    # the owned limbs agree with the single-GPU result
    want, got = gpu.ciph_to_host(whole), gpu.ciph_to_host(out)
    mine = list(sharded.owned_q(levels, rank, world, rot.qb))
    ok = all(np.array_equal(want[0][i], got[0][i]) and np.array_equal(want[1][i], got[1][i])
             for i in mine)
    ok = bool(parallel.slowest_rank([0.0 if ok else 1.0], device="cuda")[0] == 0.0)
    if rank == 0:
        print(json.dumps({
            "op": "Rotate, limbs sharded over GPUs", "n_gpus": world, "ring_degree": n,
            "levels": levels, "dnum": gpu.dnum, "special_primes": gpu.K,
            "ms_one_gpu": round(ms_one, 4), "ms_sharded": round(ms_sharded, 4),
            "speedup": round(ms_one / ms_sharded, 3),
            "received_MiB_per_rank_per_rotation": round(rot.exchange_bytes() / 2 ** 20, 1),
            "owned_limbs_match_single_gpu": ok}), flush=True)
    gpu.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
