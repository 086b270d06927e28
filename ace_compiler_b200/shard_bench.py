"""Latency of limb-sharded ciphertext operations on N GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \
        --master-addr 127.0.0.1 --master-port P -m ace_compiler_b200.shard_bench

(or plain `python -m ace_compiler_b200.shard_bench` for one GPU).  One
ciphertext at N = 2^16, L = 36, dnum = 3 is spread over the ranks by limb;
timed per operation with CUDA events on the library stream, the figure is the
slowest rank's.  Operations: rotation (two all-gathers), multiplication with
relinearisation (the same two), rescale (one broadcast of two limbs).  The
exchanges are NCCL collectives issued by the library itself.  Rank 0 prints one
JSON line.
"""
import argparse
import ctypes as C
import json
import os

import numpy as np


def main():
    import torch

    import ace_compiler_b200 as rt
    from ace_compiler_b200 import parallel, sharded

    ap = argparse.ArgumentParser()
    ap.add_argument("--levels", type=int, default=36)
    ap.add_argument("--degree", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    n, L = args.degree, args.levels
    saved = os.dup(1)
    os.dup2(2, 1)  # the library and NCCL print their greeting lines with C stdio
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist.barrier()
    gpu = rt.Runtime(n, L, 60, 56, 3, rot_idxs=(1,))
    lib = gpu.lib
    rng = np.random.default_rng(5)  # the same keys and ciphertext on every rank
    for is_rot, idx in ((False, 0), (True, 1)):
        for part in range(gpu.dnum):
            for which in (0, 1):
                key = np.stack([rng.integers(0, p, n, dtype=np.int64) for p in gpu.primes])
                gpu.import_switch_key(is_rot, idx, part, which, key)
    c0 = np.stack([rng.integers(0, p, n, dtype=np.int64) for p in gpu.primes[:L]])
    c1 = np.stack([rng.integers(0, p, n, dtype=np.int64) for p in gpu.primes[:L]])
    ct = gpu.new_ciph(c0, c1)
    ops = sharded.ShardedOps(gpu, rank, world)
    C.CDLL(None).fflush(None)
    os.dup2(saved, 1)
    stream = torch.cuda.ExternalStream(lib.Fhert_stream(), device=torch.device("cuda", local))
    rot, prod, resc = rt.CIPHERTEXT(), rt.CIPHERTEXT(), rt.CIPHERTEXT()

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        lib.Fhert_sync()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.iters):
            fn()
        e1.record(stream)
        lib.Fhert_sync()
        if world > 1:
            dist.barrier()
        dev = "cuda" if world > 1 else "cpu"
        return parallel.slowest_rank([e0.elapsed_time(e1) / args.iters], device=dev)[0]

    ms_rot = timed(lambda: ops.rotate(rot, ct, 1))
    ms_mul = timed(lambda: ops.mul_relin(prod, ct, rot))
    ms_res = timed(lambda: ops.rescale(resc, prod))
    if rank == 0:
        print(json.dumps({
            "op": "limb-sharded Rotate / HMult+relin / Rescale", "degree": n, "levels": L,
            "n_gpus": world,
            "rotate_ms": round(ms_rot, 4), "mul_relin_ms": round(ms_mul, 4),
            "rescale_ms": round(ms_res, 4),
            "hmult_relin_rescale_ms": round(ms_mul + ms_res, 4),
            "exchange_MiB_per_rank": {
                "rotate": round(ops.exchange_bytes(L, "rotate") / 2 ** 20, 2),
                "mul_relin": round(ops.exchange_bytes(L, "mul_relin") / 2 ** 20, 2),
                "rescale": round(2 * n * 8 / 2 ** 20, 2)},
            "timing": "CUDA events on the library stream, slowest rank",
        }))
    ops.close()
    for c in (ct, rot, prod, resc):
        gpu.free_ciph(c)
    gpu.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
