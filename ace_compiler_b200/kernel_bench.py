"""Micro-benchmarks of single runtime operations on one GPU.

    python -m ace_compiler_b200.kernel_bench --op ntt --levels 36 --iters 5

Each operation runs on `--polys` different polynomials in turn so that the
data touched between repetitions exceeds the L2 cache; device time comes from
CUDA events recorded around every kernel launch (Runtime.profile).  Prints one
JSON line: per-kernel launches / limbs / milliseconds, and the algorithmic
GB/s of the operation (bytes as defined per operation below).

This is also the small, self-terminating target used for profiler captures.
"""
import argparse
import ctypes as C
import json

import numpy as np

import ace_compiler_b200 as rt

W = None  # bytes per limb, set from the ring degree


def uniform(rng, primes, n):
    return np.stack([rng.integers(0, p, size=n, dtype=np.int64) for p in primes])


def main():
    global W
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="ntt",
                    choices=["ntt", "intt", "modmul", "automorphism", "rescale", "modup",
                             "moddown", "rotate", "hmult", "keyloop"])
    ap.add_argument("--degree", type=int, default=65536)
    ap.add_argument("--levels", type=int, default=36, help="L of the context and of the operands")
    ap.add_argument("--dnum", type=int, default=3)
    ap.add_argument("--polys", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    n, L = args.degree, args.levels
    gpu = rt.Runtime(n, L, 60, 56, args.dnum, rot_idxs=(1,))
    lib = gpu.lib
    W = 8 * n
    K, beta = gpu.K, -(-L // gpu.alpha)
    rng = np.random.default_rng(7)
    ext_primes = gpu.primes

    if args.op in ("rotate", "hmult", "keyloop"):
        for is_rot, idx in ((False, 0), (True, 1)):
            for part in range(gpu.dnum):
                for which in (0, 1):
                    gpu.import_switch_key(is_rot, idx, part, which, uniform(rng, ext_primes, n))

    polys, ciphs = [], []
    for _ in range(args.polys):
        if args.op in ("ntt", "intt", "moddown"):
            polys.append(gpu.new_poly(L, extended=True, data=uniform(rng, ext_primes, n),
                                      is_ntt=(args.op != "ntt")))
        elif args.op in ("rotate", "hmult", "keyloop"):
            ciphs.append(gpu.new_ciph(uniform(rng, gpu.primes[:L], n),
                                      uniform(rng, gpu.primes[:L], n)))
        else:
            polys.append(gpu.new_poly(L, data=uniform(rng, gpu.primes[:L], n)))
    out = gpu.new_poly(L, extended=(args.op == "modup"))
    out_ct, prod = rt.CIPHERTEXT(), rt.CIPHERTEXT()

    if args.op == "keyloop":
        # the key-switch loop a compiled program emits: per digit Decomp_modup, then per
        # limb tmp = key * digit; acc += tmp for both key polynomials, then two Mod_down
        ext = gpu.new_poly(L, extended=True)
        acc = [gpu.new_poly(L, extended=True) for _ in range(2)]
        down = [gpu.new_poly(L) for _ in range(2)]
        tmp = gpu.new_poly(1)
        swk = lib.Swk(True, 1)
        zeros = np.zeros((L + K, n), np.int64)

    def key_loop(i):
        c1 = C.pointer(ciphs[i % len(ciphs)]._c1_poly)
        for a in acc:
            gpu.upload(a, zeros)
        for part in range(int(lib.Num_decomp(c1))):
            lib.Decomp_modup(ext, c1, part)
            keys = (lib.Pk0_at(swk, part), lib.Pk1_at(swk, part))
            for limb in range(L + K):
                m = gpu.modulus(limb)  # operands are at the top level: limb i is prime i
                for key, a in zip(keys, acc):
                    lib.Hw_modmul(gpu.limb_ptr(tmp, 0), gpu.limb_ptr(key, limb),
                                  gpu.limb_ptr(ext, limb), m, n)
                    lib.Hw_modadd(gpu.limb_ptr(a, limb), gpu.limb_ptr(a, limb),
                                  gpu.limb_ptr(tmp, 0), m, n)
        for d, a in zip(down, acc):
            lib.Mod_down(d, a)
        lib.Fhert_sync()
        return (3 * L + 2 * beta * (L + K)) * W

    def run(i):
        if args.op == "keyloop":
            return key_loop(i)
        if args.op == "ntt":
            p = polys[i % len(polys)]
            p.contents._is_ntt = False
            lib.Conv_poly2ntt_inplace(p)
            return 2 * W * (L + K)
        if args.op == "intt":
            p = polys[i % len(polys)]
            p.contents._is_ntt = True
            lib.Conv_ntt2poly_inplace(p)
            return 2 * W * (L + K)
        if args.op == "modmul":
            a, b = polys[i % len(polys)], polys[(i + 1) % len(polys)]
            lib.Mul_poly(out, a, b)
            return 3 * W * L
        if args.op == "automorphism":
            lib.Automorphism_transform(out, polys[i % len(polys)], lib.Auto_order(1))
            return 2 * W * L
        if args.op == "rescale":
            out.contents._num_primes = L
            lib.Rescale(out, polys[i % len(polys)])
            return (2 * L - 1) * W
        if args.op == "modup":
            lib.Decomp_modup(out, polys[i % len(polys)], i % beta)
            return (L + K) * W
        if args.op == "moddown":
            lib.Mod_down(out, polys[i % len(polys)])
            return (2 * L + K) * W
        ks = (3 * L + 2 * beta * (L + K)) * W
        if args.op == "rotate":
            lib.Rotate_ciph(C.byref(out_ct), C.byref(ciphs[i % len(ciphs)]), 1)
            return ks + 3 * L * W + 4 * L * W
        lib.Mul_ciph(C.byref(prod), C.byref(ciphs[i % len(ciphs)]),
                     C.byref(ciphs[(i + 1) % len(ciphs)]))
        lib.Rescale_ciph(C.byref(out_ct), C.byref(prod))
        return 7 * L * W + ks + 6 * L * W + 2 * (2 * L - 1) * W

    for i in range(args.warmup):
        run(i)
    lib.Fhert_sync()
    with gpu.profile() as prof:
        total_bytes = sum(run(i) for i in range(args.iters))
    total_ms = sum(v[2] for v in prof.kernels.values())
    print(json.dumps({
        "op": args.op, "degree": n, "levels": L, "special_primes": K, "dnum": args.dnum,
        "iters": args.iters, "device_ms_per_op": round(total_ms / args.iters, 5),
        "ops_per_s": round(args.iters / (total_ms * 1e-3), 2),
        "algorithmic_GBs": round(total_bytes / (total_ms * 1e-3) / 1e9, 1),
        "kernels": {k: {"launches": v[0], "limbs": v[1], "ms": round(v[2], 4)}
                    for k, v in prof.kernels.items()},
    }))
    gpu.close()


if __name__ == "__main__":
    main()
