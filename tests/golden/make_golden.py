"""Writes tests/golden/ref_n64.npz from the reference CPU runtime itself.

Needs oracle/_ref/libFHErt_ant_ref.so (oracle/build_ref.sh with the reference
checkout present).  The fixture holds the parameter set, seeded inputs and the
reference's outputs for every operation on the hot path, so that the oracle and
the CUDA runtime can be checked where the reference library is not available.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests import ref_runtime as rr  # noqa: E402

N, L, Q0, SF, DNUM, ROTS = 64, 5, 60, 56, 2, (1, -2, 7)


def main():
    ref = rr.RefRuntime(N, L, Q0, SF, DNUM, rot_idxs=ROTS, seed=np.arange(16) + 42)
    rng = np.random.default_rng(2025)
    out = {"params": np.array([N, L, Q0, SF, DNUM]), "rots": np.array(ROTS),
           "primes": np.array(ref.primes, np.int64), "alpha": np.array(ref.alpha)}
    total = ref.L + ref.K
    data = rr.uniform_limbs(rng, ref.primes, N)
    out["ntt_in"] = data
    out["ntt_out"] = np.stack([ref.ntt(i, data[i]) for i in range(total)])
    out["intt_out"] = np.stack([ref.ntt(i, data[i], inverse=True) for i in range(total)])
    for i in range(total):
        rou, roup, inv, invp, ninv = ref.ntt_tables(i)
        out[f"rou_{i}"], out[f"rou_inv_{i}"] = rou, inv
    a, b = data[:L], rr.uniform_limbs(rng, ref.primes[:L], N)
    out["hw_b"] = b
    for name in ("Hw_modadd", "Hw_modsub", "Hw_modmul"):
        out[name] = np.stack([ref.hw(name, a[i], b[i], i) for i in range(L)])
    for r in ROTS:
        out[f"auto_idx_{r}"] = np.array(ref.auto_idx(r))
        out[f"auto_order_{r}"] = ref.auto_order(r)
    for level in range(2, L + 1):
        out[f"rescale_{level}"] = ref.rescale(a[:level])
    for level in (L, L - 1, 1):
        for part in range(ref.num_decomp(level)):
            out[f"modup_{level}_{part}"] = ref.decomp_modup(a[:level], part)
    ext = np.concatenate([a, data[L:]])
    out["moddown_in"] = ext
    out[f"moddown_{L}"] = ref.mod_down(ext, L)
    ext2 = np.concatenate([a[:2], data[L:]])
    out["moddown_2"] = ref.mod_down(ext2, 2)
    for is_rot, idx in [(False, 0)] + [(True, r) for r in ROTS]:
        for part in range(ref.dnum):
            for which in (0, 1):
                out[f"key_{int(is_rot)}_{idx}_{part}_{which}"] = ref.swk(is_rot, idx, part, which)
    c0, c1 = a, b
    for level in (L, 2):
        for r in ROTS:
            o0, o1 = ref.rotate(c0[:level], c1[:level], r)
            out[f"rotate_{level}_{r}_0"], out[f"rotate_{level}_{r}_1"] = o0, o1
    for level in (L, 3):
        o0, o1 = ref.mul_relin_rescale(c0[:level], c1[:level], c1[:level], c0[:level])
        out[f"mul_{level}_0"], out[f"mul_{level}_1"] = o0, o1
    np.savez_compressed(os.path.join(HERE, "ref_n64.npz"), **out)
    rr.close_ref(ref)
    print("wrote ref_n64.npz with", len(out), "arrays")


if __name__ == "__main__":
    main()
