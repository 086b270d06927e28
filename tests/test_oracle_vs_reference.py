"""The plain-C oracle against the reference CPU runtime: committed golden
vectors written by the reference (tests/golden/ref_n64.npz) and, when the
reference library is present, live comparison on a larger seeded case."""
import os

import numpy as np
import pytest

from tests import oracle_lib
from tests import ref_runtime as rr

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_n64.npz"))


def golden_key(is_rot, idx, dnum):
    return [[G[f"key_{int(is_rot)}_{idx}_{p}_{w}"] for w in (0, 1)] for p in range(dnum)]


@pytest.fixture(scope="module")
def orc():
    n, L, q0, sf, dnum = (int(v) for v in G["params"])
    o = oracle_lib.Oracle(n, L, q0, sf, dnum)
    yield o
    o.close()


def test_golden_primes_and_tables(orc):
    assert orc.primes == G["primes"].tolist()
    assert orc.alpha == int(G["alpha"])
    for i in range(orc.L + orc.K):
        rou, inv, _ = orc.tables(i)
        assert np.array_equal(rou, G[f"rou_{i}"]) and np.array_equal(inv, G[f"rou_inv_{i}"])


def test_golden_ntt_hw_auto(orc):
    for i in range(orc.L + orc.K):
        assert np.array_equal(orc.ntt(i, G["ntt_in"][i]), G["ntt_out"][i])
        assert np.array_equal(orc.ntt(i, G["ntt_in"][i], inverse=True), G["intt_out"][i])
    a, b = G["ntt_in"][:orc.L], G["hw_b"]
    for op, name in enumerate(("Hw_modadd", "Hw_modsub", "Hw_modmul")):
        for i in range(orc.L):
            assert np.array_equal(orc.hw(op, a[i], b[i], i), G[name][i])
    for r in G["rots"].tolist():
        assert orc.auto_index(r) == int(G[f"auto_idx_{r}"])
        assert np.array_equal(orc.auto_order(r), G[f"auto_order_{r}"])


def test_golden_rescale_modup_moddown(orc):
    a = G["ntt_in"][:orc.L]
    for level in range(2, orc.L + 1):
        assert np.array_equal(orc.rescale(a[:level]), G[f"rescale_{level}"])
    for level in (orc.L, orc.L - 1, 1):
        for part in range(orc.num_decomp(level)):
            assert np.array_equal(orc.decomp_modup(a[:level], part), G[f"modup_{level}_{part}"])
    ext = G["moddown_in"]
    assert np.array_equal(orc.mod_down(ext, orc.L), G[f"moddown_{orc.L}"])
    ext2 = np.concatenate([ext[:2], ext[orc.L:]])
    assert np.array_equal(orc.mod_down(ext2, 2), G["moddown_2"])


def test_golden_rotate_and_multiply(orc):
    c0, c1 = G["ntt_in"][:orc.L], G["hw_b"]
    for level in (orc.L, 2):
        for r in G["rots"].tolist():
            o0, o1 = orc.rotate(c0[:level], c1[:level], r, golden_key(True, r, orc.dnum))
            assert np.array_equal(o0, G[f"rotate_{level}_{r}_0"])
            assert np.array_equal(o1, G[f"rotate_{level}_{r}_1"])
    relin = golden_key(False, 0, orc.dnum)
    for level in (orc.L, 3):
        o0, o1 = orc.mul_relin_rescale(c0[:level], c1[:level], c1[:level], c0[:level], relin)
        assert np.array_equal(o0, G[f"mul_{level}_0"]) and np.array_equal(o1, G[f"mul_{level}_1"])


@pytest.mark.skipif(not rr.available(), reason="reference runtime not built")
def test_live_reference_n2048():
    n, L, dnum, rots = 2048, 7, 3, (3,)
    ref = rr.RefRuntime(n, L, 60, 56, dnum, rot_idxs=rots, seed=np.arange(16) + 1)
    orc = oracle_lib.Oracle(n, L, 60, 56, dnum)
    try:
        assert orc.primes == ref.primes and (orc.K, orc.alpha) == (ref.K, ref.alpha)
        rng = np.random.default_rng(8)
        c0 = rr.uniform_limbs(rng, ref.primes[:L], n)
        c1 = rr.uniform_limbs(rng, ref.primes[:L], n)
        assert np.array_equal(orc.rescale(c0), ref.rescale(c0))
        for part in range(ref.num_decomp(L)):
            assert np.array_equal(orc.decomp_modup(c0, part), ref.decomp_modup(c0, part))
        key = [[ref.swk(True, 3, p, w) for w in (0, 1)] for p in range(dnum)]
        e0, e1 = ref.rotate(c0, c1, 3)
        o0, o1 = orc.rotate(c0, c1, 3, key)
        assert np.array_equal(o0, e0) and np.array_equal(o1, e1)
        relin = [[ref.swk(False, 0, p, w) for w in (0, 1)] for p in range(dnum)]
        e0, e1 = ref.mul_relin_rescale(c0, c1, c1, c0)
        o0, o1 = orc.mul_relin_rescale(c0, c1, c1, c0, relin)
        assert np.array_equal(o0, e0) and np.array_equal(o1, e1)
    finally:
        orc.close()
        rr.close_ref(ref)


@pytest.mark.skipif(not rr.available(), reason="reference runtime not built")
@pytest.mark.parametrize("params", [(16, 4, 60, 59), (16384, 3, 60, 56), (16, 3, 33, 30)])
def test_root_table_rule_matches_reference(params):
    """ring degrees 16 and 16384 take some 2N-th roots from the reference's table
    (util/src/std_param.c:229-300); the oracle reproduces the rule behind it"""
    n, L, q0, sf = params
    ref = rr.RefRuntime(n, L, q0, sf, 2, rot_idxs=(1,), seed=np.arange(16))
    orc = oracle_lib.Oracle(n, L, q0, sf, 2)
    try:
        assert orc.primes == ref.primes
        for i in range(orc.L + orc.K):
            rou, inv, _ = orc.tables(i)
            e_rou, _, e_inv, _, _ = ref.ntt_tables(i)
            assert np.array_equal(rou, e_rou) and np.array_equal(inv, e_inv), i
    finally:
        orc.close()
        rr.close_ref(ref)
