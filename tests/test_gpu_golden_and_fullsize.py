"""CUDA runtime against the committed golden vectors of the reference
(tests/golden/ref_n64.npz), then the BASELINE-size case N=2^16, L=36, dnum=3:
bit-exact against the reference library where it is present, and
size-independent properties (round trips, permutation composition) always."""
import ctypes as C
import os

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_n64.npz"))


def test_golden_vectors_n64():
    import ace_compiler_b200 as rt
    n, L, q0, sf, dnum = (int(v) for v in G["params"])
    rots = G["rots"].tolist()
    gpu = rt.Runtime(n, L, q0, sf, dnum, rot_idxs=rots)
    try:
        assert gpu.primes == G["primes"].tolist()
        for is_rot, idx in [(False, 0)] + [(True, r) for r in rots]:
            for part in range(dnum):
                for which in (0, 1):
                    gpu.import_switch_key(is_rot, idx, part, which,
                                          G[f"key_{int(is_rot)}_{idx}_{part}_{which}"])
        a, b = G["ntt_in"][:L], G["hw_b"]
        p = gpu.new_poly(L, extended=True, data=G["ntt_in"], is_ntt=False)
        gpu.lib.Conv_poly2ntt_inplace(p)
        assert np.array_equal(gpu.download(p), G["ntt_out"])
        gpu.upload(p, G["ntt_in"])
        gpu.lib.Conv_ntt2poly_inplace(p)
        assert np.array_equal(gpu.download(p), G["intt_out"])
        gpu.free(p)
        for level in range(2, L + 1):
            src, dst = gpu.new_poly(level, data=a[:level]), gpu.new_poly(level)
            gpu.lib.Rescale(dst, src)
            assert np.array_equal(gpu.download(dst), G[f"rescale_{level}"])
            gpu.free(src); gpu.free(dst)
        for level in (L, L - 1, 1):
            src = gpu.new_poly(level, data=a[:level])
            for part in range(gpu.lib.Num_decomp(src)):
                ext = gpu.new_poly(level, extended=True)
                gpu.lib.Decomp_modup(ext, src, part)
                assert np.array_equal(gpu.download(ext), G[f"modup_{level}_{part}"])
                gpu.free(ext)
            gpu.free(src)
        ext = gpu.new_poly(L, extended=True, data=G["moddown_in"])
        out = gpu.new_poly(L)
        gpu.lib.Mod_down(out, ext)
        assert np.array_equal(gpu.download(out), G[f"moddown_{L}"])
        gpu.free(ext); gpu.free(out)
        for level in (L, 2):
            ct = gpu.new_ciph(a[:level], b[:level])
            for r in rots:
                res = rt.CIPHERTEXT()
                gpu.lib.Rotate_ciph(C.byref(res), C.byref(ct), r)
                g0, g1 = gpu.ciph_to_host(res)
                assert np.array_equal(g0, G[f"rotate_{level}_{r}_0"])
                assert np.array_equal(g1, G[f"rotate_{level}_{r}_1"])
                gpu.free_ciph(res)
            gpu.free_ciph(ct)
        for level in (L, 3):
            ca, cb = gpu.new_ciph(a[:level], b[:level]), gpu.new_ciph(b[:level], a[:level])
            prod, res = rt.CIPHERTEXT(), rt.CIPHERTEXT()
            gpu.lib.Mul_ciph(C.byref(prod), C.byref(ca), C.byref(cb))
            gpu.lib.Rescale_ciph(C.byref(res), C.byref(prod))
            g0, g1 = gpu.ciph_to_host(res)
            assert np.array_equal(g0, G[f"mul_{level}_0"]) and np.array_equal(g1, G[f"mul_{level}_1"])
            for c in (ca, cb, prod, res):
                gpu.free_ciph(c)
    finally:
        gpu.close()


@pytest.fixture(scope="module")
def full():
    import ace_compiler_b200 as rt
    gpu = rt.Runtime(65536, 36, 60, 56, 3, rot_idxs=(1, -1))
    yield gpu
    gpu.close()


def test_fullsize_round_trips(full):
    gpu = full
    rng = np.random.default_rng(31)
    data = rr.uniform_limbs(rng, gpu.primes, gpu.N)
    p = gpu.new_poly(gpu.L, extended=True, data=data, is_ntt=False)
    gpu.lib.Conv_poly2ntt_inplace(p)
    assert not np.array_equal(gpu.download(p), data)
    gpu.lib.Conv_ntt2poly_inplace(p)
    assert np.array_equal(gpu.download(p), data)
    gpu.free(p)
    # Extend then Mod_down is the identity (unittest/ut_poly.cxx:444-480)
    x = gpu.new_poly(gpu.L, data=data[:gpu.L])
    ext = gpu.new_poly(gpu.L, extended=True)
    back = gpu.new_poly(gpu.L)
    gpu.lib.Extend(ext, x)
    gpu.lib.Mod_down(back, ext)
    assert np.array_equal(gpu.download(back), data[:gpu.L])
    # automorphism by 5^1 then by 5^-1 is the identity permutation
    r1, r2 = gpu.new_poly(gpu.L), gpu.new_poly(gpu.L)
    gpu.lib.Automorphism_transform(r1, x, gpu.lib.Auto_order(1))
    gpu.lib.Automorphism_transform(r2, r1, gpu.lib.Auto_order(-1))
    assert np.array_equal(gpu.download(r2), data[:gpu.L])
    for q in (x, ext, back, r1, r2):
        gpu.free(q)


@pytest.mark.skipif(not rr.available(), reason="reference runtime not built")
def test_fullsize_against_reference(full):
    import ace_compiler_b200 as rt
    gpu = full
    ref = rr.RefRuntime(65536, 36, 60, 56, 3, rot_idxs=(1, -1), seed=np.arange(16) + 9)
    try:
        assert gpu.primes == ref.primes and gpu.K == ref.K == 12
        for is_rot, idx in ((False, 0), (True, 1)):
            for part in range(3):
                for which in (0, 1):
                    gpu.import_switch_key(is_rot, idx, part, which, ref.swk(is_rot, idx, part, which))
        rng = np.random.default_rng(32)
        c0 = rr.uniform_limbs(rng, gpu.primes[:36], gpu.N)
        c1 = rr.uniform_limbs(rng, gpu.primes[:36], gpu.N)
        ct, ct2 = gpu.new_ciph(c0, c1), gpu.new_ciph(c1, c0)
        out, prod, res = rt.CIPHERTEXT(), rt.CIPHERTEXT(), rt.CIPHERTEXT()
        gpu.lib.Rotate_ciph(C.byref(out), C.byref(ct), 1)
        g0, g1 = gpu.ciph_to_host(out)
        e0, e1 = ref.rotate(c0, c1, 1)
        assert np.array_equal(g0, e0) and np.array_equal(g1, e1)
        gpu.lib.Mul_ciph(C.byref(prod), C.byref(ct), C.byref(ct2))
        gpu.lib.Rescale_ciph(C.byref(res), C.byref(prod))
        g0, g1 = gpu.ciph_to_host(res)
        e0, e1 = ref.mul_relin_rescale(c0, c1, c1, c0)
        assert np.array_equal(g0, e0) and np.array_equal(g1, e1)
        for c in (ct, ct2, out, prod, res):
            gpu.free_ciph(c)
    finally:
        rr.close_ref(ref)
