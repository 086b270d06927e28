"""Bit-exact parity of the CUDA runtime with the reference CPU runtime
(oracle/_ref, the unmodified ANT-ACE rtlib) on seeded inputs, through the
C ABI.  One context pair per parameter set; every comparison is exact."""
import ctypes as C

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

# (degree, L, q0_bits, sf_bits, dnum, rotations)
PARAM_SETS = {
    "small_n1024": (1024, 5, 33, 30, 2, (1, -3)),
    "tile_n8192": (8192, 5, 60, 56, 3, (5,)),
    "tile_n65536": (65536, 7, 60, 56, 3, (1, 4096, -2)),
    # the prime sizes of the compiled ResNet programs: the transforms of the 46-
    # and 51-bit primes run without per-butterfly range correction
    "chain_51_46_n65536": (65536, 6, 51, 46, 3, (1, -4096)),
    "chain_51_46_n16384": (16384, 7, 51, 46, 2, (3,)),
}


@pytest.fixture(scope="module", params=list(PARAM_SETS))
def pair(request):
    if not rr.available():
        pytest.skip("reference runtime not built (oracle/build_ref.sh)")
    import ace_compiler_b200 as rt
    n, L, q0, sf, dnum, rots = PARAM_SETS[request.param]
    ref = rr.RefRuntime(n, L, q0, sf, dnum, rot_idxs=rots, seed=np.arange(16) + 7)
    gpu = rt.Runtime(n, L, q0, sf, dnum, rot_idxs=rots)
    # key material comes from the reference key generator
    for is_rot, idx in [(False, 0)] + [(True, r) for r in rots]:
        for part in range(ref.dnum):
            for which in (0, 1):
                gpu.import_switch_key(is_rot, idx, part, which, ref.swk(is_rot, idx, part, which))
    yield ref, gpu, rots
    gpu.close()
    rr.close_ref(ref)


def test_prime_chain_and_tables(pair):
    ref, gpu, _ = pair
    assert (gpu.L, gpu.K, gpu.alpha, gpu.dnum) == (ref.L, ref.K, ref.alpha, ref.dnum)
    assert gpu.primes == ref.primes
    n = gpu.N
    for idx in range(gpu.L + gpu.K):
        got = [np.zeros(n, np.int64), np.zeros(n, np.uint64), np.zeros(n, np.int64),
               np.zeros(n, np.uint64), np.zeros(1, np.int64)]
        gpu.lib.Fhert_get_ntt_tables(idx, *[a.ctypes.data_as(C.c_void_p) for a in got])
        exp = ref.ntt_tables(idx)
        for g, e in zip(got[:4], exp[:4]):
            assert np.array_equal(g, e)
        assert int(got[4][0]) == exp[4]


def test_ntt_and_intt_every_prime(pair):
    ref, gpu, _ = pair
    rng = np.random.default_rng(11)
    total = gpu.L + gpu.K
    data = rr.uniform_limbs(rng, gpu.primes, gpu.N)
    src = gpu.new_poly(total, data=data)
    dst = gpu.new_poly(total)
    for idx in range(total):
        gpu.lib.Hw_ntt(gpu.limb_ptr(dst, idx), gpu.limb_ptr(src, idx), idx, gpu.N)
    fwd = gpu.download(dst)
    for idx in range(total):
        assert np.array_equal(fwd[idx], ref.ntt(idx, data[idx])), f"NTT prime {idx}"
    for idx in range(total):
        gpu.lib.Hw_intt(gpu.limb_ptr(dst, idx), gpu.limb_ptr(src, idx), idx, gpu.N)
    inv = gpu.download(dst)
    for idx in range(total):
        assert np.array_equal(inv[idx], ref.ntt(idx, data[idx], inverse=True)), f"INTT prime {idx}"
    gpu.free(src)
    gpu.free(dst)


def test_ntt_edge_values(pair):
    """all-zero, all q-1 and a single one: the extremes of the lazy butterflies"""
    ref, gpu, _ = pair
    idx = gpu.L - 1
    q = gpu.primes[idx]
    cases = [np.zeros(gpu.N, np.int64), np.full(gpu.N, q - 1, np.int64)]
    one = np.zeros(gpu.N, np.int64)
    one[gpu.N - 1] = 1
    cases.append(one)
    p = gpu.new_poly(1)
    for data in cases:
        for inverse in (False, True):
            gpu.lib.Fhert_upload(p, 0, 1, data.ctypes.data_as(C.c_void_p))
            fn = gpu.lib.Hw_intt if inverse else gpu.lib.Hw_ntt
            fn(gpu.limb_ptr(p, 0), gpu.limb_ptr(p, 0), idx, gpu.N)  # in place
            assert np.array_equal(gpu.download(p)[0], ref.ntt(idx, data, inverse=inverse))
    gpu.free(p)


def test_batched_conversion_round_trip(pair):
    ref, gpu, _ = pair
    rng = np.random.default_rng(12)
    data = rr.uniform_limbs(rng, gpu.primes, gpu.N)
    p = gpu.new_poly(gpu.L, extended=True, data=data, is_ntt=False)
    gpu.lib.Conv_poly2ntt_inplace(p)
    fwd = gpu.download(p)
    for idx in range(gpu.L + gpu.K):
        assert np.array_equal(fwd[idx], ref.ntt(idx, data[idx]))
    gpu.lib.Conv_ntt2poly_inplace(p)
    assert np.array_equal(gpu.download(p), data)
    gpu.free(p)
    # out of place (rns_poly.c:637, rns_poly_impl.c:202) and in place, many in a row
    a = gpu.new_poly(gpu.L, data=data[: gpu.L], is_ntt=False)
    b = gpu.new_poly(gpu.L)
    for _ in range(6):
        gpu.lib.Conv_poly2ntt(b, a)
        gpu.lib.Conv_ntt2poly(a, b)
        gpu.lib.Conv_poly2ntt_inplace(a)
        gpu.lib.Conv_ntt2poly_inplace(a)
    assert np.array_equal(gpu.download(a), data[: gpu.L])
    assert np.array_equal(gpu.download(b), fwd[: gpu.L])
    gpu.free(a)
    gpu.free(b)


def test_hw_vector_ops(pair):
    ref, gpu, _ = pair
    rng = np.random.default_rng(13)
    for idx in (0, gpu.L - 1, gpu.L + gpu.K - 1):
        q = gpu.primes[idx]
        a = rng.integers(0, q, gpu.N, dtype=np.int64)
        b = rng.integers(0, q, gpu.N, dtype=np.int64)
        a[:4] = [0, q - 1, q - 1, 1]
        b[:4] = [0, q - 1, 1, q - 1]
        pa, pb, pr = (gpu.new_poly(1, data=x[None]) for x in (a, b, a))
        m = gpu.modulus(idx)
        for name in ("Hw_modadd", "Hw_modsub", "Hw_modmul"):
            getattr(gpu.lib, name)(gpu.limb_ptr(pr, 0), gpu.limb_ptr(pa, 0), gpu.limb_ptr(pb, 0), m, gpu.N)
            assert np.array_equal(gpu.download(pr)[0], ref.hw(name, a, b, idx)), name
        acc = rng.integers(0, q, gpu.N, dtype=np.int64)
        gpu.upload(pr, acc[None])
        gpu.lib.Hw_modmuladd(gpu.limb_ptr(pr, 0), gpu.limb_ptr(pa, 0), gpu.limb_ptr(pb, 0), m, gpu.N)
        assert np.array_equal(gpu.download(pr)[0], ref.hw_muladd(acc, a, b, idx))
        for s in (0, 1, q - 1, 12345678901234567 % q):
            gpu.lib.Hw_modmul_scalar(gpu.limb_ptr(pr, 0), gpu.limb_ptr(pa, 0), s, m, gpu.N)
            assert np.array_equal(gpu.download(pr)[0], ref.hw_scalar("Hw_modmul_scalar", a, s, idx))
            gpu.lib.Hw_modadd_scalar(gpu.limb_ptr(pr, 0), gpu.limb_ptr(pa, 0), s, m, gpu.N)
            assert np.array_equal(gpu.download(pr)[0], ref.hw_scalar("Hw_modadd_scalar", a, s, idx))
        for p in (pa, pb, pr):
            gpu.free(p)


def test_automorphism_tables_and_rotate(pair):
    ref, gpu, rots = pair
    rng = np.random.default_rng(14)
    q = gpu.primes[1]
    val = rng.integers(0, q, gpu.N, dtype=np.int64)
    pv = gpu.new_poly(1, data=val[None])
    pr = gpu.new_poly(1)
    for r in rots:
        assert gpu.lib.Auto_idx(r) == ref.auto_idx(r)
        order = ref.auto_order(r)
        gpu.lib.Hw_rotate(gpu.limb_ptr(pr, 0), gpu.limb_ptr(pv, 0), gpu.lib.Auto_order(r),
                          gpu.modulus(1), gpu.N)
        assert np.array_equal(gpu.download(pr)[0], ref.hw_rotate(val, order, 1))
    gpu.free(pv)
    gpu.free(pr)


def test_rescale_all_levels(pair):
    ref, gpu, _ = pair
    rng = np.random.default_rng(15)
    for level in range(2, gpu.L + 1):
        data = rr.uniform_limbs(rng, gpu.primes[:level], gpu.N)
        src = gpu.new_poly(level, data=data)
        dst = gpu.new_poly(level)
        gpu.lib.Rescale(dst, src)
        assert dst.contents._num_primes == level - 1
        assert np.array_equal(gpu.download(dst), ref.rescale(data)), f"level {level}"
        gpu.free(src)
        gpu.free(dst)


def test_decomp_modup_every_digit_and_level(pair):
    ref, gpu, _ = pair
    rng = np.random.default_rng(16)
    for level in sorted({gpu.L, gpu.L - 1, max(1, gpu.alpha), 1}):
        data = rr.uniform_limbs(rng, gpu.primes[:level], gpu.N)
        src = gpu.new_poly(level, data=data)
        assert gpu.lib.Num_decomp(src) == ref.num_decomp(level)
        for part in range(ref.num_decomp(level)):
            ext = gpu.new_poly(level, extended=True)
            gpu.lib.Decomp_modup(ext, src, part)
            assert np.array_equal(gpu.download(ext), ref.decomp_modup(data, part)), (level, part)
            gpu.free(ext)
        gpu.free(src)


def test_mod_down(pair):
    ref, gpu, _ = pair
    rng = np.random.default_rng(17)
    for level in sorted({gpu.L, 2, 1}):
        primes = gpu.primes[:level] + gpu.primes[gpu.L:]
        data = rr.uniform_limbs(rng, primes, gpu.N)
        ext = gpu.new_poly(level, extended=True, data=data)
        out = gpu.new_poly(level)
        gpu.lib.Mod_down(out, ext)
        assert np.array_equal(gpu.download(out), ref.mod_down(data, level)), f"level {level}"
        gpu.free(ext)
        gpu.free(out)


def test_rotate_ciphertext(pair):
    import ace_compiler_b200 as rt
    ref, gpu, rots = pair
    rng = np.random.default_rng(18)
    for level in sorted({gpu.L, 2}):
        c0 = rr.uniform_limbs(rng, gpu.primes[:level], gpu.N)
        c1 = rr.uniform_limbs(rng, gpu.primes[:level], gpu.N)
        ct = gpu.new_ciph(c0, c1)
        for r in rots:
            out = rt.CIPHERTEXT()
            gpu.lib.Rotate_ciph(C.byref(out), C.byref(ct), r)
            g0, g1 = gpu.ciph_to_host(out)
            e0, e1 = ref.rotate(c0, c1, r)
            assert np.array_equal(g0, e0) and np.array_equal(g1, e1), (level, r)
            gpu.free_ciph(out)
        gpu.free_ciph(ct)


def test_mul_relin_rescale(pair):
    import ace_compiler_b200 as rt
    ref, gpu, _ = pair
    rng = np.random.default_rng(19)
    for level in sorted({gpu.L, 3}):
        a0, a1, b0, b1 = (rr.uniform_limbs(rng, gpu.primes[:level], gpu.N) for _ in range(4))
        ca, cb = gpu.new_ciph(a0, a1), gpu.new_ciph(b0, b1)
        prod, res = rt.CIPHERTEXT(), rt.CIPHERTEXT()
        gpu.lib.Mul_ciph(C.byref(prod), C.byref(ca), C.byref(cb))
        gpu.lib.Rescale_ciph(C.byref(res), C.byref(prod))
        g0, g1 = gpu.ciph_to_host(res)
        e0, e1 = ref.mul_relin_rescale(a0, a1, b0, b1)
        assert np.array_equal(g0, e0) and np.array_equal(g1, e1), level
        assert res._sf_degree == 1
        for c in (ca, cb, prod, res):
            gpu.free_ciph(c)


def test_extreme_residues_through_base_conversion(pair):
    """every residue at its maximum q-1: the worst case for the lazy
    accumulators of ModUp, ModDown and the key inner product"""
    import ace_compiler_b200 as rt
    ref, gpu, rots = pair
    level = gpu.L
    top = np.stack([np.full(gpu.N, p - 1, np.int64) for p in gpu.primes])
    src = gpu.new_poly(level, data=top[:level])
    for part in range(ref.num_decomp(level)):
        ext = gpu.new_poly(level, extended=True)
        gpu.lib.Decomp_modup(ext, src, part)
        assert np.array_equal(gpu.download(ext), ref.decomp_modup(top[:level], part))
        gpu.free(ext)
    gpu.free(src)
    ext = gpu.new_poly(level, extended=True, data=top)
    out = gpu.new_poly(level)
    gpu.lib.Mod_down(out, ext)
    assert np.array_equal(gpu.download(out), ref.mod_down(top, level))
    gpu.free(ext)
    gpu.free(out)
    ct = gpu.new_ciph(top[:level], top[:level])
    res = rt.CIPHERTEXT()
    gpu.lib.Rotate_ciph(C.byref(res), C.byref(ct), rots[0])
    g0, g1 = gpu.ciph_to_host(res)
    e0, e1 = ref.rotate(top[:level], top[:level], rots[0])
    assert np.array_equal(g0, e0) and np.array_equal(g1, e1)
    gpu.free_ciph(ct)
    gpu.free_ciph(res)
