"""The call sequences the compiler emits for Rotate and for
multiply + relinearise + rescale (per-limb Hw_* loops with one shared scratch
limb, Decomp_modup per digit, two Mod_down and two Rescale calls in a row),
replayed from Python through the C ABI: the result must equal the library's
fused Rotate_ciph / Mul_ciph + Rescale_ciph and the reference, bit for bit."""
import ctypes as C

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

N, L = 4096, 9
ROTS = (1, 7)


@pytest.fixture(scope="module")
def pair():
    if not rr.available():
        pytest.skip("reference runtime not built")
    import ace_compiler_b200 as rt
    seed = np.arange(16, dtype=np.uint32) + 3
    ref = rr.RefRuntime(N, L, 60, 56, 3, rot_idxs=ROTS, seed=seed, fake_time_us=1_700_000_000_000_003)
    gpu = rt.Runtime(N, L, 60, 56, 3, rot_idxs=ROTS, keygen=True, seed=seed,
                     fake_time_us=1_700_000_000_000_003)
    yield ref, gpu, rt
    gpu.close()
    rr.close_ref(ref)


def key_switch_as_emitted(gpu, rt, src_poly, level, swk):
    """ModUp per digit, key inner product limb by limb through one scratch limb,
    then the two ModDowns: what the generated Rotate / Relinearize bodies do."""
    lib = gpu.lib
    acc0, acc1, ext = (lib.Alloc_poly(N, level, 1) for _ in range(3))
    tmp = lib.Alloc_poly(N, 1, 0)
    down0, down1 = lib.Alloc_poly(N, level, 0), lib.Alloc_poly(N, level, 0)
    for part in range(lib.Num_decomp(src_poly)):
        lib.Decomp_modup(ext, src_poly, part)
        k0, k1 = lib.Pk0_at(swk, part), lib.Pk1_at(swk, part)
        p_ofst = lib.Num_alloc(ext) - lib.Num_p(ext)
        key_p = lib.Poly_level(k0)
        limbs = [(i, i, gpu.modulus(i)) for i in range(lib.Poly_level(ext))]
        limbs += [(p_ofst + i, key_p + i, gpu.modulus(gpu.L + i)) for i in range(lib.Num_p(ext))]
        for e, k, m in limbs:
            t = lib.Coeffs(tmp, 0, N)
            lib.Hw_modmul(t, lib.Coeffs(k0, k, N), lib.Coeffs(ext, e, N), m, N)
            lib.Hw_modadd(lib.Coeffs(acc0, e, N), lib.Coeffs(acc0, e, N), t, m, N)
            lib.Hw_modmul(t, lib.Coeffs(k1, k, N), lib.Coeffs(ext, e, N), m, N)
            lib.Hw_modadd(lib.Coeffs(acc1, e, N), lib.Coeffs(acc1, e, N), t, m, N)
    lib.Mod_down(down0, acc0)
    lib.Mod_down(down1, acc1)
    for p in (acc0, acc1, ext, tmp):
        lib.Free_poly(p)
    return down0, down1


def test_rotate_as_emitted(pair):
    ref, gpu, rt = pair
    lib = gpu.lib
    rng = np.random.default_rng(21)
    for level in (L, 5, 2):
        c0 = rr.uniform_limbs(rng, gpu.primes[:level], N)
        c1 = rr.uniform_limbs(rng, gpu.primes[:level], N)
        ct = gpu.new_ciph(c0, c1)
        for rot in ROTS:
            out = rt.CIPHERTEXT()
            lib.Init_ciph_same_scale(C.byref(out), C.byref(ct), None)
            d0, d1 = key_switch_as_emitted(gpu, rt, C.pointer(ct._c1_poly), level, lib.Swk(True, rot))
            for i in range(level):
                lib.Hw_modadd(lib.Coeffs(d0, i, N), lib.Coeffs(d0, i, N),
                              lib.Coeffs(C.pointer(ct._c0_poly), i, N), gpu.modulus(i), N)
            order = lib.Auto_order(rot)
            for i in range(level):
                lib.Hw_rotate(lib.Coeffs(C.pointer(out._c0_poly), i, N), lib.Coeffs(d0, i, N), order,
                              gpu.modulus(i), N)
                lib.Hw_rotate(lib.Coeffs(C.pointer(out._c1_poly), i, N), lib.Coeffs(d1, i, N), order,
                              gpu.modulus(i), N)
            lib.Free_poly(d0)
            lib.Free_poly(d1)
            got = gpu.ciph_to_host(out)
            fused = rt.CIPHERTEXT()
            lib.Rotate_ciph(C.byref(fused), C.byref(ct), rot)
            want = ref.rotate(c0, c1, rot)
            assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]), (level, rot)
            f = gpu.ciph_to_host(fused)
            assert np.array_equal(f[0], want[0]) and np.array_equal(f[1], want[1])
            gpu.free_ciph(out)
            gpu.free_ciph(fused)
        gpu.free_ciph(ct)


def test_multiply_relinearise_rescale_as_emitted(pair):
    ref, gpu, rt = pair
    lib = gpu.lib
    rng = np.random.default_rng(22)
    for level in (L, 4):
        a0, a1, b0, b1 = (rr.uniform_limbs(rng, gpu.primes[:level], N) for _ in range(4))
        ca, cb = gpu.new_ciph(a0, a1), gpu.new_ciph(b0, b1)
        c3 = rt.CIPHERTEXT3()
        lib.Init_ciph3_up_scale(C.byref(c3), C.byref(ca), C.byref(cb))
        P = C.pointer
        tmp = lib.Alloc_poly(N, 1, 0)
        for i in range(level):
            m = gpu.modulus(i)
            co = lambda poly: lib.Coeffs(P(poly), i, N)
            lib.Hw_modmul(co(c3._c0_poly), co(ca._c0_poly), co(cb._c0_poly), m, N)
            lib.Hw_modmul(co(c3._c1_poly), co(ca._c0_poly), co(cb._c1_poly), m, N)
            lib.Hw_modmul(lib.Coeffs(tmp, 0, N), co(ca._c1_poly), co(cb._c0_poly), m, N)
            lib.Hw_modadd(co(c3._c1_poly), co(c3._c1_poly), lib.Coeffs(tmp, 0, N), m, N)
            lib.Hw_modmul(co(c3._c2_poly), co(ca._c1_poly), co(cb._c1_poly), m, N)
        lib.Free_poly(tmp)
        d0, d1 = key_switch_as_emitted(gpu, rt, P(c3._c2_poly), level, lib.Swk(False, 0))
        relin = rt.CIPHERTEXT()
        lib.Init_ciph_same_scale_ciph3(C.byref(relin), C.byref(c3))
        for i in range(level):
            m = gpu.modulus(i)
            lib.Hw_modadd(lib.Coeffs(P(relin._c0_poly), i, N), lib.Coeffs(d0, i, N),
                          lib.Coeffs(P(c3._c0_poly), i, N), m, N)
            lib.Hw_modadd(lib.Coeffs(P(relin._c1_poly), i, N), lib.Coeffs(d1, i, N),
                          lib.Coeffs(P(c3._c1_poly), i, N), m, N)
        lib.Free_poly(d0)
        lib.Free_poly(d1)
        res = rt.CIPHERTEXT()
        lib.Init_ciph_down_scale(C.byref(res), C.byref(relin))
        lib.Rescale(P(res._c0_poly), P(relin._c0_poly))
        lib.Rescale(P(res._c1_poly), P(relin._c1_poly))
        got = gpu.ciph_to_host(res)
        want = ref.mul_relin_rescale(a0, a1, b0, b1)
        assert got[0].shape[0] == level - 1
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]), level
        for p in (c3._c0_poly, c3._c1_poly, c3._c2_poly):
            lib.Free_poly_data(C.byref(p))
        for x in (ca, cb, relin, res):
            gpu.free_ciph(x)
