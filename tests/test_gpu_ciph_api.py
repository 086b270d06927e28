"""Ciphertext-level entry points beyond the compiled programs' needs, compared
bit for bit with the reference functions of the same name (called on host
structs of the same layout)."""
import ctypes as C

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

N, L = 1024, 6
ROTS = (1, -3, 5)
SEED = (np.arange(16, dtype=np.uint64) * 7919 % (2 ** 32)).astype(np.uint32)
FAKE_US = 1_700_000_111_000_007


@pytest.fixture(scope="module")
def pair():
    if not rr.available():
        pytest.skip("reference runtime not built")
    import ace_compiler_b200 as rt
    ref = rr.RefRuntime(N, L, 60, 56, 2, rot_idxs=ROTS, seed=SEED, fake_time_us=FAKE_US)
    gpu = rt.Runtime(N, L, 60, 56, 2, rot_idxs=ROTS, keygen=True, seed=SEED, fake_time_us=FAKE_US)
    yield ref, gpu, rt
    gpu.close()
    rr.close_ref(ref)


class HostCt:
    """A reference-side CIPHERTEXT / PLAINTEXT over numpy storage."""

    def __init__(self, rt, limbs0, limbs1=None, sf=2.0 ** 56, deg=1):
        self.keep = [np.ascontiguousarray(limbs0, np.int64)]
        if limbs1 is None:
            self.s = rt.PLAINTEXT()
            polys = [self.s._poly]
        else:
            self.keep.append(np.ascontiguousarray(limbs1, np.int64))
            self.s = rt.CIPHERTEXT()
            polys = [self.s._c0_poly, self.s._c1_poly]
        for p, a in zip(polys, self.keep):
            p._ring_degree, p._num_primes, p._num_alloc_primes = N, a.shape[0], a.shape[0]
            p._num_primes_p, p._is_ntt, p._data = 0, True, a.ctypes.data
        self.s._slots, self.s._scaling_factor, self.s._sf_degree = N // 2, sf ** deg, deg


def host_result(rt, ct):
    out = []
    for p in (ct._c0_poly, ct._c1_poly):
        buf = (C.c_int64 * (p._num_primes * N)).from_address(p._data)
        out.append(np.frombuffer(buf, dtype=np.int64).reshape(p._num_primes, N).copy())
    return out


def fresh(ref, gpu, rng, level, deg=1):
    vals = rng.uniform(-1, 1, N // 2) + 1j * rng.uniform(-1, 1, N // 2)
    c0, c1 = ref.encrypt(ref.encode(vals, deg, level), deg)
    return vals, c0, c1


def same(gpu, got_ct, want):
    g0, g1 = gpu.ciph_to_host(got_ct)
    return np.array_equal(g0, want[0]) and np.array_equal(g1, want[1])


def test_rotate_batch_shares_digits(pair):
    ref, gpu, rt = pair
    rng = np.random.default_rng(3)
    _, c0, c1 = fresh(ref, gpu, rng, L)
    ct = gpu.new_ciph(c0, c1)
    idx = (C.c_int32 * 4)(1, 0, -3, 5)
    outs = (rt.CIPHERTEXT * 4)()
    gpu.lib.Rotate_batch_ciph(outs, C.byref(ct), idx, 4)
    for k, r in enumerate(idx):
        want = (c0, c1) if r == 0 else ref.rotate(c0, c1, r)
        assert same(gpu, outs[k], want), r
        gpu.free_ciph(outs[k])
    gpu.free_ciph(ct)


def test_plain_operations_and_scale_management(pair):
    ref, gpu, rt = pair
    lib, rl = gpu.lib, ref.lib
    rng = np.random.default_rng(4)
    level = 5
    vals, c0, c1 = fresh(ref, gpu, rng, level)
    ptv = rng.uniform(-1, 1, N // 2) + 0j
    pt_host = ref.encode(ptv, 1, level)
    ct = gpu.new_ciph(c0, c1)
    pt = gpu.encode(ptv, 1, level)
    rc, rp = HostCt(rt, c0, c1), HostCt(rt, pt_host)

    for name in ("Mul_plain", "Add_plain"):
        got, want = rt.CIPHERTEXT(), rt.CIPHERTEXT()
        getattr(lib, name)(C.byref(got), C.byref(ct), C.byref(pt))
        getattr(rl, name)(C.byref(want), C.byref(rc.s), C.byref(rp.s))
        assert same(gpu, got, host_result(rt, want)), name
        assert (got._sf_degree, got._scaling_factor) == (want._sf_degree, want._scaling_factor)
        gpu.free_ciph(got)

    for name, arg in (("Upscale_ciph", 20), ("Mul_mono_ciph", 3 * N // 2), ("Mul_mono_ciph", 7),
                      ("Raise_mod", 0), ("Raise_mod", 4)):
        got, want = rt.CIPHERTEXT(), rt.CIPHERTEXT()
        getattr(lib, name)(C.byref(got), C.byref(ct), arg)
        getattr(rl, name).argtypes = [C.c_void_p, C.c_void_p, C.c_uint32]
        getattr(rl, name)(C.byref(want), C.byref(rc.s), arg)
        assert same(gpu, got, host_result(rt, want)), (name, arg)
        assert got._sf_degree == want._sf_degree
        gpu.free_ciph(got)

    lib.Modswitch_ciph(C.byref(ct))
    assert ct._c0_poly._num_primes == level - 1 and ct._c1_poly._num_primes == level - 1
    gpu.lib.Free_plain_data(C.byref(pt))
    gpu.free_ciph(ct)


def test_poly_arrays_views_and_precomp(pair):
    ref, gpu, rt = pair
    lib = gpu.lib
    arr = lib.Alloc_polys(3, N, 4, gpu.K)
    for i in range(3):
        assert (arr[i]._num_primes, arr[i]._num_primes_p, arr[i]._num_alloc_primes) == (4, gpu.K, 4 + gpu.K)
        assert np.count_nonzero(gpu.download(C.pointer(arr[i]))) == 0
    assert arr[1]._data - arr[0]._data == (4 + gpu.K) * N * 8
    lib.Free_polys(arr)

    a, b = gpu.new_poly(5), gpu.new_poly(3)
    res = rt.POLYNOMIAL()
    lib.Init_poly_by_opnd(C.byref(res), a, b, False)
    assert (res._num_primes, res._num_primes_p, res._is_ntt) == (3, 0, True)
    lib.Init_poly_by_opnd(C.byref(res), a, None, False)   # larger: reallocates
    assert res._num_primes == 5
    lib.Init_poly_by_opnd(C.byref(res), None, b, False)   # smaller: same storage, lower level
    assert res._num_primes == 3 and res._num_alloc_primes == 5
    lib.Free_poly_data(C.byref(res))

    views = (rt.POLYNOMIAL * gpu.dnum)()
    lib.Swk_c0(views, gpu.dnum, True, ROTS[0])
    for j in range(gpu.dnum):
        assert views[j]._data == lib.Pk0_at(lib.Swk(True, ROTS[0]), j).contents._data

    rng = np.random.default_rng(6)
    data = rr.uniform_limbs(rng, gpu.primes[:L], N)
    poly = gpu.new_poly(L, data=data)
    parts = lib.Num_decomp(poly)
    ext = lib.Alloc_polys(parts, N, L, gpu.K)
    lib.Precomp(ext, parts, poly)
    for j in range(parts):
        assert np.array_equal(gpu.download(C.pointer(ext[j])), ref.decomp_modup(data, j)), j
    lib.Free_polys(ext)
    for p in (a, b, poly):
        gpu.free(p)
