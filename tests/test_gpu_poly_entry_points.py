"""Polynomial-level entry points compared bit for bit with the reference
functions of the same name.  The reference functions are called through ctypes
on host structs of the same layout over numpy storage (Add_poly, Sub_poly,
Mul_poly: rns_poly.c:852-994; Dot_prod: rns_poly.c:516; Modswitch:
rns_poly.c:406; Swk_c0 / Swk_c1: ckks/key.h:90-124; Hw_modmuladd_scalar:
hal.c:109; Mod_down_rescale: rns_poly.c:531)."""
import ctypes as C

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

# one context with the ResNet programs' prime sizes (51 / 46 bits: the
# transforms then run without range correction), one with 60 / 56 bits
PARAM_SETS = {"n8192_51_46": (8192, 6, 51, 46, 3), "n16384_60_56": (16384, 5, 60, 56, 2)}
ROTS = (1, -2)


@pytest.fixture(scope="module", params=list(PARAM_SETS))
def pair(request):
    if not rr.available():
        pytest.skip("reference runtime not built")
    import ace_compiler_b200 as rt
    n, L, q0, sf, dnum = PARAM_SETS[request.param]
    ref = rr.RefRuntime(n, L, q0, sf, dnum, rot_idxs=ROTS, seed=np.arange(16) + 21)
    gpu = rt.Runtime(n, L, q0, sf, dnum, rot_idxs=ROTS)
    for is_rot, idx in [(False, 0)] + [(True, r) for r in ROTS]:
        for part in range(ref.dnum):
            for which in (0, 1):
                gpu.import_switch_key(is_rot, idx, part, which, ref.swk(is_rot, idx, part, which))
    yield ref, gpu, rt
    gpu.close()
    rr.close_ref(ref)


class HostPolys:
    """An array of reference-side POLYNOMIAL structs over numpy storage: `level`
    Q limbs followed directly by the special limbs when `extended`."""

    def __init__(self, rt, n, K, datas, level, extended=False, is_ntt=True):
        self.arr = (rt.POLYNOMIAL * len(datas))()
        self.keep = []
        for p, d in zip(self.arr, datas):
            a = np.ascontiguousarray(d, np.int64)
            self.keep.append(a)
            p._ring_degree, p._num_primes, p._num_alloc_primes = n, level, a.shape[0]
            p._num_primes_p = K if extended else 0
            p._is_ntt, p._data = is_ntt, a.ctypes.data

    def host(self, i=0):
        return self.keep[i]


def test_add_sub_mul_poly(pair):
    ref, gpu, rt = pair
    n, rng = gpu.N, np.random.default_rng(31)
    for level in sorted({gpu.L, 2}):
        a = rr.uniform_limbs(rng, gpu.primes[:level], n)
        b = rr.uniform_limbs(rng, gpu.primes[:level], n)
        a[:, 0] = [p - 1 for p in gpu.primes[:level]]
        b[:, 0] = [p - 1 for p in gpu.primes[:level]]
        a[:, 1] = 0
        pa, pb = gpu.new_poly(level, data=a), gpu.new_poly(level, data=b)
        for name in ("Add_poly", "Sub_poly", "Mul_poly"):
            out = gpu.new_poly(level)
            getattr(gpu.lib, name)(out, pa, pb)
            h = HostPolys(rt, n, gpu.K, [a.copy(), b.copy(), np.zeros_like(a)], level)
            f = getattr(ref.lib, name)
            f.argtypes, f.restype = [C.c_void_p] * 3, C.c_void_p
            f(C.byref(h.arr[2]), C.byref(h.arr[0]), C.byref(h.arr[1]))
            assert np.array_equal(gpu.download(out), h.host(2)), (name, level)
            gpu.free(out)
        gpu.free(pa)
        gpu.free(pb)


def test_modswitch(pair):
    ref, gpu, rt = pair
    n, rng, level = gpu.N, np.random.default_rng(32), gpu.L
    a = rr.uniform_limbs(rng, gpu.primes[:level], n)
    src = gpu.new_poly(level, data=a)
    out = gpu.new_poly(level - 1)
    gpu.lib.Modswitch(out, src)
    assert out.contents._num_primes == level - 1
    assert np.array_equal(gpu.download(out), a[: level - 1])
    gpu.lib.Modswitch(src, src)  # in place: only the level drops (rns_poly.c:406-414)
    assert src.contents._num_primes == level - 1
    assert np.array_equal(gpu.download(src), a[: level - 1])
    gpu.free(src)
    gpu.free(out)


def test_dot_prod(pair):
    ref, gpu, rt = pair
    n, K, rng = gpu.N, gpu.K, np.random.default_rng(33)
    for level in sorted({gpu.L, 2}):
        parts = ref.num_decomp(level)
        primes = gpu.primes[:level] + gpu.primes[gpu.L:]
        ext = [rr.uniform_limbs(rng, primes, n) for _ in range(parts)]
        # the second operand is a switch key: it keeps all L Q limbs, special limbs behind them
        key = [ref.swk(True, ROTS[0], j, 0) for j in range(parts)]
        d_ext = gpu.lib.Alloc_polys(parts, n, level, K)
        for j in range(parts):
            gpu.upload(C.pointer(d_ext[j]), ext[j])
            d_ext[j]._is_ntt = True
        views = (rt.POLYNOMIAL * gpu.dnum)()
        gpu.lib.Swk_c0(views, gpu.dnum, True, ROTS[0])
        out = gpu.new_poly(level, extended=True)
        gpu.lib.Dot_prod(out, d_ext, views, parts)
        h_ext = HostPolys(rt, n, K, ext, level, extended=True)
        h_key = HostPolys(rt, n, K, key, gpu.L, extended=True)
        h_out = HostPolys(rt, n, K, [np.zeros_like(ext[0])], level, extended=True)
        f = ref.lib.Dot_prod
        f.argtypes, f.restype = [C.c_void_p] * 3 + [C.c_uint32], C.c_void_p
        f(C.byref(h_out.arr[0]), h_ext.arr, h_key.arr, parts)
        assert np.array_equal(gpu.download(out), h_out.host(0)), level
        gpu.lib.Free_polys(d_ext)
        gpu.free(out)


def test_swk_views_hold_the_key_material(pair):
    ref, gpu, rt = pair
    for is_rot, idx in ((True, ROTS[1]), (False, 0)):
        for which, name in ((0, "Swk_c0"), (1, "Swk_c1")):
            views = (rt.POLYNOMIAL * gpu.dnum)()
            getattr(gpu.lib, name)(views, gpu.dnum, is_rot, idx)
            for j in range(gpu.dnum):
                assert views[j]._num_primes == gpu.L and views[j]._num_primes_p == gpu.K
                assert np.array_equal(gpu.download(C.pointer(views[j])),
                                      ref.swk(is_rot, idx, j, which)), (name, idx, j)


def test_hw_modmuladd_scalar(pair):
    ref, gpu, rt = pair
    n, rng = gpu.N, np.random.default_rng(34)
    f = ref.lib.Hw_modmuladd_scalar
    f.argtypes, f.restype = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_uint32], C.c_void_p
    for idx in (0, gpu.L - 1):
        q = gpu.primes[idx]
        acc = rr.uniform_limbs(rng, [q], n)
        a = rr.uniform_limbs(rng, [q], n)
        a[0, :2] = (q - 1, 0)
        for scalar in (q - 1, 12345, 0):
            want = acc.copy()
            f(want.ctypes.data, a.ctypes.data, scalar, ref.lib.Ref_modulus(idx), n)
            pa, pr = gpu.new_poly(1, data=a), gpu.new_poly(1, data=acc)
            gpu.lib.Hw_modmuladd_scalar(gpu.limb_ptr(pr, 0), gpu.limb_ptr(pa, 0), scalar,
                                        gpu.modulus(idx), n)
            assert np.array_equal(gpu.download(pr), want), (idx, scalar)
            gpu.free(pa)
            gpu.free(pr)


def test_mod_down_rescale(pair):
    ref, gpu, rt = pair
    n, K, rng = gpu.N, gpu.K, np.random.default_rng(35)
    f = ref.lib.Mod_down_rescale
    f.argtypes, f.restype = [C.c_void_p, C.c_void_p], C.c_void_p
    for level in sorted({gpu.L, 2}):
        primes = gpu.primes[:level] + gpu.primes[gpu.L:]
        data = rr.uniform_limbs(rng, primes, n)
        ext = gpu.new_poly(level, extended=True, data=data)
        out = gpu.new_poly(level)
        gpu.lib.Mod_down_rescale(out, ext)
        h_in = HostPolys(rt, n, K, [data.copy()], level, extended=True)
        h_out = HostPolys(rt, n, K, [np.zeros((level, n), np.int64)], level)
        f(C.byref(h_out.arr[0]), C.byref(h_in.arr[0]))
        assert out.contents._num_primes == h_out.arr[0]._num_primes == level - 1
        assert bool(out.contents._is_ntt) == bool(h_out.arr[0]._is_ntt)
        assert np.array_equal(gpu.download(out), h_out.host(0)[: level - 1]), level
        gpu.free(ext)
        gpu.free(out)


def test_rescale_in_coefficient_form(pair):
    """Rescale of an operand in coefficient form (rns_poly.c:381-399): the
    dropped limb is reduced without centring and the result stays in
    coefficient form; also in place and through Rescale_ciph."""
    ref, gpu, rt = pair
    n, K, rng = gpu.N, gpu.K, np.random.default_rng(37)
    f = ref.lib.Rescale
    f.argtypes, f.restype = [C.c_void_p, C.c_void_p], C.c_void_p
    for level in sorted({gpu.L, 2}):
        data = rr.uniform_limbs(rng, gpu.primes[:level], n)
        h_in = HostPolys(rt, n, K, [data.copy()], level, is_ntt=False)
        h_out = HostPolys(rt, n, K, [np.zeros((level, n), np.int64)], level, is_ntt=False)
        f(C.byref(h_out.arr[0]), C.byref(h_in.arr[0]))
        want = h_out.host(0)[: level - 1]
        assert h_out.arr[0]._num_primes == level - 1 and not h_out.arr[0]._is_ntt
        src = gpu.new_poly(level, data=data)
        src.contents._is_ntt = False
        out = gpu.new_poly(level)
        gpu.lib.Rescale(out, src)
        assert out.contents._num_primes == level - 1 and not out.contents._is_ntt
        assert np.array_equal(gpu.download(out), want), level
        gpu.lib.Rescale(src, src)          # in place
        assert src.contents._num_primes == level - 1 and not src.contents._is_ntt
        assert np.array_equal(gpu.download(src), want), level
        gpu.free(src)
        gpu.free(out)
    level = gpu.L
    c0 = rr.uniform_limbs(rng, gpu.primes[:level], n)
    c1 = rr.uniform_limbs(rng, gpu.primes[:level], n)
    wants = []
    for d in (c0, c1):
        h_in = HostPolys(rt, n, K, [d.copy()], level, is_ntt=False)
        h_out = HostPolys(rt, n, K, [np.zeros((level, n), np.int64)], level, is_ntt=False)
        f(C.byref(h_out.arr[0]), C.byref(h_in.arr[0]))
        wants.append(h_out.host(0)[: level - 1].copy())
    ct = gpu.new_ciph(c0, c1, sf_degree=2)
    ct._c0_poly._is_ntt = ct._c1_poly._is_ntt = False
    res = rt.CIPHERTEXT()
    gpu.lib.Rescale_ciph(C.byref(res), C.byref(ct))
    assert not res._c0_poly._is_ntt and not res._c1_poly._is_ntt
    assert res._c0_poly._num_primes == level - 1 and res._sf_degree == 1
    got0, got1 = gpu.ciph_to_host(res)
    assert np.array_equal(got0, wants[0]) and np.array_equal(got1, wants[1])
    gpu.free_ciph(ct)
    gpu.free_ciph(res)


def test_reduce_and_rescale_modup(pair):
    """ModDown, rescale and the raise of every digit in one call
    (rns_poly_impl.c:521-620): the raised digits (coefficient form), what is
    left in res, and the input left in coefficient form, against the reference."""
    ref, gpu, rt = pair
    n, K, rng = gpu.N, gpu.K, np.random.default_rng(39)

    class HostList(C.Structure):
        _fields_ = [("_type", C.c_int), ("_length", C.c_size_t), ("_p", C.POINTER(C.c_void_p))]

    f = ref.lib.Reduce_and_rescale_modup
    f.argtypes, f.restype = [C.c_void_p, C.c_void_p], C.POINTER(HostList)
    gpu.lib.Reduce_and_rescale_modup.restype = C.POINTER(HostList)
    for level in sorted({gpu.L, 2, max(2, gpu.alpha + 1)}):
        primes = gpu.primes[:level] + gpu.primes[gpu.L:]
        data = rr.uniform_limbs(rng, primes, n)
        h_in = HostPolys(rt, n, K, [data.copy()], level, extended=True)
        h_res = HostPolys(rt, n, K, [np.zeros((level, n), np.int64)], level)
        want = f(C.byref(h_res.arr[0]), C.byref(h_in.arr[0])).contents
        ext = gpu.new_poly(level, extended=True, data=data)
        res = gpu.new_poly(level)
        got = gpu.lib.Reduce_and_rescale_modup(res, ext).contents
        assert got._type == want._type and got._length == want._length >= 1
        for d in range(want._length):
            hp = C.cast(want._p[d], C.POINTER(rt.POLYNOMIAL)).contents
            gp = C.cast(got._p[d], rt.POLY)
            words = (hp._num_primes + hp._num_primes_p) * n
            host = np.ctypeslib.as_array(C.cast(hp._data, C.POINTER(C.c_int64)), (words,)).reshape(-1, n)
            assert (gp.contents._num_primes, gp.contents._num_primes_p) == (hp._num_primes, hp._num_primes_p)
            assert bool(gp.contents._is_ntt) == bool(hp._is_ntt) is False
            assert np.array_equal(gpu.download(gp), host), (level, d)
        assert res.contents._num_primes == h_res.arr[0]._num_primes == level - 1
        assert np.array_equal(gpu.download(res), h_res.host(0)[: level - 1])
        assert not ext.contents._is_ntt and not h_in.arr[0]._is_ntt
        assert np.array_equal(gpu.download(ext), h_in.host(0))
        gpu.lib.Free_precomp(C.cast(C.pointer(got), C.c_void_p))
        gpu.free(ext)
        gpu.free(res)


def test_out_of_place_conversions(pair):
    """Conv_poly2ntt (rns_poly.c:637) and Conv_ntt2poly (rns_poly_impl.c:202)
    against the reference functions on an extended polynomial: Q and special
    limbs, the source untouched."""
    ref, gpu, rt = pair
    n, K, L, rng = gpu.N, gpu.K, gpu.L, np.random.default_rng(38)
    data = rr.uniform_limbs(rng, gpu.primes, n)
    marker = rr.uniform_limbs(rng, gpu.primes, n)       # what res holds before the call
    for name, src_ntt in (("Conv_poly2ntt", False), ("Conv_ntt2poly", True)):
        f = getattr(ref.lib, name)
        f.argtypes, f.restype = [C.c_void_p, C.c_void_p], None
        h_in = HostPolys(rt, n, K, [data.copy()], L, extended=True, is_ntt=src_ntt)
        h_out = HostPolys(rt, n, K, [marker.copy()], L, extended=True, is_ntt=src_ntt)
        f(C.byref(h_out.arr[0]), C.byref(h_in.arr[0]))
        src = gpu.new_poly(L, extended=True, data=data, is_ntt=src_ntt)
        out = gpu.new_poly(L, extended=True, data=marker, is_ntt=src_ntt)
        getattr(gpu.lib, name)(out, src)
        assert bool(out.contents._is_ntt) == bool(h_out.arr[0]._is_ntt) == (not src_ntt)
        assert np.array_equal(gpu.download(out), h_out.host(0)), name
        assert np.array_equal(gpu.download(src), data)      # the source is untouched
        gpu.free(src)
        gpu.free(out)


def test_lpoly_interface(pair):
    """The single-limb interface of the LPOLY emit target (lpoly/poly.h:116-143)
    against the reference functions of the same names: every operation on the
    first and on the last prime (a special one), operands by value."""
    ref, gpu, rt = pair
    n, rng = gpu.N, np.random.default_rng(36)

    class HostLpoly(C.Structure):
        _fields_ = [("_ring_degree", C.c_uint32), ("_is_ntt", C.c_bool), ("_data", C.c_void_p)]

    def host(a, is_ntt):
        keep = np.ascontiguousarray(a, np.int64)
        return HostLpoly(n, is_ntt, keep.ctypes.data), keep

    def dev(a, is_ntt):
        p = rt.L_POLY()
        gpu.lib.Alloc_lpoly_data(C.byref(p), n)
        tmp = gpu.new_poly(1, data=a.reshape(1, n))
        gpu.lib.Copy_lpoly(C.byref(p), rt.L_POLY(n, is_ntt, tmp.contents._data))
        gpu.free(tmp)
        return p

    def down(p):
        tmp = gpu.new_poly(1)
        view = rt.L_POLY(n, False, tmp.contents._data)
        gpu.lib.Copy_lpoly(C.byref(view), p)
        out = gpu.download(tmp)[0]
        gpu.free(tmp)
        return out

    for idx in (0, gpu.L + gpu.K - 1):
        q = gpu.primes[idx]
        a = rng.integers(0, q, n, dtype=np.int64)
        b = rng.integers(0, q, n, dtype=np.int64)
        a[:2], b[:2] = (q - 1, 0), (q - 1, q - 1)
        mod_ref, mod_gpu = ref.lib.Ref_modulus(idx), gpu.modulus(idx)
        for name, scalar in (("Add_lpoly", None), ("Sub_lpoly", None), ("Mul_lpoly", None),
                             ("Mac_lpoly", None), ("Add_scalar", 12345), ("Sub_scalar", 777),
                             ("Mul_scalar", q - 2), ("Mac_scalar", 99)):
            res0 = rng.integers(0, q, n, dtype=np.int64)
            hr, keep_r = host(res0.copy(), True)
            ha, _ka = host(a, True)
            hb, _kb = host(b, True)
            f = getattr(ref.lib, name)
            f.restype = C.c_void_p
            dr, da, db = dev(res0, True), dev(a, True), dev(b, True)
            if scalar is None:
                f.argtypes = [C.c_void_p, HostLpoly, HostLpoly, C.c_void_p]
                f(C.byref(hr), ha, hb, mod_ref)
                getattr(gpu.lib, name)(C.byref(dr), da, db, mod_gpu)
            else:
                f.argtypes = [C.c_void_p, HostLpoly, C.c_int64, C.c_void_p]
                f(C.byref(hr), ha, scalar, mod_ref)
                getattr(gpu.lib, name)(C.byref(dr), da, scalar, mod_gpu)
            assert np.array_equal(down(dr), keep_r), (name, idx)
            assert bool(dr._is_ntt) == bool(hr._is_ntt)
            for p in (dr, da, db):
                gpu.lib.Free_lpoly_data(C.byref(p))
        # transforms: coefficient form -> NTT -> back
        hc, keep_c = host(a.copy(), False)
        hn, keep_n = host(np.zeros(n, np.int64), False)
        for fn in (ref.lib.Ntt, ref.lib.Intt):
            fn.argtypes, fn.restype = [C.c_void_p, HostLpoly, C.c_size_t], None
        ref.lib.Ntt(C.byref(hn), hc, idx)
        dc, dn = dev(a, False), dev(np.zeros(n, np.int64), False)
        gpu.lib.Ntt(C.byref(dn), dc, idx)
        assert dn._is_ntt and np.array_equal(down(dn), keep_n), idx
        gpu.lib.Intt(C.byref(dc), dn, idx)
        assert not dc._is_ntt and np.array_equal(down(dc), a), idx
        for p in (dc, dn):
            gpu.lib.Free_lpoly_data(C.byref(p))
    heap = gpu.lib.Alloc_lpoly(n)
    assert heap.contents._is_ntt and heap.contents._ring_degree == n
    assert np.count_nonzero(down(heap.contents)) == 0
    gpu.lib.Free_lpoly(heap)
