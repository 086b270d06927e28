"""Bootstrapping against the reference CPU runtime with the same generator
seed: the linear-transform plaintexts, the bootstrap keys and the refreshed
ciphertext must be bit-identical, and the refreshed message must agree with the
original to the precision the reference's own test accepts."""
import ctypes as C
import os

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

SEED = (np.arange(16, dtype=np.uint64) * 40503 % (2 ** 32)).astype(np.uint32)
FAKE_US = 1_700_000_000_654_321
# ring degree, limbs: 2048 has a remainder stage in the collapsed FFT
# (10 = 4 + 4 + 2 layers), 8192 splits evenly; 65536 with 32768 slots is the
# size the compiled networks and the bootstrap benchmark run at (5 collapsed
# layers per stage, 16 giant x 4 baby steps; the reference side takes a few
# minutes of host time there)
PARAMS = {"n2048": (2048, 19), "n8192": (8192, 18), "n65536": (65536, 18)}


@pytest.fixture(scope="module", params=list(PARAMS))
def pair(request):
    if not rr.available():
        pytest.skip("reference runtime not built")
    import ace_compiler_b200 as rt
    n, L = PARAMS[request.param]
    old = os.environ.get("RTLIB_DISABLE_BOOTSTRAP_PRECOM")
    os.environ["RTLIB_DISABLE_BOOTSTRAP_PRECOM"] = "0"
    try:
        ref = rr.RefRuntime(n, L, 60, 56, 3, seed=SEED, fake_time_us=FAKE_US)
        gpu = rt.Runtime(n, L, 60, 56, 3, keygen=True, seed=SEED, fake_time_us=FAKE_US)
    finally:
        if old is None:
            os.environ.pop("RTLIB_DISABLE_BOOTSTRAP_PRECOM", None)
        else:
            os.environ["RTLIB_DISABLE_BOOTSTRAP_PRECOM"] = old
    lib = ref.lib
    lib.Ref_bootstrap.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32,
                                  C.c_void_p, C.c_void_p]
    lib.Ref_bootstrap.restype = C.c_size_t
    lib.Ref_bootstrap_plain.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_void_p]
    lib.Ref_bootstrap_plain.restype = C.c_size_t
    lib.Ref_encode_slots.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32,
                                     C.c_void_p]
    if n <= 8192:
        # sparse packing (N/8 slots): its transforms and rotation keys are made now,
        # while both generators are still in step (the tests below encrypt on the
        # reference side only)
        lib.Bootstrap_precom.argtypes = [C.c_uint32]
        lib.Bootstrap_precom(n // 8)
        gpu.lib.Bootstrap_precom(n // 8)
    yield ref, gpu
    gpu.close()
    rr.close_ref(ref)


def test_transform_plaintexts_are_identical(pair):
    ref, gpu = pair
    n, limbs = gpu.N, gpu.L + gpu.K
    want = np.zeros((limbs, n), np.int64)
    got = np.zeros((limbs, n), np.int64)
    seen = 0
    for encoding in (1, 0):
        for stage in range(3):
            for index in range(64):
                lr = ref.lib.Ref_bootstrap_plain(encoding, stage, index, rr._p(want))
                lg = gpu.lib.Fhert_export_bootstrap_plain(0, encoding, stage, index, rr._p(got))
                assert lr == lg, (encoding, stage, index)
                if lr == 0:
                    continue
                seen += 1
                rows = lr + gpu.K
                assert np.array_equal(got[:rows], want[:rows]), (encoding, stage, index)
    assert seen > 30


def test_bootstrap_keys_are_identical(pair):
    ref, gpu = pair
    conj = 2 * gpu.N - 1
    rots = (C.c_int32 * 512)()
    count = gpu.lib.Fhert_bootstrap_rotations(0, rots, 512)
    assert 8 < count <= 512
    picked = [rots[0], rots[count // 2], rots[count - 1], conj]
    for rot in picked:
        for part in range(ref.dnum):
            for which in (0, 1):
                assert np.array_equal(gpu.export_switch_key(True, rot, part, which),
                                      ref.swk(True, rot, part, which)), (rot, part, which)


def test_conjugate_matches_reference(pair):
    """Conjugate_ciph (cipher.c:481) against the reference function of the same
    name on host structs; both sides hold the conjugation key of the bootstrap
    key set."""
    import ace_compiler_b200 as rt
    ref, gpu = pair
    n = gpu.N
    rng = np.random.default_rng(8)
    level = 3
    c0 = rr.uniform_limbs(rng, gpu.primes[:level], n)
    c1 = rr.uniform_limbs(rng, gpu.primes[:level], n)
    ct = gpu.new_ciph(c0, c1)
    got = rt.CIPHERTEXT()
    gpu.lib.Conjugate_ciph(C.byref(got), C.byref(ct))
    g0, g1 = gpu.ciph_to_host(got)
    keep = [np.ascontiguousarray(c0), np.ascontiguousarray(c1)]
    h, want = rt.CIPHERTEXT(), rt.CIPHERTEXT()
    for p, a in zip((h._c0_poly, h._c1_poly), keep):
        p._ring_degree, p._num_primes, p._num_alloc_primes = n, level, level
        p._num_primes_p, p._is_ntt, p._data = 0, True, a.ctypes.data
    h._slots, h._scaling_factor, h._sf_degree = n // 2, 2.0 ** 56, 1
    f = ref.lib.Conjugate_ciph
    f.argtypes, f.restype = [C.c_void_p, C.c_void_p], C.c_void_p
    f(C.byref(want), C.byref(h))
    for g, p in ((g0, want._c0_poly), (g1, want._c1_poly)):
        assert p._num_primes == level
        buf = (C.c_int64 * (level * n)).from_address(p._data)
        assert np.array_equal(g, np.frombuffer(buf, dtype=np.int64).reshape(level, n))
    gpu.free_ciph(ct)
    gpu.free_ciph(got)


def test_bootstrap_matches_reference(pair):
    ref, gpu = pair
    n, L = gpu.N, gpu.L
    rng = np.random.default_rng(5)
    values = rng.uniform(-1, 1, n // 2) + 0j
    level_in = 2
    pt_ref = ref.encode(values, 1, level_in)
    c0, c1 = ref.encrypt(pt_ref)
    out0 = np.zeros((L, n), np.int64)
    out1 = np.zeros((L, n), np.int64)
    out_level = ref.lib.Ref_bootstrap(rr._p(c0), rr._p(c1), level_in, n // 2, 0, rr._p(out0), rr._p(out1))
    assert out_level >= 2

    ct = gpu.new_ciph(c0, c1)
    res = type(ct)()
    gpu.lib.Bootstrap(C.byref(res), C.byref(ct), 0)
    g0, g1 = gpu.ciph_to_host(res)
    assert g0.shape[0] == out_level
    assert np.array_equal(g0, out0[:out_level])
    assert np.array_equal(g1, out1[:out_level])
    assert res._sf_degree == 1

    refreshed = gpu.decrypt_decode(res)
    assert np.max(np.abs(refreshed.real - values.real)) < 1e-2
    gpu.free_ciph(ct)
    gpu.free_ciph(res)


def _host_ct(rt, n, c0, c1, slots, sf_bits=56):
    keep = [np.ascontiguousarray(c0), np.ascontiguousarray(c1)]
    h = rt.CIPHERTEXT()
    for p, a in zip((h._c0_poly, h._c1_poly), keep):
        p._ring_degree, p._num_primes, p._num_alloc_primes = n, a.shape[0], a.shape[0]
        p._num_primes_p, p._is_ntt, p._data = 0, True, a.ctypes.data
    h._slots, h._scaling_factor, h._sf_degree = slots, 2.0 ** sf_bits, 1
    return h, keep


def _host_limbs(ct, n):
    out = []
    for p in (ct._c0_poly, ct._c1_poly):
        buf = (C.c_int64 * (p._num_primes * n)).from_address(p._data)
        out.append(np.frombuffer(buf, dtype=np.int64).reshape(p._num_primes, n).copy())
    return out


def test_sparse_bootstrap_matches_reference(pair):
    """N/8 slots: partial sums before CoeffsToSlots, one EvalMod, rotate-and-add
    after SlotsToCoeffs (bootstrap.c:1728-1793)."""
    ref, gpu = pair
    n, L = gpu.N, gpu.L
    if n > 8192:
        pytest.skip("sparse packing is covered at the smaller ring degrees")
    slots = n // 8
    rng = np.random.default_rng(9)
    values = np.ascontiguousarray(rng.uniform(-1, 1, slots) + 0j)
    level_in = 2
    pt = np.zeros((level_in, n), np.int64)
    ref.lib.Ref_encode_slots(rr._p(values.view(np.float64)), slots, slots, 1, level_in, rr._p(pt))
    c0, c1 = ref.encrypt(pt)
    out0, out1 = np.zeros((L, n), np.int64), np.zeros((L, n), np.int64)
    out_level = ref.lib.Ref_bootstrap(rr._p(c0), rr._p(c1), level_in, slots, 0, rr._p(out0), rr._p(out1))
    ct = gpu.new_ciph(c0, c1)
    ct._slots = slots
    res = type(ct)()
    gpu.lib.Bootstrap(C.byref(res), C.byref(ct), 0)
    g0, g1 = gpu.ciph_to_host(res)
    assert g0.shape[0] == out_level
    assert np.array_equal(g0, out0[:out_level]) and np.array_equal(g1, out1[:out_level])
    gpu.free_ciph(ct)
    gpu.free_ciph(res)


def test_staged_bootstrap_matches_reference(pair):
    """Eval_bootstrap_coeffs_to_slots_ciph / _eval_mod_ciph / _slots_to_coeffs_ciph
    (cipher.c:585-767) stage by stage against the reference functions of the same
    names, fully packed."""
    import ace_compiler_b200 as rt
    ref, gpu = pair
    n = gpu.N
    if n > 8192:
        pytest.skip("the stages are covered at the smaller ring degrees")
    rng = np.random.default_rng(10)
    values = rng.uniform(-1, 1, n // 2) + 0j
    c0, c1 = ref.encrypt(ref.encode(values, 1, 2))
    h, keep = _host_ct(rt, n, c0, c1, n // 2)
    ct = gpu.new_ciph(c0, c1)
    names = ("Eval_bootstrap_coeffs_to_slots_ciph", "Eval_bootstrap_eval_mod_ciph",
             "Eval_bootstrap_slots_to_coeffs_ciph")
    r_in, g_in = h, ct
    held = []
    for name in names:
        f = getattr(ref.lib, name)
        f.argtypes, f.restype = [C.c_void_p, C.c_void_p, C.c_uint32], C.c_void_p
        r_out, g_out = rt.CIPHERTEXT(), rt.CIPHERTEXT()
        f(C.byref(r_out), C.byref(r_in), n // 2)
        getattr(gpu.lib, name)(C.byref(g_out), C.byref(g_in), n // 2)
        want = _host_limbs(r_out, n)
        got = gpu.ciph_to_host(g_out)
        assert got[0].shape == want[0].shape, name
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]), name
        assert (g_out._sf_degree, g_out._slots) == (r_out._sf_degree, r_out._slots), name
        held.append(g_out)
        r_in, g_in = r_out, g_out
    refreshed = gpu.decrypt_decode(g_in)
    assert np.max(np.abs(refreshed.real - values.real)) < 1e-2
    gpu.free_ciph(ct)
    for g in held:
        gpu.free_ciph(g)
