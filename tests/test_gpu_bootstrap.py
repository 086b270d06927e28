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
# (10 = 4 + 4 + 2 layers), 8192 splits evenly like 65536 does
PARAMS = {"n2048": (2048, 19), "n8192": (8192, 18)}


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
