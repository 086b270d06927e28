"""Key generation, encode, encrypt, decrypt and decode against the reference
CPU runtime with the same generator seed and the same clock value: keys,
plaintexts and ciphertexts must be bit-identical, decoded values identical as
IEEE doubles."""
import ctypes as C

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

SEED = (np.arange(16, dtype=np.uint64) * 2654435761 % (2 ** 32)).astype(np.uint32)
FAKE_US = 1_700_000_000_123_456
PARAMS = {"n1024": (1024, 5, 60, 56, 2, (1, -3, 5)), "n16384": (16384, 7, 60, 56, 3, (2, 64))}


@pytest.fixture(scope="module", params=list(PARAMS))
def pair(request):
    if not rr.available():
        pytest.skip("reference runtime not built")
    import ace_compiler_b200 as rt
    n, L, q0, sf, dnum, rots = PARAMS[request.param]
    ref = rr.RefRuntime(n, L, q0, sf, dnum, rot_idxs=rots, seed=SEED, fake_time_us=FAKE_US)
    gpu = rt.Runtime(n, L, q0, sf, dnum, rot_idxs=rots, keygen=True, seed=SEED, fake_time_us=FAKE_US)
    yield ref, gpu, rots
    gpu.close()
    rr.close_ref(ref)


def test_keys_are_identical(pair):
    ref, gpu, rots = pair
    for which in range(4):
        assert np.array_equal(gpu.export_key(which), ref.export_key(which)), f"key part {which}"
    for is_rot, idx in [(False, 0)] + [(True, r) for r in rots]:
        for part in range(ref.dnum):
            for which in (0, 1):
                assert np.array_equal(gpu.export_switch_key(is_rot, idx, part, which),
                                      ref.swk(is_rot, idx, part, which)), (is_rot, idx, part, which)


def test_encode_matches(pair):
    ref, gpu, _ = pair
    rng = np.random.default_rng(41)
    slots = gpu.N // 2
    cases = [rng.uniform(-1, 1, slots) + 1j * rng.uniform(-1, 1, slots),
             rng.uniform(-1, 1, 10).astype(np.complex128),
             np.zeros(slots, np.complex128)]
    for values in cases:
        for sf_degree, level in ((1, 0), (2, gpu.L), (1, 2)):
            pt = gpu.encode(values, sf_degree, level)
            got = gpu.download(C.pointer(pt._poly))
            assert np.array_equal(got, ref.encode(values, sf_degree, level)), (len(values), sf_degree, level)
            gpu.lib.Free_plain_data(C.byref(pt))
    for value in (0.5, -1.25, 3.0e-5, 1234.5):
        pt = gpu.encode_scalar(value, 1, 3)
        assert np.array_equal(gpu.download(C.pointer(pt._poly)), ref.encode_scalar(value, 1, 3))
        gpu.lib.Free_plain_data(C.byref(pt))


def test_encrypt_decrypt_decode(pair):
    ref, gpu, rots = pair
    rng = np.random.default_rng(42)
    slots = gpu.N // 2
    values = rng.uniform(-1, 1, slots) + 1j * rng.uniform(-1, 1, slots)
    pt = gpu.encode(values, 1, gpu.L)
    plain_host = gpu.download(C.pointer(pt._poly))
    ct = gpu.encrypt(pt)
    g0, g1 = gpu.ciph_to_host(ct)
    e0, e1 = ref.encrypt(plain_host, 1)
    assert np.array_equal(g0, e0) and np.array_equal(g1, e1)
    got = gpu.decrypt_decode(ct)
    want = ref.decrypt_decode(e0, e1, 1)
    assert np.array_equal(got.view(np.float64), want.view(np.float64))
    assert np.max(np.abs(got - values)) < 1e-6
    # homomorphic rotation with our own keys decrypts to the rotated slots
    import ace_compiler_b200 as rt
    out = rt.CIPHERTEXT()
    gpu.lib.Rotate_ciph(C.byref(out), C.byref(ct), rots[0])
    rot = gpu.decrypt_decode(out)
    assert np.max(np.abs(rot - np.roll(values, -rots[0]))) < 1e-5
    gpu.free_ciph(out)
    gpu.free_ciph(ct)
    gpu.lib.Free_plain_data(C.byref(pt))
