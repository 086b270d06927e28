"""Pt_from_msg / Pt_from_msg_ofst / Free_data on a synthetic weight file:
plaintext residues must equal the reference runtime's for the same file, with
and without the device plaintext cache."""
import ctypes as C
import os

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu

N, L = 2048, 6


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    if not rr.available():
        pytest.skip("reference runtime not built")
    import ace_compiler_b200 as rt
    from ace_compiler_b200.msgfile import write_msg_file
    rng = np.random.default_rng(7)
    entries = [("w0", rng.normal(0, 0.3, 1024).astype(np.float32), 1, 0),
               ("w1", rng.normal(0, 0.3, 4096).astype(np.float32), 1, 4),
               ("b0", rng.normal(0, 0.3, 10).astype(np.float32), 2, 3),
               ("s0", np.array([0.75], np.float32), 1, 2)]
    path = str(tmp_path_factory.mktemp("msg") / "weights.msg")
    write_msg_file(path, entries)
    ref = rr.RefRuntime(N, L, 60, 56, 2)
    ref.lib.Pt_mgr_init.argtypes = [C.c_char_p]
    ref.lib.Pt_mgr_init.restype = C.c_bool
    ref.lib.Pt_from_msg.argtypes = [C.c_void_p, C.c_uint32, C.c_size_t, C.c_uint32, C.c_uint32]
    ref.lib.Pt_from_msg_ofst.argtypes = [C.c_void_p, C.c_uint32, C.c_size_t, C.c_size_t,
                                         C.c_uint32, C.c_uint32]
    assert ref.lib.Pt_mgr_init(path.encode())
    gpu = rt.Runtime(N, L, 60, 56, 2)
    yield ref, gpu, rt, path
    gpu.close()
    rr.close_ref(ref)


def ref_plain(ref, rt, index, ofst, length, scale, level):
    pt = rt.PLAINTEXT()
    if ofst is None:
        ref.lib.Pt_from_msg(C.byref(pt), index, length, scale, level)
    else:
        ref.lib.Pt_from_msg_ofst(C.byref(pt), index, ofst, length, scale, level)
    limbs = pt._poly._num_primes
    host = (C.c_int64 * (limbs * N)).from_address(pt._poly._data)
    data = np.frombuffer(host, dtype=np.int64).reshape(limbs, N).copy()
    return data, pt._slots, pt._scaling_factor, pt._sf_degree


CASES = [(0, None, 1024, 1, 0), (1, None, 1024, 1, 4), (1, 1024, 1024, 1, 4), (1, 3072, 512, 2, 5),
         (2, None, 10, 2, 3), (3, None, 1, 1, 2)]


@pytest.mark.parametrize("cache_mb", [0, 64])
def test_plaintexts_from_data_file(setup, cache_mb):
    ref, gpu, rt, path = setup
    os.environ["FHERT_PT_CACHE_MB"] = str(cache_mb)
    try:
        assert gpu.lib.Pt_mgr_init(path.encode())
        for rounds in range(2):  # the second pass is served from the cache when it is on
            for index, ofst, length, scale, level in CASES:
                pt = rt.PLAINTEXT()
                if ofst is None:
                    gpu.lib.Pt_from_msg(C.byref(pt), index, length, scale, level)
                else:
                    gpu.lib.Pt_from_msg_ofst(C.byref(pt), index, ofst, length, scale, level)
                want, slots, sf, deg = ref_plain(ref, rt, index, ofst, length, scale, level)
                got = gpu.download(C.pointer(pt._poly))
                assert np.array_equal(got, want), (index, ofst, length, scale, level)
                assert (pt._slots, pt._scaling_factor, pt._sf_degree) == (slots, sf, deg)
                gpu.lib.Free_data(C.byref(pt._poly))
                assert not pt._poly._data
        stats = [C.c_size_t() for _ in range(4)]
        gpu.lib.Fhert_pt_cache_stats(*[C.byref(s) for s in stats])
        entries, _, hits, misses = [s.value for s in stats]
        if cache_mb:
            assert (entries, hits, misses) == (len(CASES), len(CASES), len(CASES))
            # bypass: encoded afresh (the plaintext owns its limbs), the cache untouched
            gpu.lib.Fhert_pt_cache_bypass(1)
            index, ofst, length, scale, level = CASES[1]
            pt = rt.PLAINTEXT()
            gpu.lib.Pt_from_msg(C.byref(pt), index, length, scale, level)   # cached view first
            gpu.lib.Fhert_pt_cache_bypass(0)
            gpu.lib.Pt_from_msg(C.byref(pt), index, length, scale, level)
            gpu.lib.Fhert_pt_cache_bypass(1)
            gpu.lib.Pt_from_msg(C.byref(pt), index, length, scale, level)   # replaces the view
            want = ref_plain(ref, rt, index, ofst, length, scale, level)[0]
            assert np.array_equal(gpu.download(C.pointer(pt._poly)), want)
            gpu.lib.Free_data(C.byref(pt._poly))
            gpu.lib.Fhert_pt_cache_bypass(0)
            gpu.lib.Fhert_pt_cache_stats(*[C.byref(s) for s in stats])
            assert [s.value for s in stats][0] == len(CASES)
            assert [s.value for s in stats][2] == len(CASES) + 1
        else:
            assert (entries, hits) == (0, 0)
    finally:
        gpu.lib.Pt_mgr_fini()
        os.environ.pop("FHERT_PT_CACHE_MB", None)


def test_pre_encoded_plaintext_file(setup, tmp_path):
    """A DE_PLAINTEXT data file whose entries the reference's offline encoder
    entry point (Encode_plain_buffer, ckks/src/plain.c:196-217) produced:
    Pt_from_msg hands out those residues (uploaded once), Free_data leaves them."""
    from ace_compiler_b200.msgfile import write_plaintext_file
    ref, gpu, rt, _ = setup
    rng = np.random.default_rng(8)
    enc = ref.lib.Encode_plain_buffer
    enc.argtypes, enc.restype = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32], C.c_void_p
    cases = [(1024, 1, 4), (10, 2, 3), (512, 1, L)]
    buffers, want = [], []
    for k, (length, scale, level) in enumerate(cases):
        vals = np.ascontiguousarray(rng.normal(0, 0.3, length).astype(np.float32))
        buf = enc(vals.ctypes.data, length, scale, level)
        size = C.c_uint32.from_address(buf + 12).value
        raw = C.string_at(buf, 16 + size)
        assert raw[:8] == b"ANTPLAIN"
        buffers.append((f"p{k}", raw, scale, level))
        head = C.sizeof(rt.PLAINTEXT)
        want.append(np.frombuffer(raw[16 + head:16 + head + level * N * 8], dtype=np.int64)
                    .reshape(level, N).copy())
    path = str(tmp_path / "weights.pt")
    write_plaintext_file(path, buffers)
    try:
        assert gpu.lib.Pt_mgr_init(path.encode())
        for rounds in range(2):
            for k, (length, scale, level) in enumerate(cases):
                pt = rt.PLAINTEXT()
                gpu.lib.Pt_from_msg(C.byref(pt), k, length, scale, level)
                assert pt._poly._num_primes == level and pt._sf_degree == scale
                assert np.array_equal(gpu.download(C.pointer(pt._poly)), want[k]), k
                gpu.lib.Free_data(C.byref(pt._poly))
        stats = [C.c_size_t() for _ in range(4)]
        gpu.lib.Fhert_pt_cache_stats(*[C.byref(s) for s in stats])
        assert [s.value for s in stats][0] == len(cases) and [s.value for s in stats][2] == len(cases)
    finally:
        gpu.lib.Pt_mgr_fini()
