"""Rescale without allocation.

Fhert_rescale_static serves hosts that cannot let the runtime allocate device
memory while they run (a CUDA graph being captured, a fixed memory budget): it
keeps its working storage in an array built into the library.  It must give
exactly the residues of the regular Rescale entry point, call after call,
because every call reuses the same storage.  This file is collected last so
that a failure here never hides another test.
"""
import ctypes as C

import numpy as np
import pytest

from tests import ref_runtime as rr

pytestmark = pytest.mark.gpu


def _uniform(rng, primes, n):
    return np.stack([rng.integers(0, p, size=n, dtype=np.int64) for p in primes])


def test_static_rescale_matches_rescale_twice():
    import ace_compiler_b200 as rt
    n, L = 65536, 6
    gpu = rt.Runtime(n, L, 60, 56, 3)
    lib = gpu.lib
    rng = np.random.default_rng(2024)
    try:
        assert lib.Fhert_rescale_static_capacity() >= L * n
        for call, level in enumerate((L, L - 1)):  # two calls in a row, different sizes
            data = _uniform(rng, gpu.primes[:level], n)
            src = gpu.new_poly(level, data=data)
            expect = gpu.new_poly(level)
            lib.Rescale(expect, src)
            want = gpu.download(expect)
            got_poly = gpu.new_poly(level)
            rc = lib.Fhert_rescale_static(gpu.limb_ptr(got_poly, 0), gpu.limb_ptr(src, 0), level)
            assert rc == 0, f"call {call}: status {rc}"
            got_poly.contents._num_primes = level - 1
            got = gpu.download(got_poly)
            assert np.array_equal(got, want), f"call {call} differs from Rescale"
            for p in (src, expect, got_poly):
                gpu.free(p)
        # sizes beyond the built-in storage, and malformed calls, are refused
        src = gpu.new_poly(2)
        assert lib.Fhert_rescale_static(gpu.limb_ptr(src, 0), gpu.limb_ptr(src, 0), 1) == 2
        assert lib.Fhert_rescale_static(gpu.limb_ptr(src, 0), gpu.limb_ptr(src, 0), L + 1) == 2
        gpu.free(src)
    finally:
        gpu.close()


def test_static_rescale_refuses_oversize():
    import ace_compiler_b200 as rt
    # 2^17 words per limb: 21 limbs would need more than the 40 * 65536 words built in
    gpu = rt.Runtime(131072, 21, 60, 56, 3)
    try:
        src = gpu.new_poly(21)
        rc = gpu.lib.Fhert_rescale_static(gpu.limb_ptr(src, 0), gpu.limb_ptr(src, 0), 21)
        assert rc == 3
        gpu.free(src)
    finally:
        gpu.close()


def test_static_rescale_against_reference_in_place_without_allocating():
    """The same residues as the reference Rescale (rns_poly.c:310-404), also when
    the result overwrites the source; no device memory is taken from the driver
    by the call; and the call refuses while earlier calls have deferred work
    waiting, since running that work allocates."""
    if not rr.available():
        pytest.skip("reference runtime not built")
    import torch

    import ace_compiler_b200 as rt
    n, L = 8192, 5
    ref = rr.RefRuntime(n, L, 60, 56, 3, seed=np.arange(16) + 5)
    gpu = rt.Runtime(n, L, 60, 56, 3)
    lib = gpu.lib
    rng = np.random.default_rng(77)
    try:
        data = _uniform(rng, gpu.primes[:L], n)
        want = ref.rescale(data)
        src = gpu.new_poly(L, data=data)
        lib.Fhert_sync()
        # first call on the device (address look-up), then the measured one
        assert lib.Fhert_rescale_static(gpu.limb_ptr(src, 0), gpu.limb_ptr(src, 0), L) == 0
        gpu.upload(src, data)
        lib.Fhert_sync()
        free_before = torch.cuda.mem_get_info()[0]
        assert lib.Fhert_rescale_static(gpu.limb_ptr(src, 0), gpu.limb_ptr(src, 0), L) == 0  # in place
        lib.Fhert_sync()
        assert torch.cuda.mem_get_info()[0] == free_before
        src.contents._num_primes = L - 1
        assert np.array_equal(gpu.download(src), want)
        # a recorded per-limb call is waiting: refused with code 5, nothing launched
        src.contents._num_primes = L
        gpu.upload(src, data)
        other = gpu.new_poly(1, data=data[:1])
        lib.Hw_modadd(gpu.limb_ptr(other, 0), gpu.limb_ptr(other, 0), gpu.limb_ptr(src, 0),
                      gpu.modulus(0), n)
        rc = lib.Fhert_rescale_static(gpu.limb_ptr(src, 0), gpu.limb_ptr(src, 0), L)
        assert rc == 5
        lib.Fhert_sync()  # runs the waiting call
        assert lib.Fhert_rescale_static(gpu.limb_ptr(src, 0), gpu.limb_ptr(src, 0), L) == 0
        src.contents._num_primes = L - 1
        assert np.array_equal(gpu.download(src), want)
        gpu.free(src)
        gpu.free(other)
    finally:
        gpu.close()
        rr.close_ref(ref)
