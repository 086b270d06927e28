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
