"""The plain-C oracle against the reference's own known-answer vectors
(tests/golden/reference_kats.json cites the unit test each one comes from)."""
import ctypes as C
import json
import os

import numpy as np

from tests import oracle_lib

KATS = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))
LIB = oracle_lib.load()


def test_ntt_n4_known_answer():
    k = KATS["ntt_n4"]
    n, q = k["degree"], k["modulus"]
    psi = LIB.Oracle_root_of_unity(2 * n, q)
    rou, inv = np.zeros(n, np.int64), np.zeros(n, np.int64)
    LIB.Oracle_make_tables(n, q, psi, rou.ctypes.data_as(C.c_void_p), inv.ctypes.data_as(C.c_void_p))
    x = np.array(k["coeffs"], np.int64)
    LIB.Oracle_ntt_tables(x.ctypes.data_as(C.c_void_p), n, q, rou.ctypes.data_as(C.c_void_p))
    assert x.tolist() == k["ntt"]
    n_inv = LIB.Oracle_inv_mod_prime(n, q)
    LIB.Oracle_intt_tables(x.ctypes.data_as(C.c_void_p), n, q, inv.ctypes.data_as(C.c_void_p), n_inv)
    assert x.tolist() == k["coeffs"]


def test_number_theory_known_answers():
    for a, e, m, want in KATS["mod_exp"]["cases"]:
        assert LIB.Oracle_pow_mod(a, e, m) == want
    for a, m, want in KATS["mod_inv_prime"]["cases"]:
        assert LIB.Oracle_inv_mod_prime(a, m) == want
    for a, m, want in KATS["mod_inv"]["cases"]:
        assert LIB.Oracle_inv_mod(a, m) == want
    for m, want in KATS["find_generator"]["cases"]:
        assert LIB.Oracle_find_generator(m) == want
    for order, m, want in KATS["root_of_unity"]["cases"]:
        assert LIB.Oracle_root_of_unity(order, m) == want
    for p in KATS["is_prime"]["primes"]:
        assert LIB.Oracle_is_prime(p) == 1
    for c in KATS["is_prime"]["composites"]:
        assert LIB.Oracle_is_prime(c) == 0
    k = KATS["precompute_const_128"]
    hi, lo = C.c_uint64(), C.c_uint64()
    LIB.Oracle_prec128(k["modulus"], C.byref(hi), C.byref(lo))
    assert (hi.value, lo.value) == (k["hi"], k["lo"])


def test_negacyclic_product_property():
    """NTT -> pointwise product -> INTT equals the schoolbook product mod x^N+1
    (the property unittest/ut_poly.cxx:54-109 checks through CRT reconstruction)."""
    orc = oracle_lib.Oracle(16, 3, 60, 56, 3)
    rng = np.random.default_rng(3)
    for idx in range(orc.L + orc.K):
        q = orc.primes[idx]
        a = rng.integers(0, q, 16, dtype=np.int64)
        b = rng.integers(0, q, 16, dtype=np.int64)
        want = [0] * 16
        for i in range(16):
            for j in range(16):
                s = int(a[i]) * int(b[j])
                k = i + j
                if k >= 16:
                    k -= 16
                    s = -s
                want[k] = (want[k] + s) % q
        prod = orc.hw(2, orc.ntt(idx, a), orc.ntt(idx, b), idx)
        assert orc.ntt(idx, prod, inverse=True).tolist() == want
    orc.close()
