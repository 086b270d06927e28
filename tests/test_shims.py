"""Stand-ins used to build the reference runtime: the big-integer subset
against Python integers, keyed BLAKE2b against hashlib."""
import ctypes as C
import hashlib
import os
import random
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "libshims.so")


def shims():
    if not os.path.exists(LIB):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    return C.CDLL(LIB)


class MPZ(C.Structure):
    _fields_ = [("alloc", C.c_int), ("size", C.c_int), ("d", C.POINTER(C.c_uint32))]


def test_bigint_against_python_integers():
    L = shims()
    L.mpz_get_d.restype = C.c_double
    L.mpz_sizeinbase.restype = C.c_size_t
    for f in ("mpz_mul_2exp", "mpz_fdiv_q_2exp"):
        getattr(L, f).argtypes = [C.c_void_p, C.c_void_p, C.c_ulong]

    def new(v):
        m = MPZ()
        L.mpz_init(C.byref(m))
        assert L.mpz_set_str(C.byref(m), str(v).encode(), 10) == 0
        return m

    def val(m):
        v = sum(m.d[i] << (32 * i) for i in range(abs(m.size)))
        return -v if m.size < 0 else v

    rnd = random.Random(5)
    for _ in range(3000):
        bits_a, bits_b = rnd.choice([1, 31, 32, 33, 64, 65, 200, 900, 2300]), rnd.choice([1, 32, 63, 64, 130, 700])
        a = rnd.getrandbits(bits_a) * rnd.choice([1, -1])
        b = rnd.getrandbits(bits_b) * rnd.choice([1, -1])
        A, B, R = new(a), new(b), new(0)
        L.mpz_add(C.byref(R), C.byref(A), C.byref(B)); assert val(R) == a + b
        L.mpz_sub(C.byref(R), C.byref(A), C.byref(B)); assert val(R) == a - b
        L.mpz_mul(C.byref(R), C.byref(A), C.byref(B)); assert val(R) == a * b
        if b:
            L.mpz_fdiv_q(C.byref(R), C.byref(A), C.byref(B)); assert val(R) == a // b
            L.mpz_fdiv_r(C.byref(R), C.byref(A), C.byref(B)); assert val(R) == a % b
        s = rnd.randrange(0, 150)
        L.mpz_mul_2exp(C.byref(R), C.byref(A), s); assert val(R) == a << s
        L.mpz_fdiv_q_2exp(C.byref(R), C.byref(A), s); assert val(R) == a >> s
        if a:
            assert L.mpz_sizeinbase(C.byref(A), 2) == abs(a).bit_length()
        t = abs(a)
        if t.bit_length() > 53:
            t = (t >> (t.bit_length() - 53)) << (t.bit_length() - 53)
        if t.bit_length() < 1000:
            assert L.mpz_get_d(C.byref(A)) == (float(t) if a >= 0 else -float(t))
        for m in (A, B, R):
            L.mpz_clear(C.byref(m))


def test_blake2b_against_hashlib():
    L = shims()
    rnd = random.Random(6)
    for _ in range(300):
        n, k, o = rnd.choice([0, 1, 8, 64, 127, 128, 129, 500]), rnd.choice([0, 16, 64]), rnd.choice([1, 32, 64])
        msg, key = rnd.randbytes(n), rnd.randbytes(k)
        out = C.create_string_buffer(o)
        assert L.blake2b(out, C.c_size_t(o), msg, C.c_size_t(n), key, C.c_size_t(k)) == 0
        assert out.raw == hashlib.blake2b(msg, digest_size=o, key=key).digest()


def test_blake2xb_is_deterministic_and_length_bound():
    """No independent implementation is available for the XOF layering; check the
    properties the specification gives: determinism, and that outputs of different
    requested lengths are unrelated (the length is hashed into the root)."""
    L = shims()
    a, b, c = (C.create_string_buffer(n) for n in (4096, 4096, 128))
    key = bytes(range(64))
    for buf in (a, b, c):
        assert L.blake2xb(buf, C.c_size_t(len(buf)), b"\x01" * 8, C.c_size_t(8), key, C.c_size_t(64)) == 0
    assert a.raw == b.raw
    assert a.raw[:128] != c.raw
    assert len(set(a.raw[i:i + 64] for i in range(0, 4096, 64))) == 64
