"""Test-side loader for the reference CPU runtime built by oracle/build_ref.sh.

The library holds one global CKKS context per process (as the reference does),
so tests that need different parameters run the reference in a child process
via `run_isolated`.
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libFHErt_ant_ref.so")


def available():
    return os.path.exists(REF_LIB)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class RefRuntime:
    def __init__(self, degree, num_q, q0_bits=60, sf_bits=56, num_q_parts=3, input_level=0,
                 hamming_weight=192, rot_idxs=(), seed=None, fake_time_us=1_700_000_000_000_000):
        # bootstrap precomputation is not needed for primitive parity and costs minutes
        os.environ.setdefault("RTLIB_DISABLE_BOOTSTRAP_PRECOM", "1")
        self.lib = lib = C.CDLL(REF_LIB)
        lib.Ref_set_params.argtypes = [C.c_uint32] + [C.c_size_t] * 7 + [C.c_void_p, C.c_size_t]
        lib.Ref_set_fake_time.argtypes = [C.c_int64]
        lib.Ref_seed_prng.argtypes = [C.c_void_p, C.c_uint64]
        for f in ("Ref_num_q", "Ref_num_p", "Ref_part_size", "Ref_num_parts"):
            getattr(lib, f).restype = C.c_size_t
        lib.Ref_get_primes.argtypes = [C.c_void_p]
        lib.Ref_get_ntt_tables.argtypes = [C.c_size_t] + [C.c_void_p] * 5
        lib.Ref_ntt.argtypes = [C.c_size_t, C.c_void_p, C.c_int]
        lib.Ref_modulus.argtypes = [C.c_size_t]
        lib.Ref_modulus.restype = C.c_void_p
        lib.Ref_rescale.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        lib.Ref_decomp_modup.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_void_p]
        lib.Ref_mod_down.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        lib.Ref_num_decomp.argtypes = [C.c_size_t]
        lib.Ref_num_decomp.restype = C.c_uint32
        lib.Ref_auto_idx.argtypes = [C.c_int32]
        lib.Ref_auto_idx.restype = C.c_uint32
        lib.Ref_auto_order.argtypes = [C.c_int32, C.c_void_p]
        lib.Ref_get_swk.argtypes = [C.c_int, C.c_int32, C.c_uint32, C.c_int, C.c_void_p]
        lib.Ref_rotate.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int32, C.c_void_p, C.c_void_p]
        lib.Ref_mul_relin_rescale.argtypes = [C.c_void_p] * 4 + [C.c_size_t] + [C.c_void_p] * 2
        lib.Ref_relinearize.argtypes = [C.c_void_p] * 3 + [C.c_size_t] + [C.c_void_p] * 2
        lib.Ref_export_key.argtypes = [C.c_int, C.c_void_p]
        lib.Ref_encode.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32, C.c_void_p]
        lib.Ref_encode_scalar.argtypes = [C.c_double, C.c_uint32, C.c_uint32, C.c_void_p]
        lib.Ref_encrypt.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, C.c_void_p, C.c_void_p]
        lib.Ref_decrypt_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint32,
                                           C.c_void_p, C.c_size_t]
        for name in ("Hw_modadd", "Hw_modsub", "Hw_modmul", "Hw_modmuladd", "Hw_rotate"):
            getattr(lib, name).restype = C.c_void_p
        lib.Hw_modadd.argtypes = lib.Hw_modsub.argtypes = lib.Hw_modmul.argtypes = \
            [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32]
        lib.Hw_modmuladd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32]
        lib.Hw_rotate.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32]
        lib.Hw_modmul_scalar.argtypes = lib.Hw_modadd_scalar.argtypes = \
            [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_uint32]

        if fake_time_us is not None:
            lib.Ref_set_fake_time(fake_time_us)
        if seed is not None:
            s = np.asarray(seed, dtype=np.uint32)
            assert s.shape == (16,)
            lib.Ref_seed_prng(_p(s), 0)
        rot = (C.c_int32 * max(1, len(rot_idxs)))(*rot_idxs)
        lib.Ref_set_params(degree, num_q, q0_bits, sf_bits, num_q_parts, input_level,
                           hamming_weight, len(rot_idxs), rot, 0)
        lib.Ref_prepare_context()
        self.N = degree
        self.L = lib.Ref_num_q()
        self.K = lib.Ref_num_p()
        self.alpha = lib.Ref_part_size()
        self.dnum = lib.Ref_num_parts()
        pr = np.zeros(self.L + self.K, dtype=np.int64)
        lib.Ref_get_primes(_p(pr))
        self.primes = [int(v) for v in pr]

    def ntt_tables(self, idx):
        n = self.N
        rou = np.zeros(n, np.int64); roup = np.zeros(n, np.uint64)
        inv = np.zeros(n, np.int64); invp = np.zeros(n, np.uint64)
        dinv = np.zeros(1, np.int64)
        self.lib.Ref_get_ntt_tables(idx, _p(rou), _p(roup), _p(inv), _p(invp), _p(dinv))
        return rou, roup, inv, invp, int(dinv[0])

    def ntt(self, idx, data, inverse=False):
        out = np.ascontiguousarray(data, dtype=np.int64).copy()
        self.lib.Ref_ntt(idx, _p(out), 1 if inverse else 0)
        return out

    def hw(self, op, a, b, idx):
        a = np.ascontiguousarray(a, np.int64); b = np.ascontiguousarray(b, np.int64)
        res = np.zeros_like(a)
        getattr(self.lib, op)(_p(res), _p(a), _p(b), self.lib.Ref_modulus(idx), self.N)
        return res

    def hw_muladd(self, acc, a, b, idx):
        res = np.ascontiguousarray(acc, np.int64).copy()
        a = np.ascontiguousarray(a, np.int64); b = np.ascontiguousarray(b, np.int64)
        self.lib.Hw_modmuladd(_p(res), _p(a), _p(b), self.lib.Ref_modulus(idx), self.N)
        return res

    def hw_scalar(self, op, a, s, idx):
        a = np.ascontiguousarray(a, np.int64)
        res = np.zeros_like(a)
        getattr(self.lib, op)(_p(res), _p(a), s, self.lib.Ref_modulus(idx), self.N)
        return res

    def auto_order(self, rot_idx):
        out = np.zeros(self.N, np.int64)
        self.lib.Ref_auto_order(rot_idx, _p(out))
        return out

    def auto_idx(self, rot_idx):
        return self.lib.Ref_auto_idx(rot_idx)

    def hw_rotate(self, val, order, idx):
        val = np.ascontiguousarray(val, np.int64); order = np.ascontiguousarray(order, np.int64)
        res = np.zeros_like(val)
        self.lib.Hw_rotate(_p(res), _p(val), _p(order), self.lib.Ref_modulus(idx), self.N)
        return res

    def rescale(self, poly, is_ntt=True):
        poly = np.ascontiguousarray(poly, np.int64)
        out = np.zeros((poly.shape[0] - 1, self.N), np.int64)
        self.lib.Ref_rescale(_p(poly), poly.shape[0], int(is_ntt), _p(out))
        return out

    def decomp_modup(self, poly, part, is_ntt=True):
        poly = np.ascontiguousarray(poly, np.int64)
        out = np.zeros((poly.shape[0] + self.K, self.N), np.int64)
        self.lib.Ref_decomp_modup(_p(poly), poly.shape[0], int(is_ntt), part, _p(out))
        return out

    def mod_down(self, ext, level, is_ntt=True):
        ext = np.ascontiguousarray(ext, np.int64)
        assert ext.shape[0] == level + self.K
        out = np.zeros((level, self.N), np.int64)
        self.lib.Ref_mod_down(_p(ext), level, int(is_ntt), _p(out))
        return out

    def num_decomp(self, level):
        return self.lib.Ref_num_decomp(level)

    def swk(self, is_rot, rot_idx, part, which):
        out = np.zeros((self.L + self.K, self.N), np.int64)
        self.lib.Ref_get_swk(int(is_rot), rot_idx, part, which, _p(out))
        return out

    def rotate(self, c0, c1, rot_idx):
        c0 = np.ascontiguousarray(c0, np.int64); c1 = np.ascontiguousarray(c1, np.int64)
        o0 = np.zeros_like(c0); o1 = np.zeros_like(c1)
        self.lib.Ref_rotate(_p(c0), _p(c1), c0.shape[0], rot_idx, _p(o0), _p(o1))
        return o0, o1

    def mul_relin_rescale(self, a0, a1, b0, b1):
        arrs = [np.ascontiguousarray(x, np.int64) for x in (a0, a1, b0, b1)]
        level = arrs[0].shape[0]
        o0 = np.zeros((level - 1, self.N), np.int64); o1 = np.zeros_like(o0)
        self.lib.Ref_mul_relin_rescale(*[_p(x) for x in arrs], level, _p(o0), _p(o1))
        return o0, o1

    def relinearize(self, c0, c1, c2):
        arrs = [np.ascontiguousarray(x, np.int64) for x in (c0, c1, c2)]
        level = arrs[0].shape[0]
        o0 = np.zeros((level, self.N), np.int64); o1 = np.zeros_like(o0)
        self.lib.Ref_relinearize(*[_p(x) for x in arrs], level, _p(o0), _p(o1))
        return o0, o1


def _client(self):
    pass


def export_key(self, which):
    limbs = self.L + self.K if which < 2 else self.L
    out = np.zeros((limbs, self.N), np.int64)
    self.lib.Ref_export_key(which, _p(out))
    return out


def encode(self, values, sf_degree=1, level=0):
    v = np.ascontiguousarray(np.asarray(values, dtype=np.complex128))
    lv = level or self.L
    out = np.zeros((lv, self.N), np.int64)
    self.lib.Ref_encode(_p(v.view(np.float64)), len(v), sf_degree, lv, _p(out))
    return out


def encode_scalar(self, value, sf_degree=1, level=0):
    lv = level or self.L
    out = np.zeros((lv, self.N), np.int64)
    self.lib.Ref_encode_scalar(float(value), sf_degree, lv, _p(out))
    return out


def encrypt(self, plain_poly, sf_degree=1):
    pp = np.ascontiguousarray(plain_poly, np.int64)
    c0 = np.zeros_like(pp); c1 = np.zeros_like(pp)
    self.lib.Ref_encrypt(_p(pp), pp.shape[0], sf_degree, _p(c0), _p(c1))
    return c0, c1


def decrypt_decode(self, c0, c1, sf_degree=1, count=None):
    c0 = np.ascontiguousarray(c0, np.int64); c1 = np.ascontiguousarray(c1, np.int64)
    count = count or self.N // 2
    out = np.zeros(count, np.complex128)
    self.lib.Ref_decrypt_decode(_p(c0), _p(c1), c0.shape[0], sf_degree, _p(out.view(np.float64)), count)
    return out


for _f in (export_key, encode, encode_scalar, encrypt, decrypt_decode):
    setattr(RefRuntime, _f.__name__, _f)


def uniform_limbs(rng, primes, n):
    """Seeded uniform residues, one row per prime."""
    return np.stack([rng.integers(0, p, size=n, dtype=np.int64) for p in primes])


def close_ref(ref):
    ref.lib.Ref_finalize_context()
