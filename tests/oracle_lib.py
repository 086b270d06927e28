"""ctypes wrapper of the plain-C oracle (oracle/ckks_oracle.c)."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "liboracle.so")


def load():
    if not os.path.exists(LIB):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    lib = C.CDLL(LIB)
    u64, vp = C.c_uint64, C.c_void_p
    lib.Oracle_pow_mod.restype = u64
    lib.Oracle_pow_mod.argtypes = [u64, u64, u64]
    lib.Oracle_inv_mod_prime.restype = u64
    lib.Oracle_inv_mod_prime.argtypes = [u64, u64]
    lib.Oracle_inv_mod.restype = C.c_int64
    lib.Oracle_inv_mod.argtypes = [C.c_int64, C.c_int64]
    lib.Oracle_prec128.argtypes = [u64, vp, vp]
    lib.Oracle_is_prime.argtypes = [u64]
    lib.Oracle_find_generator.restype = u64
    lib.Oracle_find_generator.argtypes = [u64]
    lib.Oracle_root_of_unity.restype = u64
    lib.Oracle_root_of_unity.argtypes = [u64, u64]
    lib.Oracle_create.restype = vp
    lib.Oracle_create.argtypes = [C.c_uint32, C.c_int, C.c_size_t, C.c_size_t, C.c_int]
    lib.Oracle_destroy.argtypes = [vp]
    lib.Oracle_num_p.argtypes = [vp]
    lib.Oracle_alpha.argtypes = [vp]
    lib.Oracle_get_primes.argtypes = [vp, vp]
    lib.Oracle_get_tables.argtypes = [vp, C.c_int, vp, vp, vp]
    lib.Oracle_ntt_tables.argtypes = [vp, C.c_uint32, u64, vp]
    lib.Oracle_intt_tables.argtypes = [vp, C.c_uint32, u64, vp, u64]
    lib.Oracle_make_tables.argtypes = [C.c_uint32, u64, u64, vp, vp]
    lib.Oracle_ntt.argtypes = [vp, C.c_int, vp, C.c_int]
    lib.Oracle_hw.argtypes = [C.c_int, vp, vp, vp, u64, C.c_uint32]
    lib.Oracle_auto_index.restype = C.c_uint32
    lib.Oracle_auto_index.argtypes = [C.c_int32, C.c_uint32]
    lib.Oracle_auto_order.argtypes = [C.c_uint32, C.c_uint32, vp]
    lib.Oracle_rotate_limb.argtypes = [vp, vp, vp, C.c_uint32]
    lib.Oracle_rescale.argtypes = [vp, vp, C.c_int, vp]
    lib.Oracle_num_decomp.argtypes = [vp, C.c_int]
    lib.Oracle_decomp_modup.argtypes = [vp, vp, C.c_int, C.c_int, vp]
    lib.Oracle_mod_down.argtypes = [vp, vp, C.c_int, vp]
    lib.Oracle_switch_key.argtypes = [vp, vp, C.c_int, vp, vp, vp, vp]
    lib.Oracle_rotate.argtypes = [vp, vp, vp, C.c_int, C.c_int32, vp, vp, vp, vp]
    lib.Oracle_mul_relin_rescale.argtypes = [vp] * 5 + [C.c_int] + [vp] * 4
    return lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    def __init__(self, degree, num_q, q0_bits=60, sf_bits=56, dnum=3):
        self.lib = load()
        self.h = self.lib.Oracle_create(degree, num_q, q0_bits, sf_bits, dnum)
        self.N, self.L, self.dnum = degree, num_q, dnum
        self.K = self.lib.Oracle_num_p(self.h)
        self.alpha = self.lib.Oracle_alpha(self.h)
        pr = np.zeros(self.L + self.K, np.int64)
        self.lib.Oracle_get_primes(self.h, _p(pr))
        self.primes = [int(v) for v in pr]

    def close(self):
        self.lib.Oracle_destroy(self.h)

    def tables(self, idx):
        rou, inv, ninv = np.zeros(self.N, np.int64), np.zeros(self.N, np.int64), np.zeros(1, np.int64)
        self.lib.Oracle_get_tables(self.h, idx, _p(rou), _p(inv), _p(ninv))
        return rou, inv, int(ninv[0])

    def ntt(self, idx, data, inverse=False):
        out = np.ascontiguousarray(data, np.int64).copy()
        self.lib.Oracle_ntt(self.h, idx, _p(out), int(inverse))
        return out

    def hw(self, op, a, b, idx, acc=None):
        a = np.ascontiguousarray(a, np.int64); b = np.ascontiguousarray(b, np.int64)
        res = np.zeros_like(a) if acc is None else np.ascontiguousarray(acc, np.int64).copy()
        self.lib.Oracle_hw(op, _p(res), _p(a), _p(b), self.primes[idx], self.N)
        return res

    def auto_index(self, rot_idx):
        return self.lib.Oracle_auto_index(rot_idx, self.N)

    def auto_order(self, rot_idx):
        out = np.zeros(self.N, np.int64)
        self.lib.Oracle_auto_order(self.auto_index(rot_idx), self.N, _p(out))
        return out

    def rescale(self, poly):
        poly = np.ascontiguousarray(poly, np.int64)
        out = np.zeros((poly.shape[0] - 1, self.N), np.int64)
        self.lib.Oracle_rescale(self.h, _p(poly), poly.shape[0], _p(out))
        return out

    def num_decomp(self, level):
        return self.lib.Oracle_num_decomp(self.h, level)

    def decomp_modup(self, poly, part):
        poly = np.ascontiguousarray(poly, np.int64)
        out = np.zeros((poly.shape[0] + self.K, self.N), np.int64)
        self.lib.Oracle_decomp_modup(self.h, _p(poly), poly.shape[0], part, _p(out))
        return out

    def mod_down(self, ext, level):
        ext = np.ascontiguousarray(ext, np.int64)
        out = np.zeros((level, self.N), np.int64)
        self.lib.Oracle_mod_down(self.h, _p(ext), level, _p(out))
        return out

    @staticmethod
    def _keys(key):
        """key[part][which] -> two contiguous (dnum, L+K, N) arrays"""
        k0 = np.ascontiguousarray(np.stack([k[0] for k in key]), np.int64)
        k1 = np.ascontiguousarray(np.stack([k[1] for k in key]), np.int64)
        return k0, k1

    def rotate(self, c0, c1, rot_idx, key):
        c0 = np.ascontiguousarray(c0, np.int64); c1 = np.ascontiguousarray(c1, np.int64)
        k0, k1 = self._keys(key)
        o0, o1 = np.zeros_like(c0), np.zeros_like(c1)
        self.lib.Oracle_rotate(self.h, _p(c0), _p(c1), c0.shape[0], rot_idx, _p(k0), _p(k1),
                               _p(o0), _p(o1))
        return o0, o1

    def mul_relin_rescale(self, a0, a1, b0, b1, key):
        arrs = [np.ascontiguousarray(x, np.int64) for x in (a0, a1, b0, b1)]
        level = arrs[0].shape[0]
        k0, k1 = self._keys(key)
        o0 = np.zeros((level - 1, self.N), np.int64); o1 = np.zeros_like(o0)
        self.lib.Oracle_mul_relin_rescale(self.h, *[_p(x) for x in arrs], level, _p(k0), _p(k1),
                                          _p(o0), _p(o1))
        return o0, o1
