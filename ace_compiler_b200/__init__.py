"""Python binding of libFHErt_b200, the B200 CKKS runtime behind the ANT-ACE
runtime API (include/fhert_b200.h).

The binding is a thin ctypes mirror: function names, argument order and struct
fields are those of the C ABI, which in turn are those of the CPU runtime in
fhe-cmplr/rtlib/ant.  There is no CPU implementation in this package; loading
fails loudly when the CUDA library has not been built, and creating a context
aborts when no GPU is present.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libFHErt_b200.so")


class POLYNOMIAL(C.Structure):
    _fields_ = [
        ("_ring_degree", C.c_uint32),
        ("_num_alloc_primes", C.c_size_t),
        ("_num_primes", C.c_size_t),
        ("_num_primes_p", C.c_size_t),
        ("_is_ntt", C.c_bool),
        ("_data", C.c_void_p),
    ]


class CIPHERTEXT(C.Structure):
    _fields_ = [
        ("_c0_poly", POLYNOMIAL),
        ("_c1_poly", POLYNOMIAL),
        ("_slots", C.c_uint32),
        ("_scaling_factor", C.c_double),
        ("_sf_degree", C.c_uint32),
    ]


class CIPHERTEXT3(C.Structure):
    _fields_ = [
        ("_c0_poly", POLYNOMIAL),
        ("_c1_poly", POLYNOMIAL),
        ("_c2_poly", POLYNOMIAL),
        ("_slots", C.c_uint32),
        ("_scaling_factor", C.c_double),
        ("_sf_degree", C.c_uint32),
    ]


class PLAINTEXT(C.Structure):
    _fields_ = [
        ("_poly", POLYNOMIAL),
        ("_slots", C.c_uint32),
        ("_scaling_factor", C.c_double),
        ("_sf_degree", C.c_uint32),
    ]


class MODULUS(C.Structure):
    _fields_ = [
        ("_val", C.c_int64),
        ("_br_k", C.c_int64),
        ("_br_m", C.c_int64),
        ("_pad", C.c_int64),
        ("_prec128_lo", C.c_uint64),
        ("_prec128_hi", C.c_uint64),
    ]


POLY = C.POINTER(POLYNOMIAL)


class L_POLY(C.Structure):  # one RNS limb (ant/include/lpoly/poly.h:18-24)
    _fields_ = [("_ring_degree", C.c_uint32), ("_is_ntt", C.c_bool), ("_data", C.c_void_p)]


LPOLY = C.POINTER(L_POLY)
CIPHER = C.POINTER(CIPHERTEXT)
CIPHER3 = C.POINTER(CIPHERTEXT3)
PLAIN = C.POINTER(PLAINTEXT)
MODP = C.POINTER(MODULUS)
I64P = C.c_void_p  # device or host int64 buffers travel as raw addresses

# name -> (restype, argtypes); every symbol include/fhert_b200.h declares
SIGNATURES = {
    "Get_context_params": (C.c_void_p, []),
    "Fhert_set_context_params": (None, [C.c_uint32] + [C.c_size_t] * 7 + [C.c_void_p]),
    "Prepare_context": (None, []),
    "Finalize_context": (None, []),
    "Degree": (C.c_uint32, []),
    "Get_q_cnt": (C.c_size_t, []),
    "Get_p_cnt": (C.c_size_t, []),
    "Get_q_parts": (C.c_size_t, []),
    "Get_part_size": (C.c_size_t, []),
    "Q_modulus": (MODP, []),
    "P_modulus": (MODP, []),
    "Get_default_sc": (C.c_double, []),
    "Fhert_get_primes": (None, [C.c_void_p]),
    "Fhert_get_ntt_tables": (None, [C.c_size_t] + [C.c_void_p] * 5),
    "Alloc_poly": (POLY, [C.c_uint32, C.c_size_t, C.c_size_t]),
    "Free_poly": (None, [POLY]),
    "Alloc_poly_data": (None, [POLY, C.c_uint32, C.c_size_t, C.c_size_t]),
    "Free_poly_data": (None, [POLY]),
    "Init_poly_by_size": (None, [POLY, C.c_size_t, C.c_bool]),
    "Copy_poly": (None, [POLY, POLY]),
    "Coeffs": (C.c_void_p, [POLY, C.c_uint32, C.c_uint32]),
    "Set_coeffs": (None, [POLY, C.c_uint32, C.c_uint32, I64P]),
    "Fhert_upload": (None, [POLY, C.c_size_t, C.c_size_t, C.c_void_p]),
    "Fhert_download": (None, [POLY, C.c_size_t, C.c_size_t, C.c_void_p]),
    "Fhert_sync": (None, []),
    "Fhert_stream": (C.c_void_p, []),
    "Fhert_transfer_bytes": (None, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "Fhert_kernel_launches": (C.c_uint64, []),
    "Fhert_profile_begin": (None, []),
    "Fhert_profile_end": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "Hw_modadd": (C.c_void_p, [I64P, I64P, I64P, MODP, C.c_uint32]),
    "Hw_modsub": (C.c_void_p, [I64P, I64P, I64P, MODP, C.c_uint32]),
    "Hw_modmul": (C.c_void_p, [I64P, I64P, I64P, MODP, C.c_uint32]),
    "Hw_modmuladd": (C.c_void_p, [I64P, I64P, I64P, MODP, C.c_uint32]),
    "Hw_modmuladd_scalar": (C.c_void_p, [I64P, I64P, C.c_int64, MODP, C.c_uint32]),
    "Hw_modsub_scalar": (C.c_void_p, [I64P, I64P, C.c_int64, MODP, C.c_uint32]),
    "Alloc_lpoly_data": (None, [LPOLY, C.c_uint32]),
    "Init_lpoly_data": (None, [LPOLY, C.c_uint32, I64P]),
    "Free_lpoly_data": (None, [LPOLY]),
    "Alloc_lpoly": (LPOLY, [C.c_uint32]),
    "Free_lpoly": (None, [LPOLY]),
    "Zero_lpoly": (None, [LPOLY]),
    "Copy_lpoly": (None, [LPOLY, L_POLY]),
    "Add_lpoly": (LPOLY, [LPOLY, L_POLY, L_POLY, MODP]),
    "Add_scalar": (LPOLY, [LPOLY, L_POLY, C.c_int64, MODP]),
    "Sub_lpoly": (LPOLY, [LPOLY, L_POLY, L_POLY, MODP]),
    "Sub_scalar": (LPOLY, [LPOLY, L_POLY, C.c_int64, MODP]),
    "Mul_lpoly": (LPOLY, [LPOLY, L_POLY, L_POLY, MODP]),
    "Mul_scalar": (LPOLY, [LPOLY, L_POLY, C.c_int64, MODP]),
    "Mac_lpoly": (LPOLY, [LPOLY, L_POLY, L_POLY, MODP]),
    "Mac_scalar": (LPOLY, [LPOLY, L_POLY, C.c_int64, MODP]),
    "Ntt": (None, [LPOLY, L_POLY, C.c_size_t]),
    "Intt": (None, [LPOLY, L_POLY, C.c_size_t]),
    "Hw_modadd_scalar": (C.c_void_p, [I64P, I64P, C.c_int64, MODP, C.c_uint32]),
    "Hw_modmul_scalar": (C.c_void_p, [I64P, I64P, C.c_int64, MODP, C.c_uint32]),
    "Hw_rotate": (C.c_void_p, [I64P, I64P, I64P, MODP, C.c_uint32]),
    "Hw_ntt": (None, [I64P, I64P, C.c_size_t, C.c_uint32]),
    "Hw_intt": (None, [I64P, I64P, C.c_size_t, C.c_uint32]),
    "Conv_poly2ntt_inplace": (POLY, [POLY]),
    "Conv_ntt2poly_inplace": (POLY, [POLY]),
    "Reduce_and_rescale_modup": (C.c_void_p, [POLY, POLY]),
    "Free_precomp": (None, [C.c_void_p]),
    "Conv_poly2ntt": (None, [POLY, POLY]),
    "Conv_ntt2poly": (None, [POLY, POLY]),
    "Add_poly": (POLY, [POLY, POLY, POLY]),
    "Sub_poly": (POLY, [POLY, POLY, POLY]),
    "Mul_poly": (POLY, [POLY, POLY, POLY]),
    "Rescale": (POLY, [POLY, POLY]),
    "Modswitch": (POLY, [POLY, POLY]),
    "Num_decomp": (C.c_size_t, [POLY]),
    "Decomp": (POLY, [POLY, POLY, C.c_uint32]),
    "Mod_up": (POLY, [POLY, POLY, C.c_uint32]),
    "Decomp_modup": (POLY, [POLY, POLY, C.c_uint32]),
    "Mod_down": (POLY, [POLY, POLY]),
    "Extend": (POLY, [POLY, POLY]),
    "Dot_prod": (POLY, [POLY, POLY, POLY, C.c_size_t]),
    "Mod_down_rescale": (POLY, [POLY, POLY]),
    "Chk_level": (None, [POLY, POLY, POLY]),
    "Automorphism_transform": (POLY, [POLY, POLY, I64P]),
    "Fhert_rescale_static": (C.c_int, [I64P, I64P, C.c_size_t]),
    "Fhert_rescale_static_capacity": (C.c_size_t, []),
    "Auto_idx": (C.c_uint32, [C.c_int32]),
    "Auto_order": (C.c_void_p, [C.c_int32]),
    "Swk": (C.c_void_p, [C.c_bool, C.c_int32]),
    "Pk0_at": (POLY, [C.c_void_p, C.c_uint32]),
    "Pk1_at": (POLY, [C.c_void_p, C.c_uint32]),
    "Set_pk0": (None, [POLY, C.c_void_p, C.c_uint32]),
    "Set_pk1": (None, [POLY, C.c_void_p, C.c_uint32]),
    "Fhert_import_switch_key": (None, [C.c_bool, C.c_int32, C.c_uint32, C.c_int, C.c_void_p]),
    "Fhert_seed": (None, [C.c_void_p, C.c_uint64, C.c_int64]),
    "Encode_float": (None, [PLAIN, C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32]),
    "Encode_double": (None, [PLAIN, C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32]),
    "Encode_float_mask": (None, [PLAIN, C.c_float, C.c_size_t, C.c_uint32, C.c_uint32]),
    "Encode_double_mask": (None, [PLAIN, C.c_double, C.c_size_t, C.c_uint32, C.c_uint32]),
    "Encode_dcmplx": (None, [PLAIN, C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32]),
    "Free_plain_data": (None, [PLAIN]),
    "Encrypt": (CIPHER, [CIPHER, PLAIN]),
    "Fhert_decrypt": (None, [PLAIN, CIPHER]),
    "Fhert_decode": (None, [PLAIN, C.c_void_p, C.c_size_t]),
    "Get_msg": (C.c_void_p, [CIPHER]),
    "Fhert_export_switch_key": (None, [C.c_bool, C.c_int32, C.c_uint32, C.c_int, C.c_void_p]),
    "Fhert_export_key": (None, [C.c_int, C.c_void_p]),
    "Init_ciph_same_scale": (None, [CIPHER, CIPHER, CIPHER]),
    "Init_ciph_up_scale": (None, [CIPHER, CIPHER, CIPHER]),
    "Init_ciph_down_scale": (None, [CIPHER, CIPHER]),
    "Init_ciph3_up_scale": (None, [CIPHER3, CIPHER, CIPHER]),
    "Copy_ciph": (None, [CIPHER, CIPHER]),
    "Init_ciph_same_scale_plain": (None, [CIPHER, CIPHER, PLAIN]),
    "Init_ciph_same_scale_ciph3": (None, [CIPHER, CIPHER3]),
    "Init_ciph3_same_scale_ciph3": (None, [CIPHER3, CIPHER3, CIPHER3]),
    "Init_ciph3_same_scale": (None, [CIPHER3, CIPHER3, CIPHER3]),
    "Init_ciph_up_scale_plain": (None, [CIPHER, CIPHER, PLAIN]),
    "Init_ciph3_down_scale": (None, [CIPHER3, CIPHER3]),
    "Zero_ciph": (None, [CIPHER]),
    "Sc_degree": (C.c_uint32, [CIPHER]),
    "Get_slots": (C.c_uint32, [CIPHER]),
    "Set_slots": (None, [CIPHER, C.c_uint32]),
    "Poly_level": (C.c_size_t, [POLY]),
    "Num_p": (C.c_size_t, [POLY]),
    "Num_alloc": (C.c_size_t, [POLY]),
    "Rotate_batch_ciph": (None, [CIPHER, CIPHER, C.POINTER(C.c_int32), C.c_uint32]),
    "Add_plain": (CIPHER, [CIPHER, CIPHER, PLAIN]),
    "Mul_plain": (CIPHER, [CIPHER, CIPHER, PLAIN]),
    "Modswitch_ciph": (None, [CIPHER]),
    "Upscale_ciph": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Downscale_ciph": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Raise_mod": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Mul_mono_ciph": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Print_cipher_msg": (None, [C.c_void_p, C.c_char_p, CIPHER, C.c_uint32]),
    "Dump_cipher_msg": (None, [C.c_char_p, CIPHER, C.c_uint32]),
    "Alloc_polys": (POLY, [C.c_uint32, C.c_uint32, C.c_size_t, C.c_size_t]),
    "Free_polys": (None, [POLY]),
    "Init_poly_by_opnd": (POLY, [POLY, POLY, POLY, C.c_bool]),
    "Swk_c0": (POLY, [POLY, C.c_size_t, C.c_bool, C.c_int32]),
    "Swk_c1": (POLY, [POLY, C.c_size_t, C.c_bool, C.c_int32]),
    "Precomp": (POLY, [POLY, C.c_size_t, POLY]),
    "Fhert_shard_blocks": (None, [C.c_size_t, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "Fhert_shard_begin": (C.c_void_p, [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]),
    "Fhert_shard_mid": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int, C.c_void_p,
                               C.c_void_p]),
    "Fhert_shard_end": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int,
                               C.c_void_p, C.c_void_p]),
    "Fhert_shard_end2": (None, [C.c_void_p, I64P, I64P, I64P, I64P, C.c_int32, C.c_int, I64P, I64P]),
    "Fhert_shard_rescale_begin": (C.c_int, [I64P, I64P, C.c_size_t, C.c_int, C.c_int, I64P]),
    "Fhert_shard_rescale_end": (None, [I64P, I64P, C.c_size_t, C.c_int, C.c_int, I64P, I64P, I64P]),
    "Fhert_shard_tensor": (None, [I64P, I64P, I64P, I64P, C.c_size_t, C.c_int, C.c_int, I64P, I64P, I64P]),
    "Fhert_shard_comm_id": (C.c_int, [C.c_void_p]),
    "Fhert_shard_comm_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "Fhert_shard_comm_destroy": (None, []),
    "Fhert_shard_rotate": (CIPHER, [CIPHER, CIPHER, C.c_int32, C.c_int]),
    "Fhert_shard_mul_relin": (CIPHER, [CIPHER, CIPHER, CIPHER]),
    "Fhert_shard_rescale": (CIPHER, [CIPHER, CIPHER]),
    "Bootstrap": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Bootstrap_precom": (None, [C.c_uint32]),
    "Eval_bootstrap_ciph": (CIPHER, [CIPHER, CIPHER, C.c_uint32, C.c_uint32]),
    "Eval_bootstrap_coeffs_to_slots_ciph": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Eval_bootstrap_eval_mod_ciph": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Eval_bootstrap_slots_to_coeffs_ciph": (CIPHER, [CIPHER, CIPHER, C.c_uint32]),
    "Fhert_bootstrap_rotations": (C.c_size_t, [C.c_uint32, C.POINTER(C.c_int32), C.c_size_t]),
    "Fhert_export_bootstrap_plain": (C.c_size_t, [C.c_uint32, C.c_int, C.c_uint32, C.c_uint32,
                                                  C.c_void_p]),
    # program driver
    "Get_rt_data_info": (C.c_void_p, []),
    "Get_input_count": (C.c_int, []),
    "Get_output_count": (C.c_int, []),
    "Get_encode_scheme": (C.c_void_p, [C.c_int]),
    "Get_decode_scheme": (C.c_void_p, [C.c_int]),
    "Main_graph": (C.c_bool, []),
    "Alloc_tensor": (C.c_void_p, [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                  C.POINTER(C.c_double)]),
    "Free_tensor": (None, [C.c_void_p]),
    "Print_tensor": (None, [C.c_void_p, C.c_void_p]),
    "Prepare_input": (None, [C.c_void_p, C.c_char_p]),
    "Get_input_data": (CIPHERTEXT, [C.c_char_p, C.c_size_t]),
    "Set_output_data": (None, [C.c_char_p, C.c_size_t, CIPHER]),
    "Run_main_graph": (None, []),
    "Handle_output": (C.POINTER(C.c_double), [C.c_char_p]),
    "Pt_mgr_init": (C.c_bool, [C.c_char_p]),
    "Pt_mgr_fini": (None, []),
    "Pt_from_msg": (C.c_void_p, [C.c_void_p, C.c_uint32, C.c_size_t, C.c_uint32, C.c_uint32]),
    "Pt_from_msg_ofst": (C.c_void_p, [C.c_void_p, C.c_uint32, C.c_size_t, C.c_size_t, C.c_uint32,
                                      C.c_uint32]),
    "Free_data": (None, [C.c_void_p]),
    "Fhert_pt_cache_stats": (None, [C.POINTER(C.c_size_t)] * 4),
    "Fhert_pt_cache_bypass": (None, [C.c_int]),
    "Fhert_replay_mode": (None, [C.c_int]),
    "Fhert_replay_state": (C.c_int, [C.c_char_p, C.c_size_t, C.POINTER(C.c_uint64)]),
    "Fhert_replay_graph": (None, [C.POINTER(C.c_uint64)] * 5),
    "Validate_impl": (None, [C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_uint32, C.c_int32]),
    "Validate_value_range": (None, [C.c_bool]),
    "Within_value_range": (C.c_bool, [CIPHER, C.POINTER(C.c_double), C.c_uint32]),
    "Fhert_tm_event": (None, [C.c_uint32, C.c_uint32, C.c_int]),
    "Fhert_tm_report": (None, []),
    "Tm_start": (None, [C.c_char_p]),
    "Tm_taken": (None, [C.c_char_p]),
    "Level": (C.c_size_t, [CIPHER]),
    "Free_ciph_poly": (None, [CIPHER, C.c_uint32]),
    "Add_ciph": (CIPHER, [CIPHER, CIPHER, CIPHER]),
    "Sub_ciph": (CIPHER, [CIPHER, CIPHER, CIPHER]),
    "Mul_ciph3": (CIPHER3, [CIPHER3, CIPHER, CIPHER]),
    "Relin": (CIPHER, [CIPHER, CIPHER3]),
    "Mul_ciph": (CIPHER, [CIPHER, CIPHER, CIPHER]),
    "Rescale_ciph": (CIPHER, [CIPHER, CIPHER]),
    "Rotate_ciph": (CIPHER, [CIPHER, CIPHER, C.c_int32]),
    "Conjugate_ciph": (CIPHER, [CIPHER, CIPHER]),
}

_lib = None


def load():
    """Loads the CUDA runtime library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libFHErt_b200.so is missing: build it with `python -m ace_compiler_b200.build` "
            "(this package has no CPU implementation)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class Runtime:
    """One CKKS context on the current GPU, driven through the C ABI.

    Mirrors Prepare_context (fhe-cmplr/rtlib/ant/context/src/ckks_context.c:84)
    and exposes helpers that move numpy int64 arrays of shape (limbs, N) in and
    out of device polynomials.
    """

    def __init__(self, degree, num_q, q0_bits=60, sf_bits=56, num_q_parts=3, input_level=0,
                 hamming_weight=192, rot_idxs=(), keygen=False, seed=None, fake_time_us=-1):
        """keygen=False skips key generation (switch keys are then imported);
        seed = 16 uint32 words pins the sample generator as Fhert_seed does."""
        self.lib = load()
        previous = os.environ.get("FHERT_SKIP_KEYGEN")
        os.environ["FHERT_SKIP_KEYGEN"] = "0" if keygen else "1"
        if seed is not None:
            s = np.ascontiguousarray(seed, dtype=np.uint32)
            assert s.shape == (16,)
            self.lib.Fhert_seed(_ptr(s), 0, fake_time_us)
        rot = (C.c_int32 * max(1, len(rot_idxs)))(*rot_idxs)
        self.lib.Fhert_set_context_params(degree, num_q, q0_bits, sf_bits, num_q_parts,
                                          input_level, hamming_weight, len(rot_idxs), rot)
        try:
            self.lib.Prepare_context()
        finally:  # the switch is for this context only, not for child processes
            if previous is None:
                os.environ.pop("FHERT_SKIP_KEYGEN", None)
            else:
                os.environ["FHERT_SKIP_KEYGEN"] = previous
        self.N = self.lib.Degree()
        self.L = self.lib.Get_q_cnt()
        self.K = self.lib.Get_p_cnt()
        self.dnum = self.lib.Get_q_parts()
        self.alpha = self.lib.Get_part_size()
        pr = np.zeros(self.L + self.K, dtype=np.int64)
        self.lib.Fhert_get_primes(_ptr(pr))
        self.primes = [int(v) for v in pr]

    def close(self):
        self.lib.Finalize_context()

    def profile(self):
        """Context manager: per-kernel (launches, limbs, total ms) of the calls inside."""
        rt = self

        class _Prof:
            def __enter__(self):
                rt.lib.Fhert_profile_begin()
                self.kernels = {}
                return self

            def __exit__(self, *exc):
                buf = C.create_string_buffer(8192)
                n = rt.lib.Fhert_profile_end(buf, len(buf))
                for line in buf.raw[:n].decode().splitlines():
                    name, cnt, limbs, ms = line.split()
                    self.kernels[name] = (int(cnt), int(limbs), float(ms))
                return False

        return _Prof()

    # --- polynomials ------------------------------------------------------
    def modulus(self, idx):
        """MODULUS* of prime idx (Q chain first, then P), as generated code gets
        it from Q_modulus() / P_modulus() plus pointer arithmetic."""
        if idx < self.L:
            base, off = self.lib.Q_modulus(), idx
        else:
            base, off = self.lib.P_modulus(), idx - self.L
        addr = C.addressof(base.contents) + off * C.sizeof(MODULUS)
        return C.cast(addr, MODP)

    def new_poly(self, level, extended=False, data=None, is_ntt=True):
        p = self.lib.Alloc_poly(self.N, level, 1 if extended else 0)
        p.contents._is_ntt = is_ntt
        if data is not None:
            self.upload(p, data)
        return p

    def upload(self, poly, data):
        data = np.ascontiguousarray(data, dtype=np.int64)
        assert data.shape == (poly.contents._num_alloc_primes, self.N), data.shape
        self.lib.Fhert_upload(poly, 0, data.shape[0], _ptr(data))

    def download(self, poly):
        """All live limbs: level Q limbs followed by the special limbs."""
        p = poly.contents
        out = np.empty((p._num_primes + p._num_primes_p, self.N), dtype=np.int64)
        self.lib.Fhert_download(poly, 0, p._num_primes, _ptr(out))
        if p._num_primes_p:
            tail = out[p._num_primes:]
            self.lib.Fhert_download(poly, p._num_alloc_primes - p._num_primes_p,
                                    p._num_primes_p, _ptr(tail))
        return out

    def free(self, poly):
        self.lib.Free_poly(poly)

    def limb_ptr(self, poly, limb):
        return self.lib.Coeffs(poly, limb, self.N)

    # --- ciphertexts ------------------------------------------------------
    def new_ciph(self, c0, c1, sf_degree=1):
        """Ciphertext from two (level, N) residue arrays in NTT form."""
        ct = CIPHERTEXT()
        level = c0.shape[0]
        for poly, data in ((ct._c0_poly, c0), (ct._c1_poly, c1)):
            self.lib.Alloc_poly_data(C.byref(poly), self.N, level, 0)
            poly._is_ntt = True
            self.upload(C.pointer(poly), data)
        ct._slots = self.N // 2
        ct._scaling_factor = self.lib.Get_default_sc() ** sf_degree
        ct._sf_degree = sf_degree
        return ct

    def ciph_to_host(self, ct):
        return self.download(C.pointer(ct._c0_poly)), self.download(C.pointer(ct._c1_poly))

    def free_ciph(self, ct):
        self.lib.Free_ciph_poly(C.byref(ct), 1)

    # --- client side -------------------------------------------------------
    def encode(self, values, sf_degree=1, level=0):
        """Complex (or real) slot values -> PLAINTEXT in NTT form on the device."""
        v = np.ascontiguousarray(np.asarray(values, dtype=np.complex128))
        pt = PLAINTEXT()
        self.lib.Encode_dcmplx(C.byref(pt), _ptr(v.view(np.float64)), len(v), sf_degree, level)
        return pt

    def encode_scalar(self, value, sf_degree=1, level=0):
        pt = PLAINTEXT()
        d = C.c_double(value)
        self.lib.Encode_double(C.byref(pt), C.byref(d), 1, sf_degree, level)
        return pt

    def encrypt(self, pt):
        ct = CIPHERTEXT()
        self.lib.Encrypt(C.byref(ct), C.byref(pt))
        return ct

    def decrypt_decode(self, ct, count=None):
        count = count or self.N // 2
        pt = PLAINTEXT()
        self.lib.Fhert_decrypt(C.byref(pt), C.byref(ct))
        out = np.zeros(count, np.complex128)
        self.lib.Fhert_decode(C.byref(pt), _ptr(out.view(np.float64)), count)
        self.lib.Free_plain_data(C.byref(pt))
        return out

    def export_key(self, which):
        limbs = self.L + self.K if which < 2 else self.L
        out = np.zeros((limbs, self.N), np.int64)
        self.lib.Fhert_export_key(which, _ptr(out))
        return out

    def export_switch_key(self, is_rot, rot_idx, part, which):
        out = np.zeros((self.L + self.K, self.N), np.int64)
        self.lib.Fhert_export_switch_key(is_rot, rot_idx, part, which, _ptr(out))
        return out

    def import_switch_key(self, is_rot, rot_idx, part, which, data):
        data = np.ascontiguousarray(data, dtype=np.int64)
        assert data.shape == (self.L + self.K, self.N)
        self.lib.Fhert_import_switch_key(is_rot, rot_idx, part, which, _ptr(data))
