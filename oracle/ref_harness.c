/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * ctypes-friendly entry points into the unmodified reference runtime
 * (oracle/_ref/libFHErt_ant_ref.so).  The reference exposes most of its API
 * as `static inline` header code on its own structs; this file, compiled with
 * the reference headers, turns the pieces the parity tests need into plain
 * functions that take raw int64 buffers.  It also supplies the symbols that a
 * compiled program normally provides (Get_context_params and friends,
 * fhe-cmplr/rtlib/include/common/rt_api.h:48-80).
 *
 * Buffers are limb-major: limb i occupies [i*N, (i+1)*N).  "Extended" buffers
 * hold `level` Q limbs followed directly by K special (P) limbs.
 */
#include <complex.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "ckks/bootstrap.h"
#include "ckks/cipher.h"
#include "ckks/ciphertext.h"
#include "ckks/decryptor.h"
#include "ckks/encoder.h"
#include "ckks/encryptor.h"
#include "ckks/evaluator.h"
#include "ckks/key.h"
#include "ckks/key_gen.h"
#include "ckks/param.h"
#include "ckks/plain.h"
#include "common/common.h"
#include "common/rt_api.h"
#include "context/ckks_context.h"
#include "hal/hal.h"
#include "poly/rns_poly.h"
#include "rns_poly_impl.h"
#include "type_impl.h"
#include "util/crt.h"
#include "util/ntt.h"
#include "ntt_impl.h"
#include "crt_impl.h"

static CKKS_PARAMS* Harness_params = NULL;

CKKS_PARAMS*  Get_context_params() { return Harness_params; }
RT_DATA_INFO* Get_rt_data_info() { return NULL; }
int           Get_input_count() { return 0; }
int           Get_output_count() { return 0; }
DATA_SCHEME*  Get_encode_scheme(int idx) { return NULL; }
DATA_SCHEME*  Get_decode_scheme(int idx) { return NULL; }

void Ref_set_params(uint32_t degree, size_t num_q, size_t q0_bits,
                    size_t sf_bits, size_t num_parts, size_t input_level,
                    size_t hamming_weight, size_t num_rot,
                    const int32_t* rot_idxs, size_t sec_level) {
  free(Harness_params);
  Harness_params =
      (CKKS_PARAMS*)malloc(sizeof(CKKS_PARAMS) + num_rot * sizeof(int32_t));
  Harness_params->_provider         = LIB_ANT;
  Harness_params->_poly_degree      = degree;
  Harness_params->_sec_level        = sec_level;
  Harness_params->_mul_depth        = num_q - 1;
  Harness_params->_input_level      = input_level;
  Harness_params->_first_mod_size   = q0_bits;
  Harness_params->_scaling_mod_size = sf_bits;
  Harness_params->_num_q_parts      = num_parts;
  Harness_params->_hamming_weight   = hamming_weight;
  Harness_params->_num_rot_idx      = num_rot;
  if (num_rot) {
    memcpy(Harness_params->_rot_idxs, rot_idxs, num_rot * sizeof(int32_t));
  }
}

void Ref_prepare_context() { Prepare_context(); }
void Ref_finalize_context() { Finalize_context(); }

size_t Ref_num_q() { return Get_q_cnt(); }
size_t Ref_num_p() { return Get_p_cnt(); }
size_t Ref_part_size() { return Get_per_part_size(Get_qpart(Get_crt_context())); }
size_t Ref_num_parts() { return Get_q_parts(); }

static CRT_PRIME* Prime_at(size_t idx) {
  CRT_CONTEXT* crt = Get_crt_context();
  size_t       nq  = Get_q_cnt();
  return idx < nq ? Get_prime_at(Get_q(crt), idx)
                  : Get_prime_at(Get_p(crt), idx - nq);
}

//! primes[0..L) = Q chain, primes[L..L+K) = P chain
void Ref_get_primes(int64_t* primes) {
  size_t n = Get_q_cnt() + Get_p_cnt();
  for (size_t i = 0; i < n; i++) primes[i] = Get_modulus_val(Prime_at(i));
}

MODULUS* Ref_modulus(size_t idx) { return Get_modulus(Prime_at(idx)); }

//! twiddle tables of one prime, as the reference lays them out (ntt_impl.h:25)
void Ref_get_ntt_tables(size_t idx, int64_t* rou, uint64_t* rou_prec,
                        int64_t* rou_inv, uint64_t* rou_inv_prec,
                        int64_t* degree_inv) {
  NTT_CONTEXT* ntt = Get_ntt(Prime_at(idx));
  size_t       n   = ntt->_degree;
  memcpy(rou, Get_i64_values(ntt->_rou), n * sizeof(int64_t));
  memcpy(rou_prec, Get_ui64_values(ntt->_rou_prec), n * sizeof(uint64_t));
  memcpy(rou_inv, Get_i64_values(ntt->_rou_inv), n * sizeof(int64_t));
  memcpy(rou_inv_prec, Get_ui64_values(ntt->_rou_inv_prec),
         n * sizeof(uint64_t));
  *degree_inv = ntt->_degree_inv;
}

void Ref_ntt(size_t prime_idx, int64_t* data, int inverse) {
  NTT_CONTEXT* ntt = Get_ntt(Prime_at(prime_idx));
  VALUE_LIST   vl;
  vl._type       = I64_TYPE;
  vl._length     = ntt->_degree;
  vl._vals._i    = data;
  if (inverse) {
    Ftt_inv(&vl, ntt, &vl);
  } else {
    Ftt_fwd(&vl, ntt, &vl);
  }
}

static void Wrap_poly(POLYNOMIAL* p, int64_t* data, size_t level, size_t num_p,
                      int is_ntt) {
  memset(p, 0, sizeof(*p));
  p->_ring_degree      = Degree();
  p->_num_primes       = level;
  p->_num_primes_p     = num_p;
  p->_num_alloc_primes = level + num_p;
  p->_data             = data;
  p->_is_ntt           = is_ntt != 0;
}

void Ref_rescale(const int64_t* in, size_t level, int is_ntt, int64_t* out) {
  size_t     n = Degree();
  POLYNOMIAL src, dst;
  int64_t*   tmp = (int64_t*)malloc(level * n * sizeof(int64_t));
  Wrap_poly(&src, (int64_t*)in, level, 0, is_ntt);
  Wrap_poly(&dst, tmp, level, 0, is_ntt);
  Rescale(&dst, &src);
  memcpy(out, tmp, (level - 1) * n * sizeof(int64_t));
  free(tmp);
}

void Ref_decomp_modup(const int64_t* in, size_t level, int is_ntt,
                      uint32_t part, int64_t* out_ext) {
  POLYNOMIAL src, dst;
  Wrap_poly(&src, (int64_t*)in, level, 0, is_ntt);
  Wrap_poly(&dst, out_ext, level, Get_p_cnt(), is_ntt);
  Decomp_modup(&dst, &src, part);
}

void Ref_mod_down(const int64_t* in_ext, size_t level, int is_ntt,
                  int64_t* out) {
  POLYNOMIAL src, dst;
  Wrap_poly(&src, (int64_t*)in_ext, level, Get_p_cnt(), is_ntt);
  Wrap_poly(&dst, out, level, 0, is_ntt);
  Mod_down(&dst, &src);
}

uint32_t Ref_num_decomp(size_t level) {
  POLYNOMIAL p;
  Wrap_poly(&p, NULL, level, 0, 1);
  return (uint32_t)Num_decomp(&p);
}

uint32_t Ref_auto_idx(int32_t rot_idx) { return Auto_idx(rot_idx); }

void Ref_auto_order(int32_t rot_idx, int64_t* out) {
  memcpy(out, Auto_order(rot_idx), Degree() * sizeof(int64_t));
}

//! copies one polynomial of a switch key: all L Q limbs then K P limbs
void Ref_get_swk(int is_rot, int32_t rot_idx, uint32_t part, int which,
                 int64_t* out) {
  SW_KEY swk  = Swk(is_rot != 0, rot_idx);
  POLY   poly = which == 0 ? Pk0_at(swk, part) : Pk1_at(swk, part);
  size_t n    = Degree();
  memcpy(out, Get_poly_coeffs(poly), Poly_level(poly) * n * sizeof(int64_t));
  memcpy(out + Poly_level(poly) * n, Get_p_coeffs(poly),
         Num_p(poly) * n * sizeof(int64_t));
}

static void Wrap_ciph(CIPHERTEXT* c, int64_t* c0, int64_t* c1, size_t level,
                      double scale, uint32_t sf_degree) {
  memset(c, 0, sizeof(*c));
  Wrap_poly(&c->_c0_poly, c0, level, 0, 1);
  Wrap_poly(&c->_c1_poly, c1, level, 0, 1);
  c->_slots          = Degree() / 2;
  c->_scaling_factor = scale;
  c->_sf_degree      = sf_degree;
}

static void Export_ciph(CIPHERTEXT* c, int64_t* c0, int64_t* c1) {
  size_t bytes = Poly_level(Get_c0(c)) * Degree() * sizeof(int64_t);
  memcpy(c0, Get_poly_coeffs(Get_c0(c)), bytes);
  memcpy(c1, Get_poly_coeffs(Get_c1(c)), bytes);
}

//! Eval_fast_rotate (evaluator.c:524): key-switch, add c0, automorphism
void Ref_rotate(const int64_t* c0, const int64_t* c1, size_t level,
                int32_t rot_idx, int64_t* out0, int64_t* out1) {
  CIPHERTEXT in, out;
  Wrap_ciph(&in, (int64_t*)c0, (int64_t*)c1, level, Get_default_sc(), 1);
  memset(&out, 0, sizeof(out));
  Eval_fast_rotate(&out, &in, rot_idx, (CKKS_EVALUATOR*)Eval());
  Export_ciph(&out, out0, out1);
  Free_poly_data(Get_c0(&out));
  Free_poly_data(Get_c1(&out));
}

//! Mul_ciphertext (tensor + relinearise) then Rescale_ciphertext;
//! outputs have level-1 limbs
void Ref_mul_relin_rescale(const int64_t* a0, const int64_t* a1,
                           const int64_t* b0, const int64_t* b1, size_t level,
                           int64_t* out0, int64_t* out1) {
  CIPHERTEXT a, b, prod, res;
  double     sc = Get_default_sc();
  Wrap_ciph(&a, (int64_t*)a0, (int64_t*)a1, level, sc, 1);
  Wrap_ciph(&b, (int64_t*)b0, (int64_t*)b1, level, sc, 1);
  memset(&prod, 0, sizeof(prod));
  memset(&res, 0, sizeof(res));
  Mul_ciphertext(&prod, &a, &b, (CKKS_EVALUATOR*)Eval());
  Rescale_ciphertext(&res, &prod, (CKKS_EVALUATOR*)Eval());
  Export_ciph(&res, out0, out1);
  Free_poly_data(Get_c0(&prod));
  Free_poly_data(Get_c1(&prod));
  Free_poly_data(Get_c0(&res));
  Free_poly_data(Get_c1(&res));
}

//! relinearisation alone: (c0,c1,c2) -> (out0,out1) at the same level
void Ref_relinearize(const int64_t* c0, const int64_t* c1, const int64_t* c2,
                     size_t level, int64_t* out0, int64_t* out1) {
  POLYNOMIAL p0, p1, p2;
  CIPHERTEXT res;
  Wrap_poly(&p0, (int64_t*)c0, level, 0, 1);
  Wrap_poly(&p1, (int64_t*)c1, level, 0, 1);
  Wrap_poly(&p2, (int64_t*)c2, level, 0, 1);
  memset(&res, 0, sizeof(res));
  Relinearize_ciph3(&res, &p0, &p1, &p2, Get_default_sc(), 2, Degree() / 2,
                    (CKKS_EVALUATOR*)Eval());
  Export_ciph(&res, out0, out1);
  Free_poly_data(Get_c0(&res));
  Free_poly_data(Get_c1(&res));
}

/* ---- client side: keys, encode, encrypt, decrypt, decode ---- */

//! which: 0 secret key (coefficient form, L+K limbs), 1 secret key NTT form,
//! 2 / 3 public key polynomials (L limbs)
void Ref_export_key(int which, int64_t* out) {
  CKKS_KEY_GENERATOR* gen = (CKKS_KEY_GENERATOR*)Keygen();
  POLY                p   = which == 0   ? Get_sk_poly(gen->_secret_key)
                            : which == 1 ? Get_ntt_sk(gen->_secret_key)
                            : which == 2 ? Get_pk0(gen->_public_key)
                                         : Get_pk1(gen->_public_key);
  size_t              n   = Degree();
  memcpy(out, Get_poly_coeffs(p), Poly_level(p) * n * sizeof(int64_t));
  if (Num_p(p)) {
    memcpy(out + Poly_level(p) * n, Get_p_coeffs(p), Num_p(p) * n * sizeof(int64_t));
  }
}

//! values = len (re, im) pairs; out = level limbs in NTT form
void Ref_encode(const double* values, size_t len, uint32_t sf_degree, uint32_t level,
                int64_t* out) {
  VALUE_LIST* vec = Alloc_value_list(DCMPLX_TYPE, len);
  for (size_t i = 0; i < len; i++) {
    DCMPLX_VALUE_AT(vec, i) = values[2 * i] + values[2 * i + 1] * I;
  }
  PLAINTEXT plain;
  memset(&plain, 0, sizeof(plain));
  Encode_at_level_with_sf(&plain, (CKKS_ENCODER*)Encoder(), vec, level, 0, sf_degree);
  POLY p = Get_plain_poly(&plain);
  memcpy(out, Get_poly_coeffs(p), Poly_level(p) * Degree() * sizeof(int64_t));
  Free_poly_data(p);
  Free_value_list(vec);
}

//! as Ref_encode with an explicit slot count (sparse packing: slots < N/2)
void Ref_encode_slots(const double* values, size_t len, uint32_t slots, uint32_t sf_degree,
                      uint32_t level, int64_t* out) {
  VALUE_LIST* vec = Alloc_value_list(DCMPLX_TYPE, len);
  for (size_t i = 0; i < len; i++) {
    DCMPLX_VALUE_AT(vec, i) = values[2 * i] + values[2 * i + 1] * I;
  }
  PLAINTEXT plain;
  memset(&plain, 0, sizeof(plain));
  Encode_at_level_with_sf(&plain, (CKKS_ENCODER*)Encoder(), vec, level, slots, sf_degree);
  POLY p = Get_plain_poly(&plain);
  memcpy(out, Get_poly_coeffs(p), Poly_level(p) * Degree() * sizeof(int64_t));
  Free_poly_data(p);
  Free_value_list(vec);
}

//! scalar path of Encode_double (len == 1)
void Ref_encode_scalar(double value, uint32_t sf_degree, uint32_t level, int64_t* out) {
  PLAINTEXT plain;
  memset(&plain, 0, sizeof(plain));
  Encode_val_at_level(&plain, (CKKS_ENCODER*)Encoder(), value, level, sf_degree);
  POLY p = Get_plain_poly(&plain);
  memcpy(out, Get_poly_coeffs(p), Poly_level(p) * Degree() * sizeof(int64_t));
  Free_poly_data(p);
}

//! encrypts a plaintext polynomial (level limbs, NTT form)
void Ref_encrypt(const int64_t* plain_poly, size_t level, uint32_t sf_degree, int64_t* c0,
                 int64_t* c1) {
  PLAINTEXT  plain;
  CIPHERTEXT ciph;
  memset(&plain, 0, sizeof(plain));
  memset(&ciph, 0, sizeof(ciph));
  Wrap_poly(&plain._poly, (int64_t*)plain_poly, level, 0, 1);
  plain._slots          = Degree() / 2;
  plain._scaling_factor = pow(Get_default_sc(), sf_degree);
  plain._sf_degree      = sf_degree;
  Encrypt_msg(&ciph, (CKKS_ENCRYPTOR*)Encryptor(), &plain);
  Export_ciph(&ciph, c0, c1);
  Free_poly_data(Get_c0(&ciph));
  Free_poly_data(Get_c1(&ciph));
}

//! decrypts and decodes; out = count (re, im) pairs
void Ref_decrypt_decode(const int64_t* c0, const int64_t* c1, size_t level, uint32_t sf_degree,
                        double* out, size_t count) {
  size_t     n     = Degree();
  size_t     bytes = level * n * sizeof(int64_t);
  int64_t*   t0    = (int64_t*)malloc(bytes);
  int64_t*   t1    = (int64_t*)malloc(bytes);
  CIPHERTEXT ciph;
  PLAINTEXT  plain;
  memcpy(t0, c0, bytes);
  memcpy(t1, c1, bytes);
  Wrap_ciph(&ciph, t0, t1, level, pow(Get_default_sc(), sf_degree), sf_degree);
  memset(&plain, 0, sizeof(plain));
  Decrypt(&plain, (CKKS_DECRYPTOR*)Decryptor(), &ciph, NULL);
  VALUE_LIST* res = Alloc_value_list(DCMPLX_TYPE, count);
  Decode(res, (CKKS_ENCODER*)Encoder(), &plain);
  for (size_t i = 0; i < count; i++) {
    out[2 * i]     = creal(DCMPLX_VALUE_AT(res, i));
    out[2 * i + 1] = cimag(DCMPLX_VALUE_AT(res, i));
  }
  Free_value_list(res);
  Free_poly_data(Get_plain_poly(&plain));
  free(t0);
  free(t1);
}

//! Bootstrap (cipher.c:581): in = level limbs at scaling degree 1 with all
//! N/2 slots; returns the output level, out0/out1 must hold Get_q_cnt() limbs
size_t Ref_bootstrap(const int64_t* c0, const int64_t* c1, size_t level, uint32_t slots,
                     uint32_t level_after, int64_t* out0, int64_t* out1) {
  CIPHERTEXT in, out;
  Wrap_ciph(&in, (int64_t*)c0, (int64_t*)c1, level, Get_default_sc(), 1);
  in._slots = slots;
  memset(&out, 0, sizeof(out));
  Bootstrap(&out, &in, level_after);
  size_t out_level = Poly_level(Get_c0(&out));
  Export_ciph(&out, out0, out1);
  Free_poly_data(Get_c0(&out));
  Free_poly_data(Get_c1(&out));
  return out_level;
}

//! One plaintext of the bootstrapping linear transforms for N/2 slots:
//! writes its Q limbs then its special limbs, returns the Q limb count
//! (0 when that diagonal does not exist)
size_t Ref_bootstrap_plain(int encoding, uint32_t stage, uint32_t index, int64_t* out) {
  CKKS_BTS_CTX*    bts    = Get_bts_ctx((CKKS_EVALUATOR*)Eval());
  CKKS_BTS_PRECOM* precom = Get_bts_precom(bts, Degree() / 2);
  if (precom == NULL) return 0;
  VL_VL_PLAIN* all = encoding ? Get_u0hatt_pre_fft(precom) : Get_u0_pre_fft(precom);
  if (stage >= LIST_LEN(all)) return 0;
  VALUE_LIST* row = Get_vl_value_at(all, stage);
  if (index >= LIST_LEN(row)) return 0;
  PLAINTEXT* pt = (PLAINTEXT*)Get_ptr_value_at(row, index);
  if (pt == NULL) return 0;
  POLYNOMIAL* p = Get_plain_poly(pt);
  size_t      n = Degree();
  memcpy(out, Get_poly_coeffs(p), Poly_level(p) * n * sizeof(int64_t));
  memcpy(out + Poly_level(p) * n, Get_p_coeffs(p), Num_p(p) * n * sizeof(int64_t));
  return Poly_level(p);
}
