// Entry points of the runtime API that the committed compiled programs do not
// exercise but the compiler's emit tables and hand-written hosts may call:
// polynomial arrays, operand-shaped initialisers, key polynomial views, the
// plaintext forms of add / multiply, scale management and message dumps.
// Citations name files inside fhe-cmplr/rtlib/ant/.
#include <cmath>
#include <cstring>
#include <vector>

#include "runtime.h"

using namespace fhert;

extern "C" {

// poly/src/rns_poly.c:39-55: cnt polynomials over one block of storage; the
// first element owns the block (Free_polys releases it)
POLY_ARR Alloc_polys(uint32_t cnt, uint32_t degree, size_t num_q, size_t num_p) {
  FHERT_ASSERT(cnt > 0, "Alloc_polys: zero array size specified");
  Context* c     = ctx();
  POLY_ARR res   = (POLY_ARR)std::calloc(cnt, sizeof(POLYNOMIAL));
  size_t   words = (num_q + num_p) * (size_t)degree;
  int64_t* data  = nullptr;
  CUDA_CHECK(dev_alloc(&data, words * cnt * sizeof(int64_t), c->stream));
  CUDA_CHECK(zero_async(data, words * cnt * sizeof(int64_t), c->stream));
  for (uint32_t i = 0; i < cnt; i++) {
    res[i]._ring_degree      = degree;
    res[i]._num_primes       = num_q;
    res[i]._num_primes_p     = num_p;
    res[i]._num_alloc_primes = num_q + num_p;
    res[i]._is_ntt           = false;
    res[i]._data             = data + (size_t)i * words;
  }
  return res;
}

void Free_polys(POLY_ARR polys) {  // include/poly/rns_poly.h:182-188
  FHERT_ASSERT(polys != nullptr, "null polynomial array");
  Context* c = ctx();
  if (polys[0]._data) CUDA_CHECK(dev_free(polys[0]._data, c->stream));
  std::free(polys);
}

// include/poly/rns_poly.h:216-245: shape res after the operand of lower level
POLY Init_poly_by_opnd(POLY res, POLY opnd1, POLY opnd2, bool is_ext) {
  Context* c      = ctx();
  POLY     picked = nullptr;
  if (opnd1 == nullptr || opnd1->_num_primes == 0) picked = opnd2;
  else if (opnd2 == nullptr || opnd2->_num_primes == 0) picked = opnd1;
  else picked = opnd1->_num_primes <= opnd2->_num_primes ? opnd1 : opnd2;
  if (picked == nullptr) return res;
  if (res->_data != nullptr && res->_num_primes >= picked->_num_primes) {
    FHERT_ASSERT(res->_ring_degree == picked->_ring_degree, "unmatched size");
    res->_num_primes = picked->_num_primes;
    if (is_ext) FHERT_ASSERT(res->_num_primes_p == (size_t)c->K, "invalid p number");
  } else {
    if (res->_data != nullptr) Free_poly_data(res);
    Alloc_poly_data(res, picked->_ring_degree, picked->_num_primes, is_ext ? c->K : 0);
  }
  res->_is_ntt = true;
  return res;
}

// include/ckks/key.h:94-118: shallow views of a switch key's polynomials
POLY Swk_c0(POLY res, size_t size, bool is_rot, int32_t rot_idx) {
  SW_KEY swk = Swk(is_rot, rot_idx);
  FHERT_ASSERT(size <= swk->_num_parts, "extra size provided");
  for (size_t i = 0; i < size; i++) res[i] = swk->_parts[i]._p0;
  return res;
}
POLY Swk_c1(POLY res, size_t size, bool is_rot, int32_t rot_idx) {
  SW_KEY swk = Swk(is_rot, rot_idx);
  FHERT_ASSERT(size <= swk->_num_parts, "extra size provided");
  for (size_t i = 0; i < size; i++) res[i] = swk->_parts[i]._p1;
  return res;
}

// poly/src/rns_poly.c:459-469: all digits of input raised to Q u P; res holds
// Num_decomp(input) extended polynomials (one batch of launches for all)
POLY_ARR Precomp(POLY_ARR res, size_t size, POLY input) {
  Context* c     = ctx();
  size_t   level = input->_num_primes;
  FHERT_ASSERT(size == Num_decomp(input), "length of precompute not match");
  for (size_t j = 0; j < size; j++) Decomp_modup(&res[j], input, (uint32_t)j);
  (void)c;
  (void)level;
  return res;
}

// ckks/src/evaluator.c:98-111
CIPHER Add_plain(CIPHER res, CIPHER ciph, PLAIN plain) {
  Context* c = ctx();
  size_t level = ciph->_c0_poly._num_primes;
  FHERT_ASSERT(plain->_poly._num_primes >= level, "plaintext level below the ciphertext's");
  if (res != ciph) {
    shape_like(c, res, ciph, ciph->_scaling_factor, ciph->_sf_degree);
    Copy_poly(&res->_c1_poly, &ciph->_c1_poly);
  }
  launch_elementwise(EW_ADD, ptr2(res->_c0_poly._data), ptr2(ciph->_c0_poly._data),
                     ptr2(plain->_poly._data), 0,
                     poly_batch(c, &res->_c0_poly, &ciph->_c0_poly, &plain->_poly, level, 0));
  return res;
}

// ckks/src/evaluator.c:192-216
CIPHER Mul_plain(CIPHER res, CIPHER ciph, PLAIN plain) {
  Context* c = ctx();
  size_t level = ciph->_c0_poly._num_primes, num_p = ciph->_c0_poly._num_primes_p;
  FHERT_ASSERT(plain->_poly._num_primes >= level && plain->_poly._num_primes_p == num_p,
               "unmatched mod");
  shape_like(c, res, ciph, ciph->_scaling_factor * plain->_scaling_factor,
             ciph->_sf_degree + plain->_sf_degree);
  LimbBatch one  = poly_batch(c, &res->_c0_poly, &ciph->_c0_poly, &plain->_poly, level, num_p);
  LimbBatch both = both_polys(one);
  for (int i = one.count; i < both.count; i++) both.limb[i].sel &= (uint8_t)~2;  // one plaintext
  launch_elementwise(EW_MUL, ptr2(res->_c0_poly._data, res->_c1_poly._data),
                     ptr2(ciph->_c0_poly._data, ciph->_c1_poly._data), ptr2(plain->_poly._data), 0,
                     both);
  return res;
}

void Modswitch_ciph(CIPHER ciph) { mod_switch(ciph); }  // evaluator.c:401-409

// evaluator.c:364-378: multiply by 2^mod_size, encoded as a constant
CIPHER Upscale_ciph(CIPHER res, CIPHER ciph, uint32_t mod_size) {
  Context* c        = ctx();
  double   up_scale = std::pow(2.0, (double)mod_size);
  size_t   level = ciph->_c0_poly._num_primes, num_p = ciph->_c0_poly._num_primes_p;
  std::vector<int64_t> s = encode_value(c, 1.0, (uint32_t)level, up_scale, (uint32_t)num_p);
  std::vector<u64>     sc(s.begin(), s.end());
  sc.insert(sc.end(), s.begin(), s.end());
  double   sf  = ciph->_scaling_factor * up_scale;
  uint32_t deg = ciph->_sf_degree + 1;
  shape_like(c, res, ciph, sf, deg);
  launch_scalars(true, ptr2(res->_c0_poly._data, res->_c1_poly._data),
                 ptr2(ciph->_c0_poly._data, ciph->_c1_poly._data), sc.data(), ct_batch(c, res, ciph));
  return res;
}

// evaluator.c:380-399: bring the scale to `waterline` bits by a rescale
CIPHER Downscale_ciph(CIPHER res, CIPHER ciph, uint32_t waterline) {
  Context* c = ctx();
  FHERT_ASSERT(ciph->_c0_poly._num_primes > 1, "Downscale: multiply level is not big enough");
  uint32_t sf_bits   = (uint32_t)c->sf_bits;
  uint32_t ciph_bits = (uint32_t)std::log2(ciph->_scaling_factor);
  FHERT_ASSERT(waterline <= sf_bits, "Downscale: waterline should not larger than scaling factor");
  FHERT_ASSERT(ciph_bits > sf_bits && ciph_bits < waterline + sf_bits,
               "Downscale: waterline is set too low or the scale of input ciph is too high");
  Upscale_ciph(ciph, ciph, waterline + sf_bits - ciph_bits);
  ciph->_sf_degree += 1;
  return Rescale_ciph(res, ciph);
}

// ckks/src/cipher.c:417-450: back to scaling degree 1, then the q_0 residues
// lifted to mod_size primes (0 = all)
CIPHER Raise_mod(CIPHER res, CIPHER ciph, uint32_t mod_size) {
  Context* c = ctx();
  raise_from_level0(c, res, ciph, mod_size ? mod_size : (uint32_t)c->L);
  return res;
}

CIPHER Mul_mono_ciph(CIPHER res, CIPHER ciph, uint32_t power) {  // evaluator.c:260-286
  mul_monomial(ctx(), res, ciph, power);
  return res;
}

// ckks/src/cipher.c: decrypted real parts printed the way the reference's
// trace and dump helpers do
void Print_cipher_msg(FILE* fp, const char* name, CIPHER ciph, uint32_t len) {
  double*  msg   = Get_msg(ciph);
  uint32_t slots = ciph->_slots;
  if (len > slots) len = slots;
  std::fprintf(fp, "[%s] level %zu sf_degree %u: [", name, ciph->_c0_poly._num_primes,
               ciph->_sf_degree);
  for (uint32_t i = 0; i < len; i++) std::fprintf(fp, "%s%.6f", i ? " " : "", msg[i]);
  std::fprintf(fp, "]\n");
  std::free(msg);
}

void Dump_cipher_msg(const char* name, CIPHER ciph, uint32_t len) {
  Print_cipher_msg(stdout, name, ciph, len);
  std::fflush(stdout);
}

}  // extern "C"
