// The single-limb polynomial interface of the reference's LPOLY emit target
// (fhe-cmplr/rtlib/ant/include/lpoly/poly.h:18-143, lpoly/src/poly.c): an L_POLY
// is one RNS limb; every operation forwards to the per-limb vector entry
// points, which record and batch as they do for POLY-level programs.  The
// reference allocates limb storage with malloc in inline functions of its
// header; here the storage is device memory, so those are entry points too.
#include <cstring>

#include "runtime.h"

using namespace fhert;

extern "C" {

void Alloc_lpoly_data(LPOLY poly, uint32_t ring_degree) {  // lpoly/poly.h:63-69
  Context* c         = ctx();
  poly->_ring_degree = ring_degree;
  poly->_is_ntt      = false;
  CUDA_CHECK(dev_alloc(&poly->_data, (size_t)ring_degree * sizeof(int64_t), c->stream));
  CUDA_CHECK(cudaMemsetAsync(poly->_data, 0, (size_t)ring_degree * sizeof(int64_t), c->stream));
}

void Init_lpoly_data(LPOLY poly, uint32_t ring_degree, int64_t* data) {  // lpoly/poly.h:72-77
  poly->_ring_degree = ring_degree;
  poly->_data        = data;
  poly->_is_ntt      = false;
}

void Free_lpoly_data(LPOLY poly) {  // lpoly/poly.h:80-85
  if (poly->_data) {
    Context* c = ctx();
    CUDA_CHECK(dev_free(poly->_data, c->stream));
    poly->_data = nullptr;
  }
}

LPOLY Alloc_lpoly(uint32_t degree) {  // lpoly/poly.h:88-94
  LPOLY poly = (LPOLY)std::calloc(1, sizeof(L_POLY));
  Alloc_lpoly_data(poly, degree);
  poly->_is_ntt = true;
  return poly;
}

void Free_lpoly(LPOLY poly) {  // lpoly/poly.h:97-101
  if (!poly) return;
  Free_lpoly_data(poly);
  std::free(poly);
}

void Zero_lpoly(LPOLY poly) {  // lpoly/poly.h:104-107
  Context* c = ctx();
  CUDA_CHECK(cudaMemsetAsync(poly->_data, 0, (size_t)poly->_ring_degree * sizeof(int64_t), c->stream));
}

void Copy_lpoly(LPOLY res, L_POLY poly) {  // lpoly/poly.h:110-114
  Context* c = ctx();
  CUDA_CHECK(counted_copy(res->_data, poly._data, (size_t)res->_ring_degree * sizeof(int64_t),
                          cudaMemcpyDeviceToDevice, c->stream));
  res->_is_ntt = poly._is_ntt;
}

// lpoly/src/poly.c:13-76
LPOLY Add_lpoly(LPOLY sum, L_POLY poly1, L_POLY poly2, MODULUS* mod) {
  Hw_modadd(sum->_data, poly1._data, poly2._data, mod, sum->_ring_degree);
  sum->_is_ntt = poly1._is_ntt;
  return sum;
}
LPOLY Add_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod) {
  Hw_modadd_scalar(res->_data, poly._data, scalar, mod, res->_ring_degree);
  res->_is_ntt = poly._is_ntt;
  return res;
}
LPOLY Sub_lpoly(LPOLY res, L_POLY poly1, L_POLY poly2, MODULUS* mod) {
  Hw_modsub(res->_data, poly1._data, poly2._data, mod, res->_ring_degree);
  res->_is_ntt = poly1._is_ntt;
  return res;
}
LPOLY Sub_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod) {
  Hw_modsub_scalar(res->_data, poly._data, scalar, mod, res->_ring_degree);
  res->_is_ntt = poly._is_ntt;
  return res;
}
LPOLY Mul_lpoly(LPOLY res, L_POLY poly1, L_POLY poly2, MODULUS* mod) {
  Hw_modmul(res->_data, poly1._data, poly2._data, mod, res->_ring_degree);
  res->_is_ntt = poly1._is_ntt;
  return res;
}
LPOLY Mul_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod) {
  Hw_modmul_scalar(res->_data, poly._data, scalar, mod, res->_ring_degree);
  res->_is_ntt = poly._is_ntt;
  return res;
}
LPOLY Mac_lpoly(LPOLY res, L_POLY poly1, L_POLY poly2, MODULUS* mod) {
  Hw_modmuladd(res->_data, poly1._data, poly2._data, mod, res->_ring_degree);
  res->_is_ntt = poly1._is_ntt;
  return res;
}
LPOLY Mac_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod) {
  Hw_modmuladd_scalar(res->_data, poly._data, scalar, mod, res->_ring_degree);
  res->_is_ntt = poly._is_ntt;
  return res;
}

// lpoly/src/poly.c:78-124: idx counts the Q primes first, then the special primes
void Ntt(LPOLY res, L_POLY poly, size_t idx) {
  FHERT_ASSERT(!poly._is_ntt, "already ntt form");
  Hw_ntt(res->_data, poly._data, idx, res->_ring_degree);
  res->_is_ntt = true;
}
void Intt(LPOLY res, L_POLY poly, size_t idx) {
  FHERT_ASSERT(poly._is_ntt, "already coeffcient form");
  Hw_intt(res->_data, poly._data, idx, res->_ring_degree);
  res->_is_ntt = false;
}

}  // extern "C"
