// C ABI of libFHErt_b200: the entry points declared in include/fhert_b200.h.
// Each function keeps the contract of the CPU runtime function of the same
// name (cited in the header) and queues CUDA kernels on the library stream.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "runtime.h"

using namespace fhert;

namespace {

CKKS_PARAMS* g_params = nullptr;

inline size_t alloc_words(POLY p) { return (size_t)p->_num_alloc_primes * p->_ring_degree; }

// allocation index of the first P limb (rns_poly_impl.h:43)
inline size_t p_offset(POLY p) { return p->_num_alloc_primes - p->_num_primes_p; }

int prime_index_of(Context* c, MODULUS* m) {
  // moduli handed out by Q_modulus()/P_modulus() point into c->moduli
  if (m >= c->moduli.data() && m < c->moduli.data() + c->moduli.size())
    return (int)(m - c->moduli.data());
  for (size_t i = 0; i < c->primes.size(); i++)
    if ((u64)m->_val == c->primes[i]) return (int)i;
  FHERT_ASSERT(false, "modulus %lld is not a prime of this context", (long long)m->_val);
  return -1;
}

LimbBatch single(int prime) {
  LimbBatch b;
  b.count   = 1;
  b.limb[0] = LimbRef{0, 0, 0, (uint16_t)prime};
  return b;
}

// Q limbs [0, level) and, when present, the K special limbs, with the limb
// offsets of each operand computed from its own allocation.
LimbBatch poly_batch(Context* c, POLY res, POLY a, POLY b, size_t level, size_t num_p) {
  LimbBatch bt;
  bt.count = 0;
  for (size_t i = 0; i < level; i++)
    bt.limb[bt.count++] = LimbRef{(uint16_t)i, (uint16_t)i, (uint16_t)i, (uint16_t)i};
  for (size_t k = 0; k < num_p; k++) {
    LimbRef r;
    r.a     = (uint16_t)(p_offset(a) + k);
    r.b     = (uint16_t)(b ? p_offset(b) + k : 0);
    r.dst   = (uint16_t)(p_offset(res) + k);
    r.prime = (uint16_t)(c->L + k);
    bt.limb[bt.count++] = r;
  }
  return bt;
}

void ensure_poly(POLY res, uint32_t degree, size_t num_q, size_t num_p) {
  if (res->_data == nullptr || res->_num_alloc_primes < num_q + num_p) {
    Free_poly_data(res);
    Alloc_poly_data(res, degree, num_q, num_p);
  } else {
    res->_ring_degree  = degree;
    res->_num_primes   = num_q;
    res->_num_primes_p = num_p;
  }
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------

__attribute__((weak)) CKKS_PARAMS* Get_context_params(void) { return g_params; }

void Fhert_set_context_params(uint32_t degree, size_t num_q, size_t q0_bits, size_t sf_bits,
                              size_t num_q_parts, size_t input_level, size_t hamming_weight,
                              size_t num_rot, const int32_t* rot_idxs) {
  std::free(g_params);
  g_params = (CKKS_PARAMS*)std::malloc(sizeof(CKKS_PARAMS) + num_rot * sizeof(int32_t));
  g_params->_provider         = LIB_ANT;
  g_params->_poly_degree      = degree;
  g_params->_sec_level        = 0;
  g_params->_mul_depth        = num_q - 1;
  g_params->_input_level      = input_level;
  g_params->_first_mod_size   = q0_bits;
  g_params->_scaling_mod_size = sf_bits;
  g_params->_num_q_parts      = num_q_parts;
  g_params->_hamming_weight   = hamming_weight;
  g_params->_num_rot_idx      = num_rot;
  if (num_rot) std::memcpy(g_params->_rot_idxs, rot_idxs, num_rot * sizeof(int32_t));
}

void Prepare_context(void) {
  if (ctx_or_null()) return;
  CKKS_PARAMS* p = Get_context_params();
  FHERT_ASSERT(p != nullptr, "Get_context_params returned no parameters");
  Context* c = create_context(p);
  for (size_t i = 0; i < p->_num_rot_idx; i++) auto_index_for(c, p->_rot_idxs[i]);
  std::printf(
      "ckks_param: _provider = %d, _poly_degree = %d, mul_depth = %ld, input_lev = %ld, "
      "_first_mod_size = %ld, _scaling_mod_size = %ld, _num_q_parts = %ld, _num_p = %ld, "
      "_num_rot_idx = %ld,_hamming_weight = %ld\n",
      (int)p->_provider, (int)p->_poly_degree, (long)p->_mul_depth, (long)p->_input_level,
      (long)p->_first_mod_size, (long)p->_scaling_mod_size, (long)p->_num_q_parts,
      (long)c->K, (long)p->_num_rot_idx, (long)p->_hamming_weight);
}

void Finalize_context(void) { destroy_context(); }

uint32_t Degree(void) { return ctx()->N; }
size_t   Get_q_cnt(void) { return ctx()->L; }
size_t   Get_p_cnt(void) { return ctx()->K; }
size_t   Get_q_parts(void) { return ctx()->dnum; }
size_t   Get_part_size(void) { return ctx()->alpha; }
MODULUS* Q_modulus(void) { return ctx()->moduli.data(); }
MODULUS* P_modulus(void) { return ctx()->moduli.data() + ctx()->L; }
double   Get_default_sc(void) { return std::pow(2.0, (double)ctx()->sf_bits); }

void Fhert_get_primes(int64_t* primes) {
  Context* c = ctx();
  for (size_t i = 0; i < c->primes.size(); i++) primes[i] = (int64_t)c->primes[i];
}

void Fhert_get_ntt_tables(size_t idx, int64_t* rou, uint64_t* rou_prec, int64_t* rou_inv,
                          uint64_t* rou_inv_prec, int64_t* degree_inv) {
  Context* c = ctx();
  FHERT_ASSERT(idx < c->primes.size(), "prime index out of range");
  for (uint32_t i = 0; i < c->N; i++) {
    rou[i]          = (int64_t)c->h_fwd[idx][i].w;
    rou_prec[i]     = c->h_fwd[idx][i].wp;
    rou_inv[i]      = (int64_t)c->h_inv[idx][i].w;
    rou_inv_prec[i] = c->h_inv[idx][i].wp;
  }
  *degree_inv = (int64_t)invmod(c->N % c->primes[idx], c->primes[idx]);
}

// ---------------------------------------------------------------------------
// memory
// ---------------------------------------------------------------------------

void Alloc_poly_data(POLY poly, uint32_t degree, size_t num_q, size_t num_p) {
  Context* c              = ctx();
  poly->_ring_degree      = degree;
  poly->_num_primes       = num_q;
  poly->_num_primes_p     = num_p;
  poly->_num_alloc_primes = num_q + num_p;
  poly->_is_ntt           = false;
  size_t bytes            = alloc_words(poly) * sizeof(int64_t);
  CUDA_CHECK(cudaMallocAsync(&poly->_data, bytes, c->stream));
  CUDA_CHECK(cudaMemsetAsync(poly->_data, 0, bytes, c->stream));
}

void Free_poly_data(POLY poly) {
  // rns_poly.c:1319-1325
  if (poly->_data) {
    CUDA_CHECK(cudaFreeAsync(poly->_data, ctx()->stream));
    poly->_data = nullptr;
  }
  poly->_num_alloc_primes = 0;
}

POLY Alloc_poly(uint32_t degree, size_t num_q, size_t num_p) {
  FHERT_ASSERT(num_q > 0, "Alloc_poly: q primes should not be NULL");
  POLY poly = (POLY)std::calloc(1, sizeof(POLYNOMIAL));
  // A special part is all-or-nothing: programs compiled against the older
  // boolean third argument pass 1 to ask for the extended basis.
  Alloc_poly_data(poly, degree, num_q, num_p ? ctx()->K : 0);
  poly->_is_ntt = true;
  return poly;
}

void Free_poly(POLY poly) {
  if (!poly) return;
  Free_poly_data(poly);
  std::free(poly);
}

void Init_poly_by_size(POLY res, size_t num_q, bool is_ext) {
  Context* c     = ctx();
  size_t   num_p = is_ext ? c->K : 0;
  if (res->_data == nullptr || res->_num_alloc_primes < num_q + num_p) {
    Free_poly_data(res);
    Alloc_poly_data(res, c->N, num_q, num_p);
  } else {
    res->_ring_degree  = c->N;
    res->_num_primes   = num_q;
    res->_num_primes_p = num_p;
  }
  res->_is_ntt = true;
}

void Copy_poly(POLY res, POLY poly) {
  if (res == poly) return;
  Context* c = ctx();
  FHERT_ASSERT(res->_num_primes == poly->_num_primes && res->_num_primes_p >= poly->_num_primes_p,
               "Copy_poly: size not match");
  size_t n = poly->_ring_degree;
  CUDA_CHECK(cudaMemcpyAsync(res->_data, poly->_data, poly->_num_primes * n * sizeof(int64_t),
                             cudaMemcpyDeviceToDevice, c->stream));
  if (poly->_num_primes_p)
    CUDA_CHECK(cudaMemcpyAsync(res->_data + p_offset(res) * n, poly->_data + p_offset(poly) * n,
                               res->_num_primes_p * n * sizeof(int64_t),
                               cudaMemcpyDeviceToDevice, c->stream));
  res->_is_ntt = poly->_is_ntt;
}

int64_t* Coeffs(POLY poly, uint32_t limb, uint32_t degree) {
  return poly->_data + (size_t)limb * degree;
}

void Set_coeffs(POLY poly, uint32_t limb, uint32_t degree, int64_t* src) {
  int64_t* dst = poly->_data + (size_t)limb * degree;
  if (dst == src) return;
  CUDA_CHECK(cudaMemcpyAsync(dst, src, (size_t)degree * sizeof(int64_t),
                             cudaMemcpyDeviceToDevice, ctx()->stream));
}

void Fhert_upload(POLY poly, size_t first, size_t limbs, const int64_t* host) {
  FHERT_ASSERT(poly->_data && first + limbs <= poly->_num_alloc_primes, "upload out of range");
  size_t n = poly->_ring_degree;
  CUDA_CHECK(cudaMemcpyAsync(poly->_data + first * n, host, limbs * n * sizeof(int64_t),
                             cudaMemcpyHostToDevice, ctx()->stream));
}

void Fhert_download(POLY poly, size_t first, size_t limbs, int64_t* host) {
  FHERT_ASSERT(poly->_data && first + limbs <= poly->_num_alloc_primes,
               "download out of range");
  size_t n = poly->_ring_degree;
  CUDA_CHECK(cudaMemcpyAsync(host, poly->_data + first * n, limbs * n * sizeof(int64_t),
                             cudaMemcpyDeviceToHost, ctx()->stream));
  CUDA_CHECK(cudaStreamSynchronize(ctx()->stream));
}

void     Fhert_sync(void) { CUDA_CHECK(cudaStreamSynchronize(ctx()->stream)); }
void*    Fhert_stream(void) { return (void*)ctx()->stream; }
uint64_t Fhert_kernel_launches(void) { return ctx_or_null() ? ctx()->launches : 0; }
void     Fhert_profile_begin(void) { prof_begin(); }
size_t   Fhert_profile_end(char* buf, size_t cap) { return prof_end(buf, cap); }

// ---------------------------------------------------------------------------
// per-limb vector operations
// ---------------------------------------------------------------------------

int64_t* Hw_modadd(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  launch_elementwise(EW_ADD, res, a, b, 0, single(prime_index_of(c, m)));
  return res;
}
int64_t* Hw_modsub(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  launch_elementwise(EW_SUB, res, a, b, 0, single(prime_index_of(c, m)));
  return res;
}
int64_t* Hw_modmul(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  launch_elementwise(EW_MUL, res, a, b, 0, single(prime_index_of(c, m)));
  return res;
}
int64_t* Hw_modmuladd(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  launch_elementwise(EW_MULADD, res, a, b, 0, single(prime_index_of(c, m)));
  return res;
}
int64_t* Hw_modadd_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  launch_elementwise(EW_ADD_SCALAR, res, a, nullptr, s, single(prime_index_of(c, m)));
  return res;
}
int64_t* Hw_modmul_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  launch_elementwise(EW_MUL_SCALAR, res, a, nullptr, s, single(prime_index_of(c, m)));
  return res;
}
int64_t* Hw_rotate(int64_t* res, int64_t* val, int64_t* order, MODULUS* m, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  FHERT_ASSERT(res != val, "Hw_rotate cannot work in place");
  launch_automorphism(res, val, reinterpret_cast<const uint32_t*>(order), single(0));
  return res;
}
void Hw_ntt(int64_t* res, int64_t* val, size_t mod_idx, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N && mod_idx < c->primes.size(), "Hw_ntt: bad arguments");
  launch_ntt(val, res, single((int)mod_idx), false);
}
void Hw_intt(int64_t* res, int64_t* val, size_t mod_idx, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N && mod_idx < c->primes.size(), "Hw_intt: bad arguments");
  launch_ntt(val, res, single((int)mod_idx), true);
}

// ---------------------------------------------------------------------------
// RNS polynomial operations
// ---------------------------------------------------------------------------

POLY Conv_poly2ntt_inplace(POLY poly) {
  FHERT_ASSERT(!poly->_is_ntt, "already ntt form");
  Context* c = ctx();
  launch_ntt(poly->_data, poly->_data,
             poly_batch(c, poly, poly, poly, poly->_num_primes, poly->_num_primes_p), false);
  poly->_is_ntt = true;
  return poly;
}

POLY Conv_ntt2poly_inplace(POLY poly) {
  FHERT_ASSERT(poly->_is_ntt, "already coefficient form");
  Context* c = ctx();
  launch_ntt(poly->_data, poly->_data,
             poly_batch(c, poly, poly, poly, poly->_num_primes, poly->_num_primes_p), true);
  poly->_is_ntt = false;
  return poly;
}

static POLY binary_poly(EwOp op, POLY res, POLY a, POLY b) {
  Context* c = ctx();
  FHERT_ASSERT(a->_num_primes == b->_num_primes || op == EW_MUL || true, "size");
  size_t level = res->_num_primes;
  FHERT_ASSERT(level <= a->_num_primes && level <= b->_num_primes, "operand level too low");
  size_t num_p = res->_num_primes_p;
  FHERT_ASSERT(num_p == 0 || (a->_num_primes_p == num_p && b->_num_primes_p == num_p),
               "unmatched special limbs");
  launch_elementwise(op, res->_data, a->_data, b->_data, 0,
                     poly_batch(c, res, a, b, level, num_p));
  res->_is_ntt = a->_is_ntt;
  return res;
}

POLY Add_poly(POLY res, POLY a, POLY b) { return binary_poly(EW_ADD, res, a, b); }
POLY Sub_poly(POLY res, POLY a, POLY b) { return binary_poly(EW_SUB, res, a, b); }
POLY Mul_poly(POLY res, POLY a, POLY b) { return binary_poly(EW_MUL, res, a, b); }

POLY Modswitch(POLY res, POLY poly) {
  size_t level = poly->_num_primes;
  FHERT_ASSERT(level >= 2, "polynomial level is too small to support modswitch");
  if (res != poly) {
    ensure_poly(res, poly->_ring_degree, level - 1, poly->_num_primes_p);
    CUDA_CHECK(cudaMemcpyAsync(res->_data, poly->_data,
                               (level - 1) * poly->_ring_degree * sizeof(int64_t),
                               cudaMemcpyDeviceToDevice, ctx()->stream));
    res->_is_ntt = poly->_is_ntt;
  } else {
    res->_num_primes = level - 1;
  }
  return res;
}

POLY Rescale(POLY res, POLY poly) {
  Context* c     = ctx();
  size_t   level = poly->_num_primes;
  FHERT_ASSERT(level >= 2, "Level of rescale opnd is too small");
  FHERT_ASSERT(res->_num_primes == level && res->_data, "Rescale: primes not match");
  FHERT_ASSERT(poly->_is_ntt, "Rescale: coefficient-form input is not supported");
  const uint32_t n  = c->N;
  const int      l  = (int)level - 1;
  int64_t*       sc = scratch((size_t)level * n);  // [0] = last limb, [1..] = lifted limbs
  LimbBatch      lb = single(l);
  lb.limb[0].a      = (uint16_t)l;
  lb.limb[0].dst    = 0;
  launch_ntt(poly->_data, sc, lb, true);
  LimbBatch bt;
  bt.count = l;
  for (int i = 0; i < l; i++)
    bt.limb[i] = LimbRef{(uint16_t)(1 + i), (uint16_t)(1 + i), (uint16_t)(1 + i), (uint16_t)i};
  launch_rescale_lift(sc, sc, l, bt);
  launch_ntt(sc, sc, bt, false);
  for (int i = 0; i < l; i++) bt.limb[i] = LimbRef{(uint16_t)i, (uint16_t)(1 + i), (uint16_t)i, (uint16_t)i};
  launch_rescale_combine(res->_data, poly->_data, sc, l, bt);
  res->_is_ntt     = true;
  res->_num_primes = level - 1;  // Modswitch(res, res)
  return res;
}

size_t Num_decomp(POLY poly) {
  // crt.c:1135: ceil(level / alpha), capped by dnum
  Context* c = ctx();
  size_t   d = (poly->_num_primes + c->alpha - 1) / c->alpha;
  return d > (size_t)c->dnum ? (size_t)c->dnum : d;
}

POLY Decomp(POLY res, POLY poly, uint32_t part) {
  Context* c     = ctx();
  size_t   level = poly->_num_primes;
  size_t   start = (size_t)c->alpha * part;
  FHERT_ASSERT(start < level, "Decomp: digit out of range");
  size_t len = std::min((size_t)c->alpha, level - start);
  if (res->_data == nullptr || res->_num_alloc_primes < len) {
    Free_poly_data(res);
    Alloc_poly_data(res, c->N, len, 0);
  } else {
    res->_num_primes   = len;
    res->_num_primes_p = 0;
  }
  CUDA_CHECK(cudaMemcpyAsync(res->_data, poly->_data + start * c->N,
                             len * c->N * sizeof(int64_t), cudaMemcpyDeviceToDevice, c->stream));
  res->_is_ntt = poly->_is_ntt;
  return res;
}

// Raises the digit limbs found at src (digit_len limbs, NTT form, limb j of
// the digit at src + j*N) to all other limbs of `res` (level Q limbs + K P).
static void raise_digit(Context* c, POLY res, const int64_t* digit_src, size_t level,
                        uint32_t part, bool is_ntt) {
  const uint32_t             n     = c->N;
  const Context::ModUpTable& t     = modup_table(c, (int)level, (int)part);
  const int                  start = c->alpha * (int)part;
  int64_t*                   sc    = scratch((size_t)t.digit_len * n);
  LimbBatch                  in;
  in.count = t.digit_len;
  for (int i = 0; i < t.digit_len; i++)
    in.limb[i] = LimbRef{(uint16_t)i, 0, (uint16_t)i, (uint16_t)(start + i)};
  const int64_t* coeff = digit_src;
  if (is_ntt) {
    launch_ntt(digit_src, sc, in, true);
    coeff = sc;
  }
  LimbBatch out;
  out.count = 0;
  for (int m = 0; m < (int)level; m++) {
    if (m >= start && m < start + t.digit_len) continue;
    out.limb[out.count++] = LimbRef{(uint16_t)m, (uint16_t)m, (uint16_t)m, (uint16_t)m};
  }
  for (int k = 0; k < c->K; k++) {
    uint16_t off = (uint16_t)(p_offset(res) + k), pr = (uint16_t)(c->L + k);
    out.limb[out.count++] = LimbRef{off, pr, off, pr};
  }
  launch_base_conv(res->_data, coeff, in, out, t.d_hat_inv, t.d_hat_mod, c->L + c->K, 1);
  if (is_ntt) launch_ntt(res->_data, res->_data, out, false);
}

POLY Decomp_modup(POLY res, POLY poly, uint32_t part) {
  Context* c     = ctx();
  size_t   level = poly->_num_primes;
  FHERT_ASSERT(res->_data && res->_num_primes == level && res->_num_primes_p == (size_t)c->K,
               "Decomp_modup: result must hold level + K limbs");
  size_t start = (size_t)c->alpha * part;
  FHERT_ASSERT(start < level, "Decomp_modup: digit out of range");
  size_t len = std::min((size_t)c->alpha, level - start);
  raise_digit(c, res, poly->_data + start * c->N, level, part, poly->_is_ntt);
  CUDA_CHECK(cudaMemcpyAsync(res->_data + start * c->N, poly->_data + start * c->N,
                             len * c->N * sizeof(int64_t), cudaMemcpyDeviceToDevice, c->stream));
  res->_is_ntt = poly->_is_ntt;
  return res;
}

POLY Mod_up(POLY res, POLY old_poly, uint32_t part) {
  Context* c     = ctx();
  size_t   level = res->_num_primes;
  FHERT_ASSERT(res->_data && res->_num_primes_p == (size_t)c->K, "Mod_up: result size not match");
  size_t start = (size_t)c->alpha * part;
  size_t len   = old_poly->_num_primes;
  raise_digit(c, res, old_poly->_data, level, part, old_poly->_is_ntt);
  CUDA_CHECK(cudaMemcpyAsync(res->_data + start * c->N, old_poly->_data,
                             len * c->N * sizeof(int64_t), cudaMemcpyDeviceToDevice, c->stream));
  res->_is_ntt = old_poly->_is_ntt;
  return res;
}

POLY Mod_down(POLY res, POLY poly) {
  Context*       c     = ctx();
  const uint32_t n     = c->N;
  size_t         level = poly->_num_primes;
  if (res->_data == nullptr) Alloc_poly_data(res, n, level, 0);
  FHERT_ASSERT(res->_num_primes == level && poly->_num_primes_p == (size_t)c->K,
               "Mod_down: result size not match");
  const int K  = c->K;
  int64_t*  sc = scratch((size_t)(K + level) * n);  // [0,K) P limbs, [K, K+level) conversions
  LimbBatch in;
  in.count = K;
  for (int k = 0; k < K; k++)
    in.limb[k] = LimbRef{(uint16_t)(p_offset(poly) + k), 0, (uint16_t)k, (uint16_t)(c->L + k)};
  const int64_t* coeff = poly->_data;
  if (poly->_is_ntt) {
    launch_ntt(poly->_data, sc, in, true);
    for (int k = 0; k < K; k++) in.limb[k].a = (uint16_t)k;
    coeff = sc;
  }
  LimbBatch out;
  out.count = (int)level;
  for (int i = 0; i < (int)level; i++)
    out.limb[i] = LimbRef{(uint16_t)(K + i), (uint16_t)i, (uint16_t)(K + i), (uint16_t)i};
  launch_base_conv(sc, coeff, in, out, c->d_phat_inv, c->d_phat_mod_q, 1, K);
  if (poly->_is_ntt) launch_ntt(sc, sc, out, false);
  for (int i = 0; i < (int)level; i++)
    out.limb[i] = LimbRef{(uint16_t)i, (uint16_t)(K + i), (uint16_t)i, (uint16_t)i};
  launch_moddown_combine(res->_data, poly->_data, sc, out);
  res->_is_ntt = poly->_is_ntt;
  return res;
}

POLY Extend(POLY res, POLY poly) {
  Context* c = ctx();
  FHERT_ASSERT(res->_num_primes == poly->_num_primes && poly->_data, "Extend: size not match");
  FHERT_ASSERT(res->_num_alloc_primes == poly->_num_primes + (size_t)c->K,
               "Extend: alloc_size not match");
  size_t n = c->N;
  CUDA_CHECK(cudaMemsetAsync(res->_data + p_offset(res) * n, 0, (size_t)c->K * n * sizeof(int64_t),
                             c->stream));
  launch_mul_const(res->_data, poly->_data, c->d_p_mod_q,
                   poly_batch(c, res, poly, nullptr, poly->_num_primes, 0));
  res->_num_primes_p = c->K;
  res->_is_ntt       = poly->_is_ntt;
  return res;
}

POLY Dot_prod(POLY res, POLY a, POLY b, size_t parts) {
  Context* c = ctx();
  FHERT_ASSERT(parts >= 1 && parts <= (size_t)kMaxParts, "Dot_prod: unsupported digit count");
  size_t level = a[0]._num_primes, num_p = a[0]._num_primes_p;
  ensure_poly(res, c->N, level, num_p);
  InnerArgs args;
  args.parts = (int)parts;
  for (size_t j = 0; j < parts; j++) {
    FHERT_ASSERT(a[j]._num_alloc_primes == a[0]._num_alloc_primes &&
                     b[j]._num_alloc_primes == b[0]._num_alloc_primes,
                 "Dot_prod: operands must share a layout");
    args.ext[j]  = reinterpret_cast<const u64*>(a[j]._data);
    args.key0[j] = reinterpret_cast<const u64*>(b[j]._data);
    args.key1[j] = nullptr;
  }
  launch_inner_product(res->_data, nullptr, args, poly_batch(c, res, &a[0], &b[0], level, num_p));
  res->_is_ntt = a[0]._is_ntt;
  return res;
}

POLY Automorphism_transform(POLY res, POLY poly, int64_t* order) {
  Context* c = ctx();
  FHERT_ASSERT(poly->_is_ntt, "Automorphism_transform: coefficient form is not supported");
  FHERT_ASSERT(res->_data != poly->_data, "Automorphism_transform cannot work in place");
  launch_automorphism(res->_data, poly->_data, reinterpret_cast<const uint32_t*>(order),
                      poly_batch(c, res, poly, nullptr, poly->_num_primes, poly->_num_primes_p));
  res->_is_ntt = true;
  return res;
}

// ---------------------------------------------------------------------------
// keys and automorphism tables
// ---------------------------------------------------------------------------

uint32_t Auto_idx(int32_t rot_idx) { return auto_index_for(ctx(), rot_idx); }

int64_t* Auto_order(int32_t rot_idx) {
  Context* c = ctx();
  uint32_t k = (rot_idx == (int32_t)(2 * c->N - 1)) ? (uint32_t)rot_idx : auto_index_for(c, rot_idx);
  return reinterpret_cast<int64_t*>(auto_table(c, k));
}

static SWITCH_KEY* key_slot(Context* c, uint32_t key_id, bool create) {
  auto it = c->keys.find(key_id);
  if (it != c->keys.end()) return it->second;
  if (!create) return nullptr;
  SWITCH_KEY* k = new SWITCH_KEY();
  k->_num_parts = c->dnum;
  k->_parts     = new PUBLIC_KEY[c->dnum];
  std::memset(k->_parts, 0, sizeof(PUBLIC_KEY) * c->dnum);
  size_t words = (size_t)(c->L + c->K) * c->N;
  for (int j = 0; j < c->dnum; j++) {
    for (POLYNOMIAL* p : {&k->_parts[j]._p0, &k->_parts[j]._p1}) {
      p->_ring_degree      = c->N;
      p->_num_primes       = c->L;
      p->_num_primes_p     = c->K;
      p->_num_alloc_primes = c->L + c->K;
      p->_is_ntt           = true;
      CUDA_CHECK(cudaMalloc(&p->_data, words * sizeof(int64_t)));
    }
  }
  c->keys[key_id] = k;
  return k;
}

static uint32_t key_id_for(Context* c, bool is_rot, int32_t rot_idx) {
  if (!is_rot) return 0;
  uint32_t conj = 2 * c->N - 1;
  return rot_idx == (int32_t)conj ? conj : auto_index_for(c, rot_idx);
}

SW_KEY Swk(bool is_rot, int32_t rot_idx) {
  Context*    c = ctx();
  SWITCH_KEY* k = key_slot(c, key_id_for(c, is_rot, rot_idx), false);
  FHERT_ASSERT(k != nullptr, "cannot find %s key for index %d", is_rot ? "rotation" : "relin",
               rot_idx);
  return k;
}

POLY Pk0_at(SW_KEY swk, uint32_t part) {
  FHERT_ASSERT(part < swk->_num_parts, "idx outof bound");
  return &swk->_parts[part]._p0;
}
POLY Pk1_at(SW_KEY swk, uint32_t part) {
  FHERT_ASSERT(part < swk->_num_parts, "idx outof bound");
  return &swk->_parts[part]._p1;
}
void Set_pk0(POLY pk, SW_KEY swk, uint32_t part) { *pk = *Pk0_at(swk, part); }
void Set_pk1(POLY pk, SW_KEY swk, uint32_t part) { *pk = *Pk1_at(swk, part); }

void Fhert_import_switch_key(bool is_rot, int32_t rot_idx, uint32_t part, int which,
                             const int64_t* host) {
  Context*    c = ctx();
  SWITCH_KEY* k = key_slot(c, key_id_for(c, is_rot, rot_idx), true);
  FHERT_ASSERT(part < k->_num_parts, "digit out of range");
  POLY   p     = which == 0 ? &k->_parts[part]._p0 : &k->_parts[part]._p1;
  size_t bytes = (size_t)(c->L + c->K) * c->N * sizeof(int64_t);
  CUDA_CHECK(cudaMemcpyAsync(p->_data, host, bytes, cudaMemcpyHostToDevice, c->stream));
  CUDA_CHECK(cudaStreamSynchronize(c->stream));
}

// ---------------------------------------------------------------------------
// ciphertext level
// ---------------------------------------------------------------------------

size_t Level(CIPHER ciph) { return ciph->_c0_poly._num_primes; }

void Free_ciph_poly(CIPHER ciph, uint32_t cnt) {
  for (uint32_t i = 0; i < cnt; i++) {
    Free_poly_data(&ciph[i]._c0_poly);
    Free_poly_data(&ciph[i]._c1_poly);
  }
}

static void init_ciph(CIPHER res, uint32_t degree, size_t level, size_t num_p, double sf,
                      uint32_t sf_degree, uint32_t slots) {
  ensure_poly(&res->_c0_poly, degree, level, num_p);
  ensure_poly(&res->_c1_poly, degree, level, num_p);
  res->_c0_poly._is_ntt = true;
  res->_c1_poly._is_ntt = true;
  res->_scaling_factor  = sf;
  res->_sf_degree       = sf_degree;
  res->_slots           = slots;
}

void Init_ciph_same_scale(CIPHER res, CIPHER a, CIPHER b) {
  CIPHER low = (b != nullptr && Level(b) < Level(a)) ? b : a;
  if (low->_c0_poly._data == nullptr) {
    std::memset(res, 0, sizeof(CIPHERTEXT));
    return;
  }
  init_ciph(res, low->_c0_poly._ring_degree, Level(low), low->_c0_poly._num_primes_p,
            low->_scaling_factor, low->_sf_degree, low->_slots);
}

void Init_ciph_up_scale(CIPHER res, CIPHER a, CIPHER b) {
  CIPHER low = Level(b) < Level(a) ? b : a;
  init_ciph(res, low->_c0_poly._ring_degree, Level(low), low->_c0_poly._num_primes_p,
            a->_scaling_factor * b->_scaling_factor, a->_sf_degree + b->_sf_degree, low->_slots);
}

void Init_ciph_down_scale(CIPHER res, CIPHER a) {
  FHERT_ASSERT(a->_sf_degree >= 2, "Scale degree of result dec to zero");
  init_ciph(res, a->_c0_poly._ring_degree, Level(a), a->_c0_poly._num_primes_p,
            a->_scaling_factor / Get_default_sc(), a->_sf_degree - 1, a->_slots);
}

void Init_ciph3_up_scale(CIPHER3 res, CIPHER a, CIPHER b) {
  CIPHER low   = Level(b) < Level(a) ? b : a;
  uint32_t deg = low->_c0_poly._ring_degree;
  for (POLYNOMIAL* p : {&res->_c0_poly, &res->_c1_poly, &res->_c2_poly}) {
    ensure_poly(p, deg, Level(low), 0);
    p->_is_ntt = true;
  }
  res->_scaling_factor = a->_scaling_factor * b->_scaling_factor;
  res->_sf_degree      = a->_sf_degree + b->_sf_degree;
  res->_slots          = low->_slots;
}

void Copy_ciph(CIPHER res, CIPHER ciph) {
  if (res == ciph) return;
  init_ciph(res, ciph->_c0_poly._ring_degree, Level(ciph), ciph->_c0_poly._num_primes_p,
            ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
  Copy_poly(&res->_c0_poly, &ciph->_c0_poly);
  Copy_poly(&res->_c1_poly, &ciph->_c1_poly);
}

CIPHER Add_ciph(CIPHER res, CIPHER a, CIPHER b) {
  Init_ciph_same_scale(res, a, b);
  Add_poly(&res->_c0_poly, &a->_c0_poly, &b->_c0_poly);
  Add_poly(&res->_c1_poly, &a->_c1_poly, &b->_c1_poly);
  return res;
}

CIPHER Sub_ciph(CIPHER res, CIPHER a, CIPHER b) {
  Init_ciph_same_scale(res, a, b);
  Sub_poly(&res->_c0_poly, &a->_c0_poly, &b->_c0_poly);
  Sub_poly(&res->_c1_poly, &a->_c1_poly, &b->_c1_poly);
  return res;
}

CIPHER3 Mul_ciph3(CIPHER3 res, CIPHER a, CIPHER b) {
  // evaluator.c:137-173: c0 = a0*b0, c1 = a0*b1 + a1*b0, c2 = a1*b1
  Context* c = ctx();
  Init_ciph3_up_scale(res, a, b);
  size_t  level = res->_c0_poly._num_primes;
  POLY    r0 = &res->_c0_poly, r1 = &res->_c1_poly, r2 = &res->_c2_poly;
  Mul_poly(r0, &a->_c0_poly, &b->_c0_poly);
  Mul_poly(r1, &a->_c0_poly, &b->_c1_poly);
  launch_elementwise(EW_MULADD, r1->_data, a->_c1_poly._data, b->_c0_poly._data, 0,
                     poly_batch(c, r1, &a->_c1_poly, &b->_c0_poly, level, 0));
  Mul_poly(r2, &a->_c1_poly, &b->_c1_poly);
  return res;
}

// Hybrid key switch of one polynomial (evaluator.c:411-462): digit-wise ModUp,
// inner product with the key over Q u P, ModDown of both accumulators.
static void switch_key(Context* c, POLY out0, POLY out1, POLY in, SW_KEY swk) {
  const uint32_t n     = c->N;
  size_t         level = in->_num_primes;
  size_t         parts = Num_decomp(in);
  FHERT_ASSERT(parts <= (size_t)kMaxParts, "too many digits");
  std::vector<POLYNOMIAL> ext(parts);
  for (size_t j = 0; j < parts; j++) {
    std::memset(&ext[j], 0, sizeof(POLYNOMIAL));
    Alloc_poly_data(&ext[j], n, level, c->K);
    Decomp_modup(&ext[j], in, (uint32_t)j);
  }
  POLYNOMIAL acc0, acc1;
  std::memset(&acc0, 0, sizeof(acc0));
  std::memset(&acc1, 0, sizeof(acc1));
  Alloc_poly_data(&acc0, n, level, c->K);
  Alloc_poly_data(&acc1, n, level, c->K);
  InnerArgs args;
  args.parts = (int)parts;
  for (size_t j = 0; j < parts; j++) {
    args.ext[j]  = reinterpret_cast<const u64*>(ext[j]._data);
    args.key0[j] = reinterpret_cast<const u64*>(swk->_parts[j]._p0._data);
    args.key1[j] = reinterpret_cast<const u64*>(swk->_parts[j]._p1._data);
  }
  launch_inner_product(acc0._data, acc1._data, args,
                       poly_batch(c, &acc0, &ext[0], &swk->_parts[0]._p0, level, c->K));
  acc0._is_ntt = acc1._is_ntt = true;
  Mod_down(out0, &acc0);
  Mod_down(out1, &acc1);
  for (size_t j = 0; j < parts; j++) Free_poly_data(&ext[j]);
  Free_poly_data(&acc0);
  Free_poly_data(&acc1);
}

CIPHER Relin(CIPHER res, CIPHER3 ciph) {
  // evaluator.c:288-305
  Context* c     = ctx();
  size_t   level = ciph->_c2_poly._num_primes;
  init_ciph(res, c->N, level, 0, ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
  switch_key(c, &res->_c0_poly, &res->_c1_poly, &ciph->_c2_poly, Swk(false, 0));
  Add_poly(&res->_c0_poly, &res->_c0_poly, &ciph->_c0_poly);
  Add_poly(&res->_c1_poly, &res->_c1_poly, &ciph->_c1_poly);
  return res;
}

CIPHER Mul_ciph(CIPHER res, CIPHER a, CIPHER b) {
  CIPHERTEXT3 t;
  std::memset(&t, 0, sizeof(t));
  Mul_ciph3(&t, a, b);
  Relin(res, &t);
  Free_poly_data(&t._c0_poly);
  Free_poly_data(&t._c1_poly);
  Free_poly_data(&t._c2_poly);
  return res;
}

CIPHER Rescale_ciph(CIPHER res, CIPHER ciph) {
  // evaluator.c:344-363
  size_t level = Level(ciph);
  FHERT_ASSERT(level > 1, "rescale: multiply level is not big enough");
  init_ciph(res, ciph->_c0_poly._ring_degree, level, 0,
            ciph->_scaling_factor / Get_default_sc(), ciph->_sf_degree - 1, ciph->_slots);
  Rescale(&res->_c0_poly, &ciph->_c0_poly);
  Rescale(&res->_c1_poly, &ciph->_c1_poly);
  return res;
}

static CIPHER rotate_with_key(CIPHER res, CIPHER ciph, int32_t rot_idx, uint32_t k) {
  // evaluator.c:503-522: key switch c1, add c0, then permute both polynomials
  Context*   c     = ctx();
  size_t     level = Level(ciph);
  CIPHERTEXT t;
  std::memset(&t, 0, sizeof(t));
  init_ciph(&t, c->N, level, 0, ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
  switch_key(c, &t._c0_poly, &t._c1_poly, &ciph->_c1_poly, Swk(true, rot_idx));
  Add_poly(&t._c0_poly, &t._c0_poly, &ciph->_c0_poly);
  if (res != ciph)
    init_ciph(res, c->N, level, 0, ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
  int64_t* order = reinterpret_cast<int64_t*>(auto_table(c, k));
  Automorphism_transform(&res->_c0_poly, &t._c0_poly, order);
  Automorphism_transform(&res->_c1_poly, &t._c1_poly, order);
  Free_poly_data(&t._c0_poly);
  Free_poly_data(&t._c1_poly);
  return res;
}

CIPHER Rotate_ciph(CIPHER res, CIPHER ciph, int32_t rot_idx) {
  return rotate_with_key(res, ciph, rot_idx, auto_index_for(ctx(), rot_idx));
}

CIPHER Conjugate_ciph(CIPHER res, CIPHER ciph) {
  int32_t conj = (int32_t)(2 * ctx()->N - 1);
  return rotate_with_key(res, ciph, conj, (uint32_t)conj);
}

}  // extern "C"
