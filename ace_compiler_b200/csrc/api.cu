// C ABI of libFHErt_b200: the entry points declared in include/fhert_b200.h.
// Each function keeps the contract of the CPU runtime function of the same
// name (cited in the header) and queues CUDA kernels on the library stream.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

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
  b.limb[0] = LimbRef{0, 0, 0, (uint8_t)prime, 0};
  return b;
}

}  // namespace

namespace fhert {

// Q limbs [0, level) and, when present, the K special limbs, with the limb
// offsets of each operand computed from its own allocation.
LimbBatch poly_batch(Context* c, POLY res, POLY a, POLY b, size_t level, size_t num_p) {
  LimbBatch bt;
  bt.count = 0;
  for (size_t i = 0; i < level; i++)
    bt.limb[bt.count++] = LimbRef{(uint16_t)i, (uint16_t)i, (uint16_t)i, (uint8_t)i, 0};
  for (size_t k = 0; k < num_p; k++) {
    LimbRef r;
    r.a     = (uint16_t)(p_offset(a) + k);
    r.b     = (uint16_t)(b ? p_offset(b) + k : 0);
    r.dst   = (uint16_t)(p_offset(res) + k);
    r.prime = (uint8_t)(c->L + k);
    r.sel   = 0;
    bt.limb[bt.count++] = r;
  }
  return bt;
}

// Appends the limbs of a second polynomial (second base pointer of every
// operand) to a batch built for the first one.
LimbBatch both_polys(const LimbBatch& one) {
  LimbBatch bt = one;
  for (int i = 0; i < one.count; i++) {
    LimbRef r = one.limb[i];
    r.sel     = 7;
    bt.limb[bt.count++] = r;
  }
  return bt;
}

void ensure_poly(POLY res, uint32_t degree, size_t num_q, size_t num_p) {
  // special limbs live at the end of the allocation: a polynomial that has
  // them must own exactly num_q + num_p limbs
  if (res->_data == nullptr || (num_p ? res->_num_alloc_primes != num_q + num_p
                                      : res->_num_alloc_primes < num_q)) {
    Free_poly_data(res);
    // the callers write every limb they ask for, so the fresh storage is not
    // cleared (a program's own allocations are: Alloc_poly_data)
    Context* c              = ctx();
    res->_ring_degree       = degree;
    res->_num_primes        = num_q;
    res->_num_primes_p      = num_p;
    res->_num_alloc_primes  = num_q + num_p;
    res->_is_ntt            = false;
    CUDA_CHECK(dev_alloc(&res->_data, (num_q + num_p) * (size_t)degree * sizeof(int64_t),
                               c->stream));
  } else {
    res->_ring_degree  = degree;
    res->_num_primes   = num_q;
    res->_num_primes_p = num_p;
  }
}

}  // namespace fhert

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
  // FHERT_PIN=<n> fixes the key / encryption randomness of a program that does
  // not call Fhert_seed itself, so that two runs can be compared bit for bit
  if (const char* pin = std::getenv("FHERT_PIN")) {
    uint32_t words[16];
    long     v = std::atol(pin);
    for (int k = 0; k < 16; k++) words[k] = (uint32_t)(v * 2654435761u + 40503u * k);
    Fhert_seed(words, 0, 1700000000000000ll + v);
  }
  Context* c = create_context(p);
  for (size_t i = 0; i < p->_num_rot_idx; i++) auto_index_for(c, p->_rot_idxs[i]);
  const char* skip = std::getenv("FHERT_SKIP_KEYGEN");
  if (!(skip != nullptr && skip[0] != '\0' && skip[0] != '0')) {
    generate_keys(c);
    // ckks_context.c:141-149: deep contexts get the bootstrapping plaintexts
    // and keys for full packing right away, unless the program opts out
    const char* no_bts = std::getenv("RTLIB_DISABLE_BOOTSTRAP_PRECOM");
    if (!(no_bts != nullptr && no_bts[0] != '\0' && no_bts[0] != '0'))
      prepare_bootstrap(c, p->_poly_degree / 2);
  }
  // ckks_context.c:151-154: open the program's weight file when it names one
  RT_DATA_INFO* info = Get_rt_data_info();
  if (info != nullptr) {
    // FHERT_DATA_FILE points a program at a weight file somewhere else than
    // the path compiled into it
    const char* moved = std::getenv("FHERT_DATA_FILE");
    const char* path  = moved != nullptr && moved[0] != '\0' ? moved : info->_file_name;
    bool        ok    = Pt_mgr_init(path);
    FHERT_ASSERT(ok, "cannot open data file %s", path);
  }
  std::printf(
      "ckks_param: _provider = %d, _poly_degree = %d, mul_depth = %ld, input_lev = %ld, "
      "_first_mod_size = %ld, _scaling_mod_size = %ld, _num_q_parts = %ld, _num_p = %ld, "
      "_num_rot_idx = %ld,_hamming_weight = %ld\n",
      (int)p->_provider, (int)p->_poly_degree, (long)p->_mul_depth, (long)p->_input_level,
      (long)p->_first_mod_size, (long)p->_scaling_mod_size, (long)c->dnum,
      (long)c->K, (long)p->_num_rot_idx, (long)p->_hamming_weight);
}

void Finalize_context(void) {
  if (ctx_or_null() == nullptr) return;
  Fhert_tm_report();
  Pt_mgr_fini();
  destroy_context();
}

uint32_t Degree(void) { return ctx_noflush()->N; }
size_t   Get_q_cnt(void) { return ctx_noflush()->L; }
size_t   Get_p_cnt(void) { return ctx_noflush()->K; }
size_t   Get_q_parts(void) { return ctx_noflush()->dnum; }
size_t   Get_part_size(void) { return ctx_noflush()->alpha; }
MODULUS* Q_modulus(void) { return ctx_noflush()->moduli.data(); }
MODULUS* P_modulus(void) { return ctx_noflush()->moduli.data() + ctx_noflush()->L; }
double   Get_default_sc(void) { return std::pow(2.0, (double)ctx_noflush()->sf_bits); }

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
  CUDA_CHECK(dev_alloc(&poly->_data, bytes, c->stream));
  CUDA_CHECK(zero_async(poly->_data, bytes, c->stream));
}

void Free_poly_data(POLY poly) {
  // rns_poly.c:1319-1325
  if (poly->_data) {
    Context* c = ctx();
    if (!pt_cache_owns(poly->_data)) CUDA_CHECK(dev_free(poly->_data, c->stream));
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
  CUDA_CHECK(counted_copy(res->_data, poly->_data, poly->_num_primes * n * sizeof(int64_t),
                             cudaMemcpyDeviceToDevice, c->stream));
  if (poly->_num_primes_p)
    CUDA_CHECK(counted_copy(res->_data + p_offset(res) * n, poly->_data + p_offset(poly) * n,
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
  Context* c = ctx_noflush();
  if (degree == c->N && hw_record(c, HW_COPY, dst, src, nullptr, nullptr, 0, 0)) return;
  CUDA_CHECK(counted_copy(dst, src, (size_t)degree * sizeof(int64_t),
                             cudaMemcpyDeviceToDevice, ctx()->stream));
}

void Fhert_upload(POLY poly, size_t first, size_t limbs, const int64_t* host) {
  FHERT_ASSERT(poly->_data && first + limbs <= poly->_num_alloc_primes, "upload out of range");
  size_t n = poly->_ring_degree;
  CUDA_CHECK(counted_copy(poly->_data + first * n, host, limbs * n * sizeof(int64_t),
                             cudaMemcpyHostToDevice, ctx()->stream));
}

void Fhert_download(POLY poly, size_t first, size_t limbs, int64_t* host) {
  FHERT_ASSERT(poly->_data && first + limbs <= poly->_num_alloc_primes,
               "download out of range");
  size_t n = poly->_ring_degree;
  CUDA_CHECK(counted_copy(host, poly->_data + first * n, limbs * n * sizeof(int64_t),
                             cudaMemcpyDeviceToHost, ctx()->stream));
  CUDA_CHECK(stream_sync(ctx()->stream));
}

void     Fhert_sync(void) { CUDA_CHECK(stream_sync(ctx()->stream)); }
void*    Fhert_stream(void) { return (void*)ctx()->stream; }
uint64_t Fhert_kernel_launches(void) { return ctx_or_null() ? ctx()->launches : 0; }
void     Fhert_transfer_bytes(uint64_t* h2d, uint64_t* d2h) {
  Context* c = ctx_or_null();
  if (h2d) *h2d = c ? c->h2d_bytes : 0;
  if (d2h) *d2h = c ? c->d2h_bytes : 0;
}
void     Fhert_profile_begin(void) { prof_begin(); }
size_t   Fhert_profile_end(char* buf, size_t cap) { return prof_end(buf, cap); }


// ---------------------------------------------------------------------------
// per-limb vector operations
// ---------------------------------------------------------------------------

static int64_t* hw_binary(EwOp op, int64_t* res, int64_t* a, int64_t* b, int64_t s, MODULUS* m,
                          uint32_t degree) {
  Context* c = ctx_noflush();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  int prime = prime_index_of(c, m);
  if (hw_record(c, (HwKind)op, res, a, b, nullptr, s, prime)) return res;
  launch_elementwise(op, ptr2(res), ptr2(a), ptr2(b), s, single(prime));
  return res;
}

int64_t* Hw_modadd(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  return hw_binary(EW_ADD, res, a, b, 0, m, degree);
}
int64_t* Hw_modsub(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  return hw_binary(EW_SUB, res, a, b, 0, m, degree);
}
int64_t* Hw_modmul(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  return hw_binary(EW_MUL, res, a, b, 0, m, degree);
}
int64_t* Hw_modmuladd(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree) {
  return hw_binary(EW_MULADD, res, a, b, 0, m, degree);
}
int64_t* Hw_modadd_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree) {
  return hw_binary(EW_ADD_SCALAR, res, a, a, s, m, degree);
}
int64_t* Hw_modmul_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree) {
  return hw_binary(EW_MUL_SCALAR, res, a, a, s, m, degree);
}
int64_t* Hw_modsub_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree) {
  // hal.c:56-66: a - s = a + (-s); the scalar is reduced into [0, q) when recorded
  return hw_binary(EW_ADD_SCALAR, res, a, a, -s, m, degree);
}
int64_t* Hw_modmuladd_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree) {
  // hal.c:109-121; no compiled program emits it, so it is launched at once
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  launch_elementwise(EW_MULADD_SCALAR, ptr2(res), ptr2(a), ptr2(a), s, single(prime_index_of(c, m)));
  return res;
}
int64_t* Hw_rotate(int64_t* res, int64_t* val, int64_t* order, MODULUS* m, uint32_t degree) {
  Context* c = ctx_noflush();
  FHERT_ASSERT(degree == c->N, "degree mismatch");
  FHERT_ASSERT(res != val, "Hw_rotate cannot work in place");
  const uint32_t* table = reinterpret_cast<const uint32_t*>(order);
  if (hw_record(c, HW_ROTATE, res, val, nullptr, table, 0, 0)) return res;
  launch_automorphism(ptr2(res), ptr2(val), reinterpret_cast<const uint32_t*>(order), single(0));
  return res;
}
void Hw_ntt(int64_t* res, int64_t* val, size_t mod_idx, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N && mod_idx < c->primes.size(), "Hw_ntt: bad arguments");
  launch_ntt(ptr2(val), ptr2(res), single((int)mod_idx), false);
}
void Hw_intt(int64_t* res, int64_t* val, size_t mod_idx, uint32_t degree) {
  Context* c = ctx();
  FHERT_ASSERT(degree == c->N && mod_idx < c->primes.size(), "Hw_intt: bad arguments");
  launch_ntt(ptr2(val), ptr2(res), single((int)mod_idx), true);
}

// ---------------------------------------------------------------------------
// RNS polynomial operations
// ---------------------------------------------------------------------------

POLY Conv_poly2ntt_inplace(POLY poly) {
  FHERT_ASSERT(!poly->_is_ntt, "already ntt form");
  Context* c = ctx();
  launch_ntt(ptr2(poly->_data), ptr2(poly->_data),
             poly_batch(c, poly, poly, poly, poly->_num_primes, poly->_num_primes_p), false);
  poly->_is_ntt = true;
  return poly;
}

POLY Conv_ntt2poly_inplace(POLY poly) {
  FHERT_ASSERT(poly->_is_ntt, "already coefficient form");
  Context* c = ctx();
  launch_ntt(ptr2(poly->_data), ptr2(poly->_data),
             poly_batch(c, poly, poly, poly, poly->_num_primes, poly->_num_primes_p), true);
  poly->_is_ntt = false;
  return poly;
}

// rns_poly.c:637-669: Q and special limbs
void Conv_poly2ntt(POLY res, POLY poly) {
  FHERT_ASSERT(!poly->_is_ntt, "already ntt form");
  FHERT_ASSERT(res->_ring_degree == poly->_ring_degree && res->_num_primes == poly->_num_primes &&
                   res->_num_primes_p == poly->_num_primes_p, "size not match");
  Context* c = ctx();
  launch_ntt(ptr2(poly->_data), ptr2(res->_data),
             poly_batch(c, res, poly, poly, poly->_num_primes, poly->_num_primes_p), false);
  res->_is_ntt = true;
}

// rns_poly_impl.c:202-234: Q and special limbs
void Conv_ntt2poly(POLY res, POLY poly) {
  FHERT_ASSERT(poly->_is_ntt, "already coefficient form");
  FHERT_ASSERT(res->_ring_degree == poly->_ring_degree && res->_num_primes == poly->_num_primes &&
                   res->_num_primes_p == poly->_num_primes_p, "size not match");
  Context* c = ctx();
  launch_ntt(ptr2(poly->_data), ptr2(res->_data),
             poly_batch(c, res, poly, poly, poly->_num_primes, poly->_num_primes_p), true);
  res->_is_ntt = false;
}

static POLY binary_poly(EwOp op, POLY res, POLY a, POLY b) {
  Context* c = ctx();
  // operands in coefficient form are brought to NTT form in place, as the CPU
  // runtime does: always for a product, only on a mismatch for sums
  // (rns_poly.c:852-858, 900-906, 950-956)
  if (op == EW_MUL) {
    if (!a->_is_ntt) Conv_poly2ntt_inplace(a);
    if (!b->_is_ntt) Conv_poly2ntt_inplace(b);
  } else if (a->_is_ntt != b->_is_ntt) {
    if (!a->_is_ntt) Conv_poly2ntt_inplace(a);
    else Conv_poly2ntt_inplace(b);
  }
  size_t level = res->_num_primes;
  FHERT_ASSERT(level <= a->_num_primes && level <= b->_num_primes, "operand level too low");
  size_t num_p = res->_num_primes_p;
  FHERT_ASSERT(num_p == 0 || (a->_num_primes_p == num_p && b->_num_primes_p == num_p),
               "unmatched special limbs");
  launch_elementwise(op, ptr2(res->_data), ptr2(a->_data), ptr2(b->_data), 0,
                     poly_batch(c, res, a, b, level, num_p));
  res->_is_ntt = op == EW_MUL ? true : a->_is_ntt;
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
    if (poly->_num_primes_p)  // only the Q limbs are copied: the special limbs read as zero
      CUDA_CHECK(zero_async(res->_data, alloc_words(res) * sizeof(int64_t), ctx()->stream));
    CUDA_CHECK(counted_copy(res->_data, poly->_data,
                               (level - 1) * poly->_ring_degree * sizeof(int64_t),
                               cudaMemcpyDeviceToDevice, ctx()->stream));
    res->_is_ntt = poly->_is_ntt;
  } else {
    res->_num_primes = level - 1;
  }
  return res;
}

// Rescale of one or two polynomials of the same level in NTT form
// (rns_poly.c:310-404): inverse NTT of the dropped limb(s), centred lift and
// scaling per remaining limb, forward NTT, combine.  Each step is one launch
// for all limbs of both polynomials.
void fhert_rescale_polys(Context* c, int npoly, int64_t* const res[2],
                          const int64_t* const poly[2], size_t level) {
  const uint32_t n = c->N;
  const int      l = (int)level - 1;
  FHERT_ASSERT(npoly * l <= kMaxLimbs, "rescale batch too large");
  int64_t*  sc = scratch((size_t)npoly * level * n);  // [npoly] dropped limbs, then lifted limbs
  LimbBatch lb;
  lb.count = npoly;
  for (int g = 0; g < npoly; g++)
    lb.limb[g] = LimbRef{(uint16_t)l, 0, (uint16_t)g, (uint8_t)l, (uint8_t)g};
  launch_ntt(ptr2(poly[0], poly[1]), ptr2(sc), lb, true);
  LimbBatch bt;
  bt.count = npoly * l;
  if (ntt_can_fuse()) {
    // lift inside the first pass of the forward transform, combine inside its last
    for (int g = 0; g < npoly; g++)
      for (int i = 0; i < l; i++) {
        uint8_t sel = (uint8_t)(g ? (2 | 4) : 0);  // aux (poly) and res from the second base
        bt.limb[g * l + i] = LimbRef{(uint16_t)g, (uint16_t)i, (uint16_t)i, (uint8_t)i, sel};
      }
    NttFuse f;
    f.pro_mul  = c->d_ql_neg + (size_t)l * c->L;
    f.pro_mod  = c->d_ql_mod + (size_t)l * c->L;
    f.q_last   = c->primes[l];
    f.epi_kind = 1;
    f.epi_mul  = c->d_ql_inv + (size_t)l * c->L;
    f.aux      = ptr2(poly[0], poly[1]);
    launch_ntt_fused(ptr2(sc), sc + (size_t)npoly * n, ptr2(res[0], res[1]), bt, f);
    return;
  }
  for (int g = 0; g < npoly; g++)
    for (int i = 0; i < l; i++) {
      uint16_t t = (uint16_t)(npoly + g * l + i);
      bt.limb[g * l + i] = LimbRef{t, (uint16_t)g, t, (uint8_t)i, 0};
    }
  launch_rescale_lift(ptr2(sc), ptr2(sc), l, bt);
  launch_ntt(ptr2(sc), ptr2(sc), bt, false);
  for (int g = 0; g < npoly; g++)
    for (int i = 0; i < l; i++) {
      uint8_t sel = (uint8_t)(g ? (1 | 4) : 0);  // poly and res from the second base
      bt.limb[g * l + i] =
          LimbRef{(uint16_t)i, (uint16_t)(npoly + g * l + i), (uint16_t)i, (uint8_t)i, sel};
    }
  launch_rescale_combine(ptr2(res[0], res[1]), ptr2(poly[0], poly[1]), ptr2(sc), l, bt);
}

// The two polynomials of a ciphertext are rescaled (or brought down from the
// extended basis) by two calls in a row.  The device work of the first call
// waits for the second and both run as one batch of launches; any other entry
// point runs a waiting call on its own first (ctx()).
static void pair_run(Context* c, int kind, int npoly, int64_t* const r[2],
                     const int64_t* const x[2], size_t level, int p_limb, bool is_ntt) {
  if (kind == 1) fhert_mod_down_polys(c, npoly, r, x, p_limb, nullptr, level, is_ntt);
  else fhert_rescale_polys(c, npoly, r, x, level);
}

}  // extern "C"

namespace fhert {
void pair_flush(Context* c) {
  auto w = c->pair_wait;
  if (!w.kind) return;
  c->pair_wait.kind   = 0;
  int64_t*       r[2] = {w.res, nullptr};
  const int64_t* x[2] = {w.src, nullptr};
  pair_run(c, w.kind, 1, r, x, w.level, w.p_limb, w.is_ntt);
}
}  // namespace fhert

extern "C" {

static void pair_submit(int kind, int64_t* res, const int64_t* src, size_t level, int p_limb,
                        bool is_ntt) {
  Context* c = ctx_noflush();
  if (c->hw_pending) ctx();  // per-limb calls recorded since: everything older runs now
  auto& w = c->pair_wait;
  if (w.kind == kind && w.level == level && w.p_limb == p_limb && w.is_ntt == is_ntt &&
      w.res != res && w.res != src && w.src != res) {
    int64_t*       r[2] = {w.res, res};
    const int64_t* x[2] = {w.src, src};
    w.kind              = 0;
    pair_run(c, kind, 2, r, x, level, p_limb, is_ntt);
    return;
  }
  if (w.kind) ctx();  // an unrelated call was waiting: it runs alone
  w.kind   = kind;
  w.res    = res;
  w.src    = src;
  w.level  = level;
  w.p_limb = p_limb;
  w.is_ntt = is_ntt;
}

POLY Rescale(POLY res, POLY poly) {
  size_t level = poly->_num_primes;
  FHERT_ASSERT(level >= 2, "Level of rescale opnd is too small");
  FHERT_ASSERT(res->_num_primes == level && res->_data, "Rescale: primes not match");
  if (!poly->_is_ntt) {  // rns_poly.c:381-399: stays in coefficient form
    ctx();
    launch_rescale_coeff(ptr2(res->_data), ptr2(poly->_data), 1, (int)level);
    res->_is_ntt     = false;
    res->_num_primes = level - 1;
    return res;
  }
  pair_submit(2, res->_data, poly->_data, level, 0, true);
  res->_is_ntt     = true;
  res->_num_primes = level - 1;  // Modswitch(res, res)
  return res;
}

size_t Num_decomp(POLY poly) {
  // crt.c:1135: ceil(level / alpha), capped by dnum
  Context* c = ctx_noflush();
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
  CUDA_CHECK(counted_copy(res->_data, poly->_data + start * c->N,
                             len * c->N * sizeof(int64_t), cudaMemcpyDeviceToDevice, c->stream));
  res->_is_ntt = poly->_is_ntt;
  return res;
}

static void fhert_launch_ntt_chunked(Ptr2 in, Ptr2 out, const std::vector<LimbRef>& limbs, bool inverse) {
  for (size_t off = 0; off < limbs.size(); off += kMaxLimbs) {
    LimbBatch b;
    b.count = (int)std::min((size_t)kMaxLimbs, limbs.size() - off);
    std::copy(limbs.begin() + off, limbs.begin() + off + b.count, b.limb);
    launch_ntt(in, out, b, inverse);
  }
}

// ModUp of digits [part_begin, part_end) of a level-`level` polynomial whose Q
// limbs start at `src` (rns_poly.c:160-258).  Digit j is raised into the
// extended polynomial at ext_base + (j - part_begin) * part_stride limbs: its
// level Q limbs at limb 0.. and its K special limbs at limb p_limb...  Only the
// complement limbs are written; the digit's own limbs are left to the caller.
// One inverse-NTT launch, one base-conversion launch and one forward-NTT
// launch cover all digits.
void fhert_raise_parts(Context* c, const int64_t* src, bool is_ntt, size_t level,
                        int part_begin, int part_end, int64_t* ext_base, size_t part_stride,
                        int p_limb) {
  const uint32_t n = c->N;
  const int      K = c->K;
  const int64_t* coeff = src;
  int first = part_begin * c->alpha;
  int last  = std::min(part_end * c->alpha, (int)level);
  if (is_ntt) {
    int64_t* d = scratch(level * n);
    std::vector<LimbRef> lim;
    for (int i = first; i < last; i++)
      lim.push_back(LimbRef{(uint16_t)i, 0, (uint16_t)i, (uint8_t)i, 0});
    fhert_launch_ntt_chunked(ptr2(src), ptr2(d), lim, true);
    coeff = d;
  }
  std::vector<LimbRef> out_limbs;
  for (int pb = part_begin; pb < part_end; pb += kMaxParts) {
    ConvArgs args;
    args.groups     = std::min(kMaxParts, part_end - pb);
    args.level      = (int)level;
    args.out_total  = (int)level + K;
    args.p_limb     = p_limb;
    args.in_stride  = c->L + K;
    args.out_stride = 1;
    for (int g = 0; g < args.groups; g++) {
      int                        part = pb + g;
      const Context::ModUpTable& t    = modup_table(c, (int)level, part);
      int                        start = c->alpha * part;
      ConvGroup&                 cg    = args.g[g];
      cg.in          = reinterpret_cast<const u64*>(coeff);
      cg.out         = reinterpret_cast<u64*>(ext_base + (size_t)(part - part_begin) * part_stride * n);
      cg.inv         = t.d_hat_inv;
      cg.mat         = t.d_hat_mod;
      cg.first_limb  = start;
      cg.first_prime = start;
      cg.count       = t.digit_len;
      cg.skip_start  = start;
      cg.skip_len    = t.digit_len;
      size_t base_limb = (size_t)(part - part_begin) * part_stride;
      for (int m = 0; m < (int)level + K; m++) {
        if (m >= start && m < start + t.digit_len) continue;
        size_t limb  = base_limb + (m < (int)level ? m : p_limb + (m - (int)level));
        int    prime = m < (int)level ? m : c->L + (m - (int)level);
        FHERT_ASSERT(limb < 65536, "extended buffer too large for one launch");
        out_limbs.push_back(LimbRef{(uint16_t)limb, 0, (uint16_t)limb, (uint8_t)prime, 0});
      }
    }
    launch_base_conv(args);
  }
  if (is_ntt) fhert_launch_ntt_chunked(ptr2(ext_base), ptr2(ext_base), out_limbs, false);
}

// Hands digit `part` of the raised polynomial kept in c->raised to res: every
// limb of res becomes an alias of the kept copy in the recorder, so the
// per-limb calls recorded around it need no launch in between.
static bool modup_serve(Context* c, POLY res, POLY poly, uint32_t part) {
  auto& m = c->raised;
  if (!m.valid || m.src != poly->_data || m.level != poly->_num_primes ||
      m.is_ntt != poly->_is_ntt || (int)part >= m.parts)
    return false;
  const size_t   n = c->N, ext_limbs = m.level + c->K;
  const int64_t* digit = m.digits + (size_t)part * ext_limbs * n;
  for (size_t i = 0; i < ext_limbs; i++) {
    size_t limb = i < m.level ? i : p_offset(res) + (i - m.level);
    if (!hw_alias(c, res->_data + limb * n, digit + i * n)) return false;
  }
  res->_is_ntt = poly->_is_ntt;
  return true;
}

POLY Decomp_modup(POLY res, POLY poly, uint32_t part) {
  Context* c     = ctx_noflush();
  size_t   level = poly->_num_primes;
  FHERT_ASSERT(res->_data && res->_num_primes == level && res->_num_primes_p == (size_t)c->K,
               "Decomp_modup: result must hold level + K limbs");
  size_t start = (size_t)c->alpha * part;
  FHERT_ASSERT(start < level, "Decomp_modup: digit out of range");
  if (modup_serve(c, res, poly, part)) return res;
  c = ctx();  // deferred work first; this also drops digits kept for another polynomial
  size_t len   = std::min((size_t)c->alpha, level - start);
  int    parts = (int)((level + c->alpha - 1) / c->alpha);
  // A program raises the digits of one polynomial one after the other
  // (hal: the emitted key-switch loop), so the first call raises all of them
  // in one batch of launches and the following calls only hand them out.
  if (part == 0 && parts > 1 && !c->draining && hw_recording(c)) {
    const size_t n = c->N, ext_limbs = level + c->K;
    int64_t*     digits = nullptr;
    CUDA_CHECK(dev_alloc(&digits, (size_t)parts * ext_limbs * n * sizeof(int64_t), c->stream));
    fhert_raise_parts(c, poly->_data, poly->_is_ntt, level, 0, parts, digits, ext_limbs, (int)level);
    for (int p = 0; p < parts; p++) {  // each digit's own limbs are the polynomial's
      size_t first = (size_t)c->alpha * p, cnt = std::min((size_t)c->alpha, level - first);
      CUDA_CHECK(counted_copy(digits + ((size_t)p * ext_limbs + first) * n, poly->_data + first * n,
                                 cnt * n * sizeof(int64_t), cudaMemcpyDeviceToDevice, c->stream));
    }
    hw_free_after_replay(c, digits);
    c->raised.valid  = true;
    c->raised.src    = poly->_data;
    c->raised.level  = level;
    c->raised.is_ntt = poly->_is_ntt;
    c->raised.parts  = parts;
    c->raised.digits = digits;
    bool served = modup_serve(c, res, poly, 0);
    FHERT_ASSERT(served, "Decomp_modup: kept digits not usable");
    return res;
  }
  fhert_raise_parts(c, poly->_data, poly->_is_ntt, level, (int)part, (int)part + 1, res->_data, 0,
              (int)p_offset(res));
  CUDA_CHECK(counted_copy(res->_data + start * c->N, poly->_data + start * c->N,
                             len * c->N * sizeof(int64_t), cudaMemcpyDeviceToDevice, c->stream));
  res->_is_ntt = poly->_is_ntt;
  return res;
}

POLY Mod_up(POLY res, POLY old_poly, uint32_t part) {
  // rns_poly.c:107-158: old_poly holds only the digit's limbs (from Decomp)
  Context* c     = ctx();
  size_t   level = res->_num_primes;
  FHERT_ASSERT(res->_data && res->_num_primes_p == (size_t)c->K, "Mod_up: result size not match");
  size_t start = (size_t)c->alpha * part;
  size_t len   = old_poly->_num_primes;
  // place the digit at its own limbs of res, then raise from there
  CUDA_CHECK(counted_copy(res->_data + start * c->N, old_poly->_data,
                             len * c->N * sizeof(int64_t), cudaMemcpyDeviceToDevice, c->stream));
  fhert_raise_parts(c, res->_data, old_poly->_is_ntt, level, (int)part, (int)part + 1, res->_data, 0,
              (int)p_offset(res));
  res->_is_ntt = old_poly->_is_ntt;
  return res;
}

// ModDown of one or two extended polynomials of the same level
// (rns_poly.c:260-308): res[g] = (x[g] - Conv_P->Q(x[g] mod P)) * P^-1, plus
// add[g] when given.  ext[g] has its special limbs at limb index ext_p_limb.
void fhert_mod_down_polys(Context* c, int npoly, int64_t* const res[2],
                           const int64_t* const ext[2], int ext_p_limb,
                           const int64_t* const add[2], size_t level, bool is_ntt) {
  const uint32_t n = c->N;
  const int      K = c->K;
  FHERT_ASSERT(npoly * (int)level <= kMaxLimbs && npoly * K <= kMaxLimbs, "ModDown batch too large");
  int64_t* sc   = scratch((size_t)npoly * (K + level) * n);
  int64_t* conv = sc + (size_t)npoly * K * n;  // [npoly][level]
  if (is_ntt) {
    LimbBatch in;
    in.count = npoly * K;
    for (int g = 0; g < npoly; g++)
      for (int k = 0; k < K; k++)
        in.limb[g * K + k] = LimbRef{(uint16_t)(ext_p_limb + k), 0, (uint16_t)(g * K + k),
                                     (uint8_t)(c->L + k), (uint8_t)g};
    launch_ntt(ptr2(ext[0], ext[1]), ptr2(sc), in, true);
  }
  ConvArgs args;
  args.groups     = npoly;
  args.level      = (int)level;
  args.out_total  = (int)level;
  args.p_limb     = 0;
  args.in_stride  = 1;
  args.out_stride = K;
  for (int g = 0; g < npoly; g++) {
    ConvGroup& cg  = args.g[g];
    cg.in          = is_ntt ? reinterpret_cast<const u64*>(sc + (size_t)g * K * n)
                            : reinterpret_cast<const u64*>(ext[g] + (size_t)ext_p_limb * n);
    cg.out         = reinterpret_cast<u64*>(conv + (size_t)g * level * n);
    cg.inv         = c->d_phat_inv;
    cg.mat         = c->d_phat_mod_q;
    cg.first_limb  = 0;
    cg.first_prime = c->L;
    cg.count       = K;
    cg.skip_start  = 0;
    cg.skip_len    = 0;
  }
  launch_base_conv(args);
  if (is_ntt && ntt_can_fuse()) {
    // the ModDown tail runs inside the last pass of the forward transform
    LimbBatch out;
    out.count = npoly * (int)level;
    for (int g = 0; g < npoly; g++)
      for (int i = 0; i < (int)level; i++) {
        uint8_t sel = (uint8_t)(g ? (2 | 4) : 0);  // x (and addend) and res from the second base
        out.limb[g * level + i] =
            LimbRef{(uint16_t)(g * level + i), (uint16_t)i, (uint16_t)i, (uint8_t)i, sel};
      }
    NttFuse f;
    f.epi_kind = 2;
    f.epi_mul  = c->d_p_inv;
    f.aux      = ptr2(ext[0], npoly > 1 ? ext[1] : nullptr);
    if (add) f.add = ptr2(add[0], npoly > 1 ? add[1] : nullptr);
    launch_ntt_fused(ptr2(conv), conv, ptr2(res[0], npoly > 1 ? res[1] : nullptr), out, f);
    return;
  }
  if (is_ntt) {
    LimbBatch out;
    out.count = npoly * (int)level;
    for (int g = 0; g < npoly; g++)
      for (int i = 0; i < (int)level; i++) {
        uint16_t t = (uint16_t)(g * level + i);
        out.limb[t] = LimbRef{t, 0, t, (uint8_t)i, 0};
      }
    launch_ntt(ptr2(conv), ptr2(conv), out, false);
  }
  ModDownTail tail;
  tail.polys = npoly;
  tail.level = (int)level;
  for (int g = 0; g < 2; g++) {
    bool on     = g < npoly;
    tail.res[g] = on ? reinterpret_cast<u64*>(res[g]) : nullptr;
    tail.x[g]   = on ? reinterpret_cast<const u64*>(ext[g]) : nullptr;
    tail.t[g]   = on ? reinterpret_cast<const u64*>(conv + (size_t)g * level * n) : nullptr;
    tail.add[g] = on && add ? reinterpret_cast<const u64*>(add[g]) : nullptr;
  }
  launch_moddown_combine(tail);
}

POLY Mod_down(POLY res, POLY poly) {
  size_t level = poly->_num_primes;
  if (res->_data == nullptr) Alloc_poly_data(res, ctx()->N, level, 0);
  FHERT_ASSERT(res->_num_primes == level && poly->_num_primes_p == (size_t)ctx_noflush()->K,
               "Mod_down: result size not match");
  pair_submit(1, res->_data, poly->_data, level, (int)p_offset(poly), poly->_is_ntt);
  res->_is_ntt = poly->_is_ntt;
  return res;
}

POLY Mod_down_rescale(POLY res, POLY poly) {
  // rns_poly.c:531-603: ModDown and Rescale in one step, computed in coefficient
  // form; like the CPU runtime it leaves `poly` in coefficient form.
  Context*       c     = ctx();
  const size_t   level = poly->_num_primes, n = c->N;
  const int      K     = c->K;
  FHERT_ASSERT(res->_data && res->_num_primes == level && level > 1 &&
                   poly->_num_primes_p == (size_t)K && res->_num_primes_p == 0,
               "Mod_down_rescale: size not match");
  if (poly->_is_ntt) Conv_ntt2poly_inplace(poly);
  int64_t* conv = scratch(level * n);
  ConvArgs args;
  args.groups     = 1;
  args.level      = (int)level;
  args.out_total  = (int)level;
  args.p_limb     = 0;
  args.in_stride  = 1;
  args.out_stride = K;
  ConvGroup& cg   = args.g[0];
  cg.in           = reinterpret_cast<const u64*>(poly->_data + p_offset(poly) * n);
  cg.out          = reinterpret_cast<u64*>(conv);
  cg.inv          = c->d_phat_inv;
  cg.mat          = c->d_phat_mod_q;
  cg.first_limb   = 0;
  cg.first_prime  = c->L;
  cg.count        = K;
  cg.skip_start   = 0;
  cg.skip_len     = 0;
  launch_base_conv(args);
  launch_moddown_rescale(res->_data, poly->_data, conv, (int)level);
  res->_num_primes = level - 1;
  res->_is_ntt     = false;
  Conv_poly2ntt_inplace(res);
  return res;
}

VALUE_LIST* Reduce_and_rescale_modup(POLY res, POLY poly) {
  // rns_poly_impl.c:521-620
  Context*     c     = ctx();
  const size_t level = poly->_num_primes, n = c->N;
  const int    K     = c->K;
  FHERT_ASSERT(level > 1 && poly->_num_primes_p == (size_t)K,
               "Reduce_and_rescale_modup: size not match");
  FHERT_ASSERT(res->_data && res->_num_alloc_primes >= level,
               "Reduce_and_rescale_modup: res must hold as many limbs as poly");
  if (poly->_is_ntt) Conv_ntt2poly_inplace(poly);
  // the special limbs converted to every Q prime: the CPU runtime uses res for them
  ConvArgs args;
  args.groups     = 1;
  args.level      = (int)level;
  args.out_total  = (int)level;
  args.p_limb     = 0;
  args.in_stride  = 1;
  args.out_stride = K;
  ConvGroup& cg   = args.g[0];
  cg.in           = reinterpret_cast<const u64*>(poly->_data + p_offset(poly) * n);
  cg.out          = reinterpret_cast<u64*>(res->_data);
  cg.inv          = c->d_phat_inv;
  cg.mat          = c->d_phat_mod_q;
  cg.first_limb   = 0;
  cg.first_prime  = c->L;
  cg.count        = K;
  cg.skip_start   = 0;
  cg.skip_len     = 0;
  launch_base_conv(args);
  // ModDown and rescale in coefficient form, level - 1 limbs
  const size_t out_level = level - 1;
  int64_t*     x         = nullptr;
  CUDA_CHECK(dev_alloc(&x, out_level * n * sizeof(int64_t), c->stream));
  launch_moddown_rescale(x, poly->_data, res->_data, (int)level);
  // every digit of x raised to Q_{level-1} u P, left in coefficient form
  size_t parts = (out_level + c->alpha - 1) / c->alpha;
  if (parts > (size_t)c->dnum) parts = (size_t)c->dnum;
  POLY_ARR arr = Alloc_polys((uint32_t)parts, c->N, out_level, (size_t)K);
  fhert_raise_parts(c, x, false, out_level, 0, (int)parts, arr[0]._data, out_level + K,
                    (int)out_level);
  for (size_t d = 0; d < parts; d++) {  // a digit's own limbs are those of x
    size_t first = (size_t)c->alpha * d, cnt = std::min((size_t)c->alpha, out_level - first);
    CUDA_CHECK(counted_copy(arr[d]._data + first * n, x + first * n, cnt * n * sizeof(int64_t),
                            cudaMemcpyDeviceToDevice, c->stream));
  }
  CUDA_CHECK(dev_free(x, c->stream));
  res->_num_primes = out_level;  // Modswitch(res, res)
  VALUE_LIST* list = (VALUE_LIST*)std::calloc(1, sizeof(VALUE_LIST));
  list->_type      = 0x4000;
  list->_length    = parts;
  list->_vals._p   = (void**)std::calloc(parts, sizeof(void*));
  for (size_t d = 0; d < parts; d++) list->_vals._p[d] = &arr[d];
  return list;
}

void Free_precomp(VALUE_LIST* precomputed) {  // rns_poly_impl.c:622-630
  if (precomputed == nullptr) return;
  if (precomputed->_length > 0) Free_polys((POLY_ARR)precomputed->_vals._p[0]);
  std::free(precomputed->_vals._p);
  std::free(precomputed);
}

void Chk_level(POLY res, POLY p0, POLY p1) {
  // rns_poly.c:606-613: a diagnostic, it only prints
  if (res->_num_primes != p0->_num_primes || res->_num_primes_p != p0->_num_primes_p)
    std::printf("level not match\n");
  if (p1 && (res->_num_primes != p1->_num_primes || res->_num_primes_p != p1->_num_primes_p))
    std::printf("level not match\n");
}

POLY Extend(POLY res, POLY poly) {
  Context* c = ctx();
  FHERT_ASSERT(res->_num_primes == poly->_num_primes && poly->_data, "Extend: size not match");
  FHERT_ASSERT(res->_num_alloc_primes == poly->_num_primes + (size_t)c->K,
               "Extend: alloc_size not match");
  size_t n = c->N;
  res->_num_primes_p = c->K;
  CUDA_CHECK(zero_async(res->_data + p_offset(res) * n, (size_t)c->K * n * sizeof(int64_t),
                        c->stream));
  launch_mul_const(ptr2(res->_data), ptr2(poly->_data), c->d_p_mod_q,
                   poly_batch(c, res, poly, nullptr, poly->_num_primes, 0));
  res->_is_ntt = poly->_is_ntt;
  return res;
}

POLY Dot_prod(POLY res, POLY a, POLY b, size_t parts) {
  Context* c = ctx();
  FHERT_ASSERT(parts >= 1 && parts <= (size_t)kMaxParts, "Dot_prod: unsupported digit count");
  size_t level = a[0]._num_primes, num_p = a[0]._num_primes_p;
  FHERT_ASSERT(num_p == (size_t)c->K, "Dot_prod: operands must be extended polynomials");
  ensure_poly(res, c->N, level, num_p);
  InnerArgs args;
  std::memset(&args, 0, sizeof(args));
  args.parts      = (int)parts;
  args.level      = (int)level;
  args.alpha      = c->alpha;
  args.key_p_limb = (int)p_offset(&b[0]);
  args.ext_p_limb = (int)p_offset(&a[0]);
  args.acc_p_limb = (int)p_offset(res);
  args.in         = nullptr;
  for (size_t j = 0; j < parts; j++) {
    FHERT_ASSERT(a[j]._num_alloc_primes == a[0]._num_alloc_primes &&
                     b[j]._num_alloc_primes == b[0]._num_alloc_primes,
                 "Dot_prod: operands must share a layout");
    args.ext_ptr[j] = reinterpret_cast<const u64*>(a[j]._data);
    args.key0[j]    = reinterpret_cast<const u64*>(b[j]._data);
  }
  args.acc0 = reinterpret_cast<u64*>(res->_data);
  args.acc1 = nullptr;
  launch_inner_product(args);
  res->_is_ntt = a[0]._is_ntt;
  return res;
}

POLY Automorphism_transform(POLY res, POLY poly, int64_t* order) {
  Context* c = ctx();
  FHERT_ASSERT(poly->_is_ntt, "Automorphism_transform: coefficient form is not supported");
  FHERT_ASSERT(res->_data != poly->_data, "Automorphism_transform cannot work in place");
  launch_automorphism(ptr2(res->_data), ptr2(poly->_data), reinterpret_cast<const uint32_t*>(order),
                      poly_batch(c, res, poly, nullptr, poly->_num_primes, poly->_num_primes_p));
  res->_is_ntt = true;
  return res;
}

// ---------------------------------------------------------------------------
// keys and automorphism tables
// ---------------------------------------------------------------------------

uint32_t Auto_idx(int32_t rot_idx) { return auto_index_for(ctx(), rot_idx); }

int64_t* Auto_order(int32_t rot_idx) {
  Context* c = ctx_noflush();  // a table of the library's own: touches no program data
  uint32_t k = (rot_idx == (int32_t)(2 * c->N - 1)) ? (uint32_t)rot_idx : auto_index_for(c, rot_idx);
  return reinterpret_cast<int64_t*>(auto_table(c, k));
}

static uint32_t key_id_for(Context* c, bool is_rot, int32_t rot_idx) {
  if (!is_rot) return 0;
  uint32_t conj = 2 * c->N - 1;
  return rot_idx == (int32_t)conj ? conj : auto_index_for(c, rot_idx);
}

SW_KEY Swk(bool is_rot, int32_t rot_idx) {
  Context*    c = ctx_noflush();  // looks a key up: touches no program data
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
  CUDA_CHECK(counted_copy(p->_data, host, bytes, cudaMemcpyHostToDevice, c->stream));
  CUDA_CHECK(stream_sync(c->stream));
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

// shape of the lower-level operand; the public Init_ciph_* family with the
// reference's storage-reuse rules lives in program_api.cu
static void init_like_lower(CIPHER res, CIPHER a, CIPHER b) {
  CIPHER low = (b != nullptr && Level(b) < Level(a)) ? b : a;
  init_ciph(res, low->_c0_poly._ring_degree, Level(low), low->_c0_poly._num_primes_p,
            low->_scaling_factor, low->_sf_degree, low->_slots);
}

static void init_ciph3_product(CIPHER3 res, CIPHER a, CIPHER b) {
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

static CIPHER add_sub_ciph(EwOp op, CIPHER res, CIPHER a, CIPHER b) {
  Context* c = ctx();
  init_like_lower(res, a, b);
  size_t level = Level(res), num_p = res->_c0_poly._num_primes_p;
  FHERT_ASSERT(num_p == 0 || (a->_c0_poly._num_primes_p == num_p && b->_c0_poly._num_primes_p == num_p),
               "unmatched special limbs");
  LimbBatch one = poly_batch(c, &res->_c0_poly, &a->_c0_poly, &b->_c0_poly, level, num_p);
  launch_elementwise(op, ptr2(res->_c0_poly._data, res->_c1_poly._data),
                     ptr2(a->_c0_poly._data, a->_c1_poly._data),
                     ptr2(b->_c0_poly._data, b->_c1_poly._data), 0, both_polys(one));
  return res;
}

CIPHER Add_ciph(CIPHER res, CIPHER a, CIPHER b) { return add_sub_ciph(EW_ADD, res, a, b); }
CIPHER Sub_ciph(CIPHER res, CIPHER a, CIPHER b) { return add_sub_ciph(EW_SUB, res, a, b); }

CIPHER3 Mul_ciph3(CIPHER3 res, CIPHER a, CIPHER b) {
  // evaluator.c:137-173: c0 = a0*b0, c1 = a0*b1 + a1*b0, c2 = a1*b1
  init_ciph3_product(res, a, b);
  size_t level = res->_c0_poly._num_primes;
  launch_tensor(res->_c0_poly._data, res->_c1_poly._data, res->_c2_poly._data,
                a->_c0_poly._data, a->_c1_poly._data, b->_c0_poly._data, b->_c1_poly._data,
                (int)level);
  return res;
}

// Hybrid key switch of one polynomial (evaluator.c:411-462): ModUp of all
// digits, inner product with the key over Q u P, ModDown of both accumulators.
// out0/out1 receive level limbs; add0/add1 (optional) are added to them, which
// folds the "+ c0" of a rotation and the "+ c0, + c1" of a relinearisation
// into the last kernel.  About a dozen launches regardless of the digit count.
// Key switch of `in` whose digits were already raised into `digits`
// (parts extended polynomials of level + K limbs each).
void fhert_switch_key_raised(Context* c, int64_t* out0, int64_t* out1, const int64_t* in,
                             const int64_t* digits, int parts, size_t level, SW_KEY swk,
                             const int64_t* add0, const int64_t* add1) {
  const uint32_t n         = c->N;
  const size_t   ext_limbs = level + c->K;
  int64_t*       acc0      = nullptr;
  CUDA_CHECK(dev_alloc(&acc0, 2 * ext_limbs * n * sizeof(int64_t), c->stream));
  int64_t* acc1 = acc0 + ext_limbs * n;
  InnerArgs args;
  std::memset(&args, 0, sizeof(args));
  args.parts      = parts;
  args.level      = (int)level;
  args.alpha      = c->alpha;
  args.key_p_limb = c->L;
  args.ext_p_limb = (int)level;
  args.acc_p_limb = (int)level;
  args.in         = reinterpret_cast<const u64*>(in);  // digits' own limbs come from the input
  for (int j = 0; j < parts; j++) {
    args.ext_ptr[j] = reinterpret_cast<const u64*>(digits + (size_t)j * ext_limbs * n);
    args.key0[j]    = reinterpret_cast<const u64*>(swk->_parts[j]._p0._data);
    args.key1[j]    = reinterpret_cast<const u64*>(swk->_parts[j]._p1._data);
  }
  args.acc0 = reinterpret_cast<u64*>(acc0);
  args.acc1 = reinterpret_cast<u64*>(acc1);
  launch_inner_product(args);
  int64_t*       r[2] = {out0, out1};
  const int64_t* x[2] = {acc0, acc1};
  const int64_t* a[2] = {add0, add1};
  fhert_mod_down_polys(c, 2, r, x, (int)level, a, level, true);
  CUDA_CHECK(dev_free(acc0, c->stream));
}

void fhert_switch_key(Context* c, int64_t* out0, int64_t* out1, const int64_t* in, size_t level,
                      SW_KEY swk, const int64_t* add0, const int64_t* add1) {
  const int parts = (int)std::min<size_t>((level + c->alpha - 1) / c->alpha, c->dnum);
  FHERT_ASSERT(parts <= kMaxParts, "too many digits");
  const size_t ext_limbs = level + c->K;
  int64_t*     digits    = nullptr;
  CUDA_CHECK(dev_alloc(&digits, (size_t)parts * ext_limbs * c->N * sizeof(int64_t), c->stream));
  fhert_raise_parts(c, in, true, level, 0, parts, digits, ext_limbs, (int)level);
  fhert_switch_key_raised(c, out0, out1, in, digits, parts, level, swk, add0, add1);
  CUDA_CHECK(dev_free(digits, c->stream));
}

CIPHER Relin(CIPHER res, CIPHER3 ciph) {
  // evaluator.c:288-305
  Context* c     = ctx();
  size_t   level = ciph->_c2_poly._num_primes;
  init_ciph(res, c->N, level, 0, ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
  fhert_switch_key(c, res->_c0_poly._data, res->_c1_poly._data, ciph->_c2_poly._data, level,
             Swk(false, 0), ciph->_c0_poly._data, ciph->_c1_poly._data);
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
  Context* c     = ctx();
  size_t   level = Level(ciph);
  FHERT_ASSERT(level > 1, "rescale: multiply level is not big enough");
  FHERT_ASSERT(ciph->_c0_poly._is_ntt == ciph->_c1_poly._is_ntt, "Rescale_ciph: mixed forms");
  const bool is_ntt = ciph->_c0_poly._is_ntt;
  init_ciph(res, ciph->_c0_poly._ring_degree, level, 0,
            ciph->_scaling_factor / Get_default_sc(), ciph->_sf_degree - 1, ciph->_slots);
  int64_t*       r[2] = {res->_c0_poly._data, res->_c1_poly._data};
  const int64_t* p[2] = {ciph->_c0_poly._data, ciph->_c1_poly._data};
  if (is_ntt)
    fhert_rescale_polys(c, 2, r, p, level);
  else
    launch_rescale_coeff(ptr2(r[0], r[1]), ptr2(p[0], p[1]), 2, (int)level);
  res->_c0_poly._is_ntt = res->_c1_poly._is_ntt = is_ntt;
  res->_c0_poly._num_primes = res->_c1_poly._num_primes = level - 1;
  return res;
}

static CIPHER rotate_with_key(CIPHER res, CIPHER ciph, int32_t rot_idx, uint32_t k) {
  // evaluator.c:503-522: key switch c1, add c0, then permute both polynomials
  Context* c     = ctx();
  size_t   level = Level(ciph);
  size_t   words = level * c->N;
  int64_t* t     = nullptr;
  CUDA_CHECK(dev_alloc(&t, 2 * words * sizeof(int64_t), c->stream));
  fhert_switch_key(c, t, t + words, ciph->_c1_poly._data, level, Swk(true, rot_idx),
             ciph->_c0_poly._data, nullptr);
  if (res != ciph)
    init_ciph(res, c->N, level, 0, ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
  LimbBatch one = poly_batch(c, &res->_c0_poly, &res->_c0_poly, nullptr, level, 0);
  launch_automorphism(ptr2(res->_c0_poly._data, res->_c1_poly._data), ptr2(t, t + words),
                      auto_table(c, k), both_polys(one));
  CUDA_CHECK(dev_free(t, c->stream));
  return res;
}

// cipher.c:460-481: several rotations of one ciphertext; its digits are raised
// once and shared by all of them
void Rotate_batch_ciph(CIPHER res_arr, CIPHER ciph, const int32_t* rot_idx, uint32_t count) {
  if (count == 0) return;
  Context* c     = ctx();
  size_t   level = Level(ciph), words = level * c->N, ext_limbs = level + c->K;
  const int parts = (int)std::min<size_t>((level + c->alpha - 1) / c->alpha, c->dnum);
  int64_t *digits = nullptr, *t = nullptr;
  CUDA_CHECK(dev_alloc(&digits, (size_t)parts * ext_limbs * c->N * sizeof(int64_t), c->stream));
  CUDA_CHECK(dev_alloc(&t, 2 * words * sizeof(int64_t), c->stream));
  fhert_raise_parts(c, ciph->_c1_poly._data, true, level, 0, parts, digits, ext_limbs, (int)level);
  for (uint32_t i = 0; i < count; i++) {
    CIPHER out = &res_arr[i];
    FHERT_ASSERT(out != ciph, "Rotate_batch_ciph cannot work in place");
    if (rot_idx[i] == 0) {
      Copy_ciph(out, ciph);
      continue;
    }
    fhert_switch_key_raised(c, t, t + words, ciph->_c1_poly._data, digits, parts, level,
                            Swk(true, rot_idx[i]), ciph->_c0_poly._data, nullptr);
    init_ciph(out, c->N, level, 0, ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
    LimbBatch one = poly_batch(c, &out->_c0_poly, &out->_c0_poly, nullptr, level, 0);
    launch_automorphism(ptr2(out->_c0_poly._data, out->_c1_poly._data), ptr2(t, t + words),
                        auto_table(c, auto_index_for(c, rot_idx[i])), both_polys(one));
  }
  CUDA_CHECK(dev_free(t, c->stream));
  CUDA_CHECK(dev_free(digits, c->stream));
}

CIPHER Rotate_ciph(CIPHER res, CIPHER ciph, int32_t rot_idx) {
  return rotate_with_key(res, ciph, rot_idx, auto_index_for(ctx(), rot_idx));
}

CIPHER Conjugate_ciph(CIPHER res, CIPHER ciph) {
  int32_t conj = (int32_t)(2 * ctx()->N - 1);
  return rotate_with_key(res, ciph, conj, (uint32_t)conj);
}

}  // extern "C"
