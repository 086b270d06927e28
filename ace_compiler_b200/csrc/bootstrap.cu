// CKKS bootstrapping: mod-raise, CoeffsToSlots, approximate modular reduction
// (Chebyshev series of a scaled cosine, Paterson-Stockmeyer evaluation, double
// angle iterations) and SlotsToCoeffs, with collapsed-FFT linear transforms,
// baby-step/giant-step and hoisted rotations.
//
// The host precomputation (diagonals of the collapsed FFT stages in fp64) and
// the order of homomorphic operations follow rtlib/ant/ckks/src/bootstrap.c and
// chebyshev_impl.c of the CPU runtime step by step, so that every ciphertext
// residue is identical; citations below name those files.  On the device the
// work is arranged differently: the digits of a ciphertext are raised once per
// linear-transform stage, every baby-step sum is one fused multiply-accumulate
// launch over all giant-step rotations, and both polynomials of a ciphertext
// travel through every kernel together.
#include <algorithm>
#include <cmath>
#include <complex>
#include <cstring>
#include <set>
#include <vector>

#include "runtime.h"

using namespace fhert;

namespace {

typedef std::complex<double> cplx;
#include "sine_tables.inc"

// product with separately rounded operations, as a C compiler evaluates
// complex * complex without fused multiply-add
inline cplx cmul(cplx a, cplx b) {
  return cplx(a.real() * b.real() - a.imag() * b.imag(), a.real() * b.imag() + a.imag() * b.real());
}
inline cplx scaled(cplx a, double f) { return cplx(a.real() * f, a.imag() * f); }

// ---------------------------------------------------------------------------
// parameters
// ---------------------------------------------------------------------------

// bootstrap.c:43-62: which cosine series, by secret-key Hamming weight
const SineTable& sine_table(size_t hamming_weight) {
  const char* even_env = std::getenv("RTLIB_BTS_EVEN_POLY");
  bool        even     = even_env != nullptr && std::atoi(even_env) != 0;
  bool        light    = hamming_weight > 0 && hamming_weight <= 192;
  if (even) return light ? kSineEvenHw192 : kSineEvenDense;
  return light ? kSineHw192 : kSineDense;
}

bool sine_table_is_even(const SineTable& t) { return &t == &kSineEvenHw192 || &t == &kSineEvenDense; }

// bootstrap.c:64-79: multiplicative depth of a Paterson-Stockmeyer evaluation
uint32_t depth_by_degree(size_t degree) {
  FHERT_ASSERT(degree >= 5 && degree <= 2031, "Polynomial degree is supported from 5 to 2031");
  static const uint32_t upper[] = {4, 5, 13, 27, 59, 119, 247, 495, 1007, 2031};
  static const uint32_t depth[] = {3, 4, 5, 6, 7, 8, 9, 10, 11, 12};
  for (int i = 0; i < 10; i++)
    if (degree <= upper[i]) return depth[i];
  return 12;
}

// include/ckks/bootstrap.h: levels the modular reduction consumes
uint32_t approx_mod_depth(size_t hamming_weight) {
  const SineTable& t = sine_table(hamming_weight);
  return depth_by_degree(t.size - 1) - 1 + t.double_angle;
}

struct FftParams {  // one direction of the collapsed FFT (bootstrap.c:556-615)
  int level_budget, layers_coll, rem_coll, num_rot, b, g, num_rot_rem, b_rem, g_rem;
};

struct Precom {  // per slot count (include/ckks/bootstrap.h CKKS_BTS_PRECOM)
  uint32_t                            slots = 0;
  FftParams                           enc{}, dec{};
  std::vector<std::vector<PLAINTEXT>> c2s, s2c;  // [stage][diagonal], extended plaintexts
  bool                                keys = false;
};

// bootstrap.c:199-211
uint32_t reduce_rotation(int32_t index, uint32_t slots) {
  int32_t islots = (int32_t)slots;
  if ((slots & (slots - 1)) == 0) {
    int32_t n = (int32_t)std::log2((double)slots);
    if (index >= 0) return (uint32_t)(index - ((index >> n) << n));
    return (uint32_t)(index + islots + (((-index) >> n) << n));
  }
  return (uint32_t)((islots + index % islots) % islots);
}

// bootstrap.c:518-554: {layers per level, rows, remainder}
void select_layers(uint32_t log_slots, uint32_t budget, uint32_t out[3]) {
  uint32_t layers = (uint32_t)std::ceil((double)log_slots / budget);
  uint32_t rows = log_slots / layers, rem = log_slots % layers;
  uint32_t dim = rem ? rows + 1 : rows;
  if (dim < budget) {
    layers -= 1;
    rows = log_slots / layers;
    rem  = log_slots - rows * layers;
    dim  = rem ? rows + 1 : rows;
    while (dim != budget) {
      rows -= 1;
      rem = log_slots - rows * layers;
      dim = rem ? rows + 1 : rows;
    }
  }
  out[0] = layers;
  out[1] = rows;
  out[2] = rem;
}

FftParams fft_params(uint32_t slots, uint32_t level_budget, uint32_t dim1) {
  uint32_t dims[3];
  select_layers((uint32_t)std::log2((double)slots), level_budget, dims);
  FftParams p{};
  p.level_budget = (int)level_budget;
  p.layers_coll  = (int)dims[0];
  p.rem_coll     = (int)dims[2];
  p.num_rot      = (1 << (p.layers_coll + 1)) - 1;
  p.num_rot_rem  = (1 << (p.rem_coll + 1)) - 1;
  if (dim1 == 0 || dim1 > (uint32_t)p.num_rot)
    p.g = p.num_rot > 7 ? 1 << (p.layers_coll / 2 + 2) : 1 << (p.layers_coll / 2 + 1);
  else
    p.g = (int)dim1;
  p.b = (p.num_rot + 1) / p.g;
  if (p.rem_coll != 0) {
    p.g_rem = p.num_rot_rem > 7 ? 1 << (p.rem_coll / 2 + 2) : 1 << (p.rem_coll / 2 + 1);
    p.b_rem = (p.num_rot_rem + 1) / p.g_rem;
  }
  return p;
}

// ---------------------------------------------------------------------------
// diagonals of the FFT stages (host, fp64)
// ---------------------------------------------------------------------------

typedef std::vector<cplx>   Row;
typedef std::vector<Row>    Rows;
typedef std::vector<Rows>   Stages;

// bootstrap.c:424-516.  Every radix-2 stage is a sum of the input shifted
// right, the input itself and the input shifted left; rows [0, log) hold the
// first weights, [log, 2 log) the second, [2 log, 3 log) the third.
Rows one_level_coeffs(const Row& ksi, const std::vector<uint32_t>& rot_group, bool flag,
                      bool encoding) {
  uint32_t dim = (uint32_t)ksi.size() - 1, slots = (uint32_t)rot_group.size();
  uint32_t lg  = (uint32_t)std::log2((double)slots);
  Rows     w(3 * lg, Row(slots, cplx(0, 0)));
  for (uint32_t m = slots; m > 1; m >>= 1) {
    uint32_t s = (uint32_t)std::log2((double)m) - 1;
    Row &right = w[s], &mid = w[s + lg], &left = w[s + 2 * lg];
    uint32_t lenh = m >> 1, lenq = m << 2;
    for (uint32_t k = 0; k < slots; k += m) {
      for (uint32_t j = 0; j < lenh; j++) {
        uint32_t tw = encoding ? (lenq - rot_group[j] % lenq) * (dim / lenq)
                               : (rot_group[j] % lenq) * (dim / lenq);
        cplx one(1, 0), x = ksi[tw];
        if (flag && m == 2) {
          double a = encoding ? -M_PI / 2 : M_PI / 2;
          one      = cplx(std::cos(a), std::sin(a));
          x        = cmul(one, ksi[tw]);
        }
        mid[j + k]        = one;
        mid[j + k + lenh] = -x;
        if (encoding) {
          left[j + k]         = one;
          right[j + k + lenh] = x;
        } else {
          left[j + k]         = x;
          right[j + k + lenh] = one;
        }
      }
    }
  }
  return w;
}

// bootstrap.c:617-781: merge layers_coll consecutive stages into one matrix
// with 2^(layers+1) - 1 diagonals per level of the budget
Stages collapse(const Row& ksi, const std::vector<uint32_t>& rot_group, uint32_t level_budget,
                bool flag, bool encoding) {
  uint32_t slots = (uint32_t)rot_group.size(), lg = (uint32_t)std::log2((double)slots);
  uint32_t dims[3];
  select_layers(lg, level_budget, dims);
  int  layers = (int)dims[0], rem = (int)dims[2], budget = (int)level_budget;
  bool has_rem = rem != 0;
  uint32_t num_rot = (1u << (layers + 1)) - 1, num_rot_rem = (1u << (rem + 1)) - 1;
  Rows one = one_level_coeffs(ksi, rot_group, flag, encoding);

  Stages coeff(budget);
  for (int s = 0; s < budget; s++) {
    bool is_rem = has_rem && ((encoding && s == 0) || (!encoding && s == budget - 1));
    coeff[s].assign(is_rem ? num_rot_rem : num_rot, Row(slots, cplx(0, 0)));
  }
  for (int s = 0; s < budget; s++) {
    int  top    = encoding ? (int)lg - (budget - 1 - s) * layers - 1 : s * layers;
    bool is_rem = has_rem && ((encoding && s == 0) || (!encoding && s == budget - 1));
    int  end_l  = is_rem ? rem : layers;
    for (int l = 0; l < end_l; l++) {
      if (l == 0) {
        coeff[s][0] = one[top];
        coeff[s][1] = one[top + lg];
        coeff[s][2] = one[top + 2 * lg];
        continue;
      }
      Rows next(coeff[s].size(), Row(slots, cplx(0, 0)));
      int  width = (1 << (l + 1)) - 1;
      if (encoding) {
        const Row &r0 = one[top - l], &r1 = one[top - l + lg], &r2 = one[top - l + 2 * lg];
        for (int u = 0; u < width; u++) {
          const Row& prev = coeff[s][u];
          for (uint32_t k = 0; k < slots; k++) {
            uint32_t back = reduce_rotation((int32_t)k - (1 << (top - l)), slots);
            uint32_t fwd  = reduce_rotation((int32_t)k + (1 << (top - l)), slots);
            next[2 * u][k] += cmul(r0[k], prev[back]);
            next[2 * u + 1][k] += cmul(r1[k], prev[k]);
            next[2 * u + 2][k] += cmul(r2[k], prev[fwd]);
          }
        }
      } else {
        const Row &r0 = one[top + l], &r1 = one[top + l + lg], &r2 = one[top + l + 2 * lg];
        for (int t = 0; t < 3; t++) {
          const Row& r   = t == 0 ? r0 : (t == 1 ? r1 : r2);
          int        off = t == 0 ? 0 : (t == 1 ? 1 << l : 1 << (l + 1));
          for (int u = 0; u < width; u++) {
            const Row& prev = coeff[s][u];
            for (uint32_t k = 0; k < slots; k++) next[u + off][k] += cmul(r[k], prev[k]);
          }
        }
      }
      coeff[s].swap(next);
    }
  }
  return coeff;
}

}  // namespace

namespace {

// ---------------------------------------------------------------------------
// plaintexts of the linear transforms
// ---------------------------------------------------------------------------

// bootstrap.c:305-422: diagonal dim2 = g*i + j of every stage is rotated by the
// negated giant step i and encoded over Q_level u P so that it can multiply an
// extended ciphertext; the overall constant goes into one stage only
std::vector<std::vector<PLAINTEXT>> encode_stages(Context* c, Stages& coeffs, const FftParams& p,
                                                 double scale, uint32_t level, bool encoding) {
  const uint32_t m4 = c->N / 2;  // m / 4
  const int      budget = p.level_budget, flag_rem = p.rem_coll != 0 ? 1 : 0;
  const int      stop = flag_rem ? 0 : -1;
  std::vector<std::vector<PLAINTEXT>> out(budget);
  for (int s = 0; s < budget; s++) {
    bool is_rem = flag_rem && s == (encoding ? 0 : budget - 1);
    out[s].resize(is_rem ? p.num_rot_rem : p.num_rot);
    for (auto& pt : out[s]) std::memset(&pt, 0, sizeof(PLAINTEXT));
  }
  const int      start = encoding ? stop + 1 : 0;
  const int      end   = encoding ? budget : budget - flag_rem;
  const int      cond  = encoding ? start : end - 1;
  const uint32_t enc_level = level ? level + 1 : (uint32_t)c->L - budget + 1;
  const uint32_t dec_level = level ? level + budget : (uint32_t)c->L;

  auto emit = [&](Row& diag, uint32_t rot, uint32_t plain_level, PLAINTEXT* dst) {
    size_t len = diag.size();
    Row    turned(len);
    for (size_t k = 0; k < len; k++) turned[k] = diag[(k + rot) % len];
    encode_vector(c, dst, turned, 1, plain_level, (uint32_t)len, (uint32_t)c->K);
  };

  for (int s = start; s < end; s++) {
    uint32_t plain_level = encoding ? enc_level + s : dec_level - s;
    for (int i = 0; i < p.b; i++) {
      for (int j = 0; j < p.g; j++) {
        int dim2 = p.g * i + j;
        if (dim2 == p.num_rot) continue;
        int shift = encoding ? (s - flag_rem) * p.layers_coll + p.rem_coll : s * p.layers_coll;
        uint32_t rot = reduce_rotation(-p.g * i * (1 << shift), m4);
        Row&     diag = coeffs[s][dim2];
        if (flag_rem == 0 && s == cond)
          for (auto& v : diag) v = scaled(v, scale);
        emit(diag, rot, plain_level, &out[s][dim2]);
      }
    }
  }
  if (flag_rem) {
    int      dim1  = encoding ? stop : budget - flag_rem;
    int      shift = encoding ? 1 : 1 << (dim1 * p.layers_coll);
    uint32_t plain_level = encoding ? enc_level : dec_level - budget + flag_rem;
    for (int i = 0; i < p.b_rem; i++) {
      for (int j = 0; j < p.g_rem; j++) {
        int dim2 = p.g_rem * i + j;
        if (dim2 == p.num_rot_rem) continue;
        uint32_t rot  = reduce_rotation(-p.g_rem * i * shift, m4);
        Row&     diag = coeffs[dim1][dim2];
        for (auto& v : diag) v = scaled(v, scale);
        emit(diag, rot, plain_level, &out[dim1][dim2]);
      }
    }
  }
  return out;
}

// sparse packing (bootstrap.c:803-829): the diagonals without and with the
// extra quarter turn, one after the other
Stages merged_stages(const Row& ksi, const std::vector<uint32_t>& rot_group, uint32_t budget,
                     bool flag, bool encoding, bool fully_packed) {
  if (fully_packed) return collapse(ksi, rot_group, budget, flag, encoding);
  Stages a = collapse(ksi, rot_group, budget, false, encoding);
  Stages b = collapse(ksi, rot_group, budget, true, encoding);
  for (size_t s = 0; s < a.size(); s++)
    for (size_t d = 0; d < a[s].size(); d++) a[s][d].insert(a[s][d].end(), b[s][d].begin(), b[s][d].end());
  return a;
}

std::map<uint32_t, Precom*>& precoms(Context* c) {
  if (c->bootstrap == nullptr) c->bootstrap = new std::map<uint32_t, Precom*>();
  return *static_cast<std::map<uint32_t, Precom*>*>(c->bootstrap);
}

// bootstrap.c:1055-1197 with level budget {3, 3} and automatic inner dimension
Precom* setup(Context* c, uint32_t slots) {
  const uint32_t n = c->N, m = 2 * n;
  if (slots == 0) slots = m / 4;
  auto& table = precoms(c);
  auto  it    = table.find(slots);
  if (it != table.end()) return it->second;
  Precom* pre = new Precom();
  pre->slots  = slots;
  table[slots] = pre;

  uint32_t budget[2] = {3, 3};
  double   log_slots = std::log2((double)slots);
  for (uint32_t& b : budget) {
    if (b > log_slots) b = (uint32_t)log_slots;
    if (b < 1) b = 1;
  }
  pre->enc = fft_params(slots, budget[0], 0);
  pre->dec = fft_params(slots, budget[1], 0);

  const uint32_t slots4 = 4 * slots;
  std::vector<uint32_t> rot_group(slots);
  uint32_t five = 1;
  for (uint32_t i = 0; i < slots; i++) {
    rot_group[i] = five;
    five         = (five * 5) % slots4;
  }
  Row ksi(slots4 + 1);
  for (uint32_t i = 0; i < slots4; i++) {
    double angle = 2.0 * M_PI * i / slots4;
    ksi[i]       = cplx(std::cos(angle), std::sin(angle));
  }
  ksi[slots4] = ksi[0];

  const double q0        = (double)c->primes[0];
  const double pre_scale = q0 / std::pow(2.0, std::round(std::log2(q0)));
  const double scale_enc = pre_scale / 1.0, scale_dec = 1 / pre_scale;
  const uint32_t bts_depth = approx_mod_depth(c->hamming_weight) + budget[0] + budget[1];
  const uint32_t level_0   = (uint32_t)c->L;
  FHERT_ASSERT(level_0 > budget[0], "not enough levels");
  FHERT_ASSERT(level_0 > bts_depth, "need set a larger multiply depth");
  FHERT_ASSERT(budget[0] > 1 || budget[1] > 1, "single-level linear transforms are not supported");
  const uint32_t level_enc = level_0 - budget[0], level_dec = level_0 - bts_depth;
  const bool     full      = slots == m / 4;

  Stages enc = merged_stages(ksi, rot_group, budget[0], false, true, full);
  // fold 1/N, 1/K and sf/q0 into the encoding matrices, spread over the
  // stages to keep the encoded magnitudes balanced (bootstrap.c:831-861)
  double factor = 1.0 / n;
  factor /= sine_table(c->hamming_weight).k;
  double sf = std::pow(2.0, (double)c->sf_bits);
  factor /= std::pow(2, std::round(std::log2(q0 / sf)));
  factor = std::pow(factor, 1. / budget[0]);
  for (auto& stage : enc)
    for (auto& row : stage)
      for (auto& v : row) v = scaled(v, factor);
  pre->c2s = encode_stages(c, enc, pre->enc, scale_enc, level_enc, true);

  Stages dec = merged_stages(ksi, rot_group, budget[1], false, false, full);
  pre->s2c   = encode_stages(c, dec, pre->dec, scale_dec, level_dec, false);
  CUDA_CHECK(stream_sync(c->stream));
  return pre;
}

// bootstrap.c:218-303: rotations the two transforms use, ascending, without 0
// and N/2
void stage_rotations(std::set<int32_t>& out, const FftParams& p, uint32_t slots, uint32_t m,
                     bool encoding) {
  const int      flag_rem = p.rem_coll != 0 ? 1 : 0, stop = flag_rem ? 0 : -1;
  const uint32_t m4 = m / 4;
  const int      start = encoding ? stop + 1 : 0, end = p.level_budget;
  const uint32_t slots_value = encoding ? slots : m4;
  for (int s = start; s < end; s++) {
    int shift = encoding ? 1 << ((s - flag_rem) * p.layers_coll + p.rem_coll)
                         : 1 << (s * p.layers_coll);
    for (int j = 0; j < p.g; j++)
      out.insert((int32_t)reduce_rotation((j - ((p.num_rot + 1) / 2) + 1) * shift, slots_value));
    for (int i = 0; i < p.b; i++) out.insert((int32_t)reduce_rotation((p.g * i) * shift, m4));
  }
  if (flag_rem) {
    int s     = p.level_budget - flag_rem;
    int shift = encoding ? 1 : 1 << (s * p.layers_coll);
    for (int j = 0; j < p.g_rem; j++)
      out.insert((int32_t)reduce_rotation((j - ((p.num_rot_rem + 1) / 2) + 1) * shift, slots_value));
    for (int i = 0; i < p.b_rem; i++) out.insert((int32_t)reduce_rotation(p.g_rem * i * shift, m4));
  }
  if (slots * 4 != m)
    for (uint32_t j = 1; j < m / (slots * 4); j <<= 1) out.insert((int32_t)(j * slots));
}

std::vector<int32_t> all_rotations(Context* c, Precom* pre) {
  const uint32_t m = 2 * c->N;
  std::set<int32_t> rots;
  stage_rotations(rots, pre->enc, pre->slots, m, true);
  stage_rotations(rots, pre->dec, pre->slots, m, false);
  rots.erase(0);
  rots.erase((int32_t)(m / 4));
  return std::vector<int32_t>(rots.begin(), rots.end());
}

void keygen(Context* c, Precom* pre) {
  if (pre->keys) return;
  generate_bootstrap_keys(c, all_rotations(c, pre));
  pre->keys = true;
}

}  // namespace

namespace fhert {

// ---------------------------------------------------------------------------
// ciphertext helpers used by the evaluation below (ckks/src/evaluator.c)
// ---------------------------------------------------------------------------

struct Ct {  // owning ciphertext
  CIPHERTEXT v;
  Ct() { std::memset(&v, 0, sizeof(v)); }
  ~Ct() { Free_ciph_poly(&v, 1); }
  Ct(const Ct&)            = delete;
  Ct& operator=(const Ct&) = delete;
  CIPHER  p() { return &v; }
  size_t  level() const { return v._c0_poly._num_primes; }
};

struct DevBuf {  // stream-ordered scratch
  int64_t* p = nullptr;
  Context* c;
  DevBuf(Context* ctx_, size_t words) : c(ctx_) {
    CUDA_CHECK(dev_alloc(&p, words * sizeof(int64_t), c->stream));
  }
  ~DevBuf() { dev_free(p, c->stream); }
  DevBuf(const DevBuf&)            = delete;
  DevBuf& operator=(const DevBuf&) = delete;
};

void set_level(CIPHER ct, size_t level) {
  ct->_c0_poly._num_primes = ct->_c1_poly._num_primes = level;
}

LimbBatch ct_batch(Context* c, CIPHER res, CIPHER a) {
  return both_polys(poly_batch(c, &res->_c0_poly, &a->_c0_poly, nullptr, a->_c0_poly._num_primes,
                               a->_c0_poly._num_primes_p));
}

void shape_like(Context* c, CIPHER res, CIPHER a, double sf, uint32_t sf_degree) {
  if (res != a) {
    ensure_poly(&res->_c0_poly, c->N, a->_c0_poly._num_primes, a->_c0_poly._num_primes_p);
    ensure_poly(&res->_c1_poly, c->N, a->_c0_poly._num_primes, a->_c0_poly._num_primes_p);
    res->_c0_poly._is_ntt = res->_c1_poly._is_ntt = true;
    res->_slots = a->_slots;
  }
  res->_scaling_factor = sf;
  res->_sf_degree      = sf_degree;
}

std::vector<u64> twice(const std::vector<int64_t>& s) {  // same scalars for c0 and c1
  std::vector<u64> v(s.begin(), s.end());
  v.insert(v.end(), s.begin(), s.end());
  return v;
}

// evaluator.c:218-248: multiply by a real constant encoded at the scaling factor
void mul_const(Context* c, CIPHER res, CIPHER a, double value) {
  size_t level = a->_c0_poly._num_primes, num_p = a->_c0_poly._num_primes_p;
  double delta = std::pow(2.0, (double)c->sf_bits);
  std::vector<u64> sc = twice(encode_value(c, value, (uint32_t)level, delta, (uint32_t)num_p));
  shape_like(c, res, a, a->_scaling_factor * delta, a->_sf_degree + 1);
  launch_scalars(true, ptr2(res->_c0_poly._data, res->_c1_poly._data),
                 ptr2(a->_c0_poly._data, a->_c1_poly._data), sc.data(), ct_batch(c, res, a));
}

// evaluator.c:113-140: add per-limb constants to c0
void add_scalars(Context* c, CIPHER res, CIPHER a, const std::vector<int64_t>& scalars) {
  size_t level = a->_c0_poly._num_primes, num_p = a->_c0_poly._num_primes_p;
  if (res != a) {
    shape_like(c, res, a, a->_scaling_factor, a->_sf_degree);
    Copy_poly(&res->_c1_poly, &a->_c1_poly);
  }
  std::vector<u64> sc(scalars.begin(), scalars.begin() + level + num_p);
  launch_scalars(false, ptr2(res->_c0_poly._data), ptr2(a->_c0_poly._data), sc.data(),
                 poly_batch(c, &res->_c0_poly, &a->_c0_poly, nullptr, level, num_p));
}

void add_const(Context* c, CIPHER res, CIPHER a, double value) {
  add_scalars(c, res, a,
              encode_value(c, value, (uint32_t)a->_c0_poly._num_primes, a->_scaling_factor,
                           (uint32_t)a->_c0_poly._num_primes_p));
}

// evaluator.c:250-258
void mul_integer(Context* c, CIPHER res, CIPHER a, uint64_t power) {
  size_t level = a->_c0_poly._num_primes;
  std::vector<int64_t> s(level);
  for (size_t i = 0; i < level; i++) s[i] = (int64_t)(power % c->primes[i]);
  std::vector<u64> sc = twice(s);
  shape_like(c, res, a, a->_scaling_factor, a->_sf_degree);
  launch_scalars(true, ptr2(res->_c0_poly._data, res->_c1_poly._data),
                 ptr2(a->_c0_poly._data, a->_c1_poly._data), sc.data(), ct_batch(c, res, a));
}

// The transform of x^power on all Q primes, built once per power and kept on
// the device (the two powers a bootstrap uses come back at every bootstrap).
static POLYNOMIAL* monomial_ntt(Context* c, uint32_t reduced) {
  if (c->monomials == nullptr) c->monomials = new std::map<uint32_t, POLYNOMIAL>();
  auto& table = *static_cast<std::map<uint32_t, POLYNOMIAL>*>(c->monomials);
  auto  it    = table.find(reduced);
  if (it != table.end()) return &it->second;
  const uint32_t n = c->N, index = reduced % n;
  const size_t   level = (size_t)c->L;
  POLYNOMIAL mono{};
  Alloc_poly_data(&mono, n, level, 0);  // zero-filled
  std::vector<int64_t> one(level);
  for (size_t i = 0; i < level; i++) one[i] = reduced < n ? 1 : (int64_t)c->primes[i] - 1;
  for (size_t i = 0; i < level; i++)
    CUDA_CHECK(counted_copy(mono._data + i * n + index, &one[i], sizeof(int64_t),
                               cudaMemcpyHostToDevice, c->stream));
  CUDA_CHECK(stream_sync(c->stream));
  Conv_poly2ntt_inplace(&mono);
  return &table.emplace(reduced, mono).first->second;
}

// evaluator.c:260-286: multiply by x^power (power < 2N) through its transform
void mul_monomial(Context* c, CIPHER res, CIPHER a, uint32_t power) {
  size_t      level = a->_c0_poly._num_primes;
  POLYNOMIAL* mono  = monomial_ntt(c, power % (2 * c->N));
  shape_like(c, res, a, a->_scaling_factor, a->_sf_degree);
  // limb i of the cached transform belongs to prime i whatever the level
  LimbBatch one_poly = poly_batch(c, &res->_c0_poly, &a->_c0_poly, mono, level, 0);
  LimbBatch both     = both_polys(one_poly);
  for (int i = one_poly.count; i < both.count; i++) both.limb[i].sel &= ~2;  // one monomial
  launch_elementwise(EW_MUL, ptr2(res->_c0_poly._data, res->_c1_poly._data),
                     ptr2(a->_c0_poly._data, a->_c1_poly._data), ptr2(mono->_data), 0, both);
}

// bootstrap.c:1607-1632, cipher.c:417-446: down to scaling degree 1, keep only
// the q_0 residues, lift them to the first raise_level primes
void raise_from_level0(Context* c, CIPHER res, CIPHER ciph, uint32_t raise_level) {
  const uint32_t n = c->N;
  Ct low;
  Copy_ciph(low.p(), ciph);
  while (low.v._sf_degree > 1) Rescale_ciph(low.p(), low.p());
  set_level(low.p(), 1);
  Conv_ntt2poly_inplace(&low.v._c0_poly);
  Conv_ntt2poly_inplace(&low.v._c1_poly);
  ensure_poly(&res->_c0_poly, n, raise_level, 0);
  ensure_poly(&res->_c1_poly, n, raise_level, 0);
  res->_scaling_factor = low.v._scaling_factor;
  res->_sf_degree      = low.v._sf_degree;
  res->_slots          = ciph->_slots;
  for (POLY dst : {&res->_c0_poly, &res->_c1_poly}) {
    POLY src = dst == &res->_c0_poly ? &low.v._c0_poly : &low.v._c1_poly;
    launch_mod_raise(dst->_data, src->_data, poly_batch(c, dst, dst, nullptr, raise_level, 0));
    dst->_is_ntt = false;
    Conv_poly2ntt_inplace(dst);
  }
}

// evaluator.c:401-409
void mod_switch(CIPHER ct) {
  FHERT_ASSERT(ct->_c0_poly._num_primes >= 2, "polynomial level is too small to support modswitch");
  set_level(ct, ct->_c0_poly._num_primes - 1);
}

}  // namespace fhert

namespace {

// ---------------------------------------------------------------------------
// Chebyshev series evaluation (ckks/src/chebyshev_impl.c)
// ---------------------------------------------------------------------------

typedef std::vector<double> Coeffs;

// index of the last non-zero coefficient (chebyshev_impl.c:42-53)
uint32_t degree_of(const Coeffs& f) {
  uint32_t trailing = 1;
  for (int32_t i = (int32_t)f.size() - 1; i > 0; i--) {
    if (f[i] == 0) trailing++;
    else break;
  }
  return (uint32_t)f.size() - trailing;
}

bool is_even_series(const Coeffs& f) {
  uint32_t d = degree_of(f);
  for (uint32_t i = 1; i <= d; i += 2)
    if (f[i] != 0.) return false;
  return true;
}

// chebyshev_impl.c:71-139: split degree n as k (2^m - 1) > n
void ps_degrees(uint32_t n, uint32_t& k, uint32_t& m) {
  FHERT_ASSERT(n >= 1 && n <= 2204, "unsupported polynomial degree %u", n);
  static const uint32_t ranges[16] = {2, 11, 13, 17, 55, 59, 76, 239, 247, 284, 991, 1007, 1083, 2015, 2031, 2204};
  static const uint32_t values[16] = {1, 2, 3, 2, 3, 4, 3, 4, 5, 4, 5, 6, 5, 6, 7, 6};
  m = 0;
  for (int i = 0; i < 16; i++)
    if (n - 1 < ranges[i]) {
      m = values[i];
      break;
    }
  k = (uint32_t)std::floor(n / ((1 << m) - 1)) + 1;
}

bool differs_from_one(double v) {
  const double prec = 9.5367431640625e-07;  // 2^-20
  return 1 - prec >= v || 1 + prec <= v;
}

// chebyshev_impl.c:159-273: quotient q and remainder r of f / g in the
// Chebyshev basis; the constant terms are kept as c0 (not c0 / 2)
void long_division(Coeffs& q, Coeffs& r, const Coeffs& f, const Coeffs& g) {
  uint32_t n = degree_of(f), k = degree_of(g);
  FHERT_ASSERT(n == f.size() - 1 && k == g.size() - 1, "The dominant coefficient is zero");
  r = f;
  if (n < k) {
    q.assign(1, 0.0);
    return;
  }
  q.assign(n - k + 1, 0.0);
  auto subtract = [&](Coeffs& d) {
    double r_back = r.back(), g_back = g.back();
    if (differs_from_one(r_back))
      for (auto& x : d) x = x * r_back;
    if (differs_from_one(g_back))
      for (auto& x : d) x = x / g_back;
    for (size_t i = 0; i < r.size(); i++) r[i] = r[i] - d[i];
    if (r.size() > 1) {
      n = degree_of(r);
      r.resize(n + 1, 0.0);
    }
  };
  while (n > k) {
    q[n - k] = 2 * r.back();
    if (differs_from_one(g[k])) q[n - k] = q[n - k] / g.back();
    Coeffs d(n + 1, 0.0);
    if (k == n - k) {
      d[0] = 2 * g[n - k];
      for (uint32_t i = 1; i < 2 * k + 1; i++) d[i] = g[std::abs((int32_t)(n - k - i))];
    } else if ((int32_t)k > (int32_t)(n - k)) {
      d[0] = 2 * g[n - k];
      for (uint32_t i = 1; i < k - (n - k) + 1; i++)
        d[i] = g[std::abs((int32_t)(n - k - i))] + g[(int32_t)(n - k + i)];
      for (uint32_t i = k - (n - k) + 1; i < n + 1; i++) d[i] = g[std::abs((int32_t)(i - n + k))];
    } else {
      d[n - k] = g[0];
      for (uint32_t i = n - 2 * k; i < n + 1; i++) d[i] = g[std::abs((int32_t)(i - n + k))];
    }
    subtract(d);
  }
  if (n == k) {
    q[0] = r.back();
    if (differs_from_one(g.back())) q[0] = r.back() / g.back();
    Coeffs d = g;
    subtract(d);
  }
  q[0] = q[0] * 2;
}

struct Cheb {  // state of one Paterson-Stockmeyer evaluation
  Context*          c;
  std::vector<Ct*>  t;   // T_1 .. T_k
  std::vector<Ct*>  t2;  // T_k, T_2k, ..., T_{2^(m-1) k}
};

// chebyshev_impl.c:286-325: out = rescale(sum_i w_i * T_{i+1}) over the first
// `count` base polynomials, skipping zero weights
void weighted_sum(Cheb& st, CIPHER out, uint32_t count, const double* w) {
  Context* c = st.c;
  Ct       tmp;
  bool     first = true;
  for (uint32_t i = 0; i < count; i++) {
    if (w[i] == 0.) continue;
    mul_const(c, tmp.p(), st.t[i]->p(), w[i]);
    if (first) {
      Copy_ciph(out, tmp.p());
      first = false;
    } else {
      Add_ciph(out, out, tmp.p());
    }
  }
  FHERT_ASSERT(!first, "polynomial has no non_zero coefficient");
  Rescale_ciph(out, out);
}

// chebyshev_impl.c:327-389
void eval_quot_or_rem(Cheb& st, CIPHER out, const Coeffs& qr, uint32_t k, bool is_quotient,
                      bool in_recursion) {
  Context* c = st.c;
  Coeffs   cut = qr;
  cut.resize(k, 0.0);
  CIPHER   tk = st.t[k - 1]->p();
  uint32_t dg = degree_of(cut);
  if (dg > 0) {
    weighted_sum(st, out, dg, cut.data() + 1);
    if (is_quotient) {
      if (in_recursion) {
        // the leading coefficient is a power of two: add instead of multiplying
        double quot_last = qr.back();
        Ct     sum;
        Copy_ciph(sum.p(), tk);
        for (uint32_t i = 0; i < std::log2(quot_last); i++) Add_ciph(sum.p(), sum.p(), sum.p());
        Add_ciph(out, out, sum.p());
      } else {
        Add_ciph(out, out, tk);
        Add_ciph(out, out, tk);
      }
    } else {
      Add_ciph(out, out, tk);
    }
  } else {
    Copy_ciph(out, tk);
    if (is_quotient) {
      double   quot_last = qr.back();
      uint32_t end       = in_recursion ? (uint32_t)std::log2(quot_last) : (uint32_t)quot_last;
      for (uint32_t i = 0; i < end; i++) Add_ciph(out, out, tk);
    }
  }
  add_const(c, out, out, qr[0] / 2);
}

// chebyshev_impl.c:392-496
void ps_inner(Cheb& st, CIPHER out, const Coeffs& f, uint32_t k, uint32_t m, bool in_recursion) {
  Context* c     = st.c;
  uint32_t k2m2k = k * (1 << (m - 1)) - k;
  Coeffs   tkm(k2m2k + k + 1, 0.0);
  tkm.back() = 1;
  Coeffs div_q, div_r;
  long_division(div_q, div_r, f, tkm);

  Coeffs r2 = div_r;
  if (k2m2k <= degree_of(div_r)) {
    r2[k2m2k] = r2[k2m2k] - 1;
    r2.resize(degree_of(r2) + 1, 0.0);
  } else {
    r2.resize(k2m2k + 1, 0.0);
    r2.back() = -1;
  }
  Coeffs cq, cr;
  long_division(cq, cr, r2, div_q);
  Coeffs s2 = cr;
  s2.resize(std::max<size_t>(cr.size(), k2m2k + 1), 0.0);
  s2.back() = 1;

  Ct       cu;
  uint32_t dc     = degree_of(cq);
  bool     has_cu = false;
  if (dc >= 1) {
    if (dc == 1) {
      if (cq[1] != 1) {
        mul_const(c, cu.p(), st.t[0]->p(), cq[1]);
        Rescale_ciph(cu.p(), cu.p());
      } else {
        Copy_ciph(cu.p(), st.t[0]->p());
      }
    } else {
      weighted_sum(st, cu.p(), dc, cq.data() + 1);
    }
    add_const(c, cu.p(), cu.p(), cq[0] / 2);
    has_cu = true;
  }
  Ct qu, su;
  if (degree_of(div_q) > k) ps_inner(st, qu.p(), div_q, k, m - 1, true);
  else eval_quot_or_rem(st, qu.p(), div_q, k, true, in_recursion);
  if (degree_of(s2) > k) ps_inner(st, su.p(), s2, k, m - 1, true);
  else eval_quot_or_rem(st, su.p(), s2, k, false, in_recursion);

  CIPHER t2 = st.t2[m - 1]->p();
  if (has_cu) {
    set_level(cu.p(), t2->_c0_poly._num_primes);
    Add_ciph(out, t2, cu.p());
  } else {
    add_const(c, out, t2, cq[0] / 2);
  }
  Mul_ciph(out, out, qu.p());
  Rescale_ciph(out, out);
  Add_ciph(out, out, su.p());
}

// chebyshev_impl.c:498-678 for the interval [-1, 1]
void eval_chebyshev(Context* c, CIPHER out, CIPHER in, const Coeffs& coeffs) {
  uint32_t n    = degree_of(coeffs);
  bool     even = is_even_series(coeffs);
  FHERT_ASSERT(n >= 5, "series of degree below 5 are not supported");
  Coeffs f2(coeffs.begin(), coeffs.begin() + (coeffs.back() == 0 ? n + 1 : coeffs.size()));
  uint32_t k, m;
  ps_degrees(n, k, m);
  if (even && (k % 2 == 1)) k += 1;

  std::vector<Ct> t_store(k), t2_store(m);
  Cheb st;
  st.c = c;
  for (auto& x : t_store) st.t.push_back(&x);
  for (auto& x : t2_store) st.t2.push_back(&x);
  CIPHER t0 = st.t[0]->p();
  Copy_ciph(t0, in);
  Ct y;
  Copy_ciph(y.p(), t0);

  Ct prod;
  std::vector<int64_t> minus_one =
      encode_value(c, -1.0, (uint32_t)t0->_c0_poly._num_primes, t0->_scaling_factor,
                   (uint32_t)t0->_c0_poly._num_primes_p);
  auto double_and_shift = [&](CIPHER tj) {  // tj = 2 * prod, rescaled
    Add_ciph(tj, prod.p(), prod.p());
    Rescale_ciph(tj, tj);
  };
  for (uint32_t i = 2; i <= k; i++) {
    CIPHER tj = st.t[i - 1]->p();
    if (!(i & (i - 1))) {
      CIPHER h = st.t[i / 2 - 1]->p();
      Mul_ciph(prod.p(), h, h);
      double_and_shift(tj);
      add_scalars(c, tj, tj, minus_one);
    } else if (i % 2 == 1) {
      if (even) continue;
      Mul_ciph(prod.p(), st.t[i / 2 - 1]->p(), st.t[i / 2]->p());
      double_and_shift(tj);
      Sub_ciph(tj, tj, y.p());
    } else {
      uint32_t h1 = i / 2;
      if (even && (h1 % 2 == 1)) h1 += 1;
      uint32_t h2 = i - h1;
      Mul_ciph(prod.p(), st.t[h1 - 1]->p(), st.t[h2 - 1]->p());
      double_and_shift(tj);
      if (h1 == h2) add_scalars(c, tj, tj, minus_one);
      else Sub_ciph(tj, tj, st.t[1]->p());
    }
  }
  // bring every base polynomial to the level of T_k
  size_t low = st.t[k - 1]->level();
  for (uint32_t i = 1; i < k; i++) {
    if (even && i % 2 == 1) continue;
    set_level(st.t[i - 1]->p(), low);
  }

  Copy_ciph(st.t2[0]->p(), st.t[k - 1]->p());
  for (uint32_t i = 1; i < m; i++) {
    CIPHER prev = st.t2[i - 1]->p(), cur = st.t2[i]->p();
    Mul_ciph(prod.p(), prev, prev);
    double_and_shift(cur);
    add_scalars(c, cur, cur, minus_one);
  }
  Ct t2km1;
  Copy_ciph(t2km1.p(), st.t2[0]->p());
  for (uint32_t i = 1; i < m; i++) {
    Mul_ciph(prod.p(), t2km1.p(), st.t2[i]->p());
    double_and_shift(t2km1.p());
    Sub_ciph(t2km1.p(), t2km1.p(), st.t2[0]->p());
  }

  uint32_t k2m2k = k * (1 << (m - 1)) - k;
  f2.resize(2 * k2m2k + k + 1, 0.0);
  f2.back() = 1;
  ps_inner(st, out, f2, k, m, false);
  Sub_ciph(out, out, t2km1.p());
}

}  // namespace

namespace {

// ---------------------------------------------------------------------------
// linear transforms on extended ciphertexts (bootstrap.c:1233-1496)
// ---------------------------------------------------------------------------

// level Q limbs followed directly by the K special limbs of one buffer
LimbBatch ext_batch(Context* c, size_t level) {
  LimbBatch b;
  b.count = 0;
  for (size_t i = 0; i < level + c->K; i++) {
    uint8_t prime = (uint8_t)(i < level ? i : c->L + (i - level));
    b.limb[b.count++] = LimbRef{(uint16_t)i, (uint16_t)i, (uint16_t)i, prime, 0};
  }
  return b;
}

LimbBatch q_only(Context* c, size_t level) {
  LimbBatch b;
  b.count = 0;
  for (size_t i = 0; i < level; i++)
    b.limb[b.count++] = LimbRef{(uint16_t)i, (uint16_t)i, (uint16_t)i, (uint8_t)i, 0};
  return b;
}

// key-switch inner product of raised digits with the key of automorphism k:
// acc (two extended polynomials) = sum_j digit_j * key_j
void digits_times_key(Context* c, const int64_t* digits, const int64_t* own, size_t level,
                      int parts, uint32_t k, int64_t* acc) {
  SWITCH_KEY* key = key_slot(c, k, false);
  FHERT_ASSERT(key != nullptr, "cannot find the rotation key of automorphism %u", k);
  const size_t ext = level + c->K, n = c->N;
  InnerArgs args;
  std::memset(&args, 0, sizeof(args));
  args.parts      = parts;
  args.level      = (int)level;
  args.alpha      = c->alpha;
  args.key_p_limb = c->L;
  args.ext_p_limb = (int)level;
  args.acc_p_limb = (int)level;
  args.in         = reinterpret_cast<const u64*>(own);
  for (int j = 0; j < parts; j++) {
    args.ext_ptr[j] = reinterpret_cast<const u64*>(digits + (size_t)j * ext * n);
    args.key0[j]    = reinterpret_cast<const u64*>(key->_parts[j]._p0._data);
    args.key1[j]    = reinterpret_cast<const u64*>(key->_parts[j]._p1._data);
  }
  args.acc0 = reinterpret_cast<u64*>(acc);
  args.acc1 = reinterpret_cast<u64*>(acc + ext * n);
  launch_inner_product(args);
}

// one stage: rescale, hoisted giant-step rotations, fused baby-step sums,
// outer rotations on the extended basis, one ModDown at the end
void rotate_stage(Context* c, CIPHER ct, std::vector<PLAINTEXT>& plains, const FftParams& p,
                  const std::vector<int32_t>& rot_in, const std::vector<int32_t>& rot_out, int step,
                  bool encoding, bool is_rem) {
  const int giant = is_rem ? p.g_rem : p.g, baby = is_rem ? p.b_rem : p.b;
  const int num_rot = is_rem ? p.num_rot_rem : p.num_rot;
  const int level_idx = encoding ? p.level_budget - 1 : 0;
  if (is_rem || step != level_idx) Rescale_ciph(ct, ct);

  const size_t n = c->N, K = c->K, level = ct->_c0_poly._num_primes, ext = level + K;
  const size_t pw = ext * n;  // words of one extended polynomial
  const int    parts = (int)std::min<size_t>((level + c->alpha - 1) / c->alpha, c->dnum);
  FHERT_ASSERT(giant <= kMaxParts, "giant step %d exceeds the fused limit", giant);
  const LimbBatch eb = ext_batch(c, level), eb2 = both_polys(eb), qb = q_only(c, level);
  // both polynomials on the extended basis; the Q limbs of the first one also
  // pick up the lifted c0 while they are permuted
  LimbBatch eb2_add = eb2;
  for (int i = 0; i < eb2_add.count; i++) {
    LimbRef& r = eb2_add.limb[i];
    bool     q_of_c0 = i < (int)level;
    r.b   = q_of_c0 ? (uint16_t)i : 0;
    r.sel = (uint8_t)((r.sel & ~2) | (q_of_c0 ? 2 : 0));  // bit 1 = "add the lifted limb"
  }

  DevBuf digits(c, (size_t)parts * pw), rot(c, (size_t)giant * 2 * pw), lifted(c, 2 * pw);
  DevBuf acc(c, 2 * pw), inner(c, 2 * pw), outer(c, 2 * pw), first(c, pw), turned(c, 2 * pw);
  DevBuf low(c, level * n);
  int64_t* c0 = ct->_c0_poly._data;
  int64_t* c1 = ct->_c1_poly._data;

  // lifted = (P * c0, P * c1) on the Q limbs, zero on the special limbs
  CUDA_CHECK(zero_async(lifted.p, 2 * pw * sizeof(int64_t), c->stream));
  launch_mul_const(ptr2(lifted.p, lifted.p + pw), ptr2(c0, c1), c->d_p_mod_q, both_polys(qb));
  fhert_raise_parts(c, c1, true, level, 0, parts, digits.p, ext, (int)level);

  for (int j = 0; j < giant; j++) {
    int64_t* dst = rot.p + (size_t)j * 2 * pw;
    int32_t  val = rot_in[j];
    if (val == 0) {
      CUDA_CHECK(counted_copy(dst, lifted.p, 2 * pw * sizeof(int64_t), cudaMemcpyDeviceToDevice,
                                 c->stream));
      continue;
    }
    uint32_t k = auto_index_for(c, val);
    digits_times_key(c, digits.p, c1, level, parts, k, acc.p);
    launch_automorphism_add(ptr2(dst, dst + pw), ptr2(acc.p, acc.p + pw), lifted.p,
                            auto_table(c, k), eb2_add);
  }

  double   plain_sf     = 0;
  uint32_t plain_degree = 0;
  for (int i = 0; i < baby; i++) {
    // inner = sum_j rot_j * plain[giant * i + j]
    InnerArgs args;
    std::memset(&args, 0, sizeof(args));
    args.level      = (int)level;
    args.alpha      = c->alpha;
    args.key_p_limb = (int)level;
    args.acc_p_limb = (int)level;
    args.in         = nullptr;
    int terms = 0;
    for (int j = 0; j < giant; j++) {
      int dim2 = giant * i + j;
      if (dim2 == num_rot) continue;
      PLAINTEXT& pt = plains[dim2];
      FHERT_ASSERT(pt._poly._data != nullptr && pt._poly._num_primes >= level,
                   "missing or too shallow transform plaintext");
      args.ext_p_limb  = (int)(pt._poly._num_alloc_primes - pt._poly._num_primes_p);
      args.ext_ptr[terms] = reinterpret_cast<const u64*>(pt._poly._data);
      args.key0[terms]    = reinterpret_cast<const u64*>(rot.p + (size_t)j * 2 * pw);
      args.key1[terms]    = reinterpret_cast<const u64*>(rot.p + (size_t)j * 2 * pw + pw);
      plain_sf     = pt._scaling_factor;
      plain_degree = pt._sf_degree;
      terms++;
    }
    args.parts = terms;
    args.acc0  = reinterpret_cast<u64*>(inner.p);
    args.acc1  = reinterpret_cast<u64*>(inner.p + pw);
    launch_inner_product(args);

    if (i == 0) {
      CUDA_CHECK(counted_copy(first.p, inner.p, pw * sizeof(int64_t), cudaMemcpyDeviceToDevice,
                                 c->stream));
      CUDA_CHECK(zero_async(outer.p, pw * sizeof(int64_t), c->stream));
      CUDA_CHECK(counted_copy(outer.p + pw, inner.p + pw, pw * sizeof(int64_t),
                                 cudaMemcpyDeviceToDevice, c->stream));
      continue;
    }
    int32_t val = rot_out[i];
    if (val == 0) {
      launch_elementwise(EW_ADD, ptr2(first.p), ptr2(first.p), ptr2(inner.p), 0, eb);
      launch_elementwise(EW_ADD, ptr2(outer.p + pw), ptr2(outer.p + pw), ptr2(inner.p + pw), 0, eb);
      continue;
    }
    uint32_t k = auto_index_for(c, val);
    // c0 part stays extended: first += sigma_k(inner.c0)
    launch_automorphism(ptr2(turned.p), ptr2(inner.p), auto_table(c, k), eb);
    launch_elementwise(EW_ADD, ptr2(first.p), ptr2(first.p), ptr2(turned.p), 0, eb);
    // c1 part: back to Q, key switch, rotate, accumulate on the extended basis
    int64_t*       r[2] = {low.p, nullptr};
    const int64_t* x[2] = {inner.p + pw, nullptr};
    fhert_mod_down_polys(c, 1, r, x, (int)level, nullptr, level, true);
    fhert_raise_parts(c, low.p, true, level, 0, parts, digits.p, ext, (int)level);
    digits_times_key(c, digits.p, low.p, level, parts, k, acc.p);
    launch_automorphism(ptr2(turned.p, turned.p + pw), ptr2(acc.p, acc.p + pw), auto_table(c, k), eb2);
    launch_elementwise(EW_ADD, ptr2(outer.p, outer.p + pw), ptr2(outer.p, outer.p + pw),
                       ptr2(turned.p, turned.p + pw), 0, eb2);
  }
  launch_elementwise(EW_ADD, ptr2(outer.p), ptr2(outer.p), ptr2(first.p), 0, eb);
  int64_t*       r[2] = {c0, c1};
  const int64_t* x[2] = {outer.p, outer.p + pw};
  fhert_mod_down_polys(c, 2, r, x, (int)level, nullptr, level, true);
  ct->_scaling_factor = ct->_scaling_factor * plain_sf;
  ct->_sf_degree      = ct->_sf_degree + plain_degree;
}

// bootstrap.c:1375-1484
void linear_transform(Context* c, CIPHER result, CIPHER in, Precom* pre, bool encoding) {
  const FftParams& p     = encoding ? pre->enc : pre->dec;
  auto&            plain = encoding ? pre->c2s : pre->s2c;
  const uint32_t   order = 2 * c->N, slots = in->_slots;
  const int flag_rem = p.rem_coll != 0 ? 1 : 0, stop = flag_rem ? 0 : -1;
  const int start = encoding ? stop + 1 : 0;
  const int end   = encoding ? p.level_budget : p.level_budget - flag_rem;
  const uint32_t slots_value = encoding ? slots : order / 4;
  std::vector<std::vector<int32_t>> rot_in(p.level_budget), rot_out(p.level_budget);
  for (int i = 0; i < p.level_budget; i++) {
    bool is_rem = flag_rem && i == (encoding ? 0 : p.level_budget - 1);
    rot_in[i].assign((is_rem ? p.num_rot_rem : p.num_rot) + 1, 0);
    rot_out[i].assign(p.b + p.b_rem, 0);
  }
  for (int s = start; s < end; s++) {
    int shift = encoding ? (s - flag_rem) * p.layers_coll + p.rem_coll : s * p.layers_coll;
    for (int j = 0; j < p.g; j++)
      rot_in[s][j] = (int32_t)reduce_rotation((j - ((p.num_rot + 1) / 2) + 1) * (1 << shift), slots_value);
    for (int i = 0; i < p.b; i++)
      rot_out[s][i] = (int32_t)reduce_rotation((p.g * i) * (1 << shift), order / 4);
  }
  if (flag_rem) {
    int s     = encoding ? stop : p.level_budget - flag_rem;
    int shift = encoding ? 1 : 1 << (s * p.layers_coll);
    for (int j = 0; j < p.g_rem; j++)
      rot_in[s][j] = (int32_t)reduce_rotation((j - ((p.num_rot_rem + 1) / 2) + 1) * shift, slots_value);
    for (int i = 0; i < p.b_rem; i++)
      rot_out[s][i] = (int32_t)reduce_rotation((p.g_rem * i) * shift, order / 4);
  }
  Copy_ciph(result, in);
  if (encoding)
    for (int s = end - 1; s > start - 1; s--) {
      rotate_stage(c, result, plain[s], p, rot_in[s], rot_out[s], s, true, false);
      trace_sum("c2s stage", result);
    }
  else
    for (int s = start; s < end; s++) {
      rotate_stage(c, result, plain[s], p, rot_in[s], rot_out[s], s, false, false);
      trace_sum("s2c stage", result);
    }
  if (flag_rem) {
    int s = encoding ? stop : p.level_budget - flag_rem;
    rotate_stage(c, result, plain[s], p, rot_in[s], rot_out[s], s, encoding, true);
  }
}

}  // namespace

namespace {

// ---------------------------------------------------------------------------
// the bootstrap itself (bootstrap.c:1504-1830)
// ---------------------------------------------------------------------------

void approx_mod(Context* c, CIPHER ct) {
  const SineTable& tab = sine_table(c->hamming_weight);
  if (sine_table_is_even(tab)) add_const(c, ct, ct, -1. / (4. * tab.k));
  Coeffs coeffs(tab.coeff, tab.coeff + tab.size);
  eval_chebyshev(c, ct, ct, coeffs);
  // double-angle iterations: cos(2x) = 2 cos^2(x) - 1, scaled
  int r = tab.double_angle;
  for (int j = 1; j < r + 1; j++) {
    Mul_ciph(ct, ct, ct);
    Add_ciph(ct, ct, ct);
    add_const(c, ct, ct, -1.0 / std::pow(2.0 * M_PI, std::pow(2.0, j - r)));
    Rescale_ciph(ct, ct);
  }
}

// bootstrap.c:1795-1824: back to the message's scale, optionally dropping the imaginary part
void finish_bootstrap(Context* c, CIPHER res, int deg) {
  const char* clear_env  = std::getenv("RT_BTS_CLEAR_IMAG");
  bool        clear_imag = clear_env != nullptr && std::atoi(clear_env) != 0;
  if (clear_imag && deg >= 1) {
    Ct conj;
    Conjugate_ciph(conj.p(), res);
    Add_ciph(res, res, conj.p());
    uint64_t ratio = (uint64_t)std::pow(2., deg - 1);
    if (ratio > 1) mul_integer(c, res, res, ratio);
  } else {
    mul_integer(c, res, res, (uint64_t)std::pow(2., deg));
  }
  while (res->_sf_degree > 1) Rescale_ciph(res, res);
}

void bootstrap_impl(Context* c, CIPHER res, CIPHER ciph, uint32_t level_after, Precom* pre) {
  const uint32_t n = c->N, m = 2 * n, slots = ciph->_slots;
  const uint32_t bts_depth =
      approx_mod_depth(c->hamming_weight) + pre->enc.level_budget + pre->dec.level_budget;
  if (!level_after) level_after = (uint32_t)c->L - bts_depth;
  FHERT_ASSERT(level_after <= (uint32_t)c->L - bts_depth,
               "The level set after bootstrapping is excessively high");
  if (ciph->_c0_poly._num_primes - (ciph->_sf_degree - 1) >= level_after) {
    if (res != ciph) Copy_ciph(res, ciph);
    return;
  }
  const double sf  = std::pow(2.0, (double)c->sf_bits);
  const int    deg = (int)std::round(std::log2((double)c->primes[0] / sf));

  const uint32_t raise_level = level_after + bts_depth;
  Ct raised;
  raise_from_level0(c, raised.p(), ciph, raise_level);

  Ct enc;
  if (slots == m / 4) {
    linear_transform(c, enc.p(), raised.p(), pre, true);
    Ct conj, diff;
    Conjugate_ciph(conj.p(), enc.p());
    trace_sum("conj", conj.p());
    Sub_ciph(diff.p(), enc.p(), conj.p());
    Add_ciph(enc.p(), enc.p(), conj.p());
    trace_sum("sum", enc.p());
    mul_monomial(c, diff.p(), diff.p(), 3 * m / 4);
    trace_sum("diff", diff.p());
    while (enc.v._sf_degree > 1) {
      Rescale_ciph(enc.p(), enc.p());
      Rescale_ciph(diff.p(), diff.p());
    }
    approx_mod(c, enc.p());
    approx_mod(c, diff.p());
    mul_monomial(c, diff.p(), diff.p(), m / 4);
    Add_ciph(enc.p(), enc.p(), diff.p());
    linear_transform(c, res, enc.p(), pre, false);
  } else {
    Ct tmp;
    for (uint32_t j = 1; j < n / (2 * slots); j <<= 1) {
      Rotate_ciph(tmp.p(), raised.p(), (int32_t)(j * slots));
      Add_ciph(raised.p(), raised.p(), tmp.p());
    }
    linear_transform(c, enc.p(), raised.p(), pre, true);
    Ct conj;
    Conjugate_ciph(conj.p(), enc.p());
    Add_ciph(enc.p(), enc.p(), conj.p());
    while (enc.v._sf_degree > 1) Rescale_ciph(enc.p(), enc.p());
    approx_mod(c, enc.p());
    linear_transform(c, res, enc.p(), pre, false);
    Ct rot;
    Rotate_ciph(rot.p(), res, (int32_t)slots);
    Add_ciph(res, res, rot.p());
  }

  finish_bootstrap(c, res, deg);
}

// ---------------------------------------------------------------------------
// the bootstrap in three separately callable stages (cipher.c:585-767).  The
// full-packed case carries the imaginary-part ciphertext from the first stage
// to the second in a per-thread state, as the CPU runtime does.
// ---------------------------------------------------------------------------

struct StageState {
  bool       active = false, full_packed = false;
  uint32_t   slots  = 0;
  bool       has_diff = false;
  CIPHERTEXT diff{};
};
thread_local StageState g_stage;

void clear_stage_state() {
  if (g_stage.has_diff) Free_ciph_poly(&g_stage.diff, 1);
  g_stage = StageState();
}

Precom* ensure_precom(Context* c, uint32_t slots) {  // cipher.c:491-517
  auto& table = precoms(c);
  if (table.find(slots) == table.end()) prepare_bootstrap(c, slots);
  auto it = table.find(slots);
  FHERT_ASSERT(it != table.end(), "Bootstrap precom is unavailable after Bootstrap_precom");
  keygen(c, it->second);
  return it->second;
}

void rescale_to_degree_one(CIPHER ct, CIPHER paired) {  // cipher.c:546-563 with AUTO_SCALE off
  while (ct->_sf_degree > 1) {
    Rescale_ciph(ct, ct);
    if (paired != nullptr) Rescale_ciph(paired, paired);
  }
}

}  // namespace

namespace fhert {

void prepare_bootstrap(Context* c, uint32_t slots) {
  uint32_t depth = approx_mod_depth(c->hamming_weight) + 3 + 3;
  if ((uint32_t)(c->L - 1) <= depth) return;  // context too shallow to bootstrap
  Precom* pre = setup(c, slots);
  keygen(c, pre);
}

void free_bootstrap(Context* c) {
  if (c->monomials != nullptr) {
    auto* monos = static_cast<std::map<uint32_t, POLYNOMIAL>*>(c->monomials);
    for (auto& kv : *monos) Free_poly_data(&kv.second);
    delete monos;
    c->monomials = nullptr;
  }
  if (c->bootstrap == nullptr) return;
  auto* table = static_cast<std::map<uint32_t, Precom*>*>(c->bootstrap);
  for (auto& kv : *table) {
    for (auto* group : {&kv.second->c2s, &kv.second->s2c})
      for (auto& stage : *group)
        for (auto& pt : stage)
          if (pt._poly._data) Free_poly_data(&pt._poly);
    delete kv.second;
  }
  delete table;
  c->bootstrap = nullptr;
}

}  // namespace fhert

extern "C" {

// ckks/src/cipher.c:565-583
CIPHER Bootstrap(CIPHER res, CIPHER ciph, uint32_t level_after_bts) {
  Context* c = ctx();
  FHERT_ASSERT(ciph->_c0_poly._num_primes > 0, "Input cipher level is exhausted");
  uint32_t slots = ciph->_slots;
  auto&    table = precoms(c);
  if (table.find(slots) == table.end()) prepare_bootstrap(c, slots);
  auto it = table.find(slots);
  FHERT_ASSERT(it != table.end(), "Bootstrap precom is unavailable: the context needs more than %u levels",
               approx_mod_depth(c->hamming_weight) + 6);
  keygen(c, it->second);
  bootstrap_impl(c, res, ciph, level_after_bts, it->second);
  return res;
}

// ant/context/src/ckks_context.c:239-262
void Bootstrap_precom(uint32_t num_slots) { prepare_bootstrap(ctx(), num_slots); }

// ckks/src/cipher.c:565-579
CIPHER Eval_bootstrap_ciph(CIPHER res, CIPHER ciph, uint32_t level_after_bts, uint32_t num_slots) {
  Context* c = ctx();
  FHERT_ASSERT(ciph->_c0_poly._num_primes > 0, "Input cipher level is exhausted");
  ensure_precom(c, num_slots ? num_slots : ciph->_slots);
  bootstrap_impl(c, res, ciph, level_after_bts, ensure_precom(c, ciph->_slots));
  return res;
}

// ckks/src/cipher.c:585-665: raise to the full modulus, CoeffsToSlots, split
// into real and imaginary parts (the latter is kept for the next stage)
CIPHER Eval_bootstrap_coeffs_to_slots_ciph(CIPHER res, CIPHER ciph, uint32_t num_slots) {
  Context* c = ctx();
  clear_stage_state();
  const uint32_t n = c->N, m = 2 * n;
  const uint32_t slots = num_slots ? num_slots : ciph->_slots;
  Precom*        pre   = ensure_precom(c, slots);
  Ct raised;
  raise_from_level0(c, raised.p(), ciph, (uint32_t)c->L);
  raised.v._slots = slots;
  const bool full = slots == m / 4;
  if (!full) {
    Ct tmp;
    for (uint32_t j = 1; j < n / (2 * slots); j <<= 1) {
      Rotate_ciph(tmp.p(), raised.p(), (int32_t)(j * slots));
      Add_ciph(raised.p(), raised.p(), tmp.p());
    }
  }
  linear_transform(c, res, raised.p(), pre, true);
  Ct conj;
  Conjugate_ciph(conj.p(), res);
  if (full) {
    std::memset(&g_stage.diff, 0, sizeof(g_stage.diff));
    g_stage.has_diff = true;
    Sub_ciph(&g_stage.diff, res, conj.p());
    Add_ciph(res, res, conj.p());
    mul_monomial(c, &g_stage.diff, &g_stage.diff, 3 * m / 4);
    rescale_to_degree_one(res, &g_stage.diff);
  } else {
    Add_ciph(res, res, conj.p());
    rescale_to_degree_one(res, nullptr);
  }
  g_stage.active      = true;
  g_stage.full_packed = full;
  g_stage.slots       = slots;
  return res;
}

// ckks/src/cipher.c:667-709: the approximate modular reduction of both parts
CIPHER Eval_bootstrap_eval_mod_ciph(CIPHER res, CIPHER ciph, uint32_t num_slots) {
  Context*       c     = ctx();
  const uint32_t slots = num_slots ? num_slots : ciph->_slots;
  ensure_precom(c, slots);
  const bool pair = g_stage.active && g_stage.full_packed && g_stage.has_diff && g_stage.slots == slots;
  if (pair) {
    if (res != ciph) Copy_ciph(res, ciph);
    approx_mod(c, res);
    approx_mod(c, &g_stage.diff);
    mul_monomial(c, &g_stage.diff, &g_stage.diff, slots);
    Add_ciph(res, res, &g_stage.diff);
    Free_ciph_poly(&g_stage.diff, 1);
    g_stage.has_diff = false;
  } else {
    rescale_to_degree_one(ciph, nullptr);
    if (res != ciph) Copy_ciph(res, ciph);
    approx_mod(c, res);
  }
  return res;
}

// ckks/src/cipher.c:711-767: SlotsToCoeffs and the way back to the message's scale
CIPHER Eval_bootstrap_slots_to_coeffs_ciph(CIPHER res, CIPHER ciph, uint32_t num_slots) {
  Context*       c     = ctx();
  const uint32_t m     = 2 * c->N;
  const uint32_t slots = num_slots ? num_slots : ciph->_slots;
  Precom*        pre   = ensure_precom(c, slots);
  linear_transform(c, res, ciph, pre, false);
  if (slots != m / 4) {
    Ct rot;
    Rotate_ciph(rot.p(), res, (int32_t)slots);
    Add_ciph(res, res, rot.p());
  }
  const double sf  = std::pow(2.0, (double)c->sf_bits);
  const int    deg = (int)std::round(std::log2((double)c->primes[0] / sf));
  finish_bootstrap(c, res, deg);
  clear_stage_state();
  return res;
}

size_t Fhert_bootstrap_rotations(uint32_t slots, int32_t* out, size_t cap) {
  Context* c     = ctx();
  auto&    table = precoms(c);
  auto     it    = table.find(slots ? slots : c->N / 2);
  if (it == table.end()) return 0;
  std::vector<int32_t> r = all_rotations(c, it->second);
  for (size_t i = 0; i < r.size() && i < cap; i++) out[i] = r[i];
  return r.size();
}

size_t Fhert_export_bootstrap_plain(uint32_t slots, int encoding, uint32_t stage, uint32_t index,
                                    int64_t* host) {
  Context* c     = ctx();
  auto&    table = precoms(c);
  auto     it    = table.find(slots ? slots : c->N / 2);
  if (it == table.end()) return 0;
  auto& all = encoding ? it->second->c2s : it->second->s2c;
  if (stage >= all.size() || index >= all[stage].size()) return 0;
  POLY p = &all[stage][index]._poly;
  if (p->_data == nullptr) return 0;
  Fhert_download(p, 0, p->_num_primes, host);
  Fhert_download(p, p->_num_alloc_primes - p->_num_primes_p, p->_num_primes_p,
                 host + p->_num_primes * (size_t)c->N);
  return p->_num_primes;
}

}  // extern "C"
