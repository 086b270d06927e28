// Client-side entry points of the C ABI: seeding, encode, encrypt, decrypt,
// decode and key export.  Citations name files inside fhe-cmplr/rtlib/ant/.
#include <algorithm>
#include <cmath>
#include <complex>
#include <cstring>
#include <vector>

#include "runtime.h"

using namespace fhert;

namespace {

typedef std::complex<double> cplx;

constexpr int64_t kMax64 = (int64_t)(((u64)1 << 63) - ((u64)1 << 9)) - 1;

uint32_t reverse_bits(uint32_t v, int bits) {
  uint32_t r = 0;
  for (int i = 0; i < bits; i++) r |= ((v >> i) & 1u) << (bits - 1 - i);
  return r;
}

// util/src/ntt.c:562-590: roots e^(2 pi i k / 2N) and the powers of 5 mod 2N
void ensure_fft_tables(Context* c) {
  if (!c->fft_rou_re.empty()) return;
  size_t m = 2ull * c->N;
  c->fft_rou_re.resize(m);
  c->fft_rou_im.resize(m);
  for (size_t i = 0; i < m; i++) {
    double angle     = 2 * M_PI * i / m;
    c->fft_rou_re[i] = std::cos(angle);
    c->fft_rou_im[i] = std::sin(angle);
  }
  size_t slots = c->N / 2;
  c->fft_rot_group.resize(slots);
  c->fft_rot_group[0] = 1;
  for (size_t i = 1; i < slots; i++)
    c->fft_rot_group[i] = (uint32_t)((5ull * c->fft_rot_group[i - 1]) % m);
}

// complex product with the textbook formula and separately rounded operations,
// as the C compiler of the CPU runtime evaluates it
inline cplx cmul(cplx a, cplx b) {
  double re = a.real() * b.real() - a.imag() * b.imag();
  double im = a.real() * b.imag() + a.imag() * b.real();
  return cplx(re, im);
}

// util/src/ntt.c:633-675
void embedding_inv(Context* c, std::vector<cplx>& v) {
  size_t len = v.size(), m = 2ull * c->N;
  int    lg  = 0;
  while ((1ull << lg) < len) lg++;
  for (int logm = lg; logm > 0; logm--) {
    size_t idx_mod = 1ull << (logm + 2), gap = m / idx_mod, num1 = 1ull << logm,
           num2 = 1ull << (logm - 1);
    for (size_t j = 0; j < len; j += num1) {
      for (size_t i = 0; i < num2; i++) {
        size_t e = j + i, o = j + i + num2;
        size_t r = (idx_mod - (c->fft_rot_group[i] % idx_mod)) * gap;
        cplx   plus = v[e] + v[o], minus = v[e] - v[o];
        minus = cmul(minus, cplx(c->fft_rou_re[r], c->fft_rou_im[r]));
        v[e]  = plus;
        v[o]  = minus;
      }
    }
  }
  std::vector<cplx> out(len);
  for (size_t i = 0; i < len; i++) out[i] = v[reverse_bits((uint32_t)i, lg)];
  double d = (double)len;
  for (size_t i = 0; i < len; i++) v[i] = cplx(out[i].real() / d, out[i].imag() / d);
}

// util/src/ntt.c:598-631
void embedding(Context* c, std::vector<cplx>& v) {
  size_t len = v.size(), m = 2ull * c->N;
  int    lg  = 0;
  while ((1ull << lg) < len) lg++;
  std::vector<cplx> res(len);
  for (size_t i = 0; i < len; i++) res[i] = v[reverse_bits((uint32_t)i, lg)];
  for (int logm = 1; logm <= lg; logm++) {
    size_t idx_mod = 1ull << (logm + 2), gap = m / idx_mod, num = 1ull << (logm - 1);
    for (size_t j = 0; j < len; j += (1ull << logm)) {
      for (size_t i = 0; i < num; i++) {
        size_t e = j + i, o = j + i + num;
        size_t r = (c->fft_rot_group[i] % idx_mod) * gap;
        cplx   w = cmul(cplx(c->fft_rou_re[r], c->fft_rou_im[r]), res[o]);
        cplx   plus = res[e] + w, minus = res[e] - w;
        res[e] = plus;
        res[o] = minus;
      }
    }
  }
  v.swap(res);
}

void init_plain(Context* c, PLAIN plain, size_t level, double scale, uint32_t sf_degree,
                uint32_t slots = 0, size_t num_p = 0) {
  POLY p = &plain->_poly;
  // special limbs sit at the end of the allocation, so an extended plaintext
  // needs storage of exactly level + K limbs
  if (p->_data == nullptr || (num_p ? p->_num_alloc_primes != level + num_p
                                    : p->_num_alloc_primes < level)) {
    Free_poly_data(p);
    Alloc_poly_data(p, c->N, level, num_p);
  } else {
    p->_num_primes   = level;
    p->_num_primes_p = num_p;
  }
  plain->_scaling_factor = scale;
  plain->_sf_degree      = sf_degree;
  plain->_slots          = slots ? slots : c->N / 2;
}

// level Q limbs, then num_p special limbs stored right behind them
LimbBatch q_batch(size_t level, size_t num_p = 0, int first_p_prime = 0) {
  LimbBatch b;
  b.count = (int)(level + num_p);
  for (size_t i = 0; i < level; i++)
    b.limb[i] = LimbRef{(uint16_t)i, (uint16_t)i, (uint16_t)i, (uint8_t)i, 0};
  for (size_t k = 0; k < num_p; k++) {
    uint16_t at = (uint16_t)(level + k);
    b.limb[level + k] = LimbRef{at, at, at, (uint8_t)(first_p_prime + k), 0};
  }
  return b;
}

}  // namespace

namespace fhert {

// ckks/src/encoder.c:473-520: residues of one real value at the given scale,
// on level Q limbs followed by num_p special limbs
std::vector<int64_t> encode_value(Context* c, double value, uint32_t level, double scale,
                                  uint32_t num_p) {
  FHERT_ASSERT(level > 0 && level <= (uint32_t)c->L, "level should not be larger than q_cnt");
  FHERT_ASSERT(num_p == 0 || num_p == (uint32_t)c->K, "invalid p cnt");
  int32_t log_scale  = (int32_t)std::log2(std::fabs(value * scale));
  int32_t log_valid  = log_scale <= 61 ? log_scale : 61;
  int32_t log_approx = log_scale - log_valid;
  double  scaled     = value / std::pow(2, log_approx) * scale;
  int64_t val_int    = (int64_t)scaled;
  std::vector<int64_t> res(level + num_p);
  for (uint32_t i = 0; i < level + num_p; i++) {
    int64_t q = (int64_t)c->primes[i < level ? i : c->L + (i - level)], r = val_int % q;
    res[i] = r < 0 ? r + q : r;
  }
  if (log_approx > 0) {
    // scale back up by 2^log_approx in steps of at most 61 then 60 bits
    for (uint32_t i = 0; i < level; i++) {
      u64     q = c->primes[i];
      int32_t left = log_approx, step = left <= 61 ? left : 61;
      u64     f = (1ull << step) % q;
      left -= step;
      while (left > 0) {
        step = left <= 60 ? left : 60;
        f    = mulmod(f, (1ull << step) % q, q);
        left -= step;
      }
      res[i] = (int64_t)mulmod((u64)res[i], f, q);
    }
  }
  return res;
}

// ckks/src/encoder.c:234-325; slots = 0 means N/2, num_p = K also fills the
// special limbs (the plaintexts of the bootstrapping linear transforms)
void encode_vector(Context* c, PLAIN plain, std::vector<cplx>& values, uint32_t sf_degree,
                   uint32_t level, uint32_t slots, uint32_t num_p, const float* reals,
                   size_t real_count) {
  ensure_fft_tables(c);
  const uint32_t n = c->N;
  if (slots == 0) slots = n / 2;
  FHERT_ASSERT(slots <= n / 2 && (slots & (slots - 1)) == 0, " slot size > N/2 ");
  FHERT_ASSERT(num_p == 0 || num_p == (uint32_t)c->K, "invalid p cnt");
  const uint32_t gap = n / (slots * 2);
  if (level == 0) level = c->L;
  FHERT_ASSERT(level <= (uint32_t)c->L, "level should not be larger than mul_depth + 1");
  const size_t count = reals != nullptr ? real_count : values.size();
  FHERT_ASSERT(count <= slots, "slot size is too small");
  FHERT_ASSERT(sf_degree >= 1, "invalid scaling factor for encode");
  const double delta = std::pow(2.0, (double)c->sf_bits);
  init_plain(c, plain, level, std::pow(delta, (double)sf_degree), sf_degree, slots, num_p);
  int64_t* d_msg = nullptr;
  u64*     d_pow = nullptr;
  CUDA_CHECK(dev_alloc(&d_msg, n * sizeof(int64_t), c->stream));
  // inverse embedding, scaling and rounding run on the device with the host
  // routine's arithmetic (encode_gpu.cu)
  encode_message_on_device(c, values.data(), count, slots, d_msg, reals);
  std::vector<u64> powp;
  if (sf_degree > 1) {
    // Delta^(d-1) modulo every prime (encoder.c:297-312)
    powp.assign(c->L + c->K, 1);
    for (uint32_t i = 0; i < level; i++) {
      u64 q = c->primes[i], p = (u64)(int64_t)delta % q;
      for (uint32_t d = 2; d < sf_degree; d++) p = mulmod(p, (u64)(int64_t)delta % q, q);
      powp[i] = p;
    }
    CUDA_CHECK(dev_alloc(&d_pow, powp.size() * sizeof(u64), c->stream));
    CUDA_CHECK(counted_copy(d_pow, powp.data(), powp.size() * sizeof(u64),
                               cudaMemcpyHostToDevice, c->stream));
  }
  launch_encode_split(plain->_poly._data, d_msg, d_pow, q_batch(level, num_p, c->L));
  // powp lives on the host stack (a captured copy reads its own snapshot instead)
  if (d_pow && !image_capturing()) CUDA_CHECK(stream_sync(c->stream));
  CUDA_CHECK(dev_free(d_msg, c->stream));
  if (d_pow) CUDA_CHECK(dev_free(d_pow, c->stream));
  plain->_poly._is_ntt = false;
  Conv_poly2ntt_inplace(&plain->_poly);
}

}  // namespace fhert

namespace {

// ckks/src/encoder.c:473-575: one value on every coefficient of every limb
void encode_scalar(Context* c, PLAIN plain, double value, uint32_t sf_degree, uint32_t level) {
  if (level == 0) level = c->L;
  const double delta = std::pow(2.0, (double)c->sf_bits), scale = std::pow(delta, sf_degree);
  init_plain(c, plain, level, scale, sf_degree);
  std::vector<int64_t> res = encode_value(c, value, level, scale, 0);
  // fill every limb with its residue: one clear, one launch for all limbs
  POLY p = &plain->_poly;
  CUDA_CHECK(zero_async(p->_data, (size_t)level * c->N * sizeof(int64_t), c->stream));
  std::vector<u64> sc(res.begin(), res.end());
  launch_scalars(false, ptr2(p->_data), ptr2(p->_data), sc.data(), q_batch(level));
  p->_is_ntt = true;
}

}  // namespace

extern "C" {

void Fhert_seed(const uint32_t seed[16], uint64_t counter, int64_t fake_time_us) {
  seed_prng(seed, counter, fake_time_us);
}

// ckks/src/cipher.c:172-186: would msg still fit the modulus at the
// ciphertext's level and scale
bool Within_value_range(CIPHER ciph, double* msg, uint32_t len) {
  Context* c     = ctx();
  uint32_t slots = ciph->_slots;
  FHERT_ASSERT(len <= slots, "length of msg should less than slots");
  ensure_fft_tables(c);
  std::vector<cplx> v(slots, cplx(0, 0));
  for (uint32_t i = 0; i < len; i++) v[i] = cplx(msg[i], 0.0);
  embedding_inv(c, v);
  double top = 0.0;
  for (auto& x : v) {
    top = std::max(top, std::fabs(x.real() * ciph->_scaling_factor));
    top = std::max(top, std::fabs(x.imag() * ciph->_scaling_factor));
  }
  int32_t bits  = (int32_t)std::log2(std::max(top, 2.2250738585072014e-308)) + 1;
  int32_t valid = (int32_t)c->q0_bits + ((int32_t)ciph->_c0_poly._num_primes - 1) * (int32_t)c->sf_bits;
  return bits < valid;
}

void Free_plain_data(PLAIN plain) { Free_poly_data(&plain->_poly); }

void Encode_double(PLAIN plain, double* input, size_t len, uint32_t sc_degree, uint32_t level) {
  Context* c = ctx();
  if (len == 1) {
    encode_scalar(c, plain, *input, sc_degree, level);
    return;
  }
  std::vector<cplx> v(len);
  for (size_t i = 0; i < len; i++) v[i] = cplx(input[i], 0.0);
  encode_vector(c, plain, v, sc_degree, level);
}

void Encode_float(PLAIN plain, float* input, size_t len, uint32_t sc_degree, uint32_t level) {
  Context* c = ctx();
  if (len == 1) {
    encode_scalar(c, plain, (double)*input, sc_degree, level);
    return;
  }
  std::vector<cplx> none;  // the floats are widened to complex doubles on the device
  encode_vector(c, plain, none, sc_degree, level, 0, 0, input, len);
}

void Encode_dcmplx(PLAIN plain, double* re_im, size_t len, uint32_t sc_degree, uint32_t level) {
  std::vector<cplx> v(len);
  for (size_t i = 0; i < len; i++) v[i] = cplx(re_im[2 * i], re_im[2 * i + 1]);
  encode_vector(ctx(), plain, v, sc_degree, level);
}

void Encode_double_mask(PLAIN plain, double cst, size_t len, uint32_t sc_degree, uint32_t level) {
  std::vector<double> m(len, cst);
  Encode_double(plain, m.data(), len, sc_degree, level);
}

void Encode_float_mask(PLAIN plain, float cst, size_t len, uint32_t sc_degree, uint32_t level) {
  std::vector<float> m(len, cst);
  Encode_float(plain, m.data(), len, sc_degree, level);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// encrypt / decrypt / decode
// ---------------------------------------------------------------------------

namespace {

// triangle sample vector as an RNS polynomial (coefficient form) at `level`
void error_poly(Context* c, POLY e, size_t level) {
  std::vector<int64_t> tri(c->N);
  sample_triangle(tri.data(), c->N);
  int64_t* d = nullptr;
  CUDA_CHECK(dev_alloc(&d, c->N * sizeof(int64_t), c->stream));
  CUDA_CHECK(counted_copy(d, tri.data(), c->N * sizeof(int64_t), cudaMemcpyHostToDevice,
                             c->stream));
  Alloc_poly_data(e, c->N, level, 0);
  launch_small_to_rns(e->_data, d, q_batch(level));
  CUDA_CHECK(stream_sync(c->stream));
  CUDA_CHECK(dev_free(d, c->stream));
  e->_is_ntt = false;
}

// little-endian multiword helpers for the CRT reconstruction of Decode
typedef std::vector<u64> Big;

void big_mul_add(Big& acc, const Big& a, u64 m) {  // acc += a * m
  u64 carry = 0;
  for (size_t i = 0; i < acc.size(); i++) {
    u128 t = (u128)(i < a.size() ? a[i] : 0) * m + acc[i] + carry;
    acc[i] = (u64)t;
    carry  = (u64)(t >> 64);
  }
}

int big_cmp(const Big& a, const Big& b) {
  for (size_t i = a.size(); i-- > 0;) {
    u64 x = a[i], y = i < b.size() ? b[i] : 0;
    if (x != y) return x > y ? 1 : -1;
  }
  return 0;
}

void big_sub(Big& a, const Big& b) {  // a -= b, a >= b
  u64 borrow = 0;
  for (size_t i = 0; i < a.size(); i++) {
    u64  y = i < b.size() ? b[i] : 0;
    u128 t = (u128)a[i] - y - borrow;
    a[i]   = (u64)t;
    borrow = (u64)(t >> 64) & 1;
  }
}

// magnitude -> double, truncating toward zero (the conversion the CPU runtime
// gets from its big-integer library, encoder.c:681)
double big_to_double(const Big& a) {
  int top = (int)a.size() - 1;
  while (top >= 0 && a[top] == 0) top--;
  if (top < 0) return 0.0;
  int  bits = top * 64 + (64 - __builtin_clzll(a[top]));
  if (bits <= 53) return (double)a[0];
  int  shift = bits - 53;  // keep the top 53 bits
  int  w = shift / 64, b = shift % 64;
  u64  lo = a[w] >> b;
  if (b && w + 1 <= top) lo |= a[w + 1] << (64 - b);
  lo &= (1ull << 53) - 1;
  return std::ldexp((double)lo, shift);
}

}  // namespace

extern "C" {

// ckks/src/encryptor.c:19-89
CIPHER Encrypt(CIPHER res, PLAIN plain) {
  Context* c = ctx();
  FHERT_ASSERT(c->pk._p0._data != nullptr, "Encrypt: no public key (keys were not generated)");
  POLY   m     = &plain->_poly;
  size_t level = m->_num_primes;
  FHERT_ASSERT(m->_num_primes_p == 0, "Encrypt_msg: plain should not be extended");
  for (POLYNOMIAL* p : {&res->_c0_poly, &res->_c1_poly}) {
    if (p->_data == nullptr || p->_num_alloc_primes < level) {
      Free_poly_data(p);
      Alloc_poly_data(p, c->N, level, 0);
    } else {
      p->_num_primes   = level;
      p->_num_primes_p = 0;
    }
  }
  res->_scaling_factor = plain->_scaling_factor;
  res->_sf_degree      = plain->_sf_degree;
  res->_slots          = plain->_slots;
  POLYNOMIAL u{}, e1{}, e2{};
  error_poly(c, &u, level);
  error_poly(c, &e1, level);
  error_poly(c, &e2, level);
  POLYNOMIAL pk0 = c->pk._p0, pk1 = c->pk._p1;  // views at the ciphertext's level
  pk0._num_primes = pk1._num_primes = level;
  Mul_poly(&res->_c0_poly, &pk0, &u);
  Add_poly(&res->_c0_poly, &e1, &res->_c0_poly);
  Add_poly(&res->_c0_poly, &res->_c0_poly, m);
  Mul_poly(&res->_c1_poly, &pk1, &u);
  Add_poly(&res->_c1_poly, &e2, &res->_c1_poly);
  Free_poly_data(&u);
  Free_poly_data(&e1);
  Free_poly_data(&e2);
  return res;
}

// ckks/src/decryptor.c:19-66 (two-polynomial ciphertexts)
void Fhert_decrypt(PLAIN res, CIPHER ciph) {
  Context* c     = ctx();
  size_t   level = ciph->_c0_poly._num_primes;
  FHERT_ASSERT(c->sk_ntt._data != nullptr, "Decrypt: no secret key");
  FHERT_ASSERT(ciph->_c0_poly._num_primes_p == 0, "Decrypt: ciph should not be extended");
  init_plain(c, res, level, ciph->_scaling_factor, ciph->_sf_degree);
  res->_slots    = ciph->_slots;
  POLYNOMIAL sk  = c->sk_ntt, c1 = ciph->_c1_poly, c0 = ciph->_c0_poly;
  sk._num_primes = c1._num_primes = c0._num_primes = level;
  sk._num_primes_p = 0;
  Mul_poly(&res->_poly, &c1, &sk);
  Add_poly(&res->_poly, &c0, &res->_poly);
}

// ckks/src/encoder.c:657-704: out receives `count` complex values as
// (re, im) pairs; the plaintext is left in coefficient form
void Fhert_decode(PLAIN plain, double* out, size_t count) {
  Context* c = ctx();
  ensure_fft_tables(c);
  POLY           poly  = &plain->_poly;
  const uint32_t n     = c->N, half = n / 2;
  const size_t   level = poly->_num_primes;
  const uint32_t slots = plain->_slots ? plain->_slots : half;
  const uint32_t gap   = half / slots;
  FHERT_ASSERT(count <= slots, "res size larger than decode size");
  if (poly->_is_ntt) Conv_ntt2poly_inplace(poly);
  std::vector<int64_t> host(level * n);
  Fhert_download(poly, 0, level, host.data());
  // Q = prod q_i, Qhat_i = Q / q_i, and (Qhat_i^-1 mod q_i)
  size_t words = level + 1;
  Big    big_q(words, 0);
  big_q[0] = 1;
  for (size_t i = 0; i < level; i++) {
    Big t(words, 0);
    big_mul_add(t, big_q, c->primes[i]);
    big_q = t;
  }
  std::vector<Big> hat(level, Big(words, 0));
  std::vector<u64> hat_inv(level);
  for (size_t i = 0; i < level; i++) {
    hat[i][0] = 1;
    u64 qi = c->primes[i], h = 1;
    for (size_t k = 0; k < level; k++) {
      if (k == i) continue;
      Big t(words, 0);
      big_mul_add(t, hat[i], c->primes[k]);
      hat[i] = t;
      h      = mulmod(h, c->primes[k] % qi, qi);
    }
    hat_inv[i] = invmod(h, qi);
  }
  Big half_q = big_q;  // floor(Q / 2)
  for (size_t i = 0; i < words; i++)
    half_q[i] = (half_q[i] >> 1) | (i + 1 < words ? half_q[i + 1] << 63 : 0);
  auto coeff_to_double = [&](uint32_t idx) {
    Big acc(words + 1, 0);
    for (size_t i = 0; i < level; i++) {
      u64 y = mulmod((u64)host[i * n + idx], hat_inv[i], c->primes[i]);
      big_mul_add(acc, hat[i], y);
    }
    while (big_cmp(acc, big_q) >= 0) big_sub(acc, big_q);
    if (big_cmp(acc, half_q) > 0) {
      Big neg = big_q;
      neg.resize(words + 1, 0);
      big_sub(neg, acc);
      return -big_to_double(neg);
    }
    return big_to_double(acc);
  };
  std::vector<cplx> msg(slots);
  double            factor = plain->_scaling_factor;
  for (uint32_t i = 0; i < slots; i++) {
    double re = coeff_to_double(i * gap) / factor;
    double im = coeff_to_double(i * gap + half) / factor;
    msg[i]    = cplx(re, im);
  }
  embedding(c, msg);
  for (size_t i = 0; i < count; i++) {
    out[2 * i]     = msg[i].real();
    out[2 * i + 1] = msg[i].imag();
  }
}

// cipher.c Get_msg: decrypt and decode, real parts; the caller frees the result
double* Get_msg(CIPHER ciph) {
  PLAINTEXT plain;
  std::memset(&plain, 0, sizeof(plain));
  Fhert_decrypt(&plain, ciph);
  size_t              slots = plain._slots;
  std::vector<double> tmp(2 * slots);
  Fhert_decode(&plain, tmp.data(), slots);
  Free_poly_data(&plain._poly);
  double* out = (double*)std::malloc(slots * sizeof(double));
  for (size_t i = 0; i < slots; i++) out[i] = tmp[2 * i];
  return out;
}

// key material for inspection and parity checks: L Q limbs then K P limbs
void Fhert_export_switch_key(bool is_rot, int32_t rot_idx, uint32_t part, int which,
                             int64_t* host) {
  SW_KEY k = Swk(is_rot, rot_idx);
  POLY   p = which == 0 ? Pk0_at(k, part) : Pk1_at(k, part);
  Fhert_download(p, 0, p->_num_alloc_primes, host);
}

// which: 0 = secret key (coefficient form, L+K limbs), 1 = secret key in NTT
// form, 2 / 3 = public key polynomials (L limbs)
void Fhert_export_key(int which, int64_t* host) {
  Context* c = ctx();
  POLY     p = which == 0 ? &c->sk_s : which == 1 ? &c->sk_ntt : which == 2 ? &c->pk._p0 : &c->pk._p1;
  FHERT_ASSERT(p->_data != nullptr, "keys were not generated");
  Fhert_download(p, 0, p->_num_alloc_primes, host);
}

}  // extern "C"
