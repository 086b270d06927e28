// Key generation, encoding, encryption, decryption and decoding.
//
// Sampling and the floating-point embedding run on the host exactly as in the
// CPU runtime (same generators, same order of draws, same libm and the same
// order of floating-point operations), all polynomial arithmetic runs on the
// device through the same entry points a compiled program uses.  Citations name
// files inside fhe-cmplr/rtlib/ant/.
#include <algorithm>
#include <cmath>
#include <complex>
#include <cstring>
#include <vector>

#include "runtime.h"

namespace fhert {

namespace {

constexpr int kThreads = 256;

// include/util/modular.h:278-280
constexpr int64_t kMax64 = (int64_t)(((u64)1 << 63) - ((u64)1 << 9)) - 1;

__global__ void __launch_bounds__(kThreads)
encode_split_kernel(u64* __restrict__ poly, const int64_t* __restrict__ msg,
                    const u64* __restrict__ scale_pow, LimbBatch batch,
                    const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const int64_t    q  = (int64_t)m.q;
  const u64        sp = scale_pow ? scale_pow[lr.prime] : 1;
  u64*             pr = poly + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    int64_t v = msg[i];
    // values above half of the 64-bit bound stand for negatives (crt.c:1161-1184)
    if (v > (kMax64 >> 1)) v -= kMax64;
    int64_t r = v % q;
    if (r < 0) r += q;
    u64 out = (u64)r;
    if (scale_pow) out = mul_mod(out, sp, m);
    pr[i] = out;
  }
}

__global__ void __launch_bounds__(kThreads)
small_to_rns_kernel(u64* __restrict__ poly, const int64_t* __restrict__ vals, LimbBatch batch,
                    const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64     q  = mods[lr.prime].q;
  u64*          pr = poly + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    int64_t v = vals[i];
    pr[i]     = v < 0 ? (u64)(v + (int64_t)q) : (u64)v;
  }
}

inline dim3 grid_for(uint32_t n, int limbs) {
  return dim3((n + kThreads * 2 - 1) / (kThreads * 2), limbs);
}

}  // namespace

void launch_encode_split(int64_t* poly, const int64_t* msg, const u64* scale_pow,
                         const LimbBatch& batch) {
  Context* c = ctx();
  encode_split_kernel<<<grid_for(c->N, batch.count), kThreads, 0, c->stream>>>(
      (u64*)poly, msg, scale_pow, batch, c->d_mod, c->N);
  c->launches++;
  CUDA_CHECK(cudaGetLastError());
}

void launch_small_to_rns(int64_t* poly, const int64_t* vals, const LimbBatch& batch) {
  Context* c = ctx();
  small_to_rns_kernel<<<grid_for(c->N, batch.count), kThreads, 0, c->stream>>>(
      (u64*)poly, vals, batch, c->d_mod, c->N);
  c->launches++;
  CUDA_CHECK(cudaGetLastError());
}

// ---- key storage --------------------------------------------------------------

SWITCH_KEY* key_slot(Context* c, uint32_t key_id, bool create) {
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

namespace {

// all limbs of a polynomial with level Q limbs and num_p special limbs laid
// out back to back (allocation = level + num_p)
LimbBatch dense_batch(Context* c, size_t level, size_t num_p) {
  LimbBatch b;
  b.count = 0;
  for (size_t i = 0; i < level; i++)
    b.limb[b.count++] = LimbRef{(uint16_t)i, (uint16_t)i, (uint16_t)i, (uint8_t)i, 0};
  for (size_t k = 0; k < num_p; k++) {
    uint16_t off = (uint16_t)(level + k);
    b.limb[b.count++] = LimbRef{off, off, off, (uint8_t)(c->L + k), 0};
  }
  return b;
}

// device copy of a host sample vector, freed in stream order by the caller
int64_t* upload_samples(Context* c, const std::vector<int64_t>& v) {
  int64_t* d = nullptr;
  CUDA_CHECK(dev_alloc(&d, v.size() * sizeof(int64_t), c->stream));
  CUDA_CHECK(counted_copy(d, v.data(), v.size() * sizeof(int64_t), cudaMemcpyHostToDevice,
                             c->stream));
  // the host vector may go out of scope before the copy is consumed
  CUDA_CHECK(stream_sync(c->stream));
  return d;
}

// Triangle error as an RNS polynomial in coefficient form
// (Sample_triangle + Transform_value_to_rns_poly(.., true))
void sample_error_poly(Context* c, POLY e) {
  std::vector<int64_t> tri(c->N);
  sample_triangle(tri.data(), c->N);
  int64_t* d = upload_samples(c, tri);
  launch_small_to_rns(e->_data, d, dense_batch(c, e->_num_primes, e->_num_primes_p));
  CUDA_CHECK(dev_free(d, c->stream));
  e->_is_ntt = false;
}

// Uniform polynomial: Q limbs then P limbs, one generator stream
// (poly/src/rns_poly.c:1149-1170)
void sample_uniform_poly(Context* c, POLY a) {
  size_t               limbs = a->_num_primes + a->_num_primes_p;
  std::vector<int64_t> host(limbs * c->N);
  for (size_t i = 0; i < a->_num_primes; i++)
    sample_uniform(host.data() + i * c->N, c->N, c->primes[i]);
  for (size_t k = 0; k < a->_num_primes_p; k++)
    sample_uniform(host.data() + (a->_num_primes + k) * c->N, c->N, c->primes[c->L + k]);
  CUDA_CHECK(counted_copy(a->_data, host.data(), host.size() * sizeof(int64_t),
                             cudaMemcpyHostToDevice, c->stream));
  CUDA_CHECK(stream_sync(c->stream));
}

// ckks/src/key_gen.c:127-200.  new_key may be in coefficient or NTT form and
// may lack special limbs; old_key is in NTT form over Q u P.
void generate_switching_key(Context* c, SWITCH_KEY* res, POLY new_key, POLY old_key) {
  const uint32_t n = c->N;
  POLYNOMIAL     e{}, pmuls{};
  Alloc_poly_data(&e, n, c->L, c->K);
  for (int part = 0; part < c->dnum; part++) {
    e._is_ntt = false;
    POLY b = &res->_parts[part]._p0, a = &res->_parts[part]._p1;
    sample_uniform_poly(c, a);
    a->_is_ntt = true;
    Mul_poly(b, a, old_key);
    // P * new_key on the limbs of this digit, zero elsewhere (rns_poly.c:823-850)
    Alloc_poly_data(&pmuls, n, c->L, c->K);
    int       start = c->alpha * part, end = std::min(start + c->alpha, c->L);
    LimbBatch digit;
    digit.count = 0;
    for (int i = start; i < end; i++)
      digit.limb[digit.count++] = LimbRef{(uint16_t)i, 0, (uint16_t)i, (uint8_t)i, 0};
    launch_mul_const(ptr2(pmuls._data), ptr2(new_key->_data), c->d_p_mod_q, digit);
    pmuls._is_ntt = new_key->_is_ntt;
    sample_error_poly(c, &e);
    Add_poly(&e, &e, &pmuls);
    Sub_poly(b, &e, b);
    Free_poly_data(&pmuls);
  }
  Free_poly_data(&e);
}

uint32_t inverse_mod_2n(uint32_t v, uint32_t n) {
  // number_theory.c:57-80 with modulus 2N
  int64_t m = 2ll * n, a = v % m, y = 0, x = 1, mod = m;
  while (a > 1) {
    int64_t t = mod, q = a / t;
    mod = a % t;
    a   = t;
    t   = y;
    y   = x - q * y;
    x   = t;
  }
  if (x < 0) x += m;
  return (uint32_t)x;
}

}  // namespace

// key_gen.c:235-262 with is_fast: the key switches from the rotated secret key
// to the secret key, so that the automorphism can be applied after the switch
void generate_rotation_key(Context* c, uint32_t auto_idx, bool conjugate) {
  SWITCH_KEY* key = key_slot(c, auto_idx, true);
  uint32_t    gen = conjugate ? auto_idx : inverse_mod_2n(auto_idx, c->N);
  POLYNOMIAL  rotated{};
  Alloc_poly_data(&rotated, c->N, c->L, c->K);
  Automorphism_transform(&rotated, &c->sk_ntt, reinterpret_cast<int64_t*>(auto_table(c, gen)));
  generate_switching_key(c, key, &c->sk_s, &rotated);
  Free_poly_data(&rotated);
}

// key_gen.c:15-38, 72-125, 204-214, 291-353
void generate_keys(Context* c) {
  const uint32_t n = c->N;
  const int      L = c->L, K = c->K;
  // secret key: one ternary vector, lifted to every Q prime; the special limbs
  // are derived from the q_0 residue (rns_poly.c:1172-1210)
  std::vector<int64_t> tern(n), host((size_t)(L + K) * n);
  sample_ternary(tern.data(), n, c->hamming_weight);
  for (int i = 0; i < L; i++)
    for (uint32_t k = 0; k < n; k++)
      host[(size_t)i * n + k] = tern[k] < 0 ? tern[k] + (int64_t)c->primes[i] : tern[k];
  const u64 q0 = c->primes[0];
  for (int j = 0; j < K; j++) {
    u64 p = c->primes[L + j];
    for (uint32_t k = 0; k < n; k++) {
      u64 v = (u64)host[k], r = v % p;
      if (v > (q0 >> 1)) {
        u64 d = q0 % p;
        r     = r >= d ? r - d : r + p - d;
      }
      host[(size_t)(L + j) * n + k] = (int64_t)r;
    }
  }
  Alloc_poly_data(&c->sk_s, n, L, K);
  Alloc_poly_data(&c->sk_ntt, n, L, K);
  CUDA_CHECK(counted_copy(c->sk_s._data, host.data(), host.size() * sizeof(int64_t),
                             cudaMemcpyHostToDevice, c->stream));
  CUDA_CHECK(stream_sync(c->stream));
  Copy_poly(&c->sk_ntt, &c->sk_s);
  c->sk_ntt._is_ntt = false;
  Conv_poly2ntt_inplace(&c->sk_ntt);

  // public key: pk1 uniform, pk0 = -pk1*s + e
  POLYNOMIAL err{};
  Alloc_poly_data(&err, n, L, 0);
  sample_error_poly(c, &err);
  Alloc_poly_data(&c->pk._p0, n, L, 0);
  Alloc_poly_data(&c->pk._p1, n, L, 0);
  sample_uniform_poly(c, &c->pk._p1);
  c->pk._p1._is_ntt = true;
  Mul_poly(&c->pk._p0, &c->pk._p1, &c->sk_ntt);
  launch_elementwise(EW_MUL_SCALAR, ptr2(c->pk._p0._data), ptr2(c->pk._p0._data),
                     ptr2(c->pk._p0._data), -1, dense_batch(c, L, 0));
  Add_poly(&c->pk._p0, &c->pk._p0, &err);
  Free_poly_data(&err);

  // relinearisation key: switches s^2 to s
  POLYNOMIAL s2{};
  Alloc_poly_data(&s2, n, L, 0);
  Mul_poly(&s2, &c->sk_ntt, &c->sk_ntt);
  generate_switching_key(c, key_slot(c, 0, true), &s2, &c->sk_ntt);
  Free_poly_data(&s2);

  // one rotation key per new automorphism index, in the order of the
  // program's rotation list
  CKKS_PARAMS* p = Get_context_params();
  for (size_t i = 0; i < p->_num_rot_idx; i++) {
    uint32_t k = auto_index_for(c, p->_rot_idxs[i]);
    if (c->keys.count(k)) continue;
    generate_rotation_key(c, k, false);
  }
  CUDA_CHECK(stream_sync(c->stream));
}

// bootstrap.c:1199-1231: keys for the rotations of the linear transforms, in
// ascending order of rotation, then the conjugation key
void generate_bootstrap_keys(Context* c, const std::vector<int32_t>& rotations) {
  FHERT_ASSERT(c->sk_s._data != nullptr, "bootstrap keys need the secret key of this context");
  for (int32_t r : rotations) {
    uint32_t k = auto_index_for(c, r);
    if (c->keys.count(k)) continue;
    generate_rotation_key(c, k, false);
  }
  uint32_t conj = 2 * c->N - 1;
  if (!c->keys.count(conj)) generate_rotation_key(c, conj, true);
  CUDA_CHECK(stream_sync(c->stream));
}

void free_keys(Context* c) {
  for (POLYNOMIAL* p : {&c->sk_s, &c->sk_ntt, &c->pk._p0, &c->pk._p1})
    if (p->_data) Free_poly_data(p);
}

}  // namespace fhert
