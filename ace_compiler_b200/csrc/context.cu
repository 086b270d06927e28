// Host side of the CKKS context: prime chain, roots of unity, twiddle tables,
// rescale / ModUp / ModDown constants, automorphism tables.  Every constant is
// chosen exactly as the CPU runtime chooses it, because NTT-domain residues
// depend on the primes, on the 2N-th roots and on the (approximate) base
// conversion constants; the citations name the function being matched inside
// fhe-cmplr/rtlib/ant/.
#include <sched.h>

#include <cmath>
#include <cstdio>
#include <unordered_map>
#include <vector>
#include <cstring>

#include "runtime.h"

namespace fhert {

static Context* g_ctx = nullptr;

// The thread that drives the library issues tens of thousands of launches per
// second; it should run on the CPU cores next to its GPU.  Restricts the
// calling thread (and what it starts later) to the cores of the GPU's NUMA
// node that it is already allowed to use.  FHERT_NUMA_BIND=0 leaves the
// affinity alone; so does anything unexpected in sysfs.
static void bind_to_gpu_numa_node(int dev) {
  const char* env = std::getenv("FHERT_NUMA_BIND");
  if (env != nullptr && env[0] == '0') return;
  char bus[32] = {0};
  if (cudaDeviceGetPCIBusId(bus, sizeof(bus), dev) != cudaSuccess) return;
  for (char* p = bus; *p; p++)
    if (*p >= 'A' && *p <= 'F') *p = (char)(*p - 'A' + 'a');
  char path[160];
  std::snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/numa_node", bus);
  FILE* f = std::fopen(path, "r");
  if (f == nullptr) return;
  int node = -1;
  if (std::fscanf(f, "%d", &node) != 1) node = -1;
  std::fclose(f);
  if (node < 0) return;
  std::snprintf(path, sizeof(path), "/sys/devices/system/node/node%d/cpulist", node);
  f = std::fopen(path, "r");
  if (f == nullptr) return;
  cpu_set_t allowed, wanted;
  CPU_ZERO(&wanted);
  if (sched_getaffinity(0, sizeof(allowed), &allowed) != 0) {
    std::fclose(f);
    return;
  }
  int lo = 0, hi = 0, picked = 0;
  while (std::fscanf(f, "%d", &lo) == 1) {  // "0-31,64-95"
    hi = lo;
    int ch = std::fgetc(f);
    if (ch == '-') {
      if (std::fscanf(f, "%d", &hi) != 1) break;
      ch = std::fgetc(f);
    }
    for (int cpu = lo; cpu <= hi && cpu < CPU_SETSIZE; cpu++)
      if (CPU_ISSET(cpu, &allowed)) {
        CPU_SET(cpu, &wanted);
        picked++;
      }
    if (ch != ',') break;
  }
  std::fclose(f);
  if (picked > 0) sched_setaffinity(0, sizeof(wanted), &wanted);
}

Context* ctx() {
  FHERT_ASSERT(g_ctx != nullptr, "no context: call Prepare_context first");
  // deferred work runs first, oldest first: a waiting Mod_down / Rescale was
  // queued before any per-limb call recorded after it.  The launches of that
  // work come back through here; they must not start the younger work early.
  if ((g_ctx->pair_wait.kind || g_ctx->hw_pending) && !g_ctx->draining) {
    g_ctx->draining = true;
    if (g_ctx->pair_wait.kind) pair_flush(g_ctx);
    if (g_ctx->hw_pending) hw_replay(g_ctx);
    g_ctx->draining = false;
  }
  return g_ctx;
}
Context* ctx_noflush() {
  FHERT_ASSERT(g_ctx != nullptr, "no context: call Prepare_context first");
  return g_ctx;
}
Context* ctx_or_null() { return g_ctx; }

// ---- number theory --------------------------------------------------------

u64 mulmod(u64 a, u64 b, u64 q) { return (u64)((u128)a * b % q); }

u64 powmod(u64 a, u64 e, u64 q) {
  u64 r = 1 % q;
  a %= q;
  while (e) {
    if (e & 1) r = mulmod(r, a, q);
    a = mulmod(a, a, q);
    e >>= 1;
  }
  return r;
}

u64 invmod(u64 a, u64 q) { return powmod(a, q - 2, q); }  // q prime

// Deterministic Miller-Rabin for 64-bit integers.  The CPU runtime runs 200
// random rounds (util/src/number_theory.c:165-190); both accept exactly the
// primes.
bool is_prime(u64 n) {
  if (n < 2) return false;
  static const u64 small[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
  for (u64 p : small) {
    if (n == p) return true;
    if (n % p == 0) return false;
  }
  u64 d = n - 1;
  int r = 0;
  while ((d & 1) == 0) {
    d >>= 1;
    r++;
  }
  for (u64 a : small) {
    u64 x = powmod(a, d, n);
    if (x == 1 || x == n - 1) continue;
    bool comp = true;
    for (int i = 1; i < r; i++) {
      x = mulmod(x, x, n);
      if (x == n - 1) {
        comp = false;
        break;
      }
    }
    if (comp) return false;
  }
  return true;
}

u64 shoup(u64 w, u64 q) { return (u64)(((u128)w << 64) / q); }

// util/src/crt.c:42-67
static u64 first_prime(uint32_t n, size_t bits) {
  u64 order = 2ull * n;
  u64 p     = (1ull << bits) + order + 1;
  while (!is_prime(p)) p += order;
  return p;
}
static u64 previous_prime(u64 p, u64 order) {
  p -= order;
  while (!is_prime(p)) p -= order;
  return p;
}
static u64 next_prime(u64 p, u64 order) {
  // the reference starts from p + order and steps once more before testing
  p += order;
  do {
    p += order;
  } while (!is_prime(p));
  return p;
}

// util/src/crt.c:112-148
static std::vector<u64> generate_q_primes(size_t count, size_t q0_bits, size_t sf_bits,
                                          uint32_t n) {
  std::vector<u64> q(count);
  u64              order = 2ull * n;
  u64              first = first_prime(n, sf_bits);
  q[count - 1]           = first;
  u64 q_next = first, q_prev = first;
  if (count > 1) {
    uint32_t cnt = 0;
    for (size_t i = count - 2; i >= 1; i--) {
      if ((cnt & 1) == 0) {
        q_prev = previous_prime(q_prev, order);
        q[i]   = q_prev;
      } else {
        q_next = next_prime(q_next, order);
        q[i]   = q_next;
      }
      cnt++;
    }
  }
  if (q0_bits == sf_bits) {
    q[0] = previous_prime(q_prev, order);
  } else {
    q[0] = previous_prime(first_prime(n, q0_bits), order);
  }
  return q;
}

// bit length of a product of 64-bit factors
static size_t product_bits(const std::vector<u64>& f) {
  std::vector<u64> big(1, 1);
  for (u64 v : f) {
    u64 carry = 0;
    for (size_t i = 0; i < big.size(); i++) {
      u128 t = (u128)big[i] * v + carry;
      big[i] = (u64)t;
      carry  = (u64)(t >> 64);
    }
    if (carry) big.push_back(carry);
  }
  return (big.size() - 1) * 64 + (64 - __builtin_clzll(big.back()));
}

// util/src/number_theory.c:97-139: smallest primitive root
static u64 find_generator(u64 q) {
  u64              phi = q - 1;
  std::vector<u64> factors;
  u64              number = phi;
  for (u64 i = 2; i <= (u64)std::sqrt((double)number); i++) {
    if (number % i == 0) {
      factors.push_back(i);
      while (number % i == 0) number /= i;
    }
  }
  if (number > 1) factors.push_back(number);
  for (u64 r = 2; r <= phi; r++) {
    bool ok = true;
    for (u64 f : factors) {
      if (powmod(r, phi / f, q) == 1) {
        ok = false;
        break;
      }
    }
    if (ok) return r;
  }
  FHERT_ASSERT(false, "no generator for %llu", (unsigned long long)q);
  return 0;
}

// The CPU runtime keeps a table of 2N-th roots for the prime chains of two ring
// degrees (util/src/std_param.c:229-300, orders 32 and 32768); every entry is
// the smallest primitive root of that order, and the primes covered are the
// first few lattice primes (= 1 mod order) below and above 2^60, 2^59 and 2^50.
// This reproduces which primes the table covers.
static bool root_table_covers(u64 order, u64 q) {
  struct Span { u64 order; int bits, below, above; };
  static const Span spans[] = {{32, 60, 9, 0},     {32, 59, 10, 11},    {32, 50, 2, 3},
                               {32768, 60, 10, 0}, {32768, 59, 12, 13}};
  for (const Span& s : spans) {
    if (s.order != order) continue;
    u64 c = (1ull << s.bits) + 1;
    for (int found = 0; found < s.below;) {
      c -= order;
      if (is_prime(c)) {
        if (c == q) return true;
        found++;
      }
    }
    c = (1ull << s.bits) + 1;
    for (int found = 0; found < s.above;) {
      c += order;
      if (is_prime(c)) {
        if (c == q) return true;
        found++;
      }
    }
  }
  return false;
}

// util/src/number_theory.c:141-162: table value when the table covers the prime,
// else generator^((q-1)/order) with the smallest generator
static u64 root_of_unity(u64 order, u64 q) {
  FHERT_ASSERT((q - 1) % order == 0, "modulus-1 not divisible by order");
  u64 g    = find_generator(q);
  u64 root = powmod(g, (q - 1) / order, q);
  if (!root_table_covers(order, q)) return root;
  u64 sq = mulmod(root, root, q), cur = root, best = root;
  for (u64 k = 0; k < order / 2; k++) {  // all odd powers of root
    if (cur < best) best = cur;
    cur = mulmod(cur, sq, q);
  }
  return best;
}

static uint32_t bit_reverse(uint32_t v, int bits) {
  uint32_t r = 0;
  for (int i = 0; i < bits; i++) r |= ((v >> i) & 1u) << (bits - 1 - i);
  return r;
}

static void init_modulus(MODULUS* m, u64 q) {
  // include/util/modular.h:67-72
  m->_val  = (int64_t)q;
  m->_br_k = 2 * ((int64_t)std::log2((double)q) + 1);
  m->_br_m = (int64_t)(((u128)1 << m->_br_k) / q);
  // floor(2^128 / q) = floor((2^128 - 1) / q) for q not a power of two
  m->_prec128 = ~(u128)0 / q;
}

DevModulus make_dev_modulus(u64 q, uint32_t n) {
  DevModulus d;
  u128       mu = ~(u128)0 / q;
  d.q           = q;
  d.mu_hi       = (u64)(mu >> 64);
  d.mu_lo       = (u64)mu;
  d.bits        = 64 - __builtin_clzll(q);
  d.pad         = 0;
  d.bar         = (u64)(((u128)1 << (d.bits - 1 + 64)) / q);
  d.n_inv       = n ? invmod(n % q, q) : 0;
  d.n_inv_p     = n ? shoup(d.n_inv, q) : 0;
  return d;
}

template <typename T>
static T* upload(const std::vector<T>& v) {
  T* d = nullptr;
  if (v.empty()) return d;
  if (image_capturing()) image_capture_break("a table built on first use");
  CUDA_CHECK(cudaMalloc(&d, v.size() * sizeof(T)));
  CUDA_CHECK(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
  // a copy from pageable memory may still be in flight when cudaMemcpy returns,
  // and the library stream is not ordered against the default stream: tables
  // built on first use are read by the very next kernel
  CUDA_CHECK(cudaStreamSynchronize(0));
  return d;
}

static Twiddle tw_of(u64 w, u64 q) {
  Twiddle t;
  t.w  = w;
  t.wp = shoup(w, q);
  return t;
}

// ---- ModUp tables  (util/src/crt.c:459-566) --------------------------------

const Context::ModUpTable& modup_table(Context* c, int level, int digit) {
  auto key = std::make_pair(level, digit);
  auto it  = c->modup.find(key);
  if (it != c->modup.end()) return it->second;
  Context::ModUpTable t;
  int                 start = digit * c->alpha;
  int                 end   = std::min(start + c->alpha, level);
  FHERT_ASSERT(start < level, "digit %d empty at level %d", digit, level);
  t.digit_len = end - start;
  t.out_count = level - t.digit_len + c->K;
  int              total = c->L + c->K;
  std::vector<Twiddle> hat_inv(t.digit_len);
  std::vector<u64> hat_mod((size_t)t.digit_len * total, 0);
  for (int i = 0; i < t.digit_len; i++) {
    u64 qi  = c->primes[start + i];
    u64 hat = 1;
    for (int k = start; k < end; k++)
      if (k != start + i) hat = mulmod(hat, c->primes[k] % qi, qi);
    u64 inv            = invmod(hat, qi);
    hat_inv[i]         = tw_of(inv, qi);
    for (int m = 0; m < total; m++) {
      bool is_q = m < c->L;
      if (is_q && (m >= level || (m >= start && m < end))) continue;
      u64 pm = c->primes[m];
      u64 h  = 1;
      for (int k = start; k < end; k++)
        if (k != start + i) h = mulmod(h, c->primes[k] % pm, pm);
      hat_mod[(size_t)i * total + m] = h;
    }
  }
  t.d_hat_inv = upload(hat_inv);
  t.d_hat_mod = upload(hat_mod);
  return c->modup.emplace(key, t).first->second;
}

// ---- automorphism tables  (util/src/number_theory.c:206-230, NTT form) ------

uint32_t* auto_table(Context* c, uint32_t k) {
  auto it = c->auto_tables.find(k);
  if (it != c->auto_tables.end()) return it->second;
  uint32_t              n = c->N, logn = c->logN;
  uint64_t              m = 2ull * n;
  std::vector<uint32_t> tab(n);
  for (uint32_t j = 0; j < n; j++) {
    uint64_t jt  = 2ull * j + 1;
    uint64_t idx = ((jt * k) % m) >> 1;
    tab[bit_reverse(j, logn)] = bit_reverse((uint32_t)idx, logn);
  }
  uint32_t* d = upload(tab);
  c->auto_tables[k] = d;
  return d;
}

// util/src/number_theory.c:192-204 with modulus 2N
static uint32_t find_automorphism_index(int32_t rot_idx, uint32_t n) {
  u64 m = 2ull * n;
  if (rot_idx == 0) return 1;
  if (rot_idx == (int32_t)(m - 1)) return (uint32_t)rot_idx;
  u64 gen = 5;
  if (rot_idx < 0) {
    // inverse of 5 modulo 2N (2N is a power of two): extended Euclid
    int64_t a = 5, mod = (int64_t)m, y = 0, x = 1;
    while (a > 1) {
      int64_t t = mod, qq = a / t;
      mod = a % t;
      a   = t;
      t   = y;
      y   = x - qq * y;
      x   = t;
    }
    if (x < 0) x += (int64_t)m;
    gen = (u64)x;
  }
  u64 e = (u64)std::llabs((long long)rot_idx), r = 1, b = gen % m;
  while (e) {
    if (e & 1) r = r * b % m;
    b = b * b % m;
    e >>= 1;
  }
  return (uint32_t)r;
}

uint32_t auto_index_for(Context* c, int32_t rot_idx) {
  auto it = c->auto_idx.find(rot_idx);
  if (it != c->auto_idx.end()) return it->second;
  uint32_t k           = find_automorphism_index(rot_idx, c->N);
  c->auto_idx[rot_idx] = k;
  return k;
}

// ---- context construction ---------------------------------------------------

Context* create_context(const CKKS_PARAMS* p) {
  FHERT_ASSERT(g_ctx == nullptr, "context exists already");
  int dev_count = 0;
  cudaError_t e = cudaGetDeviceCount(&dev_count);
  FHERT_ASSERT(e == cudaSuccess && dev_count > 0,
               "no CUDA device available (%s); this runtime has no CPU path",
               cudaGetErrorString(e));
  Context* c = new Context();
  c->N       = p->_poly_degree;
  FHERT_ASSERT(c->N >= 4 && (c->N & (c->N - 1)) == 0, "ring degree must be a power of two");
  c->logN           = 31 - __builtin_clz(c->N);
  c->L              = (int)p->_mul_depth + 1;
  c->dnum           = (int)p->_num_q_parts;
  // util/src/std_param.c:356-363: digit count when the program leaves it open
  if (c->dnum == 0) c->dnum = p->_mul_depth > 3 ? 3 : (p->_mul_depth == 0 ? 1 : 2);
  c->q0_bits        = p->_first_mod_size;
  c->sf_bits        = p->_scaling_mod_size;
  c->hamming_weight = p->_hamming_weight;
  c->input_level    = p->_input_level;
  FHERT_ASSERT(c->dnum >= 1, "num_q_parts must be positive");
  c->alpha = (c->L + c->dnum - 1) / c->dnum;  // util/src/crt.c:419
  FHERT_ASSERT((size_t)c->L > (size_t)c->alpha * (c->dnum - 1), "invalid number of q parts");
  FHERT_ASSERT(c->alpha <= kMaxDigit, "digit of %d primes exceeds the supported %d",
               c->alpha, kMaxDigit);

  std::vector<u64> q = generate_q_primes(c->L, c->q0_bits, c->sf_bits, c->N);
  // K = ceil(bits(largest digit product) / 60)   (crt.c:416-457)
  size_t max_bits = 0;
  for (int j = 0; j < c->dnum; j++) {
    std::vector<u64> f;
    for (int i = j * c->alpha; i < (j + 1) * c->alpha && i < c->L; i++) f.push_back(q[i]);
    max_bits = std::max(max_bits, product_bits(f));
  }
  c->K = (int)((max_bits + 59) / 60);
  // P primes: successive previous primes below first(60), skipping Q (crt.c:71-103)
  std::vector<u64> pp;
  {
    u64 order = 2ull * c->N;
    u64 prev  = first_prime(c->N, 60);
    for (int i = 0; i < c->K; i++) {
      u64  cand;
      bool in_q;
      do {
        cand = previous_prime(prev, order);
        in_q = false;
        for (u64 v : q) in_q |= (v == cand);
        prev = cand;
      } while (in_q);
      pp.push_back(cand);
    }
  }
  c->primes = q;
  c->primes.insert(c->primes.end(), pp.begin(), pp.end());
  const int total = c->L + c->K;
  FHERT_ASSERT(total <= kMaxLimbs, "too many limbs (%d)", total);
  c->moduli.resize(total);
  c->primes_below_2_60 = std::getenv("FHERT_NO_FAST_ACC") == nullptr;
  for (int i = 0; i < total; i++) {
    // the lazy reductions keep up to 9q in a 64-bit word (modarith.cuh)
    FHERT_ASSERT(c->primes[i] < 0xFFFFFFFFFFFFFFFFull / 9, "primes must be below 2^64 / 9");
    if (c->primes[i] >= (1ull << 60)) c->primes_below_2_60 = false;
    init_modulus(&c->moduli[i], c->primes[i]);
  }

  // FHERT_SPIN=1: the driver's waits of this process busy-wait instead of sleeping
  if (const char* spin = std::getenv("FHERT_SPIN")) {
    if (spin[0] == '1' && cudaSetDeviceFlags(cudaDeviceScheduleSpin) != cudaSuccess) cudaGetLastError();
  }
  CUDA_CHECK(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  // keep freed blocks cached in the stream-ordered pool
  {
    int dev = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    bind_to_gpu_numa_node(dev);
    cudaMemPool_t pool;
    CUDA_CHECK(cudaDeviceGetDefaultMemPool(&pool, dev));
    uint64_t thresh = ~0ull;
    CUDA_CHECK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh));
  }

  // twiddles (util/src/ntt.c:91-138): rou[brv(i)] = psi^i, rou_inv[brv(i)] = psi^-i
  const uint32_t          n = c->N;
  std::vector<DevModulus> dm(total);
  std::vector<Twiddle>    fwd((size_t)total * n), inv((size_t)total * n), inv_last(total * 2);
  c->psi.resize(total);
  c->h_fwd.resize(total);
  c->h_inv.resize(total);
  for (int i = 0; i < total; i++) {
    u64 qi     = c->primes[i];
    dm[i]      = make_dev_modulus(qi, n);
    u64 psi    = root_of_unity(2ull * n, qi);
    u64 psi_iv = invmod(psi, qi);
    c->psi[i]  = psi;
    Twiddle* f = &fwd[(size_t)i * n];
    Twiddle* v = &inv[(size_t)i * n];
    u64      pw = 1, pwi = 1;
    for (uint32_t k = 0; k < n; k++) {
      uint32_t r = bit_reverse(k, c->logN);
      f[r]       = tw_of(pw, qi);
      v[r]       = tw_of(pwi, qi);
      pw         = mulmod(pw, psi, qi);
      pwi        = mulmod(pwi, psi_iv, qi);
    }
    inv_last[2 * i]     = tw_of(dm[i].n_inv, qi);
    inv_last[2 * i + 1] = tw_of(mulmod(v[1].w, dm[i].n_inv, qi), qi);
    c->h_fwd[i].assign(f, f + n);
    c->h_inv[i].assign(v, v + n);
  }
  c->d_mod      = upload(dm);
  c->d_fwd      = upload(fwd);
  c->d_inv      = upload(inv);
  c->d_inv_last = upload(inv_last);

  // rescale constants (crt.c:291-353); row l = prime being dropped
  const int            L = c->L, K = c->K;
  std::vector<Twiddle> ql_inv((size_t)L * L), ql_neg((size_t)L * L);
  std::vector<u64>     ql_mod((size_t)L * L, 0);
  for (int l = 1; l < L; l++) {
    for (int i = 0; i < l; i++) {
      u64 qi = q[i], ql = q[l];
      u64 iv                    = invmod(ql % qi, qi);
      ql_inv[(size_t)l * L + i] = tw_of(iv, qi);
      // floor(Qhat_l * (Qhat_l^-1 mod q_l) / q_l) mod q_i  ==  -q_l^-1 mod q_i
      // because Qhat_l * (Qhat_l^-1 mod q_l) = 1 + c*q_l and Qhat_l = 0 mod q_i
      ql_neg[(size_t)l * L + i] = tw_of(iv == 0 ? 0 : qi - iv, qi);
      ql_mod[(size_t)l * L + i] = ql % qi;
    }
  }
  c->d_ql_inv = upload(ql_inv);
  c->d_ql_neg = upload(ql_neg);
  c->d_ql_mod = upload(ql_mod);

  // ModDown / Extend constants (crt.c:357-414)
  std::vector<Twiddle> phat_inv(K), p_inv(L), p_mod_q(L);
  std::vector<u64>     phat_mod_q((size_t)L * K);
  for (int k = 0; k < K; k++) {
    u64 pk = pp[k], hat = 1;
    for (int j = 0; j < K; j++)
      if (j != k) hat = mulmod(hat, pp[j] % pk, pk);
    phat_inv[k] = tw_of(invmod(hat, pk), pk);
  }
  for (int i = 0; i < L; i++) {
    u64 qi = q[i], P = 1;
    for (int k = 0; k < K; k++) P = mulmod(P, pp[k] % qi, qi);
    p_mod_q[i] = tw_of(P, qi);
    p_inv[i]   = tw_of(invmod(P, qi), qi);
    for (int k = 0; k < K; k++) {
      u64 hat = 1;
      for (int j = 0; j < K; j++)
        if (j != k) hat = mulmod(hat, pp[j] % qi, qi);
      phat_mod_q[(size_t)i * K + k] = hat;
    }
  }
  c->d_phat_inv   = upload(phat_inv);
  c->d_phat_mod_q = upload(phat_mod_q);
  c->d_p_inv      = upload(p_inv);
  c->d_p_mod_q    = upload(p_mod_q);

  g_ctx = c;
  return c;
}

void destroy_context() {
  Context* c = g_ctx;
  if (!c) return;
  image_replay_release();  // its blocks join the common lists, released below
  hw_release(c);
  free_encode_tables(c);
  free_bootstrap(c);
  free_keys(c);
  release_prng();
  if (c->scratch) dev_free(c->scratch, c->stream);
  c->scratch = nullptr;
  for (int64_t*& r : c->ring) {
    if (r) dev_free(r, c->stream);
    r = nullptr;
  }
  dev_release_all(c->stream);
  cudaStreamSynchronize(c->stream);
  cudaFree(c->d_mod);
  cudaFree(c->d_fwd);
  cudaFree(c->d_inv);
  cudaFree(c->d_inv_last);
  cudaFree(c->d_ql_inv);
  cudaFree(c->d_ql_neg);
  cudaFree(c->d_ql_mod);
  cudaFree(c->d_phat_inv);
  cudaFree(c->d_phat_mod_q);
  cudaFree(c->d_p_inv);
  cudaFree(c->d_p_mod_q);
  for (auto& kv : c->modup) {
    cudaFree(kv.second.d_hat_inv);
    cudaFree(kv.second.d_hat_mod);
  }
  for (auto& kv : c->auto_tables) cudaFree(kv.second);
  for (auto& kv : c->keys) {
    SWITCH_KEY* k = kv.second;
    for (size_t j = 0; j < k->_num_parts; j++) {
      cudaFree(k->_parts[j]._p0._data);
      cudaFree(k->_parts[j]._p1._data);
    }
    delete[] k->_parts;
    delete k;
  }
  if (c->scratch) cudaFree(c->scratch);
  cudaStreamDestroy(c->stream);
  delete c;
  g_ctx = nullptr;
}

// ---- per-kernel timing ------------------------------------------------------

const char* const kKernelNames[KID_COUNT] = {
    "ntt_strided", "ntt_contig", "ntt_small", "intt_strided", "intt_contig", "intt_small",
    "elementwise", "automorphism", "mul_const", "rescale_lift", "rescale_combine",
    "base_conv", "moddown_combine", "inner_product", "mod_raise", "tensor", "hw_batch", "encode"};

struct ProfState {
  bool                                    on = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pool;
  std::vector<int>                        ids;
  std::vector<int>                        limbs;
  size_t                                  used = 0;
};
static ProfState g_prof;

void prof_before(KernelId id) {
  if (!g_prof.on) return;
  if (g_prof.used == g_prof.pool.size()) {
    cudaEvent_t a, b;
    CUDA_CHECK(cudaEventCreate(&a));
    CUDA_CHECK(cudaEventCreate(&b));
    g_prof.pool.emplace_back(a, b);
  }
  g_prof.ids.push_back((int)id);
  CUDA_CHECK(cudaEventRecord(g_prof.pool[g_prof.used].first, ctx()->stream));
}

void prof_after(KernelId, int limbs) {
  if (!g_prof.on) return;
  g_prof.limbs.push_back(limbs);
  CUDA_CHECK(cudaEventRecord(g_prof.pool[g_prof.used].second, ctx()->stream));
  g_prof.used++;
}

bool prof_running() { return g_prof.on; }

void prof_begin() {
  g_prof.on   = true;
  g_prof.used = 0;
  g_prof.ids.clear();
  g_prof.limbs.clear();
}

// writes "name launches limbs total_ms" lines into buf; returns bytes written
size_t prof_end(char* buf, size_t cap) {
  CUDA_CHECK(stream_sync(ctx()->stream));
  g_prof.on = false;
  double ms[KID_COUNT]  = {0};
  long   cnt[KID_COUNT] = {0};
  long   lim[KID_COUNT] = {0};
  for (size_t i = 0; i < g_prof.used; i++) {
    float t = 0;
    CUDA_CHECK(cudaEventElapsedTime(&t, g_prof.pool[i].first, g_prof.pool[i].second));
    ms[g_prof.ids[i]] += t;
    cnt[g_prof.ids[i]]++;
    lim[g_prof.ids[i]] += g_prof.limbs[i];
  }
  size_t off = 0;
  for (int k = 0; k < KID_COUNT; k++) {
    if (!cnt[k]) continue;
    int w = std::snprintf(buf + off, cap > off ? cap - off : 0, "%s %ld %ld %.6f\n",
                          kKernelNames[k], cnt[k], lim[k], ms[k]);
    if (w < 0 || off + (size_t)w >= cap) break;
    off += (size_t)w;
  }
  return off;
}

// ---- device memory kept in per-size lists -----------------------------------
namespace {
struct DevPool {
  std::unordered_map<size_t, std::vector<void*>> free_by_size;
  std::unordered_map<void*, size_t>              size_of;
  size_t                                         held = 0;  // bytes waiting in the lists
};
DevPool g_pool;     // everybody's blocks
DevPool g_private;  // blocks of a captured program run
bool    g_private_mode = false;
int     g_pool_enabled = -1;
size_t  g_pool_cap     = (size_t)32 << 30;
bool pool_enabled() {
  if (g_pool_enabled < 0) {
    const char* e  = std::getenv("FHERT_POOL");
    g_pool_enabled = !(e != nullptr && e[0] == '0');
    if (const char* mb = std::getenv("FHERT_POOL_MB"))
      g_pool_cap = (size_t)std::strtoull(mb, nullptr, 10) << 20;
  }
  return g_pool_enabled != 0;
}
bool take_from(DevPool& pool, size_t bytes, void** ptr) {
  auto it = pool.free_by_size.find(bytes);
  if (it == pool.free_by_size.end() || it->second.empty()) return false;
  *ptr = it->second.back();
  it->second.pop_back();
  pool.held -= bytes;
  return true;
}
}  // namespace

cudaError_t dev_alloc(void** ptr, size_t bytes, cudaStream_t stream) {
  if (!pool_enabled()) return cudaMallocAsync(ptr, bytes, stream);
  if (bytes == 0) bytes = 256;
  bytes = (bytes + 255) & ~(size_t)255;
  if (g_private_mode) {
    // the block freed longest ago: whoever gets it waits for its former user
    // (the dependences of a captured run go by address), so the longer ago the
    // better; and during a capture only when a few younger ones are waiting behind
    // it: a size class with a single block would chain every user of that size to
    // the one before (FHERT_REPLAY_DEPTH, default 8; ResNet-20: 1010 / 945 / 920 ms
    // per image with 0 / 3 / 8)
    static const size_t depth = [] {
      const char* e = std::getenv("FHERT_REPLAY_DEPTH");
      return e != nullptr ? (size_t)std::strtoul(e, nullptr, 10) : (size_t)8;
    }();
    auto it       = g_private.free_by_size.find(bytes);
    size_t  have  = it != g_private.free_by_size.end() ? it->second.size() : 0;
    cudaError_t err = cudaErrorMemoryAllocation;
    if (have <= (image_capturing() ? depth : 0)) {
      err = cudaMalloc(ptr, bytes);
      if (err == cudaSuccess) {
        g_private.size_of[*ptr] = bytes;
        return err;
      }
      cudaGetLastError();  // out of memory: fall back to the oldest free block, if any
    }
    if (have > 0) {
      *ptr = it->second.front();
      it->second.erase(it->second.begin());
      g_private.held -= bytes;
      return cudaSuccess;
    }
    if (!image_capturing()) return err;
    // no room for the captured run's own blocks: what was captured so far is
    // launched, the rest of the run is launched directly from the common lists
    image_capture_break("out of device memory for the blocks of the captured run");
  }
  if (take_from(g_pool, bytes, ptr)) return cudaSuccess;
  cudaError_t err = cudaMallocAsync(ptr, bytes, stream);
  if (err == cudaErrorMemoryAllocation) {  // make room with what the lists hold
    cudaGetLastError();
    dev_release_all(stream);
    cudaStreamSynchronize(stream);
    err = cudaMallocAsync(ptr, bytes, stream);
  }
  if (err == cudaSuccess) g_pool.size_of[*ptr] = bytes;
  return err;
}

cudaError_t dev_free(void* ptr, cudaStream_t stream) {
  if (ptr == nullptr) return cudaSuccess;
  auto mine = g_private.size_of.find(ptr);
  if (mine != g_private.size_of.end()) {  // never trimmed: a replay may still use it
    g_private.free_by_size[mine->second].push_back(ptr);
    g_private.held += mine->second;
    return cudaSuccess;
  }
  auto it = g_pool.size_of.find(ptr);
  if (it == g_pool.size_of.end()) return cudaFreeAsync(ptr, stream);  // not from the lists
  if (g_private_mode && image_capturing()) {
    // the captured kernels used this block: from now on only a replay may
    g_private.size_of[ptr] = it->second;
    g_private.free_by_size[it->second].push_back(ptr);
    g_private.held += it->second;
    g_pool.size_of.erase(it);
    return cudaSuccess;
  }
  g_pool.free_by_size[it->second].push_back(ptr);
  g_pool.held += it->second;
  // sizes no longer in use pile up; not while a capture runs (a free would become a node)
  if (g_pool.held > g_pool_cap && !image_capturing()) dev_release_all(stream);
  return cudaSuccess;
}

void dev_release_all(cudaStream_t stream) {
  for (auto& kv : g_pool.free_by_size)
    for (void* p : kv.second) {
      g_pool.size_of.erase(p);
      cudaFreeAsync(p, stream);
    }
  g_pool.free_by_size.clear();
  g_pool.held = 0;
}

void dev_private_mode(bool on) { g_private_mode = on && pool_enabled(); }

bool dev_take_private(void* ptr) {
  auto mine = g_private.size_of.find(ptr);
  if (mine == g_private.size_of.end()) return false;
  auto& list = g_private.free_by_size[mine->second];
  for (size_t i = list.size(); i-- > 0;)
    if (list[i] == ptr) {
      list.erase(list.begin() + (long)i);
      g_private.held -= mine->second;
      return true;
    }
  return false;
}

void dev_private_to_common(cudaStream_t stream) {
  // cudaFreeAsync accepts blocks that came from cudaMalloc, so the common
  // lists may hold them and give them back to the driver like their own
  for (auto& kv : g_private.size_of) g_pool.size_of[kv.first] = kv.second;
  for (auto& kv : g_private.free_by_size) {
    auto& list = g_pool.free_by_size[kv.first];
    list.insert(list.end(), kv.second.begin(), kv.second.end());
  }
  g_pool.held += g_private.held;
  g_private = DevPool();
  if (g_pool.held > g_pool_cap) dev_release_all(stream);
}

int64_t* scratch(size_t words) {
  Context* c = ctx();
  if (dag_active()) {
    const unsigned slot = c->ring_next++ % Context::kScratchRing;
    if (c->ring_words[slot] < words) {
      if (c->ring[slot]) CUDA_CHECK(dev_free(c->ring[slot], c->stream));
      CUDA_CHECK(dev_alloc(&c->ring[slot], words * sizeof(int64_t), c->stream));
      c->ring_words[slot] = words;
    }
    return c->ring[slot];
  }
  if (c->scratch_words < words) {
    // the old block may still be in use by queued kernels: free it in stream order
    if (c->scratch) CUDA_CHECK(dev_free(c->scratch, c->stream));
    CUDA_CHECK(dev_alloc(&c->scratch, words * sizeof(int64_t), c->stream));
    c->scratch_words = words;
  }
  return c->scratch;
}

}  // namespace fhert
