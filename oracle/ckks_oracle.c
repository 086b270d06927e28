/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the RNS-polynomial path of the
 * ANT-ACE CKKS runtime, used by tests, smoke() and the benchmark's CPU
 * baseline as a checker.  Nothing in the shipped library links or calls it.
 *
 * Each function names the reference code it restates, as <file>:<line> inside
 * fhe-cmplr/rtlib/ant/.  The restatement is pinned two ways (tests/
 * test_oracle_*.py): against the known-answer vectors of the reference's own
 * unit tests (unittest/ut_ntt.cxx:15-19, ut_test_number_theory.cxx:14-106)
 * and, where the reference library could be built (oracle/build_ref.sh),
 * against that library on seeded inputs.
 *
 * Layout: polynomials are limb-major int64 arrays; an "extended" polynomial is
 * `level` Q limbs followed directly by K special limbs.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef unsigned __int128 u128;
typedef uint64_t          u64;

typedef struct {
  uint32_t n, logn;
  int      L, K, dnum, alpha;
  u64*     primes;   /* L + K */
  u64*     rou;      /* (L+K) x n, rou[brv(i)] = psi^i      (util/src/ntt.c:91-138) */
  u64*     rou_inv;  /* (L+K) x n, rou_inv[brv(i)] = psi^-i */
  u64*     n_inv;    /* N^-1 mod each prime */
} ORACLE_CTX;

/* ---- modular arithmetic (include/util/modular.h:126-256) ------------------ */

static u64 Mul_mod(u64 a, u64 b, u64 q) { return (u64)((u128)a * b % q); }
static u64 Add_mod(u64 a, u64 b, u64 q) {
  u64 s = a + b;
  return s >= q ? s - q : s;
}
static u64 Sub_mod(u64 a, u64 b, u64 q) { return a >= b ? a - b : a + q - b; }

u64 Oracle_pow_mod(u64 a, u64 e, u64 q) {
  u64 r = 1 % q;
  a %= q;
  while (e) {
    if (e & 1) r = Mul_mod(r, a, q);
    a = Mul_mod(a, a, q);
    e >>= 1;
  }
  return r;
}

/* util/src/number_theory.c:52-55: inverse modulo a prime by Fermat */
u64 Oracle_inv_mod_prime(u64 a, u64 q) { return Oracle_pow_mod(a, q - 2, q); }

/* util/src/number_theory.c:57-80: extended Euclid, any modulus */
int64_t Oracle_inv_mod(int64_t val, int64_t modulus) {
  int64_t m = modulus, a = val % modulus, y = 0, x = 1;
  if (modulus == 1) return 0;
  while (a > 1) {
    int64_t t = m, q = a / t;
    m = a % t;
    a = t;
    t = y;
    y = x - q * y;
    x = t;
  }
  return x < 0 ? x + modulus : x;
}

/* include/util/modular.h:296-322: centred lift from old_mod to new_mod */
static u64 Switch_mod(u64 v, u64 old_mod, u64 new_mod) {
  u64 r = v % new_mod;
  if (v > (old_mod >> 1)) r = Sub_mod(r, old_mod % new_mod, new_mod);
  return r;
}

/* include/util/modular.h:41-57: floor(2^128 / mod) as (hi, lo) */
void Oracle_prec128(u64 mod, u64* hi, u64* lo) {
  u128 v = ~(u128)0 / mod; /* equals floor(2^128/mod) unless mod is a power of two */
  *hi = (u64)(v >> 64);
  *lo = (u64)v;
}

/* ---- primes and roots ------------------------------------------------------ */

/* util/src/number_theory.c:165-190 decides primality with 200 random
 * Miller-Rabin rounds; the deterministic base set below is exact below 2^64. */
int Oracle_is_prime(u64 n) {
  static const u64 bases[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
  if (n < 2) return 0;
  for (int i = 0; i < 12; i++) {
    if (n == bases[i]) return 1;
    if (n % bases[i] == 0) return 0;
  }
  u64 d = n - 1;
  int r = 0;
  while (!(d & 1)) {
    d >>= 1;
    r++;
  }
  for (int i = 0; i < 12; i++) {
    u64 x = Oracle_pow_mod(bases[i], d, n);
    if (x == 1 || x == n - 1) continue;
    int composite = 1;
    for (int j = 1; j < r && composite; j++) {
      x = Mul_mod(x, x, n);
      if (x == n - 1) composite = 0;
    }
    if (composite) return 0;
  }
  return 1;
}

/* util/src/crt.c:42-67 */
static u64 First_prime(uint32_t n, size_t bits) {
  u64 order = 2ull * n, p = (1ull << bits) + order + 1;
  while (!Oracle_is_prime(p)) p += order;
  return p;
}
static u64 Prev_prime(u64 p, u64 order) {
  do p -= order;
  while (!Oracle_is_prime(p));
  return p;
}
static u64 Next_prime(u64 p, u64 order) {
  p += order; /* the reference skips the first candidate above p */
  do p += order;
  while (!Oracle_is_prime(p));
  return p;
}

/* util/src/number_theory.c:97-139: smallest primitive root of a prime */
u64 Oracle_find_generator(u64 q) {
  u64 phi = q - 1, number = phi, factors[64];
  int nf = 0;
  for (u64 i = 2; i <= (u64)sqrt((double)number); i++) {
    if (number % i == 0) {
      factors[nf++] = i;
      while (number % i == 0) number /= i;
    }
  }
  if (number > 1) factors[nf++] = number;
  for (u64 r = 2; r <= phi; r++) {
    int ok = 1;
    for (int i = 0; i < nf && ok; i++)
      if (Oracle_pow_mod(r, phi / factors[i], q) == 1) ok = 0;
    if (ok) return r;
  }
  return 0;
}

/* util/src/std_param.c:229-300: the reference tabulates 2N-th roots for the
 * prime chains of ring degrees 16 and 16384; each entry is the smallest
 * primitive root of that order and the covered primes are the first lattice
 * primes (1 mod order) below / above 2^60, 2^59 and 2^50. */
static int Root_table_covers(u64 order, u64 q) {
  static const struct { u64 order; int bits, below, above; } spans[] = {
      {32, 60, 9, 0}, {32, 59, 10, 11}, {32, 50, 2, 3}, {32768, 60, 10, 0}, {32768, 59, 12, 13}};
  for (int s = 0; s < 5; s++) {
    if (spans[s].order != order) continue;
    u64 c = (1ull << spans[s].bits) + 1;
    for (int found = 0; found < spans[s].below;) {
      c -= order;
      if (Oracle_is_prime(c)) {
        if (c == q) return 1;
        found++;
      }
    }
    c = (1ull << spans[s].bits) + 1;
    for (int found = 0; found < spans[s].above;) {
      c += order;
      if (Oracle_is_prime(c)) {
        if (c == q) return 1;
        found++;
      }
    }
  }
  return 0;
}

/* util/src/number_theory.c:141-162 */
u64 Oracle_root_of_unity(u64 order, u64 q) {
  u64 root = Oracle_pow_mod(Oracle_find_generator(q), (q - 1) / order, q);
  if (!Root_table_covers(order, q)) return root;
  u64 sq = Mul_mod(root, root, q), cur = root, best = root;
  for (u64 k = 0; k < order / 2; k++) {
    if (cur < best) best = cur;
    cur = Mul_mod(cur, sq, q);
  }
  return best;
}

static uint32_t Brv(uint32_t v, int bits) {
  uint32_t r = 0;
  for (int i = 0; i < bits; i++) r |= ((v >> i) & 1u) << (bits - 1 - i);
  return r;
}

static size_t Product_bits(const u64* f, int cnt) {
  u64 big[32] = {1};
  int len     = 1;
  for (int k = 0; k < cnt; k++) {
    u64 carry = 0;
    for (int i = 0; i < len; i++) {
      u128 t = (u128)big[i] * f[k] + carry;
      big[i] = (u64)t;
      carry  = (u64)(t >> 64);
    }
    if (carry) big[len++] = carry;
  }
  return (size_t)(len - 1) * 64 + (64 - (size_t)__builtin_clzll(big[len - 1]));
}

/* util/src/crt.c:112-148 (Q chain), 416-457 (K), 71-103 (P chain); tables of
 * util/src/ntt.c:34-138 */
ORACLE_CTX* Oracle_create(uint32_t n, int num_q, size_t q0_bits, size_t sf_bits, int dnum) {
  ORACLE_CTX* c = (ORACLE_CTX*)calloc(1, sizeof(ORACLE_CTX));
  c->n          = n;
  c->logn       = 31 - __builtin_clz(n);
  c->L          = num_q;
  c->dnum       = dnum;
  c->alpha      = (num_q + dnum - 1) / dnum;
  u64  order    = 2ull * n;
  u64* q        = (u64*)calloc(num_q, sizeof(u64));
  u64  first    = First_prime(n, sf_bits);
  q[num_q - 1]  = first;
  u64 q_prev = first, q_next = first;
  if (num_q > 1) {
    unsigned cnt = 0;
    for (int i = num_q - 2; i >= 1; i--, cnt++) {
      if ((cnt & 1) == 0)
        q[i] = q_prev = Prev_prime(q_prev, order);
      else
        q[i] = q_next = Next_prime(q_next, order);
    }
  }
  q[0] = q0_bits == sf_bits ? Prev_prime(q_prev, order)
                            : Prev_prime(First_prime(n, q0_bits), order);
  size_t max_bits = 0;
  for (int j = 0; j < dnum; j++) {
    int start = j * c->alpha, len = 0;
    while (len < c->alpha && start + len < num_q) len++;
    size_t b = Product_bits(q + start, len);
    if (b > max_bits) max_bits = b;
  }
  c->K      = (int)((max_bits + 59) / 60);
  c->primes = (u64*)calloc(num_q + c->K, sizeof(u64));
  memcpy(c->primes, q, num_q * sizeof(u64));
  u64 prev = First_prime(n, 60);
  for (int i = 0; i < c->K; i++) {
    u64 cand;
    int in_q;
    do {
      cand = Prev_prime(prev, order);
      in_q = 0;
      for (int j = 0; j < num_q; j++) in_q |= (q[j] == cand);
      prev = cand;
    } while (in_q);
    c->primes[num_q + i] = cand;
  }
  free(q);
  int total  = num_q + c->K;
  c->rou     = (u64*)calloc((size_t)total * n, sizeof(u64));
  c->rou_inv = (u64*)calloc((size_t)total * n, sizeof(u64));
  c->n_inv   = (u64*)calloc(total, sizeof(u64));
  for (int i = 0; i < total; i++) {
    u64 p = c->primes[i], psi = Oracle_root_of_unity(order, p);
    u64 psi_inv = Oracle_inv_mod_prime(psi, p), pw = 1, pwi = 1;
    for (uint32_t k = 0; k < n; k++) {
      uint32_t r                 = Brv(k, c->logn);
      c->rou[(size_t)i * n + r]     = pw;
      c->rou_inv[(size_t)i * n + r] = pwi;
      pw                         = Mul_mod(pw, psi, p);
      pwi                        = Mul_mod(pwi, psi_inv, p);
    }
    c->n_inv[i] = Oracle_inv_mod_prime(n % p, p);
  }
  return c;
}

void Oracle_destroy(ORACLE_CTX* c) {
  if (!c) return;
  free(c->primes);
  free(c->rou);
  free(c->rou_inv);
  free(c->n_inv);
  free(c);
}

int  Oracle_num_p(ORACLE_CTX* c) { return c->K; }
int  Oracle_alpha(ORACLE_CTX* c) { return c->alpha; }
void Oracle_get_primes(ORACLE_CTX* c, int64_t* out) {
  for (int i = 0; i < c->L + c->K; i++) out[i] = (int64_t)c->primes[i];
}
void Oracle_get_tables(ORACLE_CTX* c, int idx, int64_t* rou, int64_t* rou_inv, int64_t* n_inv) {
  memcpy(rou, c->rou + (size_t)idx * c->n, c->n * sizeof(u64));
  memcpy(rou_inv, c->rou_inv + (size_t)idx * c->n, c->n * sizeof(u64));
  *n_inv = (int64_t)c->n_inv[idx];
}

/* ---- NTT (util/src/ntt.c:167-241 forward, 245-330 inverse) ------------------ */

/* generic forms on explicit tables, so that the N=4 known-answer vectors of
 * unittest/ut_ntt.cxx can be run with their own prime */
void Oracle_ntt_tables(int64_t* data, uint32_t n, u64 q, const u64* rou) {
  u64*     x = (u64*)data;
  uint32_t t = n >> 1;
  for (uint32_t m = 1; m < n; m <<= 1, t >>= 1) {
    for (uint32_t i = 0; i < m; i++) {
      u64 w = rou[m + i];
      for (uint32_t j1 = 2 * i * t, j2 = j1 + t; j1 < j2; j1++) {
        u64 v     = Mul_mod(x[j1 + t], w, q);
        u64 lo    = x[j1];
        x[j1]     = Add_mod(lo, v, q);
        x[j1 + t] = Sub_mod(lo, v, q);
      }
    }
  }
}

void Oracle_intt_tables(int64_t* data, uint32_t n, u64 q, const u64* rou_inv, u64 n_inv) {
  u64*     x = (u64*)data;
  uint32_t t = 1;
  for (uint32_t m = n >> 1; m >= 1; m >>= 1, t <<= 1) {
    for (uint32_t i = 0; i < m; i++) {
      u64 w = rou_inv[m + i];
      for (uint32_t j1 = 2 * i * t, j2 = j1 + t; j1 < j2; j1++) {
        u64 lo = x[j1], hi = x[j1 + t];
        x[j1]     = Add_mod(lo, hi, q);
        x[j1 + t] = Mul_mod(Sub_mod(lo, hi, q), w, q);
      }
    }
  }
  /* the reference folds N^-1 into its first stage; the product is the same */
  for (uint32_t i = 0; i < n; i++) x[i] = Mul_mod(x[i], n_inv, q);
}

/* twiddle table of one prime for a given 2N-th root (util/src/ntt.c:91-138) */
void Oracle_make_tables(uint32_t n, u64 q, u64 psi, int64_t* rou, int64_t* rou_inv) {
  int logn = 31 - __builtin_clz(n);
  u64 psi_inv = Oracle_inv_mod_prime(psi, q), pw = 1, pwi = 1;
  for (uint32_t k = 0; k < n; k++) {
    uint32_t r = Brv(k, logn);
    rou[r]     = (int64_t)pw;
    rou_inv[r] = (int64_t)pwi;
    pw         = Mul_mod(pw, psi, q);
    pwi        = Mul_mod(pwi, psi_inv, q);
  }
}

void Oracle_ntt(ORACLE_CTX* c, int prime_idx, int64_t* data, int inverse) {
  size_t off = (size_t)prime_idx * c->n;
  if (inverse)
    Oracle_intt_tables(data, c->n, c->primes[prime_idx], c->rou_inv + off, c->n_inv[prime_idx]);
  else
    Oracle_ntt_tables(data, c->n, c->primes[prime_idx], c->rou + off);
}

/* ---- per-limb vector ops (hal/src/hal.c:15-138) ---------------------------- */

void Oracle_hw(int op, int64_t* res, const int64_t* a, const int64_t* b, u64 q, uint32_t n) {
  for (uint32_t i = 0; i < n; i++) {
    u64 x = (u64)a[i], y = (u64)b[i], r;
    switch (op) {
      case 0: r = Add_mod(x, y, q); break;
      case 1: r = Sub_mod(x, y, q); break;
      case 2: r = Mul_mod(x, y, q); break;
      default: r = Add_mod((u64)res[i], Mul_mod(x, y, q), q); break; /* muladd */
    }
    res[i] = (int64_t)r;
  }
}

/* util/src/number_theory.c:192-204 with the modulus 2N */
uint32_t Oracle_auto_index(int32_t rot_idx, uint32_t n) {
  u64 m = 2ull * n;
  if (rot_idx == 0) return 1;
  if ((u64)(int64_t)rot_idx == m - 1) return (uint32_t)rot_idx;
  u64 gen = rot_idx < 0 ? (u64)Oracle_inv_mod(5, (int64_t)m) : 5;
  u64 e = (u64)llabs((long long)rot_idx), r = 1, b = gen % m;
  while (e) {
    if (e & 1) r = r * b % m;
    b = b * b % m;
    e >>= 1;
  }
  return (uint32_t)r;
}

/* util/src/number_theory.c:206-230, NTT form */
void Oracle_auto_order(uint32_t k, uint32_t n, int64_t* order) {
  int logn = 31 - __builtin_clz(n);
  u64 m    = 2ull * n;
  for (uint32_t j = 0; j < n; j++) {
    u64 idx                = (((2ull * j + 1) * k) % m) >> 1;
    order[Brv(j, logn)] = (int64_t)Brv((uint32_t)idx, logn);
  }
}

void Oracle_rotate_limb(int64_t* res, const int64_t* val, const int64_t* order, uint32_t n) {
  for (uint32_t i = 0; i < n; i++) res[i] = val[order[i]];
}

/* ---- rescale (poly/src/rns_poly.c:310-404, constants util/src/crt.c:291-353) -- */

void Oracle_rescale(ORACLE_CTX* c, const int64_t* poly, int level, int64_t* out) {
  uint32_t n    = c->n;
  int      l    = level - 1;
  u64      ql   = c->primes[l];
  int64_t* last = (int64_t*)malloc(n * sizeof(int64_t));
  int64_t* t    = (int64_t*)malloc(n * sizeof(int64_t));
  memcpy(last, poly + (size_t)l * n, n * sizeof(int64_t));
  Oracle_ntt(c, l, last, 1);
  for (int i = 0; i < l; i++) {
    u64 qi     = c->primes[i];
    u64 ql_inv = Oracle_inv_mod_prime(ql % qi, qi);
    /* floor(Qhat_l (Qhat_l^-1 mod q_l) / q_l) mod q_i equals -q_l^-1 mod q_i */
    u64 neg = ql_inv ? qi - ql_inv : 0;
    for (uint32_t k = 0; k < n; k++)
      t[k] = (int64_t)Mul_mod(Switch_mod((u64)last[k], ql, qi), neg, qi);
    Oracle_ntt(c, i, t, 0);
    for (uint32_t k = 0; k < n; k++)
      out[(size_t)i * n + k] =
          (int64_t)Add_mod(Mul_mod((u64)poly[(size_t)i * n + k], ql_inv, qi), (u64)t[k], qi);
  }
  free(last);
  free(t);
}

/* ---- ModUp (poly/src/rns_poly.c:160-258, tables util/src/crt.c:459-566) ------ */

int Oracle_num_decomp(ORACLE_CTX* c, int level) {
  int d = (level + c->alpha - 1) / c->alpha;
  return d > c->dnum ? c->dnum : d;
}

void Oracle_decomp_modup(ORACLE_CTX* c, const int64_t* poly, int level, int part, int64_t* ext) {
  uint32_t n     = c->n;
  int      start = part * c->alpha, end = start + c->alpha;
  if (end > level) end = level;
  int      dl = end - start;
  int64_t* y  = (int64_t*)malloc((size_t)dl * n * sizeof(int64_t));
  for (int i = 0; i < dl; i++) {
    u64 qi = c->primes[start + i], hat = 1;
    memcpy(y + (size_t)i * n, poly + (size_t)(start + i) * n, n * sizeof(int64_t));
    Oracle_ntt(c, start + i, y + (size_t)i * n, 1);
    for (int k = start; k < end; k++)
      if (k != start + i) hat = Mul_mod(hat, c->primes[k] % qi, qi);
    u64 inv = Oracle_inv_mod_prime(hat, qi);
    for (uint32_t k = 0; k < n; k++)
      y[(size_t)i * n + k] = (int64_t)Mul_mod((u64)y[(size_t)i * n + k], inv, qi);
  }
  for (int m = 0; m < level + c->K; m++) {
    int      prime_idx = m < level ? m : c->L + (m - level);
    int64_t* dst       = ext + (size_t)m * n;
    if (m >= start && m < end) {
      memcpy(dst, poly + (size_t)m * n, n * sizeof(int64_t));
      continue;
    }
    u64 pm = c->primes[prime_idx], hat[64];
    for (int i = 0; i < dl; i++) {
      hat[i] = 1;
      for (int k = start; k < end; k++)
        if (k != start + i) hat[i] = Mul_mod(hat[i], c->primes[k] % pm, pm);
    }
    for (uint32_t k = 0; k < n; k++) {
      u128 sum = 0;
      for (int i = 0; i < dl; i++) sum += (u128)(u64)y[(size_t)i * n + k] * hat[i];
      dst[k] = (int64_t)(u64)(sum % pm);
    }
    Oracle_ntt(c, prime_idx, dst, 0);
  }
  free(y);
}

/* ---- ModDown (rns_poly.c:260-308, rns_poly_impl.c:287-339, crt.c:357-414) ---- */

void Oracle_mod_down(ORACLE_CTX* c, const int64_t* ext, int level, int64_t* out) {
  uint32_t n = c->n;
  int      K = c->K;
  int64_t* y = (int64_t*)malloc((size_t)K * n * sizeof(int64_t));
  int64_t* t = (int64_t*)malloc(n * sizeof(int64_t));
  for (int k = 0; k < K; k++) {
    u64 pk = c->primes[c->L + k], hat = 1;
    memcpy(y + (size_t)k * n, ext + (size_t)(level + k) * n, n * sizeof(int64_t));
    Oracle_ntt(c, c->L + k, y + (size_t)k * n, 1);
    for (int j = 0; j < K; j++)
      if (j != k) hat = Mul_mod(hat, c->primes[c->L + j] % pk, pk);
    u64 inv = Oracle_inv_mod_prime(hat, pk);
    for (uint32_t d = 0; d < n; d++)
      y[(size_t)k * n + d] = (int64_t)Mul_mod((u64)y[(size_t)k * n + d], inv, pk);
  }
  for (int i = 0; i < level; i++) {
    u64 qi = c->primes[i], P = 1, hat[64];
    for (int k = 0; k < K; k++) {
      P      = Mul_mod(P, c->primes[c->L + k] % qi, qi);
      hat[k] = 1;
      for (int j = 0; j < K; j++)
        if (j != k) hat[k] = Mul_mod(hat[k], c->primes[c->L + j] % qi, qi);
    }
    u64 p_inv = Oracle_inv_mod_prime(P, qi);
    for (uint32_t d = 0; d < n; d++) {
      u128 sum = 0;
      for (int k = 0; k < K; k++) sum += (u128)(u64)y[(size_t)k * n + d] * hat[k];
      t[d] = (int64_t)(u64)(sum % qi);
    }
    Oracle_ntt(c, i, t, 0);
    for (uint32_t d = 0; d < n; d++)
      out[(size_t)i * n + d] =
          (int64_t)Mul_mod(Sub_mod((u64)ext[(size_t)i * n + d], (u64)t[d], qi), p_inv, qi);
  }
  free(y);
  free(t);
}

/* ---- hybrid key switch (ckks/src/evaluator.c:411-462) -------------------------
 * key0/key1: dnum polynomials each, every one L Q limbs followed by K P limbs. */
void Oracle_switch_key(ORACLE_CTX* c, const int64_t* in, int level, const int64_t* key0,
                       const int64_t* key1, int64_t* out0, int64_t* out1) {
  uint32_t n      = c->n;
  int      parts  = Oracle_num_decomp(c, level), K = c->K;
  size_t   ext_sz = (size_t)(level + K) * n, key_sz = (size_t)(c->L + K) * n;
  int64_t* ext    = (int64_t*)malloc(ext_sz * sizeof(int64_t));
  int64_t* acc0   = (int64_t*)calloc(ext_sz, sizeof(int64_t));
  int64_t* acc1   = (int64_t*)calloc(ext_sz, sizeof(int64_t));
  for (int j = 0; j < parts; j++) {
    Oracle_decomp_modup(c, in, level, j, ext);
    for (int m = 0; m < level + K; m++) {
      int    key_limb = m < level ? m : c->L + (m - level);
      u64    p        = c->primes[key_limb];
      size_t eo = (size_t)m * n, ko = (size_t)j * key_sz + (size_t)key_limb * n;
      Oracle_hw(3, acc0 + eo, ext + eo, key0 + ko, p, n);
      Oracle_hw(3, acc1 + eo, ext + eo, key1 + ko, p, n);
    }
  }
  Oracle_mod_down(c, acc0, level, out0);
  Oracle_mod_down(c, acc1, level, out1);
  free(ext);
  free(acc0);
  free(acc1);
}

/* evaluator.c:503-530: key switch c1, add c0, permute both */
void Oracle_rotate(ORACLE_CTX* c, const int64_t* c0, const int64_t* c1, int level,
                   int32_t rot_idx, const int64_t* key0, const int64_t* key1, int64_t* out0,
                   int64_t* out1) {
  uint32_t n  = c->n;
  size_t   sz = (size_t)level * n;
  int64_t* t0 = (int64_t*)malloc(sz * sizeof(int64_t));
  int64_t* t1 = (int64_t*)malloc(sz * sizeof(int64_t));
  int64_t* order = (int64_t*)malloc(n * sizeof(int64_t));
  Oracle_switch_key(c, c1, level, key0, key1, t0, t1);
  Oracle_auto_order(Oracle_auto_index(rot_idx, n), n, order);
  for (int i = 0; i < level; i++) {
    size_t o = (size_t)i * n;
    Oracle_hw(0, t0 + o, t0 + o, c0 + o, c->primes[i], n);
    Oracle_rotate_limb(out0 + o, t0 + o, order, n);
    Oracle_rotate_limb(out1 + o, t1 + o, order, n);
  }
  free(t0);
  free(t1);
  free(order);
}

/* evaluator.c:137-190 (tensor product), 288-305 (relinearise), 344-363 (rescale);
 * outputs hold level-1 limbs */
void Oracle_mul_relin_rescale(ORACLE_CTX* c, const int64_t* a0, const int64_t* a1,
                              const int64_t* b0, const int64_t* b1, int level,
                              const int64_t* key0, const int64_t* key1, int64_t* out0,
                              int64_t* out1) {
  uint32_t n  = c->n;
  size_t   sz = (size_t)level * n;
  int64_t *d0 = (int64_t*)malloc(sz * 8), *d1 = (int64_t*)malloc(sz * 8),
          *d2 = (int64_t*)malloc(sz * 8), *r0 = (int64_t*)malloc(sz * 8),
          *r1 = (int64_t*)malloc(sz * 8);
  for (int i = 0; i < level; i++) {
    size_t o = (size_t)i * n;
    u64    q = c->primes[i];
    Oracle_hw(2, d0 + o, a0 + o, b0 + o, q, n);
    Oracle_hw(2, d1 + o, a0 + o, b1 + o, q, n);
    Oracle_hw(3, d1 + o, a1 + o, b0 + o, q, n);
    Oracle_hw(2, d2 + o, a1 + o, b1 + o, q, n);
  }
  Oracle_switch_key(c, d2, level, key0, key1, r0, r1);
  for (int i = 0; i < level; i++) {
    size_t o = (size_t)i * n;
    Oracle_hw(0, r0 + o, r0 + o, d0 + o, c->primes[i], n);
    Oracle_hw(0, r1 + o, r1 + o, d1 + o, c->primes[i], n);
  }
  Oracle_rescale(c, r0, level, out0);
  Oracle_rescale(c, r1, level, out1);
  free(d0);
  free(d1);
  free(d2);
  free(r0);
  free(r1);
}
