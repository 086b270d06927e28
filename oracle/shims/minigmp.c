/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * Implementation of the mpz subset declared in the stand-in gmp.h of this
 * directory: sign-magnitude integers on little-endian 32-bit limbs, schoolbook
 * multiplication and Knuth's algorithm D for division.  Written for clarity,
 * not speed; the reference runtime uses big integers only for one-time table
 * construction and for the CRT reconstruction inside Decode.
 */
#include "gmp.h"

#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#define ABS(x) ((x) < 0 ? -(x) : (x))

static void Reserve(mpz_ptr x, int n) {
  if (n <= x->_mp_alloc) return;
  int cap = x->_mp_alloc ? x->_mp_alloc : 4;
  while (cap < n) cap *= 2;
  x->_mp_d     = (uint32_t*)realloc(x->_mp_d, (size_t)cap * sizeof(uint32_t));
  x->_mp_alloc = cap;
}

static int Norm(const uint32_t* d, int n) {
  while (n > 0 && d[n - 1] == 0) n--;
  return n;
}

/* magnitude compare */
static int Cmp_mag(const uint32_t* a, int an, const uint32_t* b, int bn) {
  if (an != bn) return an > bn ? 1 : -1;
  for (int i = an - 1; i >= 0; i--) {
    if (a[i] != b[i]) return a[i] > b[i] ? 1 : -1;
  }
  return 0;
}

/* r = a + b (magnitudes); r has room for max(an,bn)+1 limbs; returns size */
static int Add_mag(uint32_t* r, const uint32_t* a, int an, const uint32_t* b,
                   int bn) {
  if (an < bn) {
    const uint32_t* t = a;
    a                 = b;
    b                 = t;
    int tn            = an;
    an                = bn;
    bn                = tn;
  }
  uint64_t c = 0;
  int      i = 0;
  for (; i < bn; i++) {
    c += (uint64_t)a[i] + b[i];
    r[i] = (uint32_t)c;
    c >>= 32;
  }
  for (; i < an; i++) {
    c += a[i];
    r[i] = (uint32_t)c;
    c >>= 32;
  }
  if (c) r[i++] = (uint32_t)c;
  return i;
}

/* r = a - b (magnitudes, a >= b); returns normalised size */
static int Sub_mag(uint32_t* r, const uint32_t* a, int an, const uint32_t* b,
                   int bn) {
  int64_t c = 0;
  int     i = 0;
  for (; i < bn; i++) {
    c += (int64_t)a[i] - b[i];
    r[i] = (uint32_t)c;
    c >>= 32;
  }
  for (; i < an; i++) {
    c += a[i];
    r[i] = (uint32_t)c;
    c >>= 32;
  }
  return Norm(r, an);
}

void mpz_init(mpz_ptr x) {
  x->_mp_alloc = 0;
  x->_mp_size  = 0;
  x->_mp_d     = NULL;
}

void mpz_clear(mpz_ptr x) {
  free(x->_mp_d);
  x->_mp_d     = NULL;
  x->_mp_alloc = 0;
  x->_mp_size  = 0;
}

void mpz_inits(mpz_ptr x, ...) {
  va_list ap;
  va_start(ap, x);
  while (x != NULL) {
    mpz_init(x);
    x = va_arg(ap, mpz_ptr);
  }
  va_end(ap);
}

void mpz_clears(mpz_ptr x, ...) {
  va_list ap;
  va_start(ap, x);
  while (x != NULL) {
    mpz_clear(x);
    x = va_arg(ap, mpz_ptr);
  }
  va_end(ap);
}

void mpz_set(mpz_ptr r, mpz_srcptr a) {
  if (r == a) return;
  int n = ABS(a->_mp_size);
  Reserve(r, n);
  if (n) memcpy(r->_mp_d, a->_mp_d, (size_t)n * sizeof(uint32_t));
  r->_mp_size = a->_mp_size;
}

void mpz_set_ui(mpz_ptr r, unsigned long v) {
  Reserve(r, 2);
  r->_mp_d[0] = (uint32_t)v;
  r->_mp_d[1] = (uint32_t)((uint64_t)v >> 32);
  r->_mp_size = Norm(r->_mp_d, 2);
}

void mpz_set_si(mpz_ptr r, long v) {
  if (v >= 0) {
    mpz_set_ui(r, (unsigned long)v);
  } else {
    mpz_set_ui(r, 0UL - (unsigned long)v);
    r->_mp_size = -r->_mp_size;
  }
}

void mpz_set_d(mpz_ptr r, double d) {
  int neg = d < 0;
  if (neg) d = -d;
  d = floor(d);
  if (!(d >= 1.0)) {
    r->_mp_size = 0;
    return;
  }
  int    e;
  double m = frexp(d, &e); /* d = m * 2^e, 0.5 <= m < 1 */
  /* 53 significant bits */
  uint64_t mant  = (uint64_t)ldexp(m, 53);
  int      shift = e - 53;
  mpz_set_ui(r, mant);
  if (shift > 0) {
    mpz_mul_2exp(r, r, (unsigned long)shift);
  } else if (shift < 0) {
    mpz_fdiv_q_2exp(r, r, (unsigned long)(-shift));
  }
  if (neg) r->_mp_size = -r->_mp_size;
}

void mpz_init_set(mpz_ptr r, mpz_srcptr a) {
  mpz_init(r);
  mpz_set(r, a);
}
void mpz_init_set_si(mpz_ptr r, long v) {
  mpz_init(r);
  mpz_set_si(r, v);
}
void mpz_init_set_ui(mpz_ptr r, unsigned long v) {
  mpz_init(r);
  mpz_set_ui(r, v);
}
void mpz_init_set_d(mpz_ptr r, double d) {
  mpz_init(r);
  mpz_set_d(r, d);
}

int mpz_set_str(mpz_ptr r, const char* str, int base) {
  if (base == 0) base = 10;
  int neg = 0;
  while (*str == ' ') str++;
  if (*str == '-') {
    neg = 1;
    str++;
  }
  mpz_set_ui(r, 0);
  if (*str == 0) return -1;
  for (; *str; str++) {
    int c = *str, v;
    if (c >= '0' && c <= '9')
      v = c - '0';
    else if (c >= 'a' && c <= 'z')
      v = c - 'a' + 10;
    else if (c >= 'A' && c <= 'Z')
      v = c - 'A' + 10;
    else
      return -1;
    if (v >= base) return -1;
    mpz_mul_ui(r, r, (unsigned long)base);
    mpz_add_ui(r, r, (unsigned long)v);
  }
  if (neg) r->_mp_size = -r->_mp_size;
  return 0;
}

/* signed add of (a) and (sign_b * |b|) */
static void Add_signed(mpz_ptr r, mpz_srcptr a, const uint32_t* bd, int bsize) {
  int an = ABS(a->_mp_size), bn = ABS(bsize);
  int n = (an > bn ? an : bn) + 1;
  /* work in a temporary so that r may alias a or b */
  uint32_t* t = (uint32_t*)malloc((size_t)n * sizeof(uint32_t));
  int       rn, rneg;
  if ((a->_mp_size < 0) == (bsize < 0)) {
    rn   = Add_mag(t, a->_mp_d, an, bd, bn);
    rneg = a->_mp_size < 0;
  } else {
    int c = Cmp_mag(a->_mp_d, an, bd, bn);
    if (c == 0) {
      rn   = 0;
      rneg = 0;
    } else if (c > 0) {
      rn   = Sub_mag(t, a->_mp_d, an, bd, bn);
      rneg = a->_mp_size < 0;
    } else {
      rn   = Sub_mag(t, bd, bn, a->_mp_d, an);
      rneg = bsize < 0;
    }
  }
  Reserve(r, rn);
  if (rn) memcpy(r->_mp_d, t, (size_t)rn * sizeof(uint32_t));
  r->_mp_size = rneg ? -rn : rn;
  free(t);
}

void mpz_add(mpz_ptr r, mpz_srcptr a, mpz_srcptr b) {
  Add_signed(r, a, b->_mp_d, b->_mp_size);
}

void mpz_sub(mpz_ptr r, mpz_srcptr a, mpz_srcptr b) {
  Add_signed(r, a, b->_mp_d, -b->_mp_size);
}

void mpz_add_ui(mpz_ptr r, mpz_srcptr a, unsigned long b) {
  uint32_t d[2] = {(uint32_t)b, (uint32_t)((uint64_t)b >> 32)};
  Add_signed(r, a, d, Norm(d, 2));
}

void mpz_sub_ui(mpz_ptr r, mpz_srcptr a, unsigned long b) {
  uint32_t d[2] = {(uint32_t)b, (uint32_t)((uint64_t)b >> 32)};
  Add_signed(r, a, d, -Norm(d, 2));
}

static void Mul_raw(mpz_ptr r, const uint32_t* a, int an, const uint32_t* b,
                    int bn, int neg) {
  if (an == 0 || bn == 0) {
    r->_mp_size = 0;
    return;
  }
  int       n = an + bn;
  uint32_t* t = (uint32_t*)calloc((size_t)n, sizeof(uint32_t));
  for (int i = 0; i < an; i++) {
    uint64_t c  = 0;
    uint64_t ai = a[i];
    for (int j = 0; j < bn; j++) {
      c += ai * b[j] + t[i + j];
      t[i + j] = (uint32_t)c;
      c >>= 32;
    }
    t[i + bn] = (uint32_t)c;
  }
  n = Norm(t, n);
  Reserve(r, n);
  memcpy(r->_mp_d, t, (size_t)n * sizeof(uint32_t));
  r->_mp_size = neg ? -n : n;
  free(t);
}

void mpz_mul(mpz_ptr r, mpz_srcptr a, mpz_srcptr b) {
  Mul_raw(r, a->_mp_d, ABS(a->_mp_size), b->_mp_d, ABS(b->_mp_size),
          (a->_mp_size < 0) != (b->_mp_size < 0));
}

void mpz_mul_ui(mpz_ptr r, mpz_srcptr a, unsigned long b) {
  uint32_t d[2] = {(uint32_t)b, (uint32_t)((uint64_t)b >> 32)};
  Mul_raw(r, a->_mp_d, ABS(a->_mp_size), d, Norm(d, 2), a->_mp_size < 0);
}

void mpz_mul_si(mpz_ptr r, mpz_srcptr a, long b) {
  unsigned long m    = b < 0 ? 0UL - (unsigned long)b : (unsigned long)b;
  uint32_t      d[2] = {(uint32_t)m, (uint32_t)((uint64_t)m >> 32)};
  Mul_raw(r, a->_mp_d, ABS(a->_mp_size), d, Norm(d, 2),
          (a->_mp_size < 0) != (b < 0));
}

void mpz_addmul(mpz_ptr r, mpz_srcptr a, mpz_srcptr b) {
  mpz_t t;
  mpz_init(t);
  mpz_mul(t, a, b);
  mpz_add(r, r, t);
  mpz_clear(t);
}

void mpz_addmul_ui(mpz_ptr r, mpz_srcptr a, unsigned long b) {
  mpz_t t;
  mpz_init(t);
  mpz_mul_ui(t, a, b);
  mpz_add(r, r, t);
  mpz_clear(t);
}

/* Truncating division of magnitudes: q = n / d, rem = n % d.
 * q has room for nn limbs, rem for dn limbs.  Returns through *qn, *rn the
 * normalised sizes.  d must be non-zero and normalised. */
static void Divmod_mag(uint32_t* q, int* qn, uint32_t* rem, int* rn,
                       const uint32_t* n, int nn, const uint32_t* d, int dn) {
  if (Cmp_mag(n, nn, d, dn) < 0) {
    *qn = 0;
    if (nn) memcpy(rem, n, (size_t)nn * sizeof(uint32_t));
    *rn = nn;
    return;
  }
  if (dn == 1) {
    uint64_t r = 0, dv = d[0];
    for (int i = nn - 1; i >= 0; i--) {
      uint64_t cur = (r << 32) | n[i];
      q[i]         = (uint32_t)(cur / dv);
      r            = cur % dv;
    }
    *qn    = Norm(q, nn);
    rem[0] = (uint32_t)r;
    *rn    = r ? 1 : 0;
    return;
  }
  /* Knuth algorithm D */
  int       s  = __builtin_clz(d[dn - 1]);
  uint32_t* vn = (uint32_t*)malloc((size_t)dn * sizeof(uint32_t));
  uint32_t* un = (uint32_t*)malloc((size_t)(nn + 1) * sizeof(uint32_t));
  if (s) {
    for (int i = dn - 1; i > 0; i--) vn[i] = (d[i] << s) | (d[i - 1] >> (32 - s));
    vn[0]  = d[0] << s;
    un[nn] = n[nn - 1] >> (32 - s);
    for (int i = nn - 1; i > 0; i--) un[i] = (n[i] << s) | (n[i - 1] >> (32 - s));
    un[0] = n[0] << s;
  } else {
    memcpy(vn, d, (size_t)dn * sizeof(uint32_t));
    memcpy(un, n, (size_t)nn * sizeof(uint32_t));
    un[nn] = 0;
  }
  const uint64_t b = 1ULL << 32;
  for (int j = nn - dn; j >= 0; j--) {
    uint64_t num  = ((uint64_t)un[j + dn] << 32) | un[j + dn - 1];
    uint64_t qhat = num / vn[dn - 1];
    uint64_t rhat = num % vn[dn - 1];
    while (qhat >= b || qhat * vn[dn - 2] > ((rhat << 32) | un[j + dn - 2])) {
      qhat--;
      rhat += vn[dn - 1];
      if (rhat >= b) break;
    }
    int64_t  borrow = 0;
    uint64_t carry  = 0;
    for (int i = 0; i < dn; i++) {
      uint64_t p = qhat * vn[i] + carry;
      carry      = p >> 32;
      int64_t t  = (int64_t)un[i + j] - (int64_t)(uint32_t)p + borrow;
      un[i + j]  = (uint32_t)t;
      borrow     = t >> 32;
    }
    int64_t t  = (int64_t)un[j + dn] - (int64_t)carry + borrow;
    un[j + dn] = (uint32_t)t;
    if (t < 0) {
      qhat--;
      uint64_t c = 0;
      for (int i = 0; i < dn; i++) {
        c += (uint64_t)un[i + j] + vn[i];
        un[i + j] = (uint32_t)c;
        c >>= 32;
      }
      un[j + dn] += (uint32_t)c;
    }
    q[j] = (uint32_t)qhat;
  }
  *qn = Norm(q, nn - dn + 1);
  if (s) {
    for (int i = 0; i < dn - 1; i++) rem[i] = (un[i] >> s) | (un[i + 1] << (32 - s));
    rem[dn - 1] = un[dn - 1] >> s;
  } else {
    memcpy(rem, un, (size_t)dn * sizeof(uint32_t));
  }
  *rn = Norm(rem, dn);
  free(vn);
  free(un);
}

/* floor division; q and/or r may be NULL */
static void Fdiv_qr(mpz_ptr q, mpz_ptr r, mpz_srcptr n, mpz_srcptr d) {
  int nn = ABS(n->_mp_size), dn = ABS(d->_mp_size);
  if (dn == 0) {
    fprintf(stderr, "minigmp: division by zero\n");
    abort();
  }
  int       nneg = n->_mp_size < 0, dneg = d->_mp_size < 0;
  uint32_t* qt = (uint32_t*)calloc((size_t)nn + 2, sizeof(uint32_t));
  uint32_t* rt = (uint32_t*)calloc((size_t)(dn > nn ? dn : nn) + 2, sizeof(uint32_t));
  int       qn, rn;
  Divmod_mag(qt, &qn, rt, &rn, n->_mp_d, nn, d->_mp_d, dn);
  /* truncated: n = qt*d + rt with sign(rt)=sign(n), sign(qt)=nneg^dneg */
  int qneg = nneg != dneg;
  int rneg = nneg;
  if (rn != 0 && qneg) {
    /* floor: q = -(|q|+1), r = r + d  i.e. |r'| = |d| - |r| with sign of d */
    uint32_t one = 1;
    qn           = Add_mag(qt, qt, qn, &one, 1);
    uint32_t* t2 = (uint32_t*)calloc((size_t)dn + 1, sizeof(uint32_t));
    rn           = Sub_mag(t2, d->_mp_d, dn, rt, rn);
    memcpy(rt, t2, (size_t)dn * sizeof(uint32_t));
    free(t2);
    rneg = dneg;
  }
  if (q) {
    Reserve(q, qn);
    if (qn) memcpy(q->_mp_d, qt, (size_t)qn * sizeof(uint32_t));
    q->_mp_size = qneg ? -qn : qn;
  }
  if (r) {
    Reserve(r, rn);
    if (rn) memcpy(r->_mp_d, rt, (size_t)rn * sizeof(uint32_t));
    r->_mp_size = rneg ? -rn : rn;
  }
  free(qt);
  free(rt);
}

void mpz_fdiv_q(mpz_ptr q, mpz_srcptr n, mpz_srcptr d) { Fdiv_qr(q, NULL, n, d); }
void mpz_fdiv_r(mpz_ptr r, mpz_srcptr n, mpz_srcptr d) { Fdiv_qr(NULL, r, n, d); }

unsigned long mpz_fdiv_q_ui(mpz_ptr q, mpz_srcptr n, unsigned long d) {
  mpz_t dd, r;
  mpz_init_set_ui(dd, d);
  mpz_init(r);
  Fdiv_qr(q, r, n, dd);
  unsigned long res = mpz_get_ui(r);
  mpz_clears(dd, r, NULL);
  return res;
}

unsigned long mpz_fdiv_r_ui(mpz_ptr r, mpz_srcptr n, unsigned long d) {
  mpz_t dd;
  mpz_init_set_ui(dd, d);
  Fdiv_qr(NULL, r, n, dd);
  unsigned long res = mpz_get_ui(r);
  mpz_clear(dd);
  return res;
}

void mpz_mul_2exp(mpz_ptr r, mpz_srcptr a, unsigned long bits) {
  int an = ABS(a->_mp_size);
  if (an == 0) {
    r->_mp_size = 0;
    return;
  }
  int       ws = (int)(bits / 32), bs = (int)(bits % 32);
  int       n = an + ws + 1;
  uint32_t* t = (uint32_t*)calloc((size_t)n, sizeof(uint32_t));
  for (int i = 0; i < an; i++) {
    uint64_t v = (uint64_t)a->_mp_d[i] << bs;
    t[i + ws] |= (uint32_t)v;
    t[i + ws + 1] |= (uint32_t)(v >> 32);
  }
  int neg = a->_mp_size < 0;
  n       = Norm(t, n);
  Reserve(r, n);
  memcpy(r->_mp_d, t, (size_t)n * sizeof(uint32_t));
  r->_mp_size = neg ? -n : n;
  free(t);
}

void mpz_fdiv_q_2exp(mpz_ptr q, mpz_srcptr n, unsigned long bits) {
  mpz_t d;
  mpz_init_set_ui(d, 1);
  mpz_mul_2exp(d, d, bits);
  Fdiv_qr(q, NULL, n, d);
  mpz_clear(d);
}

void mpz_powm(mpz_ptr r, mpz_srcptr b, mpz_srcptr e, mpz_srcptr m) {
  mpz_t base, acc;
  mpz_init(base);
  mpz_init_set_ui(acc, 1);
  mpz_fdiv_r(base, b, m);
  int en = ABS(e->_mp_size);
  for (int i = 0; i < en * 32; i++) {
    if ((e->_mp_d[i / 32] >> (i % 32)) & 1u) {
      mpz_mul(acc, acc, base);
      mpz_fdiv_r(acc, acc, m);
    }
    mpz_mul(base, base, base);
    mpz_fdiv_r(base, base, m);
  }
  mpz_fdiv_r(acc, acc, m);
  mpz_set(r, acc);
  mpz_clears(base, acc, NULL);
}

void mpz_pow_ui(mpz_ptr r, mpz_srcptr b, unsigned long e) {
  mpz_t base, acc;
  mpz_init_set(base, b);
  mpz_init_set_ui(acc, 1);
  while (e) {
    if (e & 1) mpz_mul(acc, acc, base);
    e >>= 1;
    if (e) mpz_mul(base, base, base);
  }
  mpz_set(r, acc);
  mpz_clears(base, acc, NULL);
}

void mpz_sqrt(mpz_ptr r, mpz_srcptr a) {
  /* Newton iteration on integers: floor(sqrt(a)) */
  if (a->_mp_size <= 0) {
    r->_mp_size = 0;
    return;
  }
  mpz_t x, y, t;
  mpz_init_set_ui(x, 1);
  mpz_mul_2exp(x, x, (mpz_sizeinbase(a, 2) + 1) / 2);
  mpz_init(y);
  mpz_init(t);
  for (;;) {
    mpz_fdiv_q(t, a, x);
    mpz_add(y, x, t);
    mpz_fdiv_q_2exp(y, y, 1);
    if (mpz_cmp(y, x) >= 0) break;
    mpz_set(x, y);
  }
  mpz_set(r, x);
  mpz_clears(x, y, t, NULL);
}

int mpz_invert(mpz_ptr r, mpz_srcptr a, mpz_srcptr m) {
  /* extended Euclid on (a mod m, m) */
  mpz_t r0, r1, s0, s1, q, t, t2;
  mpz_inits(r0, r1, s0, s1, q, t, t2, NULL);
  mpz_set(r0, m);
  if (r0->_mp_size < 0) r0->_mp_size = -r0->_mp_size;
  mpz_fdiv_r(r1, a, r0);
  mpz_set_ui(s0, 0);
  mpz_set_ui(s1, 1);
  while (r1->_mp_size != 0) {
    Fdiv_qr(q, t, r0, r1);
    mpz_set(r0, r1);
    mpz_set(r1, t);
    mpz_mul(t2, q, s1);
    mpz_sub(t, s0, t2);
    mpz_set(s0, s1);
    mpz_set(s1, t);
  }
  int ok = (r0->_mp_size == 1 && r0->_mp_d[0] == 1);
  if (ok) {
    mpz_set(t, m);
    if (t->_mp_size < 0) t->_mp_size = -t->_mp_size;
    mpz_fdiv_r(r, s0, t);
  }
  mpz_clears(r0, r1, s0, s1, q, t, t2, NULL);
  return ok;
}

int mpz_cmp(mpz_srcptr a, mpz_srcptr b) {
  int an = a->_mp_size < 0, bn = b->_mp_size < 0;
  if (an != bn) return an ? -1 : 1;
  int c = Cmp_mag(a->_mp_d, ABS(a->_mp_size), b->_mp_d, ABS(b->_mp_size));
  return an ? -c : c;
}

int mpz_cmp_si(mpz_srcptr a, long b) {
  mpz_t t;
  mpz_init_set_si(t, b);
  int c = mpz_cmp(a, t);
  mpz_clear(t);
  return c;
}

unsigned long mpz_get_ui(mpz_srcptr a) {
  int      n = ABS(a->_mp_size);
  uint64_t v = 0;
  if (n > 0) v = a->_mp_d[0];
  if (n > 1) v |= (uint64_t)a->_mp_d[1] << 32;
  return v;
}

long mpz_get_si(mpz_srcptr a) {
  uint64_t v = mpz_get_ui(a);
  if (a->_mp_size < 0) return (long)(0UL - v);
  return (long)(v & 0x7fffffffffffffffULL);
}

int mpz_fits_slong_p(mpz_srcptr a) {
  int n = ABS(a->_mp_size);
  if (n > 2) return 0;
  uint64_t v = mpz_get_ui(a);
  if (a->_mp_size < 0) return v <= 0x8000000000000000ULL;
  return v <= 0x7fffffffffffffffULL;
}

size_t mpz_sizeinbase(mpz_srcptr a, int base) {
  int n = ABS(a->_mp_size);
  if (n == 0) return 1;
  size_t bits = (size_t)(n - 1) * 32 + (32 - (size_t)__builtin_clz(a->_mp_d[n - 1]));
  if (base == 2) return bits;
  /* may overestimate by one, as the real function is allowed to */
  return (size_t)((double)bits * log(2.0) / log((double)base)) + 1;
}

/* top 64 bits of |a| (truncated), and the exponent e with |a| ~ top * 2^e */
static uint64_t Top64(mpz_srcptr a, long* e) {
  int    n    = ABS(a->_mp_size);
  size_t bits = mpz_sizeinbase(a, 2);
  if (bits <= 64) {
    *e = 0;
    return mpz_get_ui(a);
  }
  size_t   shift = bits - 64;
  int      ws = (int)(shift / 32), bs = (int)(shift % 32);
  uint64_t lo = a->_mp_d[ws], mid = ws + 1 < n ? a->_mp_d[ws + 1] : 0,
           hi = ws + 2 < n ? a->_mp_d[ws + 2] : 0;
  unsigned __int128 v = ((unsigned __int128)hi << 64) | (mid << 32) | lo;
  *e                  = (long)shift;
  return (uint64_t)(v >> bs);
}

double mpz_get_d(mpz_srcptr a) {
  if (a->_mp_size == 0) return 0.0;
  long     e;
  uint64_t top = Top64(a, &e);
  /* truncate toward zero to 53 significant bits */
  int lz = __builtin_clzll(top);
  if (lz < 11) top &= ~((1ULL << (11 - lz)) - 1);
  double d = ldexp((double)top, (int)e);
  return a->_mp_size < 0 ? -d : d;
}

double mpz_get_d_2exp(signed long* exp, mpz_srcptr a) {
  if (a->_mp_size == 0) {
    *exp = 0;
    return 0.0;
  }
  long     e;
  uint64_t top = Top64(a, &e);
  int      lz  = __builtin_clzll(top);
  if (lz < 11) top &= ~((1ULL << (11 - lz)) - 1);
  int    e2;
  double m = frexp((double)top, &e2);
  *exp     = e + e2;
  return a->_mp_size < 0 ? -m : m;
}

static void Print_dec(FILE* fp, mpz_srcptr a) {
  if (a->_mp_size == 0) {
    fputc('0', fp);
    return;
  }
  mpz_t t;
  mpz_init_set(t, a);
  if (t->_mp_size < 0) {
    fputc('-', fp);
    t->_mp_size = -t->_mp_size;
  }
  size_t cap = (size_t)t->_mp_size * 10 + 2;
  char*  buf = (char*)malloc(cap);
  size_t pos = 0;
  while (t->_mp_size != 0) {
    unsigned long r = mpz_fdiv_q_ui(t, t, 1000000000UL);
    for (int i = 0; i < 9; i++) {
      buf[pos++] = (char)('0' + r % 10);
      r /= 10;
    }
  }
  while (pos > 1 && buf[pos - 1] == '0') pos--;
  while (pos > 0) fputc(buf[--pos], fp);
  free(buf);
  mpz_clear(t);
}

static int Vgmp_fprintf(FILE* fp, const char* fmt, va_list ap) {
  /* handles literal text, %Zd, %ld, %d, %s, %f -- enough for the runtime's
   * diagnostic prints */
  for (const char* p = fmt; *p; p++) {
    if (*p != '%') {
      fputc(*p, fp);
      continue;
    }
    p++;
    if (*p == 'Z' && p[1] == 'd') {
      p++;
      Print_dec(fp, va_arg(ap, mpz_srcptr));
    } else if (*p == 'l' && p[1] == 'd') {
      p++;
      fprintf(fp, "%ld", va_arg(ap, long));
    } else if (*p == 'd') {
      fprintf(fp, "%d", va_arg(ap, int));
    } else if (*p == 's') {
      fputs(va_arg(ap, const char*), fp);
    } else if (*p == 'f') {
      fprintf(fp, "%f", va_arg(ap, double));
    } else if (*p == '%') {
      fputc('%', fp);
    } else {
      fputc('%', fp);
      fputc(*p, fp);
    }
  }
  return 0;
}

int gmp_fprintf(FILE* fp, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  int r = Vgmp_fprintf(fp, fmt, ap);
  va_end(ap);
  return r;
}

int gmp_printf(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  int r = Vgmp_fprintf(stdout, fmt, ap);
  va_end(ap);
  return r;
}
