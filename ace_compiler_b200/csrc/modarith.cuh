// 64-bit modular arithmetic for RNS limbs, device side.
//
// All moduli are NTT-friendly primes below 2^64 / 9 (60-bit primes and a little
// above), so that the lazy forms used here (up to 8q in the butterflies, up to
// 9q before the last correction of a 128-bit reduction) fit a 64-bit word.
// Residues that leave a kernel are always canonical, in [0, q): that is the
// only property the CPU runtime's results depend on
// (fhe-cmplr/rtlib/ant/include/util/modular.h:126-256 reduces after every
// operation), so any reduction that yields the canonical representative of the
// same integer reproduces it bit for bit.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace fhert {

typedef unsigned long long u64;

// Per-prime constants kept in device memory (one entry per Q or P prime).
struct DevModulus {
  u64      q;        // modulus
  u64      mu_hi;    // floor(2^128 / q), high and low words
  u64      mu_lo;
  u64      bar;      // floor(2^(bits-1+64) / q), single-word Barrett constant
  uint32_t bits;     // bit length of q
  uint32_t pad;
  u64      n_inv;    // N^-1 mod q and its Shoup companion
  u64      n_inv_p;
};

__device__ __forceinline__ u64 add_mod(u64 a, u64 b, u64 q) {
  u64 s = a + b;
  return s >= q ? s - q : s;
}

__device__ __forceinline__ u64 sub_mod(u64 a, u64 b, u64 q) {
  return a >= b ? a - b : a + q - b;
}

// Shoup multiplication by a constant w with companion wp = floor(w*2^64/q).
// Valid for any 64-bit a; result in [0, 2q).
__device__ __forceinline__ u64 mul_shoup_lazy(u64 a, u64 w, u64 wp, u64 q) {
  u64 hi = __umul64hi(a, wp);
  return a * w - hi * q;
}

// As above, result canonical in [0, q)  (modular.h:249-256).
__device__ __forceinline__ u64 mul_shoup(u64 a, u64 w, u64 wp, u64 q) {
  u64 r = mul_shoup_lazy(a, w, wp, q);
  return r >= q ? r - q : r;
}

// Exact 128-bit product of a, b < 2^61 from four 32x32 multiplies: with the high
// halves below 2^29 the two middle products sum without overflow, so the only
// carry is the one out of the low word.
__device__ __forceinline__ void mul_wide_128(u64 a, u64 b, u64& hi, u64& lo) {
  uint32_t a0 = (uint32_t)a, a1 = (uint32_t)(a >> 32), b0 = (uint32_t)b, b1 = (uint32_t)(b >> 32);
  u64      t, mid, top;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(t) : "r"(a0), "r"(b0));
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(mid) : "r"(a1), "r"(b0));
  asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(mid) : "r"(a0), "r"(b1));
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(top) : "r"(a1), "r"(b1));
  lo = t + (mid << 32);
  hi = top + (mid >> 32) + (lo < t);
}

// floor(a*b / 2^64) or up to 2 less, from three 32x32 products: the exact
// 64x64 high product costs the half-rate multiplier pipe about 16 cycles per
// warp, this one 6.
__device__ __forceinline__ u64 mulhi_under(u64 a, u64 b) {
  uint32_t a0 = (uint32_t)a, a1 = (uint32_t)(a >> 32), b0 = (uint32_t)b, b1 = (uint32_t)(b >> 32);
  uint32_t m1 = __umulhi(a1, b0), m2 = __umulhi(a0, b1);
  u64      t;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(t) : "r"(a1), "r"(b1));
  return t + m1 + m2;
}

// Canonical a*b mod q for a, b < 2^61 (product below 2^122).  Single-word
// Barrett: the quotient estimate is taken from the product shifted right by
// bits-1, multiplied by bar = floor(2^(bits-1+64)/q); with the three-product
// high multiply it undershoots the true quotient by at most 4.
__device__ __forceinline__ u64 mul_mod(u64 a, u64 b, const DevModulus& m) {
  u64 hi, lo;
  mul_wide_128(a, b, hi, lo);
  uint32_t s  = m.bits - 1;
  u64      x1 = (hi << (64 - s)) | (lo >> s);
  u64      qh = mulhi_under(x1, m.bar);
  u64      r  = lo - qh * m.q;
  if (r >= 4 * m.q) r -= 4 * m.q;
  if (r >= 2 * m.q) r -= 2 * m.q;
  if (r >= m.q) r -= m.q;
  return r;
}

// Canonical reduction of a 128-bit value (hi:lo) < 2^127 with the two-word
// constant mu = floor(2^128/q)  (modular.h:185-224 does the same job).  The
// quotient estimate drops the low partial products and takes the two high
// products from three 32-bit multiplies each: it undershoots by at most 7, so
// the remainder lies in [0, 9q), and 9q < 2^64 for every prime below 2^60.8.
__device__ __forceinline__ u64 reduce_128(u64 hi, u64 lo, const DevModulus& m) {
  u64 qh = hi * m.mu_hi + mulhi_under(hi, m.mu_lo) + mulhi_under(lo, m.mu_hi);
  u64 r  = lo - qh * m.q;
  if (r >= 8 * m.q) r -= 8 * m.q;
  if (r >= 4 * m.q) r -= 4 * m.q;
  if (r >= 2 * m.q) r -= 2 * m.q;
  if (r >= m.q) r -= m.q;
  return r;
}

// acc(hi:lo) += a*b
__device__ __forceinline__ void mac_128(u64& hi, u64& lo, u64 a, u64 b) {
  u64 ph, pl;
  mul_wide_128(a, b, ph, pl);
  lo += pl;
  hi += ph + (lo < pl);
}

// Lazy 64x64 multiply-accumulate on 30-bit halves, for operands below 2^60.
// With a = a1*2^30 + a0 and b = b1*2^30 + b0 (all halves below 2^30) the four
// partial products are below 2^60 and are summed in four separate 64-bit
// accumulators, one IMAD.WIDE each and no carry handling:
//   s00 += a0*b0, s01 += a0*b1, s10 += a1*b0, s11 += a1*b1.
// Up to 16 terms fit.  acc4_fold rebuilds the 128-bit sum
//   hi:lo = s11*2^60 + (s01 + s10)*2^30 + s00.
struct Acc4 {
  u64 s00, s01, s10, s11;
};

__device__ __forceinline__ void acc4_zero(Acc4& c) { c.s00 = c.s01 = c.s10 = c.s11 = 0; }

// acc += a * b as one 32x32+64 multiply-add
__device__ __forceinline__ void mad_wide(u64& acc, uint32_t a, uint32_t b) {
  asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(acc) : "r"(a), "r"(b));
}

__device__ __forceinline__ void acc4_mac_halves(Acc4& c, uint32_t a0, uint32_t a1, uint32_t b0,
                                                uint32_t b1) {
  mad_wide(c.s00, a0, b0);
  mad_wide(c.s01, a0, b1);
  mad_wide(c.s10, a1, b0);
  mad_wide(c.s11, a1, b1);
}

__device__ __forceinline__ void acc4_mac(Acc4& c, u64 a, u64 b) {
  acc4_mac_halves(c, (uint32_t)a & 0x3fffffffu, (uint32_t)(a >> 30),
                  (uint32_t)b & 0x3fffffffu, (uint32_t)(b >> 30));
}

__device__ __forceinline__ void acc4_add_shifted(u64& hi, u64& lo, u64 v, int sh) {
  u64 t = v << sh;
  lo += t;
  hi += (v >> (64 - sh)) + (lo < t);
}

__device__ __forceinline__ void acc4_fold(const Acc4& c, u64& hi, u64& lo) {
  lo = c.s00;
  hi = 0;
  acc4_add_shifted(hi, lo, c.s01, 30);
  acc4_add_shifted(hi, lo, c.s10, 30);
  acc4_add_shifted(hi, lo, c.s11, 60);
}

// Centred lift of a residue mod q_old into [0, q_new)  (modular.h:296-322):
// values above floor(q_old/2) stand for negative numbers, so the result is
// (v mod q_new) or (v - q_old mod q_new).  old_mod_new = q_old mod q_new.
__device__ __forceinline__ u64 switch_modulus(u64 v, u64 q_old,
                                              const DevModulus& m_new,
                                              u64 old_mod_new) {
  u64 r = reduce_128(0, v, m_new);
  if (v > (q_old >> 1)) r = sub_mod(r, old_mod_new, m_new.q);
  return r;
}

}  // namespace fhert
