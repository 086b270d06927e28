// Device code of the negacyclic NTT / inverse NTT (kernels and butterflies).
//
// Dataflow and twiddle indexing follow the CPU runtime exactly
// (fhe-cmplr/rtlib/ant/util/src/ntt.c:167-241 forward, 245-330 inverse):
// forward = Cooley-Tukey, natural order in, bit-reversed order out, stage
// m = 1, 2, .., N/2 uses twiddle table entry m + i for butterfly group i;
// inverse = Gentleman-Sande in the opposite order with N^-1 applied.  Residues
// written by the last pass are canonical, which makes them equal to the CPU
// runtime's.
//
// What bounds these kernels is the half-rate 32-bit multiplier pipe: every
// 32x32 multiply-add occupies it for two cycles per warp, 64-bit additions
// and compares run on the full-rate integer pipe beside it.  The butterflies
// are therefore written to need as few multiplies as possible:
//   * the Shoup quotient floor(b*w'/2^64) is taken from three partial
//     products instead of the exact four-product-and-carry sequence
//     (it may come out up to 2 too small, the product then lies in [0, 4q));
//   * b*w - quotient*q is one accumulation chain against -q (two wide and
//     four low multiply-adds, no separate subtraction);
//   * primes with enough headroom below 2^64 skip the per-butterfly range
//     correction altogether: forward values grow by 4q per stage (at most
//     (1 + 4 logN) q), inverse values double per stage (at most 2^(logN+1) q),
//     and one reduction at the very end makes them canonical.  Wider primes
//     keep a Harvey-style conditional subtraction with the range [0, 8q)
//     forward and [0, 4q) inverse.
//
// Three kernels per direction:
//   small    N <= 4096: one CTA per limb, whole limb in shared memory.
//   strided  first logN-8 stages: a CTA owns TC adjacent columns of the
//            (N/256) x 256 view of the limb; every thread keeps 8 rows in
//            registers and does up to three stages between exchanges.
//   contig   last 8 stages: a warp owns one contiguous 256-word block.
// The inverse runs contig first, then strided.  Between the two passes the
// values stay lazy (not canonical).
#pragma once
#include "runtime.h"

namespace fhert {
namespace nttk {

typedef unsigned int u32;

constexpr int kContigLog   = 8;    // stages handled by the contiguous kernel
constexpr int kContigBlock = 256;
constexpr int kWarpsPerCta = 4;    // contiguous kernel: independent warps per CTA

__device__ __forceinline__ u32 lo32(u64 x) { return (u32)x; }
__device__ __forceinline__ u32 hi32(u64 x) { return (u32)(x >> 32); }
__device__ __forceinline__ u64 pack64(u32 l, u32 h) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(l), "r"(h));
  return r;
}

// Per-limb constants kept in registers.
struct Mod {
  u64 q, nq, q2, q4;  // q, 2^64 - q, 2q, 4q
};
__device__ __forceinline__ Mod make_mod(u64 q) {
  Mod m;
  m.q  = q;
  m.nq = 0 - q;
  m.q2 = q << 1;
  m.q4 = q << 2;
  return m;
}

// addend + b*w + h*nq  (mod 2^64): two wide and four low multiply-adds
__device__ __forceinline__ u64 mul_chain(u64 addend, u64 b, u64 w, u64 h, u64 nq) {
  u64 t;
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(t) : "r"(lo32(b)), "r"(lo32(w)), "l"(addend));
  asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(t) : "r"(lo32(h)), "r"(lo32(nq)));
  u32 tl = lo32(t), th = hi32(t);
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(lo32(b)), "r"(hi32(w)));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(hi32(b)), "r"(lo32(w)));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(lo32(h)), "r"(hi32(nq)));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(hi32(h)), "r"(lo32(nq)));
  return pack64(tl, th);
}

// b*w mod q for any 64-bit b, result in [0, 4q)
__device__ __forceinline__ u64 shoup4(u64 b, const Twiddle t, const Mod m) {
  return mul_chain(0, b, t.w, mulhi_under(b, t.wp), m.nq);
}

__device__ __forceinline__ u64 csub(u64 v, u64 bound) { return v >= bound ? v - bound : v; }

// [0, 4q) -> [0, q)
__device__ __forceinline__ u64 canon_4q(u64 v, const Mod m) { return csub(csub(v, m.q2), m.q); }

// any 64-bit v -> [0, q); r = floor(2^64 / q)
__device__ __forceinline__ u64 canon_any(u64 v, const Mod m, u64 r) {
  u64 e = mulhi_under(v, r);  // floor(v/q) - {0..3}
  u64 t;
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(t) : "r"(lo32(e)), "r"(lo32(m.nq)), "l"(v));
  u32 th = hi32(t);
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(lo32(e)), "r"(hi32(m.nq)));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(hi32(e)), "r"(lo32(m.nq)));
  return canon_4q(pack64(lo32(t), th), m);
}

// Work fused into a forward transform (all optional).
//
// Prologue of the strided pass, the lift of a rescale (rns_poly.c:351-366): the
// source limb holds residues modulo q_last in coefficient form; the value that
// enters the transform under prime i is
//   switch_modulus(v, q_last -> q_i) * mul[i].
struct NttPro {
  const Twiddle* mul = nullptr;  // [prime]; nullptr = no prologue
  const u64*     mod = nullptr;  // [prime] q_last mod q_i
  u64            q_last = 0;
};
// Epilogue of the contiguous pass on the canonical transform output t:
//   kind 1 (rescale, rns_poly.c:367-383):  res = aux * mul[i] + t
//   kind 2 (ModDown, rns_poly.c:293-304):  res = (aux - t) * mul[i] (+ add)
// aux is limb LimbRef::b of aux.p[sel bit 1]; add uses the same limb index and
// selector, a null base means no addend.
struct NttEpi {
  int            kind = 0;
  const Twiddle* mul  = nullptr;  // [prime]
  Ptr2           aux{{nullptr, nullptr}};
  Ptr2           add{{nullptr, nullptr}};
};

__device__ __forceinline__ u64 add_canon(u64 a, u64 b, u64 q) { return csub(a + b, q); }

// Cooley-Tukey.  WIDE: a, b in [0, 8q) -> [0, 8q).  Otherwise no correction:
// the bound of both values grows by 4q.
template <bool WIDE>
__device__ __forceinline__ void ct_bfly(u64& a, u64& b, const Twiddle t, const Mod m) {
  u64 x = WIDE ? csub(a, m.q4) : a;
  u64 v = shoup4(b, t, m);
  a     = x + v;
  b     = x - v + m.q4;
}

// Gentleman-Sande.  WIDE: a, b in [0, 4q) -> [0, 4q), mq = 4q.  Otherwise no
// correction: mq is a multiple of q not below the bound of b, the sum doubles.
template <bool WIDE>
__device__ __forceinline__ void gs_bfly(u64& a, u64& b, const Twiddle t, const Mod m, u64 mq) {
  u64 s = a + b;
  u64 d = a - b + mq;
  a     = WIDE ? csub(s, m.q4) : s;
  b     = shoup4(d, t, m);
}

__device__ __forceinline__ Twiddle ld_tw(const Twiddle* p) {
  ulonglong2 v = __ldg(reinterpret_cast<const ulonglong2*>(p));
  Twiddle    t;
  t.w  = v.x;
  t.wp = v.y;
  return t;
}

// Where a round takes its twiddles from.  get<L>(jb, hp) returns the twiddle of
// local stage L with index jb + hp inside the stage (jb is the part that
// depends on the thread, hp the unrolled butterfly-group number).
struct TwGlobal {
  const Twiddle* tw;   // the prime's table
  uint32_t       node; // (1 << s0) + blk: the transform's node in the table's tree order
  template <int L>
  __device__ __forceinline__ Twiddle get(uint32_t jb, int hp) const {
    return ld_tw(tw + ((size_t)node << L) + jb + hp);
  }
};
// Multiple of q covering the inputs of inverse stage k (1 = first stage done,
// inputs canonical): bound of the values after k-1 uncorrected stages is
// 2^k q for k >= 2 and q for k = 1.
__device__ __forceinline__ u64 inv_cover(const Mod m, int k) { return k <= 1 ? m.q : m.q << k; }

// One register round of R consecutive forward stages starting at local stage
// L0 of a 2^S-point transform.  The thread holds the 8 elements
// base | (e << LOWPOS), e = 0..7, with LOWPOS = S - L0 - R.  The twiddle of
// local stage l for element index idx is entry idx >> (S - l) of that stage
// (table entry (1 << (s0 + l)) + (blk << l) + (idx >> (S - l))).
template <bool WIDE, int R, int S, int L0, typename TW, int U = 0>
__device__ __forceinline__ void fwd_round(u64 (&x)[8], int base, const TW tws, const Mod m) {
  if constexpr (U < R) {
    constexpr int  bit = R - 1 - U;
    constexpr int  l   = L0 + U;
    // the register field starts at bit S - L0 - R, so the element offset
    // (hp << (bit+1)) shifted there and then right by S - l is hp itself
    const uint32_t jb  = (uint32_t)base >> (S - l);
#pragma unroll
    for (int hp = 0; hp < (8 >> (bit + 1)); hp++) {
      Twiddle t = tws.template get<l>(jb, hp);
#pragma unroll
      for (int lp = 0; lp < (1 << bit); lp++) {
        int lo = (hp << (bit + 1)) | lp;
        ct_bfly<WIDE>(x[lo], x[lo | (1 << bit)], t, m);
      }
    }
    fwd_round<WIDE, R, S, L0, TW, U + 1>(x, base, tws, m);
  }
}

// Inverse round: same stages, processed from the highest local stage down.
// KBASE - l is the 1-based count of the inverse stage (for the cover of the
// uncorrected form).  When LAST is set and the round reaches local stage 0,
// the final butterfly applies N^-1 (fin[0] = N^-1, fin[1] = rou_inv[1]*N^-1)
// and leaves canonical values.
template <bool WIDE, int R, int S, int L0, int KBASE, bool LAST, typename TW, int U = R - 1>
__device__ __forceinline__ void inv_round(u64 (&x)[8], int base, const TW tws, const Mod m,
                                          const Twiddle* fin) {
  if constexpr (U >= 0) {
    constexpr int bit = R - 1 - U;
    constexpr int l   = L0 + U;
    const u64     mq  = WIDE ? m.q4 : inv_cover(m, KBASE - l);
    if constexpr (LAST && l == 0) {
      Twiddle n_inv = ld_tw(fin), w_n = ld_tw(fin + 1);
#pragma unroll
      for (int hp = 0; hp < (8 >> (bit + 1)); hp++) {
#pragma unroll
        for (int lp = 0; lp < (1 << bit); lp++) {
          int lo = (hp << (bit + 1)) | lp;
          int hi = lo | (1 << bit);
          u64 sum = x[lo] + x[hi];
          u64 dif = x[lo] - x[hi] + mq;
          x[lo]   = canon_4q(shoup4(sum, n_inv, m), m);
          x[hi]   = canon_4q(shoup4(dif, w_n, m), m);
        }
      }
    } else {
      const uint32_t jb = (uint32_t)base >> (S - l);
#pragma unroll
      for (int hp = 0; hp < (8 >> (bit + 1)); hp++) {
        Twiddle t = tws.template get<l>(jb, hp);
#pragma unroll
        for (int lp = 0; lp < (1 << bit); lp++) {
          int lo = (hp << (bit + 1)) | lp;
          gs_bfly<WIDE>(x[lo], x[lo | (1 << bit)], t, m, mq);
        }
      }
    }
    inv_round<WIDE, R, S, L0, KBASE, LAST, TW, U - 1>(x, base, tws, m, fin);
  }
}

// Bank swizzle for a 256-word block accessed with the three lane patterns of
// the contiguous kernel (lanes over index bits {0..4}, {0,1,5,6,7}, {3..7}):
// a permutation inside each aligned 16-word group that keeps every half-warp
// on 16 distinct 8-byte banks.  It is linear over XOR, so for an index made of
// disjoint bit fields swz(a | b) = swz(a) ^ swz(b): the per-element part is a
// compile-time constant.
__host__ __device__ constexpr int swz(int i) {
  return i ^ (((i >> 4) & 1) << 1) ^ (((i >> 5) & 1) << 2) ^ (((i >> 6) & 1) << 3) ^ ((i >> 6) & 1);
}

__device__ __forceinline__ u64 lds64(u32 addr) {
  u64 v;
  asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts64(u32 addr, u64 v) {
  asm volatile("st.shared.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}

// ---- contiguous 256-point blocks (global stages logN-8 .. logN-1) ----------
//
// One warp per block; the warp's 2 KiB of shared memory is aligned to its size
// so that the swizzled byte address is (block base ^ swizzled offset).

template <bool INV, bool WIDE, int EPI>
__device__ __forceinline__ void contig_block(const u64* __restrict__ src, u64* __restrict__ dst,
                                             u32 sbase, const TwGlobal tw, const Mod m, u64 rq,
                                             int g, const u64* aux, const u64* add,
                                             const Twiddle emul) {
  u64 x[8];
  // byte addresses inside the warp's block for the three lane patterns
  const int b1 = g;                              // elements e*32 + g
  const int b2 = ((g >> 2) << 5) | (g & 3);      // elements b2 | e<<2
  const int b3 = g << 3;                         // elements g*8 + e
  const u32 a1 = sbase ^ (u32)(swz(b1) << 3);
  const u32 a2 = sbase ^ (u32)(swz(b2) << 3);
  const u32 a3 = sbase ^ (u32)(swz(b3) << 3);
  if constexpr (!INV) {
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = src[e * 32 + g];
    fwd_round<WIDE, 3, kContigLog, 0>(x, b1, tw, m);
#pragma unroll
    for (int e = 0; e < 8; e++) sts64(a1 ^ (u32)(swz(e << 5) << 3), x[e]);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = lds64(a2 ^ (u32)(swz(e << 2) << 3));
    fwd_round<WIDE, 3, kContigLog, 3>(x, b2, tw, m);
#pragma unroll
    for (int e = 0; e < 8; e++) sts64(a2 ^ (u32)(swz(e << 2) << 3), x[e]);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = lds64(a3 ^ (u32)(swz(e) << 3));
    fwd_round<WIDE, 2, kContigLog, 6>(x, b3, tw, m);
#pragma unroll
    for (int e = 0; e < 8; e++) {
      u64 v = WIDE ? canon_4q(csub(x[e], m.q4), m) : canon_any(x[e], m, rq);
      sts64(a3 ^ (u32)(swz(e) << 3), v);
    }
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) {
      u64 t = lds64(a1 ^ (u32)(swz(e << 5) << 3));
      if (EPI == 1) {
        t = add_canon(canon_4q(shoup4(aux[e * 32 + g], emul, m), m), t, m.q);
      } else if (EPI == 2) {
        u64 x = aux[e * 32 + g];
        t     = canon_4q(shoup4(x >= t ? x - t : x + m.q - t, emul, m), m);
        if (add != nullptr) t = add_canon(t, add[e * 32 + g], m.q);
      }
      dst[e * 32 + g] = t;
    }
  } else {
    // inverse stage counts 1..8 are local stages 7..0: KBASE = 8
#pragma unroll
    for (int e = 0; e < 8; e++) sts64(a1 ^ (u32)(swz(e << 5) << 3), src[e * 32 + g]);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = lds64(a3 ^ (u32)(swz(e) << 3));
    inv_round<WIDE, 2, kContigLog, 6, 8, false>(x, b3, tw, m, nullptr);
#pragma unroll
    for (int e = 0; e < 8; e++) sts64(a3 ^ (u32)(swz(e) << 3), x[e]);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = lds64(a2 ^ (u32)(swz(e << 2) << 3));
    inv_round<WIDE, 3, kContigLog, 3, 8, false>(x, b2, tw, m, nullptr);
#pragma unroll
    for (int e = 0; e < 8; e++) sts64(a2 ^ (u32)(swz(e << 2) << 3), x[e]);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = lds64(a1 ^ (u32)(swz(e << 5) << 3));
    inv_round<WIDE, 3, kContigLog, 0, 8, false>(x, b1, tw, m, nullptr);
#pragma unroll
    for (int e = 0; e < 8; e++) dst[e * 32 + g] = x[e];
  }
}

// narrow = no range correction is needed over the whole transform
__device__ __forceinline__ bool fwd_narrow(uint32_t bits) { return bits <= 57; }
__device__ __forceinline__ bool inv_narrow(uint32_t bits, int logn) { return bits + logn + 1 <= 64; }

template <bool INV, int EPI>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
ntt_contig_kernel(Ptr2 in, Ptr2 out, LimbBatch batch, const Twiddle* __restrict__ tables,
                  const DevModulus* __restrict__ mods, uint32_t n, int logn, NttEpi epi) {
  __shared__ __align__(2048) u64 sm[kWarpsPerCta * kContigBlock];
  const LimbRef    lr   = batch.limb[blockIdx.y];
  const DevModulus dm   = mods[lr.prime];
  const Mod        m    = make_mod(dm.q);
  const Twiddle*   tw   = tables + (size_t)lr.prime * n;
  const int        warp = threadIdx.x >> 5;
  const int        g    = threadIdx.x & 31;
  const uint32_t   blk  = blockIdx.x * kWarpsPerCta + warp;  // block in limb
  const size_t     off  = (size_t)blk * kContigBlock;
  const u64*       src  = ((lr.sel & 1) ? in.p[1] : in.p[0]) + (size_t)lr.a * n + off;
  u64*             dst  = ((lr.sel & 4) ? out.p[1] : out.p[0]) + (size_t)lr.dst * n + off;
  const u32 sbase = (u32)__cvta_generic_to_shared(sm) + (u32)warp * (kContigBlock * 8);
  const int s0    = logn - kContigLog;

  const bool narrow = INV ? inv_narrow(dm.bits, logn) : fwd_narrow(dm.bits);
  const u64* aux  = nullptr;
  const u64* add  = nullptr;
  Twiddle    emul{0, 0};
  if (EPI != 0) {
    const size_t aoff = (size_t)lr.b * n + off;
    aux  = ((lr.sel & 2) ? epi.aux.p[1] : epi.aux.p[0]) + aoff;
    add  = (lr.sel & 2) ? epi.add.p[1] : epi.add.p[0];
    if (add != nullptr) add += aoff;
    emul = ld_tw(epi.mul + lr.prime);
  }
  const TwGlobal tws{tw, (1u << s0) + blk};
  if (narrow)
    contig_block<INV, false, EPI>(src, dst, sbase, tws, m, dm.mu_hi, g, aux, add, emul);
  else
    contig_block<INV, true, EPI>(src, dst, sbase, tws, m, dm.mu_hi, g, aux, add, emul);
}

// ---- strided columns (global stages 0 .. logN-9) ---------------------------
//
// S1 = logN - 8 stages on 2^S1 rows; TC columns per CTA; threads = TC * 2^(S1-3).
// Rounds cover local stages [l0, l0+R): forward ascending from 0 with R = 3
// while three are left, inverse descending with the odd-sized round first.

// the lift of a rescale: residue modulo q_last (centred) -> residue modulo q, times w
__device__ __forceinline__ u64 lift_value(u64 v, u64 q_last, u64 last_mod_q, const Twiddle w,
                                          const Mod m, u64 rq) {
  u64 r = canon_any(v, m, rq);
  if (v > (q_last >> 1)) r = r >= last_mod_q ? r - last_mod_q : r + m.q - last_mod_q;
  return canon_4q(shoup4(r, w, m), m);
}

struct LiftArgs {
  bool    on;
  u64     q_last, last_mod_q, rq;
  Twiddle w;
};

template <bool WIDE, int S1, int TC, int L0>
__device__ __forceinline__ void strided_fwd(u64 (&x)[8], const u64* __restrict__ src,
                                            u64* __restrict__ dst, u64* sm, int g, int c,
                                            const Twiddle* tw, const Mod m, const LiftArgs lift) {
  constexpr int R      = (S1 - L0 < 3) ? (S1 - L0) : 3;
  constexpr int LOWPOS = S1 - L0 - R;
  const int base = ((g >> LOWPOS) << (LOWPOS + 3)) | (g & ((1 << LOWPOS) - 1));
  if constexpr (L0 == 0) {
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = src[(size_t)(base | (e << LOWPOS)) << kContigLog];
    if (lift.on) {
#pragma unroll
      for (int e = 0; e < 8; e++)
        x[e] = lift_value(x[e], lift.q_last, lift.last_mod_q, lift.w, m, lift.rq);
    }
  } else {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = sm[(base | (e << LOWPOS)) * TC + c];
  }
  fwd_round<WIDE, R, S1, L0>(x, base, TwGlobal{tw, 1u}, m);
  if constexpr (L0 + R < S1) {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; e++) sm[(base | (e << LOWPOS)) * TC + c] = x[e];
    strided_fwd<WIDE, S1, TC, L0 + R>(x, src, dst, sm, g, c, tw, m, lift);
  } else {
#pragma unroll
    for (int e = 0; e < 8; e++) dst[(size_t)(base | (e << LOWPOS)) << kContigLog] = x[e];
  }
}

// HI = stages [0, HI) are still to do; the first call has HI = S1.
template <bool WIDE, int S1, int TC, int HI>
__device__ __forceinline__ void strided_inv(u64 (&x)[8], const u64* __restrict__ src,
                                            u64* __restrict__ dst, u64* sm, int g, int c,
                                            const Twiddle* tw, const Mod m, const Twiddle* fin) {
  constexpr int R      = (HI % 3 == 0) ? 3 : HI % 3;
  constexpr int L0     = HI - R;
  constexpr int LOWPOS = S1 - L0 - R;
  const int base = ((g >> LOWPOS) << (LOWPOS + 3)) | (g & ((1 << LOWPOS) - 1));
  if constexpr (HI == S1) {
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = src[(size_t)(base | (e << LOWPOS)) << kContigLog];
  } else {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = sm[(base | (e << LOWPOS)) * TC + c];
  }
  // inverse stage count of local stage l: 8 contiguous stages came first
  inv_round<WIDE, R, S1, L0, kContigLog + S1, true>(x, base, TwGlobal{tw, 1u}, m, fin);
  if constexpr (L0 > 0) {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; e++) sm[(base | (e << LOWPOS)) * TC + c] = x[e];
    strided_inv<WIDE, S1, TC, L0>(x, src, dst, sm, g, c, tw, m, fin);
  } else {
#pragma unroll
    for (int e = 0; e < 8; e++) dst[(size_t)(base | (e << LOWPOS)) << kContigLog] = x[e];
  }
}

template <bool INV, int S1, int TC>
__global__ void __launch_bounds__(TC << (S1 - 3))
ntt_strided_kernel(Ptr2 in, Ptr2 out, LimbBatch batch, const Twiddle* __restrict__ tables,
                   const DevModulus* __restrict__ mods, const Twiddle* __restrict__ inv_last,
                   uint32_t n, NttPro pro) {
  extern __shared__ u64 sm_dyn[];
  constexpr int    logn = S1 + kContigLog;
  const LimbRef    lr   = batch.limb[blockIdx.y];
  const DevModulus dm   = mods[lr.prime];
  const Mod        m    = make_mod(dm.q);
  const Twiddle*   tw   = tables + (size_t)lr.prime * n;
  const Twiddle*   fin  = inv_last + (size_t)lr.prime * 2;
  const int        c    = threadIdx.x & (TC - 1);
  const int        g    = threadIdx.x / TC;  // 0 .. 2^(S1-3)-1
  const size_t     col  = (size_t)blockIdx.x * TC + c;
  const u64*       src  = ((lr.sel & 1) ? in.p[1] : in.p[0]) + (size_t)lr.a * n + col;
  u64*             dst  = ((lr.sel & 4) ? out.p[1] : out.p[0]) + (size_t)lr.dst * n + col;
  u64              x[8];
  const bool narrow = INV ? inv_narrow(dm.bits, logn) : fwd_narrow(dm.bits);
  if constexpr (!INV) {
    LiftArgs lift{false, 0, 0, 0, Twiddle{0, 0}};
    if (pro.mul != nullptr) {
      lift.on         = true;
      lift.q_last     = pro.q_last;
      lift.last_mod_q = pro.mod[lr.prime];
      lift.rq         = dm.mu_hi;
      lift.w          = ld_tw(pro.mul + lr.prime);
    }
    if (narrow)
      strided_fwd<false, S1, TC, 0>(x, src, dst, sm_dyn, g, c, tw, m, lift);
    else
      strided_fwd<true, S1, TC, 0>(x, src, dst, sm_dyn, g, c, tw, m, lift);
  } else {
    if (narrow)
      strided_inv<false, S1, TC, S1>(x, src, dst, sm_dyn, g, c, tw, m, fin);
    else
      strided_inv<true, S1, TC, S1>(x, src, dst, sm_dyn, g, c, tw, m, fin);
  }
}

// ---- small transforms: whole limb in shared memory -------------------------
// Always the corrected (wide) butterflies: valid for every prime below 2^61.

template <bool INV>
__global__ void ntt_small_kernel(Ptr2 in, Ptr2 out, LimbBatch batch,
                                 const Twiddle* __restrict__ tables,
                                 const DevModulus* __restrict__ mods,
                                 const Twiddle* __restrict__ inv_last, uint32_t n, int logn) {
  extern __shared__ u64 sm_dyn[];
  const LimbRef  lr  = batch.limb[blockIdx.x];
  const Mod      m   = make_mod(mods[lr.prime].q);
  const Twiddle* tw  = tables + (size_t)lr.prime * n;
  const Twiddle* fin = inv_last + (size_t)lr.prime * 2;
  const u64*     src = ((lr.sel & 1) ? in.p[1] : in.p[0]) + (size_t)lr.a * n;
  u64*           dst = ((lr.sel & 4) ? out.p[1] : out.p[0]) + (size_t)lr.dst * n;
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) sm_dyn[i] = src[i];
  __syncthreads();
  const uint32_t half = n >> 1;
  if (!INV) {
    for (int l = 0; l < logn; l++) {
      int tlog = logn - 1 - l;  // t = 2^tlog
      for (uint32_t bf = threadIdx.x; bf < half; bf += blockDim.x) {
        uint32_t i  = bf >> tlog;
        uint32_t j1 = ((i << (tlog + 1))) | (bf & ((1u << tlog) - 1));
        Twiddle  t  = ld_tw(tw + (1u << l) + i);
        u64 a = sm_dyn[j1], b = sm_dyn[j1 + (1u << tlog)];
        ct_bfly<true>(a, b, t, m);
        sm_dyn[j1]                 = a;
        sm_dyn[j1 + (1u << tlog)] = b;
      }
      __syncthreads();
    }
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x)
      dst[i] = canon_4q(csub(sm_dyn[i], m.q4), m);
  } else {
    for (int l = logn - 1; l >= 0; l--) {
      int tlog = logn - 1 - l;
      for (uint32_t bf = threadIdx.x; bf < half; bf += blockDim.x) {
        uint32_t i  = bf >> tlog;
        uint32_t j1 = ((i << (tlog + 1))) | (bf & ((1u << tlog) - 1));
        u64 a = sm_dyn[j1], b = sm_dyn[j1 + (1u << tlog)];
        if (l == 0) {
          Twiddle n_inv = ld_tw(fin), w_n = ld_tw(fin + 1);
          u64     sum = a + b, dif = a - b + m.q4;
          a = canon_4q(shoup4(sum, n_inv, m), m);
          b = canon_4q(shoup4(dif, w_n, m), m);
        } else {
          Twiddle t = ld_tw(tw + (1u << l) + i);
          gs_bfly<true>(a, b, t, m, m.q4);
        }
        sm_dyn[j1]                 = a;
        sm_dyn[j1 + (1u << tlog)] = b;
      }
      __syncthreads();
    }
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = sm_dyn[i];
  }
}

constexpr int kSmallMaxLog = 12;

// Tables and geometry of one transform launch.
struct NttTables {
  const Twiddle*    fwd;
  const Twiddle*    inv;
  const Twiddle*    inv_last;
  const DevModulus* mods;
  uint32_t          n;
  int               logn;
};

template <bool INV, int S1, int TC>
inline void launch_strided_t(Ptr2 in, Ptr2 out, const LimbBatch& b, const NttTables& t,
                             cudaStream_t stream, const NttPro& pro) {
  static bool attr_done = false;
  const size_t smem = ((size_t)TC << S1) * sizeof(u64);
  if (!attr_done && smem > 48 * 1024) {
    cudaFuncSetAttribute(ntt_strided_kernel<INV, S1, TC>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_done = true;
  }
  dim3 grid(kContigBlock / TC, b.count);
  ntt_strided_kernel<INV, S1, TC><<<grid, TC << (S1 - 3), smem, stream>>>(
      in, out, b, INV ? t.inv : t.fwd, t.mods, t.inv_last, t.n, pro);
}

template <bool INV, int TC>
inline void launch_strided(Ptr2 in, Ptr2 out, const LimbBatch& b, const NttTables& t,
                           cudaStream_t stream, const NttPro& pro = NttPro()) {
  switch (t.logn - kContigLog) {
    case 5: launch_strided_t<INV, 5, TC>(in, out, b, t, stream, pro); break;
    case 6: launch_strided_t<INV, 6, TC>(in, out, b, t, stream, pro); break;
    case 7: launch_strided_t<INV, 7, TC>(in, out, b, t, stream, pro); break;
    case 8: launch_strided_t<INV, 8, TC>(in, out, b, t, stream, pro); break;
    case 9: launch_strided_t<INV, 9, TC>(in, out, b, t, stream, pro); break;
    default: FHERT_ASSERT(false, "ring degree 2^%d has no transform kernel", t.logn);
  }
}

template <bool INV>
inline void launch_contig(Ptr2 in, Ptr2 out, const LimbBatch& b, const NttTables& t,
                          cudaStream_t stream, const NttEpi& epi = NttEpi()) {
  dim3 grid(t.n / (kContigBlock * kWarpsPerCta), b.count);
  const Twiddle* tab = INV ? t.inv : t.fwd;
  if (INV || epi.kind == 0)
    ntt_contig_kernel<INV, 0><<<grid, kWarpsPerCta * 32, 0, stream>>>(in, out, b, tab, t.mods, t.n,
                                                                       t.logn, epi);
  else if (epi.kind == 1)
    ntt_contig_kernel<false, 1><<<grid, kWarpsPerCta * 32, 0, stream>>>(in, out, b, tab, t.mods,
                                                                         t.n, t.logn, epi);
  else
    ntt_contig_kernel<false, 2><<<grid, kWarpsPerCta * 32, 0, stream>>>(in, out, b, tab, t.mods,
                                                                         t.n, t.logn, epi);
}

template <bool INV>
inline void launch_small(Ptr2 in, Ptr2 out, const LimbBatch& b, const NttTables& t,
                         cudaStream_t stream) {
  size_t smem    = (size_t)t.n * sizeof(u64);
  int    threads = t.n / 2 < 512 ? (t.n / 2 < 32 ? 32 : t.n / 2) : 512;
  ntt_small_kernel<INV><<<b.count, threads, smem, stream>>>(in, out, b, INV ? t.inv : t.fwd,
                                                             t.mods, t.inv_last, t.n, t.logn);
}

}  // namespace nttk
}  // namespace fhert
