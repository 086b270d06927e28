// Element-wise, permutation, rescale, base-conversion and key inner-product
// kernels over limb-major RNS polynomials.  Kernels take a LimbBatch (or a
// compact group descriptor) so that one launch covers all limbs -- and, for a
// ciphertext, both polynomials -- of an operation; the x dimension of the grid
// walks the N coefficients of a limb, the y dimension the limbs.
#include <algorithm>

#include "runtime.h"

namespace fhert {

namespace {

constexpr int kThreads = 256;

inline dim3 grid_for(uint32_t n, int per_thread, int limbs) {
  uint32_t per_block = kThreads * per_thread;
  return dim3((n + per_block - 1) / per_block, limbs);
}

__device__ __forceinline__ const u64* sel_a(const Ptr2& p, const LimbRef& lr, uint32_t n) {
  return p.p[lr.sel & 1] + (size_t)lr.a * n;
}
__device__ __forceinline__ const u64* sel_b(const Ptr2& p, const LimbRef& lr, uint32_t n) {
  return p.p[(lr.sel >> 1) & 1] + (size_t)lr.b * n;
}
__device__ __forceinline__ u64* sel_d(const Ptr2& p, const LimbRef& lr, uint32_t n) {
  return p.p[(lr.sel >> 2) & 1] + (size_t)lr.dst * n;
}

// ---- element-wise (hal/src/hal.c:15-121, poly/src/rns_poly.c:852-1054) ------

template <int OP>
__global__ void __launch_bounds__(kThreads)
ew_kernel(Ptr2 res, Ptr2 a, Ptr2 b, u64 scalar, LimbBatch batch,
          const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const u64*       pa = sel_a(a, lr, n);
  const u64*       pb = sel_b(b, lr, n);
  u64*             pr = sel_d(res, lr, n);
  u64              sc = 0;
  if (OP == EW_ADD_SCALAR || OP == EW_MUL_SCALAR || OP == EW_MULADD_SCALAR) {
    // scalars arrive as signed 64-bit values; bring into [0, q)
    int64_t s = (int64_t)scalar % (int64_t)m.q;
    sc        = s < 0 ? (u64)(s + (int64_t)m.q) : (u64)s;
  }
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    u64 x = pa[i], r;
    if (OP == EW_ADD) r = add_mod(x, pb[i], m.q);
    else if (OP == EW_SUB) r = sub_mod(x, pb[i], m.q);
    else if (OP == EW_MUL) r = mul_mod(x, pb[i], m);
    else if (OP == EW_MULADD) r = add_mod(pr[i], mul_mod(x, pb[i], m), m.q);
    else if (OP == EW_ADD_SCALAR) r = add_mod(x, sc, m.q);
    else if (OP == EW_MULADD_SCALAR) r = add_mod(pr[i], mul_mod(x, sc, m), m.q);
    else r = mul_mod(x, sc, m);
    pr[i] = r;
  }
}

// one reduced scalar per limb of the batch, passed by value
// (rns_poly.c Scalars_integer_add_poly / Scalars_integer_multiply_poly)
struct ScalarList {
  u64 v[kMaxLimbs];
};

template <bool MUL>
__global__ void __launch_bounds__(kThreads)
ew_scalars_kernel(Ptr2 res, Ptr2 a, ScalarList sc, LimbBatch batch,
                  const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const u64        s  = sc.v[blockIdx.y];
  const u64*       pa = sel_a(a, lr, n);
  u64*             pr = sel_d(res, lr, n);
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = MUL ? mul_mod(pa[i], s, m) : add_mod(pa[i], s, m.q);
}

// ---- automorphism in NTT form: a pure gather (hal.c:123-138) ----------------

__global__ void __launch_bounds__(kThreads)
automorphism_kernel(Ptr2 res, Ptr2 val, const uint32_t* __restrict__ table, LimbBatch batch,
                    uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64*    pv = sel_a(val, lr, n);
  u64*          pr = sel_d(res, lr, n);
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = pv[__ldg(table + i)];
}

// res[i] = val[table[i]] (+ add[table[i]] on limbs flagged with sel bit 1, the
// addend limb index in lr.b): the "+ P*c0" of a hoisted rotation on the
// extended basis, folded into the gather
__global__ void __launch_bounds__(kThreads)
automorphism_add_kernel(Ptr2 res, Ptr2 val, const u64* __restrict__ add,
                        const uint32_t* __restrict__ table, LimbBatch batch,
                        const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef lr  = batch.limb[blockIdx.y];
  const u64*    pv  = sel_a(val, lr, n);
  u64*          pr  = sel_d(res, lr, n);
  const bool    has = (lr.sel & 2) != 0;
  const u64*    pa  = add + (size_t)lr.b * n;
  const u64     q   = mods[lr.prime].q;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    uint32_t t = __ldg(table + i);
    u64      x = pv[t];
    if (has) x = add_mod(x, pa[t], q);
    pr[i] = x;
  }
}

__global__ void __launch_bounds__(kThreads)
mul_const_kernel(Ptr2 res, Ptr2 val, const Twiddle* __restrict__ consts, LimbBatch batch,
                 const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64     q  = mods[lr.prime].q;
  const Twiddle c  = consts[lr.prime];
  const u64*    pv = sel_a(val, lr, n);
  u64*          pr = sel_d(res, lr, n);
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = mul_shoup(pv[i], c.w, c.wp, q);
}

// ---- tensor product (ckks/src/evaluator.c:137-173) ---------------------------
// limb index = prime index = blockIdx.y; the middle term is summed in 128 bits
// and reduced once.

__global__ void __launch_bounds__(kThreads)
tensor_kernel(u64* __restrict__ d0, u64* __restrict__ d1, u64* __restrict__ d2,
              const u64* __restrict__ a0, const u64* __restrict__ a1,
              const u64* __restrict__ b0, const u64* __restrict__ b1,
              const DevModulus* __restrict__ mods, uint32_t n, int first_prime) {
  const DevModulus m   = mods[first_prime + blockIdx.y];
  const size_t     off = (size_t)blockIdx.y * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    u64 x0 = a0[off + i], x1 = a1[off + i], y0 = b0[off + i], y1 = b1[off + i];
    d0[off + i] = mul_mod(x0, y0, m);
    d2[off + i] = mul_mod(x1, y1, m);
    u64 hi = 0, lo = 0;
    mac_128(hi, lo, x0, y1);
    mac_128(hi, lo, x1, y0);
    d1[off + i] = reduce_128(hi, lo, m);
  }
}

// ---- rescale (rns_poly.c:351-383) -------------------------------------------

__global__ void __launch_bounds__(kThreads)
rescale_lift_kernel(Ptr2 tmp, Ptr2 last, u64 q_last, const Twiddle* __restrict__ neg_row,
                    const u64* __restrict__ mod_row, LimbBatch batch,
                    const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const Twiddle    w  = neg_row[lr.prime];
  const u64        om = mod_row[lr.prime];
  const u64*       pl = sel_b(last, lr, n);
  u64*             pt = sel_d(tmp, lr, n);
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    u64 s = switch_modulus(pl[i], q_last, m, om);
    pt[i] = mul_shoup(s, w.w, w.wp, m.q);
  }
}

__global__ void __launch_bounds__(kThreads)
rescale_combine_kernel(Ptr2 res, Ptr2 poly, Ptr2 tmp, const Twiddle* __restrict__ inv_row,
                       LimbBatch batch, const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64     q  = mods[lr.prime].q;
  const Twiddle w  = inv_row[lr.prime];
  const u64*    pp = sel_a(poly, lr, n);
  const u64*    pt = sel_b(tmp, lr, n);
  u64*          pr = sel_d(res, lr, n);
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = add_mod(mul_shoup(pp[i], w.w, w.wp, q), pt[i], q);
}

// ---- approximate base conversion --------------------------------------------
// One thread per coefficient; the scaled inputs y_i stay in registers (padded
// with zeros up to NIN), the conversion matrix of the CTA's output chunk sits
// in shared memory.  blockIdx.y selects the chunk of outputs, blockIdx.z the
// group (digit for ModUp, polynomial for ModDown).  With FAST the sums use the
// carry-free 32-bit-half accumulators (all primes below 2^60, NIN <= 16).

constexpr int kMaxOutChunk = 18;

template <int NIN, bool FAST>
__global__ void __launch_bounds__(kThreads)
base_conv_kernel(ConvArgs args, int chunk, int num_q, const DevModulus* __restrict__ mods,
                 uint32_t n) {
  // FAST keeps the matrix pre-split into 30-bit halves (x = low, y = high)
  __shared__ uint2 sm_mat[kMaxOutChunk * NIN];
  const ConvGroup  g         = args.g[blockIdx.z];
  const int        out_count = args.out_total - g.skip_len;
  const int        o_beg     = blockIdx.y * chunk;
  if (o_beg >= out_count) return;
  const int o_end = min(o_beg + chunk, out_count);
  for (int t = threadIdx.x; t < (o_end - o_beg) * NIN; t += kThreads) {
    int o = t / NIN, i = t - o * NIN;
    int m = o_beg + o;
    m     = m < g.skip_start ? m : m + g.skip_len;
    int prime = m < args.level ? m : num_q + (m - args.level);
    u64 v = i < g.count
                ? g.mat[(size_t)i * args.in_stride + (size_t)prime * args.out_stride]
                : 0;
    sm_mat[t] = FAST ? make_uint2((uint32_t)v & 0x3fffffffu, (uint32_t)(v >> 30))
                     : make_uint2((uint32_t)v, (uint32_t)(v >> 32));
  }
  __syncthreads();
  const uint32_t c = blockIdx.x * kThreads + threadIdx.x;
  if (c >= n) return;
  uint32_t y0[NIN], y1[NIN];  // halves of y_i: 30-bit split (FAST) or 32-bit split
#pragma unroll
  for (int i = 0; i < NIN; i++) {
    u64 y = 0;
    if (i < g.count) {
      const Twiddle w = g.inv[i];
      y = mul_shoup(g.in[(size_t)(g.first_limb + i) * n + c], w.w, w.wp,
                    mods[g.first_prime + i].q);
    }
    y0[i] = FAST ? ((uint32_t)y & 0x3fffffffu) : (uint32_t)y;
    y1[i] = FAST ? (uint32_t)(y >> 30) : (uint32_t)(y >> 32);
  }
  for (int o = o_beg; o < o_end; o++) {
    int m     = o < g.skip_start ? o : o + g.skip_len;
    if ((args.skip_mask >> m) & 1) continue;
    int prime = m < args.level ? m : num_q + (m - args.level);
    int limb  = m < args.level ? m : args.p_limb + (m - args.level);
    const DevModulus md  = mods[prime];
    const uint2*     row = sm_mat + (o - o_beg) * NIN;
    u64              hi, lo;
    if (FAST) {
      Acc4 acc;
      acc4_zero(acc);
#pragma unroll
      for (int i = 0; i < NIN; i++) {
        const uint2 b = row[i];
        acc4_mac_halves(acc, y0[i], y1[i], b.x, b.y);
      }
      acc4_fold(acc, hi, lo);
    } else {
      hi = lo = 0;
#pragma unroll
      for (int i = 0; i < NIN; i++) {
        const uint2 b = row[i];
        mac_128(hi, lo, ((u64)y1[i] << 32) | y0[i], ((u64)b.y << 32) | b.x);
      }
    }
    g.out[(size_t)limb * n + c] = reduce_128(hi, lo, md);
  }
}

// ---- ModDown tail (rns_poly.c:293-304), optionally adding a polynomial -------

__global__ void __launch_bounds__(kThreads)
moddown_combine_kernel(ModDownTail a, const Twiddle* __restrict__ p_inv,
                       const DevModulus* __restrict__ mods, uint32_t n) {
  const int     g   = blockIdx.z;
  if ((a.skip_mask >> blockIdx.y) & 1) return;
  const u64     q   = mods[blockIdx.y].q;
  const Twiddle w   = p_inv[blockIdx.y];
  const size_t  off = (size_t)blockIdx.y * n;
  const u64*    px  = a.x[g] + off;
  const u64*    pt  = a.t[g] + off;
  const u64*    pa  = a.add[g] ? a.add[g] + off : nullptr;
  u64*          pr  = a.res[g] + off;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    u64 r = mul_shoup(sub_mod(px[i], pt[i], q), w.w, w.wp, q);
    if (pa) r = add_mod(r, pa[i], q);
    pr[i] = r;
  }
}

// ---- fused ModDown + Rescale tail, coefficient form (rns_poly.c:556-596) -----

// Sub_mul_const_mod of the CPU runtime (modular.h:266-276) on operands where
// val2 may exceed the modulus: the signed difference gets the modulus added
// once when negative and may stay negative; the Shoup product then runs on its
// two's-complement image exactly as the 128-bit host arithmetic does.
__device__ __forceinline__ u64 sub_mul_const_exact(u64 v1, u64 v2, u64 w, u64 wp, u64 q) {
  long long s = (long long)v1 - (long long)v2;
  if (s < 0) s += (long long)q;
  u64 lo = (u64)s;
  u64 qt = __umul64hi(lo, wp) - (s < 0 ? wp : 0);  // ((2^128 + s) * wp >> 64) mod 2^64
  u64 y  = lo * w - qt * q;
  return y >= q ? y - q : y;
}

__global__ void __launch_bounds__(kThreads)
moddown_rescale_kernel(u64* __restrict__ res, const u64* __restrict__ x,
                       const u64* __restrict__ t, int last, const Twiddle* __restrict__ p_inv,
                       const Twiddle* __restrict__ ql_inv_row,
                       const DevModulus* __restrict__ mods, uint32_t n) {
  const int     i    = blockIdx.y;  // output limb, i < last
  const u64     q    = mods[i].q, ql = mods[last].q;
  const Twiddle pi   = p_inv[i], pl = p_inv[last], wi = ql_inv_row[i];
  const u64*    xi   = x + (size_t)i * n;
  const u64*    ti   = t + (size_t)i * n;
  const u64*    xl   = x + (size_t)last * n;
  const u64*    tl   = t + (size_t)last * n;
  u64*          ri   = res + (size_t)i * n;
  for (uint32_t k = blockIdx.x * kThreads + threadIdx.x; k < n; k += gridDim.x * kThreads) {
    u64 last_new = mul_shoup(sub_mod(xl[k], tl[k], ql), pl.w, pl.wp, ql);
    u64 nv       = mul_shoup(sub_mod(xi[k], ti[k], q), pi.w, pi.wp, q);
    ri[k]        = sub_mul_const_exact(nv, last_new, wi.w, wi.wp, q);
  }
}

// Rescale of a polynomial in coefficient form (rns_poly.c:381-399): the dropped
// limb is reduced as it stands (no centring, unlike the NTT-form branch),
// res_i = (x_i - (x_last mod q_i)) * q_last^-1 mod q_i.  blockIdx.y runs over
// the limbs of `polys` polynomials of `last` output limbs each.
__global__ void __launch_bounds__(kThreads)
rescale_coeff_kernel(Ptr2 res, Ptr2 x, int last, const Twiddle* __restrict__ ql_inv_row,
                     const DevModulus* __restrict__ mods, uint32_t n) {
  const int        g  = blockIdx.y / last, i = blockIdx.y % last;
  const DevModulus md = mods[i];
  const Twiddle    wi = ql_inv_row[i];
  const u64*       xi = (g ? x.p[1] : x.p[0]) + (size_t)i * n;
  const u64*       xl = (g ? x.p[1] : x.p[0]) + (size_t)last * n;
  u64*             ri = (g ? res.p[1] : res.p[0]) + (size_t)i * n;
  for (uint32_t k = blockIdx.x * kThreads + threadIdx.x; k < n; k += gridDim.x * kThreads)
    ri[k] = mul_shoup(sub_mod(xi[k], reduce_128(0, xl[k], md), md.q), wi.w, wi.wp, md.q);
}

// ---- key inner product (rns_poly.c:516, rns_poly_impl.c:13-160) --------------
// One reduction per output word; two coefficients per thread (16-byte loads).

// The kernel streams its operands once, so what it needs is bytes in flight:
// the digits are taken U at a time and all operands of a group are loaded
// before the first multiply; registers are capped for four resident CTAs per
// SM.  EXACT: there are exactly U digits (the key switch: up to four); else
// any number, in groups of U (a group that reaches past the last digit loads
// nothing for the missing ones and multiplies zeros).
template <bool TWO, bool FAST, int U, bool EXACT>
__global__ void __launch_bounds__(kThreads, 4)
inner_product_kernel(InnerArgs a, int num_q, const DevModulus* __restrict__ mods, uint32_t n) {
  const int        m     = blockIdx.y;  // limb among level Q limbs then K P limbs
  if ((a.skip_mask >> m) & 1) return;
  const bool       is_q  = m < a.level;
  const int        prime = is_q ? m : num_q + (m - a.level);
  const DevModulus md    = mods[prime];
  const size_t e_off = (size_t)(is_q ? m : a.ext_p_limb + (m - a.level)) * n;
  const size_t k_off = (size_t)(is_q ? m : a.key_p_limb + (m - a.level)) * n;
  const size_t d_off = (size_t)(is_q ? m : a.acc_p_limb + (m - a.level)) * n;
  const int    own   = (a.in != nullptr && is_q) ? m / a.alpha : -1;
  const uint32_t pairs = n >> 1;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < pairs; i += gridDim.x * kThreads) {
    Acc4 c00, c01, c10, c11;
    u64  h[4] = {0, 0, 0, 0}, l[4] = {0, 0, 0, 0};
    if (FAST) {
      acc4_zero(c00);
      acc4_zero(c01);
      acc4_zero(c10);
      acc4_zero(c11);
    }
#pragma unroll 1
    for (int base = 0; base < (EXACT ? U : a.parts); base += U) {
      ulonglong2 e[U], k0[U], k1[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int j = base + u;
        if (!EXACT) e[u] = k0[u] = k1[u] = make_ulonglong2(0, 0);
        if (EXACT || j < a.parts) {
          const u64* es = (j == own) ? a.in + (size_t)m * n : a.ext_ptr[j] + e_off;
          e[u]  = reinterpret_cast<const ulonglong2*>(es)[i];
          // keys are read once per key switch: streamed past the L2 lines that the
          // twiddle tables and the polynomials in flight should keep
          k0[u] = __ldcs(reinterpret_cast<const ulonglong2*>(a.key0[j] + k_off) + i);
          if (TWO) k1[u] = __ldcs(reinterpret_cast<const ulonglong2*>(a.key1[j] + k_off) + i);
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        if (FAST) {
          acc4_mac(c00, e[u].x, k0[u].x);
          acc4_mac(c01, e[u].y, k0[u].y);
          if (TWO) {
            acc4_mac(c10, e[u].x, k1[u].x);
            acc4_mac(c11, e[u].y, k1[u].y);
          }
        } else {
          mac_128(h[0], l[0], e[u].x, k0[u].x);
          mac_128(h[1], l[1], e[u].y, k0[u].y);
          if (TWO) {
            mac_128(h[2], l[2], e[u].x, k1[u].x);
            mac_128(h[3], l[3], e[u].y, k1[u].y);
          }
        }
      }
    }
    if (FAST) {
      acc4_fold(c00, h[0], l[0]);
      acc4_fold(c01, h[1], l[1]);
      if (TWO) {
        acc4_fold(c10, h[2], l[2]);
        acc4_fold(c11, h[3], l[3]);
      }
    }
    ulonglong2 r;
    r.x = reduce_128(h[0], l[0], md);
    r.y = reduce_128(h[1], l[1], md);
    reinterpret_cast<ulonglong2*>(a.acc0 + d_off)[i] = r;
    if (TWO) {
      r.x = reduce_128(h[2], l[2], md);
      r.y = reduce_128(h[3], l[3], md);
      reinterpret_cast<ulonglong2*>(a.acc1 + d_off)[i] = r;
    }
  }
}

// ---- mod-raise (rns_poly.c:1101-1125) ----------------------------------------

__global__ void __launch_bounds__(kThreads)
mod_raise_kernel(u64* __restrict__ res, const u64* __restrict__ src, u64 q0,
                 LimbBatch batch, const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const u64        om = q0 % m.q;
  u64*             pr = res + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = lr.prime == 0 ? src[i] : switch_modulus(src[i], q0, m, om);
}

inline void after_launch(Context* c, KernelId id, int limbs) {
  prof_after(id, limbs);
  c->launches++;
  CUDA_CHECK(cudaGetLastError());
}

}  // namespace

void launch_elementwise(EwOp op, Ptr2 res, Ptr2 a, Ptr2 b, int64_t scalar,
                        const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  DagScope dag(DAG_ELEMENTWISE);
  {
    const bool two  = op == EW_ADD || op == EW_SUB || op == EW_MUL || op == EW_MULADD;
    const bool accu = op == EW_MULADD || op == EW_MULADD_SCALAR;
    dag.batch(batch, c->N, &res, &a, two ? &b : nullptr, accu);
  }
  dag.commit();
  prof_before(KID_ELEMENTWISE);
  dim3 g = grid_for(c->N, 2, batch.count);
#define EW_CASE(OP)                                                                        \
  case OP:                                                                                 \
    ew_kernel<OP><<<g, kThreads, 0, c->stream>>>(res, a, b, (u64)scalar, batch, c->d_mod,  \
                                                 c->N);                                    \
    break;
  switch (op) {
    EW_CASE(EW_ADD)
    EW_CASE(EW_SUB)
    EW_CASE(EW_MUL)
    EW_CASE(EW_MULADD)
    EW_CASE(EW_ADD_SCALAR)
    EW_CASE(EW_MUL_SCALAR)
    EW_CASE(EW_MULADD_SCALAR)
  }
#undef EW_CASE
  after_launch(c, KID_ELEMENTWISE, batch.count);
}

void launch_scalars(bool mul, Ptr2 res, Ptr2 a, const u64* per_limb, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  ScalarList sc;
  for (int i = 0; i < batch.count; i++) sc.v[i] = per_limb[i];
  DagScope dag(DAG_PER_LIMB_CONST);
  dag.batch(batch, c->N, &res, &a, nullptr);
  dag.commit();
  prof_before(KID_ELEMENTWISE);
  dim3 g = grid_for(c->N, 2, batch.count);
  if (mul) ew_scalars_kernel<true><<<g, kThreads, 0, c->stream>>>(res, a, sc, batch, c->d_mod, c->N);
  else ew_scalars_kernel<false><<<g, kThreads, 0, c->stream>>>(res, a, sc, batch, c->d_mod, c->N);
  after_launch(c, KID_ELEMENTWISE, batch.count);
}

void launch_automorphism(Ptr2 res, Ptr2 val, const uint32_t* table, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  DagScope dag(DAG_AUTOMORPHISM);
  dag.batch(batch, c->N, &res, &val, nullptr);
  dag.commit();
  prof_before(KID_AUTOMORPHISM);
  automorphism_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      res, val, table, batch, c->N);
  after_launch(c, KID_AUTOMORPHISM, batch.count);
}

void launch_automorphism_add(Ptr2 res, Ptr2 val, const int64_t* add, const uint32_t* table,
                             const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  DagScope dag(DAG_AUTOMORPHISM);
  dag.batch(batch, c->N, &res, &val, nullptr);
  if (dag.live)
    for (int i = 0; i < batch.count; i++)
      if (batch.limb[i].sel & 2)
        dag.set.read(add + (size_t)batch.limb[i].b * c->N, (size_t)c->N * sizeof(int64_t));
  dag.commit();
  prof_before(KID_AUTOMORPHISM);
  automorphism_add_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      res, val, reinterpret_cast<const u64*>(add), table, batch, c->d_mod, c->N);
  after_launch(c, KID_AUTOMORPHISM, batch.count);
}

void launch_mul_const(Ptr2 res, Ptr2 val, const Twiddle* consts, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  DagScope dag(DAG_PER_LIMB_CONST);
  dag.batch(batch, c->N, &res, &val, nullptr);
  dag.commit();
  prof_before(KID_MUL_CONST);
  mul_const_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      res, val, consts, batch, c->d_mod, c->N);
  after_launch(c, KID_MUL_CONST, batch.count);
}

void launch_tensor_range(int64_t* d0, int64_t* d1, int64_t* d2, const int64_t* a0,
                         const int64_t* a1, const int64_t* b0, const int64_t* b1, int first_prime,
                         int count) {
  if (count == 0) return;
  Context* c = ctx();
  DagScope dag(DAG_TENSOR);
  if (dag.live) {
    const size_t bytes = (size_t)count * c->N * sizeof(int64_t);
    for (const int64_t* r : {a0, a1, b0, b1}) dag.set.read(r, bytes);
    for (int64_t* w : {d0, d1, d2}) dag.set.write(w, bytes);
  }
  dag.commit();
  prof_before(KID_TENSOR);
  tensor_kernel<<<grid_for(c->N, 2, count), kThreads, 0, c->stream>>>(
      (u64*)d0, (u64*)d1, (u64*)d2, (const u64*)a0, (const u64*)a1, (const u64*)b0,
      (const u64*)b1, c->d_mod, c->N, first_prime);
  after_launch(c, KID_TENSOR, count);
}

void launch_tensor(int64_t* d0, int64_t* d1, int64_t* d2, const int64_t* a0,
                   const int64_t* a1, const int64_t* b0, const int64_t* b1, int level) {
  launch_tensor_range(d0, d1, d2, a0, a1, b0, b1, 0, level);
}

void launch_rescale_lift(Ptr2 tmp, Ptr2 last, int l, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_RESCALE_LIFT);
  rescale_lift_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      tmp, last, c->primes[l], c->d_ql_neg + (size_t)l * c->L, c->d_ql_mod + (size_t)l * c->L,
      batch, c->d_mod, c->N);
  after_launch(c, KID_RESCALE_LIFT, batch.count);
}

void launch_rescale_combine(Ptr2 res, Ptr2 poly, Ptr2 tmp, int l, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_RESCALE_COMBINE);
  rescale_combine_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      res, poly, tmp, c->d_ql_inv + (size_t)l * c->L, batch, c->d_mod, c->N);
  after_launch(c, KID_RESCALE_COMBINE, batch.count);
}

template <int NIN>
static void base_conv_dispatch(Context* c, const ConvArgs& args, dim3 grid, int chunk) {
  if (c->primes_below_2_60)
    base_conv_kernel<NIN, true><<<grid, kThreads, 0, c->stream>>>(args, chunk, c->L, c->d_mod,
                                                                  c->N);
  else
    base_conv_kernel<NIN, false><<<grid, kThreads, 0, c->stream>>>(args, chunk, c->L, c->d_mod,
                                                                   c->N);
}

void launch_base_conv(const ConvArgs& args) {
  Context* c = ctx();
  int max_in = 0, max_out = 0, total_out = 0;
  for (int g = 0; g < args.groups; g++) {
    max_in  = std::max(max_in, args.g[g].count);
    max_out = std::max(max_out, args.out_total - args.g[g].skip_len);
    total_out += args.out_total - args.g[g].skip_len;
  }
  if (max_out <= 0 || args.groups == 0) return;
  FHERT_ASSERT(max_in <= kMaxDigit, "base conversion from %d limbs unsupported", max_in);
  int  chunks = (max_out + kMaxOutChunk - 1) / kMaxOutChunk;
  int  chunk  = (max_out + chunks - 1) / chunks;
  dim3 grid((c->N + kThreads - 1) / kThreads, chunks, args.groups);
  DagScope dag(DAG_BASE_CONV);
  if (dag.live) {
    const size_t w = (size_t)c->N * sizeof(u64);
    for (int g = 0; g < args.groups; g++) {
      const ConvGroup& cg = args.g[g];
      dag.set.read(cg.in + (size_t)cg.first_limb * c->N, (size_t)cg.count * w);
      for (int m = 0; m < args.out_total; m++) {
        if (m >= cg.skip_start && m < cg.skip_start + cg.skip_len) continue;
        if ((args.skip_mask >> m) & 1) continue;
        int limb = m < args.level ? m : args.p_limb + (m - args.level);
        dag.set.write(cg.out + (size_t)limb * c->N, w);
      }
    }
  }
  dag.commit();
  prof_before(KID_BASE_CONV);
  if (max_in <= 2) base_conv_dispatch<2>(c, args, grid, chunk);
  else if (max_in <= 4) base_conv_dispatch<4>(c, args, grid, chunk);
  else if (max_in <= 6) base_conv_dispatch<6>(c, args, grid, chunk);
  else if (max_in <= 8) base_conv_dispatch<8>(c, args, grid, chunk);
  else if (max_in <= 12) base_conv_dispatch<12>(c, args, grid, chunk);
  else base_conv_dispatch<16>(c, args, grid, chunk);
  after_launch(c, KID_BASE_CONV, total_out);
}

void launch_moddown_combine(const ModDownTail& args) {
  if (args.level == 0 || args.polys == 0) return;
  Context* c = ctx();
  prof_before(KID_MODDOWN_COMBINE);
  dim3 g = grid_for(c->N, 2, args.level);
  g.z    = args.polys;
  moddown_combine_kernel<<<g, kThreads, 0, c->stream>>>(args, c->d_p_inv, c->d_mod, c->N);
  after_launch(c, KID_MODDOWN_COMBINE, args.level * args.polys);
}

void launch_moddown_rescale(int64_t* res, const int64_t* x, const int64_t* t, int level) {
  if (level < 2) return;
  Context* c    = ctx();
  const int last = level - 1;
  prof_before(KID_MODDOWN_COMBINE);
  moddown_rescale_kernel<<<grid_for(c->N, 2, last), kThreads, 0, c->stream>>>(
      (u64*)res, (const u64*)x, (const u64*)t, last, c->d_p_inv,
      c->d_ql_inv + (size_t)last * c->L, c->d_mod, c->N);
  after_launch(c, KID_MODDOWN_COMBINE, last);
}

void launch_rescale_coeff(Ptr2 res, Ptr2 x, int polys, int level) {
  if (level < 2) return;
  Context*  c    = ctx();
  const int last = level - 1;
  prof_before(KID_RESCALE_COMBINE);
  rescale_coeff_kernel<<<grid_for(c->N, 2, polys * last), kThreads, 0, c->stream>>>(
      res, x, last, c->d_ql_inv + (size_t)last * c->L, c->d_mod, c->N);
  after_launch(c, KID_RESCALE_COMBINE, polys * last);
}

void launch_inner_product(const InnerArgs& args) {
  Context* c     = ctx();
  int      limbs = args.level + c->K;
  FHERT_ASSERT(args.parts >= 1 && args.parts <= kMaxParts, "unsupported digit count");
  DagScope dag(DAG_INNER_PRODUCT);
  if (dag.live) {
    const size_t n = c->N, w = n * sizeof(u64);
    for (int m = 0; m < limbs; m++) {
      if ((args.skip_mask >> m) & 1) continue;
      const bool   is_q  = m < args.level;
      const size_t e_off = (size_t)(is_q ? m : args.ext_p_limb + (m - args.level)) * n;
      const size_t k_off = (size_t)(is_q ? m : args.key_p_limb + (m - args.level)) * n;
      const size_t d_off = (size_t)(is_q ? m : args.acc_p_limb + (m - args.level)) * n;
      const int    own   = (args.in != nullptr && is_q) ? m / args.alpha : -1;
      for (int j = 0; j < args.parts; j++) {
        dag.set.read(j == own ? args.in + (size_t)m * n : args.ext_ptr[j] + e_off, w);
        // the "key" operands are switching keys in a key switch, but rotated
        // ciphertext polynomials in the baby-step sums of the bootstrap
        dag.set.read(args.key0[j] + k_off, w);
        if (args.acc1 != nullptr) dag.set.read(args.key1[j] + k_off, w);
      }
      dag.set.write(args.acc0 + d_off, w);
      if (args.acc1 != nullptr) dag.set.write(args.acc1 + d_off, w);
    }
  }
  dag.commit();
  prof_before(KID_INNER_PRODUCT);
  dim3 g    = grid_for(c->N, 4, limbs);
  bool fast = c->primes_below_2_60;
  bool two  = args.acc1 != nullptr;
#define IP_CASE(TWO_, FAST_, U_, EXACT_)                                                       \
  inner_product_kernel<TWO_, FAST_, U_, EXACT_><<<g, kThreads, 0, c->stream>>>(args, c->L,      \
                                                                              c->d_mod, c->N)
#define IP_GROUPS(TWO_, FAST_)                                 \
  do {                                                         \
    if (args.parts == 1) IP_CASE(TWO_, FAST_, 1, true);        \
    else if (args.parts == 2) IP_CASE(TWO_, FAST_, 2, true);   \
    else if (args.parts == 3) IP_CASE(TWO_, FAST_, 3, true);   \
    else if (args.parts == 4) IP_CASE(TWO_, FAST_, 4, true);   \
    else IP_CASE(TWO_, FAST_, 2, false);                       \
  } while (0)
  if (two && fast) IP_GROUPS(true, true);
  else if (two) IP_GROUPS(true, false);
  else if (fast) IP_GROUPS(false, true);
  else IP_GROUPS(false, false);
#undef IP_GROUPS
#undef IP_CASE
  after_launch(c, KID_INNER_PRODUCT, limbs);
}

void launch_mod_raise(int64_t* res, const int64_t* src, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  DagScope dag(DAG_PER_LIMB_CONST);
  if (dag.live) {
    const size_t w = (size_t)c->N * sizeof(int64_t);
    dag.set.read(src, w);
    for (int i = 0; i < batch.count; i++) dag.set.write(res + (size_t)batch.limb[i].dst * c->N, w);
  }
  dag.commit();
  prof_before(KID_MOD_RAISE);
  mod_raise_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      (u64*)res, (const u64*)src, c->primes[0], batch, c->d_mod, c->N);
  after_launch(c, KID_MOD_RAISE, batch.count);
}

}  // namespace fhert
