// Element-wise, permutation, rescale, base-conversion and key inner-product
// kernels over limb-major RNS polynomials.  Every kernel takes a LimbBatch so
// that one launch covers all limbs of an operation; the x dimension of the
// grid walks the N coefficients of a limb, the y dimension the limbs.
#include "runtime.h"

namespace fhert {

namespace {

constexpr int kThreads = 256;

inline dim3 grid_for(uint32_t n, int per_thread, int limbs) {
  uint32_t per_block = kThreads * per_thread;
  return dim3((n + per_block - 1) / per_block, limbs);
}

// ---- element-wise (hal/src/hal.c:15-121, poly/src/rns_poly.c:852-1054) ------

template <int OP>
__global__ void __launch_bounds__(kThreads)
ew_kernel(u64* __restrict__ res, const u64* __restrict__ a, const u64* __restrict__ b,
          u64 scalar, LimbBatch batch, const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const u64*       pa = a + (size_t)lr.a * n;
  const u64*       pb = b ? b + (size_t)lr.b * n : nullptr;
  u64*             pr = res + (size_t)lr.dst * n;
  u64              sc = 0;
  if (OP == EW_ADD_SCALAR || OP == EW_MUL_SCALAR) {
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
    else r = mul_mod(x, sc, m);
    pr[i] = r;
  }
}

// ---- automorphism in NTT form: a pure gather (hal.c:123-138) ----------------

__global__ void __launch_bounds__(kThreads)
automorphism_kernel(u64* __restrict__ res, const u64* __restrict__ val,
                    const uint32_t* __restrict__ table, LimbBatch batch, uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64*    pv = val + (size_t)lr.a * n;
  u64*          pr = res + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = pv[__ldg(table + i)];
}

__global__ void __launch_bounds__(kThreads)
mul_const_kernel(u64* __restrict__ res, const u64* __restrict__ val,
                 const Twiddle* __restrict__ consts, LimbBatch batch,
                 const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64     q  = mods[lr.prime].q;
  const Twiddle c  = consts[lr.prime];
  const u64*    pv = val + (size_t)lr.a * n;
  u64*          pr = res + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = mul_shoup(pv[i], c.w, c.wp, q);
}

// ---- rescale (rns_poly.c:351-383) -------------------------------------------

__global__ void __launch_bounds__(kThreads)
rescale_lift_kernel(u64* __restrict__ tmp, const u64* __restrict__ last, u64 q_last,
                    const Twiddle* __restrict__ neg_row, const u64* __restrict__ mod_row,
                    LimbBatch batch, const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const Twiddle    w  = neg_row[lr.prime];
  const u64        om = mod_row[lr.prime];
  u64*             pt = tmp + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    u64 s = switch_modulus(last[i], q_last, m, om);
    pt[i] = mul_shoup(s, w.w, w.wp, m.q);
  }
}

__global__ void __launch_bounds__(kThreads)
rescale_combine_kernel(u64* __restrict__ res, const u64* __restrict__ poly,
                       const u64* __restrict__ tmp, const Twiddle* __restrict__ inv_row,
                       LimbBatch batch, const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64     q  = mods[lr.prime].q;
  const Twiddle w  = inv_row[lr.prime];
  const u64*    pp = poly + (size_t)lr.a * n;
  const u64*    pt = tmp + (size_t)lr.b * n;
  u64*          pr = res + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = add_mod(mul_shoup(pp[i], w.w, w.wp, q), pt[i], q);
}

// ---- approximate base conversion --------------------------------------------
// One thread per coefficient; y_i kept in registers, the conversion matrix in
// shared memory.  blockIdx.y selects a chunk of kOutChunk output limbs.

constexpr int kOutChunk = 12;

__global__ void __launch_bounds__(kThreads)
base_conv_kernel(u64* __restrict__ out, const u64* __restrict__ in, LimbBatch in_limbs,
                 LimbBatch out_limbs, const Twiddle* __restrict__ inv,
                 const u64* __restrict__ mat, int in_stride, int out_stride,
                 const DevModulus* __restrict__ mods, uint32_t n) {
  __shared__ u64 sm_mat[kOutChunk * kMaxDigit];
  const int      nin   = in_limbs.count;
  const int      o_beg = blockIdx.y * kOutChunk;
  const int      o_end = min(o_beg + kOutChunk, out_limbs.count);
  for (int t = threadIdx.x; t < (o_end - o_beg) * nin; t += kThreads) {
    int o = t / nin, i = t - o * nin;
    sm_mat[o * kMaxDigit + i] =
        mat[(size_t)i * in_stride + (size_t)out_limbs.limb[o_beg + o].b * out_stride];
  }
  __syncthreads();
  const uint32_t c = blockIdx.x * kThreads + threadIdx.x;
  if (c >= n) return;
  u64 y[kMaxDigit];
#pragma unroll
  for (int i = 0; i < kMaxDigit; i++) {
    if (i < nin) {
      const LimbRef lr = in_limbs.limb[i];
      const Twiddle w  = inv[i];
      y[i] = mul_shoup(in[(size_t)lr.a * n + c], w.w, w.wp, mods[lr.prime].q);
    }
  }
  for (int o = o_beg; o < o_end; o++) {
    const LimbRef    lo = out_limbs.limb[o];
    const DevModulus m  = mods[lo.prime];
    u64              hi = 0, lw = 0;
#pragma unroll
    for (int i = 0; i < kMaxDigit; i++)
      if (i < nin) mac_128(hi, lw, y[i], sm_mat[(o - o_beg) * kMaxDigit + i]);
    out[(size_t)lo.dst * n + c] = reduce_128(hi, lw, m);
  }
}

__global__ void __launch_bounds__(kThreads)
moddown_combine_kernel(u64* __restrict__ res, const u64* __restrict__ x,
                       const u64* __restrict__ t, const Twiddle* __restrict__ p_inv,
                       LimbBatch batch, const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef lr = batch.limb[blockIdx.y];
  const u64     q  = mods[lr.prime].q;
  const Twiddle w  = p_inv[lr.prime];
  const u64*    px = x + (size_t)lr.a * n;
  const u64*    pt = t + (size_t)lr.b * n;
  u64*          pr = res + (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads)
    pr[i] = mul_shoup(sub_mod(px[i], pt[i], q), w.w, w.wp, q);
}

// ---- key inner product (rns_poly.c:516, rns_poly_impl.c:13-160) --------------
// 128-bit accumulation over the digits, one reduction per output word.

template <bool TWO>
__global__ void __launch_bounds__(kThreads)
inner_product_kernel(u64* __restrict__ acc0, u64* __restrict__ acc1, InnerArgs args,
                     LimbBatch batch, const DevModulus* __restrict__ mods, uint32_t n) {
  const LimbRef    lr = batch.limb[blockIdx.y];
  const DevModulus m  = mods[lr.prime];
  const size_t     oa = (size_t)lr.a * n, ob = (size_t)lr.b * n, od = (size_t)lr.dst * n;
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    u64 h0 = 0, l0 = 0, h1 = 0, l1 = 0;
    for (int j = 0; j < args.parts; j++) {
      u64 e = args.ext[j][oa + i];
      mac_128(h0, l0, e, __ldg(args.key0[j] + ob + i));
      if (TWO) mac_128(h1, l1, e, __ldg(args.key1[j] + ob + i));
    }
    acc0[od + i] = reduce_128(h0, l0, m);
    if (TWO) acc1[od + i] = reduce_128(h1, l1, m);
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

#define U64P(p) reinterpret_cast<u64*>(p)
#define CU64P(p) reinterpret_cast<const u64*>(p)

void launch_elementwise(EwOp op, int64_t* res, const int64_t* a, const int64_t* b,
                        int64_t scalar, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_ELEMENTWISE);
  dim3     g = grid_for(c->N, 2, batch.count);
#define EW_CASE(OP)                                                                     \
  case OP:                                                                              \
    ew_kernel<OP><<<g, kThreads, 0, c->stream>>>(U64P(res), CU64P(a), CU64P(b),         \
                                                 (u64)scalar, batch, c->d_mod, c->N);   \
    break;
  switch (op) {
    EW_CASE(EW_ADD)
    EW_CASE(EW_SUB)
    EW_CASE(EW_MUL)
    EW_CASE(EW_MULADD)
    EW_CASE(EW_ADD_SCALAR)
    EW_CASE(EW_MUL_SCALAR)
  }
#undef EW_CASE
  after_launch(c, KID_ELEMENTWISE, batch.count);
}

void launch_automorphism(int64_t* res, const int64_t* val, const uint32_t* table,
                         const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_AUTOMORPHISM);
  automorphism_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      U64P(res), CU64P(val), table, batch, c->N);
  after_launch(c, KID_AUTOMORPHISM, batch.count);
}

void launch_mul_const(int64_t* res, const int64_t* val, const Twiddle* consts,
                      const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_MUL_CONST);
  mul_const_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      U64P(res), CU64P(val), consts, batch, c->d_mod, c->N);
  after_launch(c, KID_MUL_CONST, batch.count);
}

void launch_rescale_lift(int64_t* tmp, const int64_t* last, int l, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_RESCALE_LIFT);
  rescale_lift_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      U64P(tmp), CU64P(last), c->primes[l], c->d_ql_neg + (size_t)l * c->L,
      c->d_ql_mod + (size_t)l * c->L, batch, c->d_mod, c->N);
  after_launch(c, KID_RESCALE_LIFT, batch.count);
}

void launch_rescale_combine(int64_t* res, const int64_t* poly, const int64_t* tmp, int l,
                            const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_RESCALE_COMBINE);
  rescale_combine_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      U64P(res), CU64P(poly), CU64P(tmp), c->d_ql_inv + (size_t)l * c->L, batch, c->d_mod,
      c->N);
  after_launch(c, KID_RESCALE_COMBINE, batch.count);
}

void launch_base_conv(int64_t* out, const int64_t* in, const LimbBatch& in_limbs,
                      const LimbBatch& out_limbs, const Twiddle* inv, const u64* mat,
                      int in_stride, int out_stride) {
  if (out_limbs.count == 0) return;
  Context* c = ctx();
  prof_before(KID_BASE_CONV);
  FHERT_ASSERT(in_limbs.count <= kMaxDigit, "base conversion from %d limbs unsupported",
               in_limbs.count);
  dim3 g((c->N + kThreads - 1) / kThreads, (out_limbs.count + kOutChunk - 1) / kOutChunk);
  base_conv_kernel<<<g, kThreads, 0, c->stream>>>(U64P(out), CU64P(in), in_limbs, out_limbs,
                                                  inv, mat, in_stride, out_stride, c->d_mod,
                                                  c->N);
  after_launch(c, KID_BASE_CONV, out_limbs.count);
}

void launch_moddown_combine(int64_t* res, const int64_t* x, const int64_t* t,
                            const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_MODDOWN_COMBINE);
  moddown_combine_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      U64P(res), CU64P(x), CU64P(t), c->d_p_inv, batch, c->d_mod, c->N);
  after_launch(c, KID_MODDOWN_COMBINE, batch.count);
}

void launch_inner_product(int64_t* acc0, int64_t* acc1, const InnerArgs& args,
                          const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_INNER_PRODUCT);
  dim3     g = grid_for(c->N, 2, batch.count);
  if (acc1)
    inner_product_kernel<true><<<g, kThreads, 0, c->stream>>>(U64P(acc0), U64P(acc1), args,
                                                              batch, c->d_mod, c->N);
  else
    inner_product_kernel<false><<<g, kThreads, 0, c->stream>>>(U64P(acc0), nullptr, args,
                                                               batch, c->d_mod, c->N);
  after_launch(c, KID_INNER_PRODUCT, batch.count);
}

void launch_mod_raise(int64_t* res, const int64_t* src, const LimbBatch& batch) {
  if (batch.count == 0) return;
  Context* c = ctx();
  prof_before(KID_MOD_RAISE);
  mod_raise_kernel<<<grid_for(c->N, 2, batch.count), kThreads, 0, c->stream>>>(
      U64P(res), CU64P(src), c->primes[0], batch, c->d_mod, c->N);
  after_launch(c, KID_MOD_RAISE, batch.count);
}

}  // namespace fhert
