// Negacyclic NTT / inverse NTT over one or many RNS limbs.
//
// Dataflow and twiddle indexing follow the CPU runtime exactly
// (fhe-cmplr/rtlib/ant/util/src/ntt.c:167-241 forward, 245-330 inverse):
// forward = Cooley-Tukey, natural order in, bit-reversed order out, stage
// m = 1, 2, .., N/2 uses twiddle table entry m + i for butterfly group i;
// inverse = Gentleman-Sande in the opposite order with N^-1 applied.  The
// butterflies here are lazy (values stay below 4q forward, 2q inverse) and
// N^-1 is folded into the last inverse stage; the residues written out are
// canonical, which makes them equal to the CPU runtime's.
//
// Three kernels per direction:
//   small    N <= 4096: one CTA per limb, whole limb in shared memory.
//   strided  first logN-8 stages: a CTA owns 16 adjacent columns of the
//            (N/256) x 256 view of the limb; every thread keeps 8 rows in
//            registers and does up to three stages between exchanges.
//   contig   last 8 stages: a warp owns one contiguous 256-word block.
// The inverse runs contig first, then strided.
#include "runtime.h"

namespace fhert {

namespace {

constexpr int kContigLog   = 8;    // stages handled by the contiguous kernel
constexpr int kContigBlock = 256;
constexpr int kTileCols    = 16;   // columns per CTA in the strided kernel
constexpr int kBlocksPerCta = 16;  // 256-word blocks per CTA, contiguous kernel

// ---- butterflies ---------------------------------------------------------

// Cooley-Tukey, Harvey lazy form: a, b in [0,4q) -> a+wb, a-wb in [0,4q)
__device__ __forceinline__ void ct_bfly(u64& a, u64& b, const Twiddle& t, u64 q) {
  u64 two_q = q << 1;
  u64 x     = a >= two_q ? a - two_q : a;
  u64 v     = mul_shoup_lazy(b, t.w, t.wp, q);
  a         = x + v;
  b         = x - v + two_q;
}

// Gentleman-Sande, lazy: a, b in [0,2q) -> a+b, (a-b)w in [0,2q)
__device__ __forceinline__ void gs_bfly(u64& a, u64& b, const Twiddle& t, u64 q) {
  u64 two_q = q << 1;
  u64 s     = a + b;
  u64 d     = a - b + two_q;
  a         = s >= two_q ? s - two_q : s;
  b         = mul_shoup_lazy(d, t.w, t.wp, q);
}

__device__ __forceinline__ u64 canon4(u64 v, u64 q) {
  u64 two_q = q << 1;
  if (v >= two_q) v -= two_q;
  if (v >= q) v -= q;
  return v;
}

__device__ __forceinline__ Twiddle ld_tw(const Twiddle* p) {
  ulonglong2 v = __ldg(reinterpret_cast<const ulonglong2*>(p));
  Twiddle    t;
  t.w  = v.x;
  t.wp = v.y;
  return t;
}

// One register round of R consecutive forward stages starting at local stage
// l0 of a 2^s-point transform.  The thread holds the 8 elements
// base | (e << lowpos), e = 0..7, with lowpos = s - l0 - R.  tw_stage(l)
// gives the table index of the first twiddle of local stage l:
// (1 << (s0 + l)) + (blk << l); the group inside the block is idx >> (s - l).
template <int R>
__device__ __forceinline__ void fwd_round(u64 (&x)[8], int base, int lowpos, int s,
                                          int l0, int s0, uint32_t blk,
                                          const Twiddle* tw, u64 q) {
#pragma unroll
  for (int u = 0; u < R; u++) {
    const int bit = R - 1 - u;
    const int l   = l0 + u;
    uint32_t  tb  = (1u << (s0 + l)) + (blk << l);
#pragma unroll
    for (int hp = 0; hp < (8 >> (bit + 1)); hp++) {
      int     idx = base | ((hp << (bit + 1)) << lowpos);
      Twiddle t   = ld_tw(tw + tb + (idx >> (s - l)));
#pragma unroll
      for (int lp = 0; lp < (1 << bit); lp++) {
        int lo = (hp << (bit + 1)) | lp;
        ct_bfly(x[lo], x[lo | (1 << bit)], t, q);
      }
    }
  }
}

// Inverse round: same stages, processed from the highest local stage down.
// When `last` is set and the round reaches local stage 0 of global stage 0,
// the final butterfly applies N^-1 (fin[0] = N^-1, fin[1] = rou_inv[1]*N^-1)
// and leaves canonical values.
template <int R>
__device__ __forceinline__ void inv_round(u64 (&x)[8], int base, int lowpos, int s,
                                          int l0, int s0, uint32_t blk,
                                          const Twiddle* tw, u64 q, bool last,
                                          const Twiddle* fin) {
#pragma unroll
  for (int u = R - 1; u >= 0; u--) {
    const int bit = R - 1 - u;
    const int l   = l0 + u;
    uint32_t  tb  = (1u << (s0 + l)) + (blk << l);
    if (last && l == 0) {
      Twiddle n_inv = ld_tw(fin), w_n = ld_tw(fin + 1);
      u64     two_q = q << 1;
#pragma unroll
      for (int hp = 0; hp < (8 >> (bit + 1)); hp++) {
#pragma unroll
        for (int lp = 0; lp < (1 << bit); lp++) {
          int lo = (hp << (bit + 1)) | lp;
          int hi = lo | (1 << bit);
          u64 sum = x[lo] + x[hi];
          u64 dif = x[lo] - x[hi] + two_q;
          x[lo]   = mul_shoup(sum, n_inv.w, n_inv.wp, q);
          x[hi]   = mul_shoup(dif, w_n.w, w_n.wp, q);
        }
      }
    } else {
#pragma unroll
      for (int hp = 0; hp < (8 >> (bit + 1)); hp++) {
        int     idx = base | ((hp << (bit + 1)) << lowpos);
        Twiddle t   = ld_tw(tw + tb + (idx >> (s - l)));
#pragma unroll
        for (int lp = 0; lp < (1 << bit); lp++) {
          int lo = (hp << (bit + 1)) | lp;
          gs_bfly(x[lo], x[lo | (1 << bit)], t, q);
        }
      }
    }
  }
}

// Bank swizzle for a 256-word block accessed with the three lane patterns of
// the contiguous kernel (lanes over index bits {0..4}, {0,1,5,6,7}, {3..7}):
// a permutation inside each aligned 16-word group that keeps every half-warp
// on 16 distinct 8-byte banks.
__device__ __forceinline__ int swz(int i) {
  int b4 = (i >> 4) & 1, b5 = (i >> 5) & 1, b6 = (i >> 6) & 1;
  return i ^ (b4 << 1) ^ (b5 << 2) ^ (b6 << 3) ^ b6;
}

// ---- contiguous 256-point blocks (global stages logN-8 .. logN-1) ----------

template <bool INV>
__global__ void __launch_bounds__(kBlocksPerCta * 32)
ntt_contig_kernel(Ptr2 in, Ptr2 out, LimbBatch batch,
                  const Twiddle* __restrict__ tables, const DevModulus* __restrict__ mods,
                  const Twiddle* __restrict__ inv_last, uint32_t n, int logn) {
  __shared__ u64 sm[kBlocksPerCta * kContigBlock];
  const LimbRef  lr    = batch.limb[blockIdx.y];
  const u64      q     = mods[lr.prime].q;
  const Twiddle* tw    = tables + (size_t)lr.prime * n;
  const int      warp  = threadIdx.x >> 5;
  const int      g     = threadIdx.x & 31;
  const uint32_t blk   = blockIdx.x * kBlocksPerCta + warp;  // block in limb
  const size_t   off   = (size_t)blk * kContigBlock;
  const u64*     src   = in.p[lr.sel & 1] + (size_t)lr.a * n + off;
  u64*           dst   = out.p[(lr.sel >> 2) & 1] + (size_t)lr.dst * n + off;
  u64*           s     = sm + warp * kContigBlock;
  const int      s0    = logn - kContigLog;
  // the last inverse stage lives here only when the whole transform is 256
  // points or fewer, which the small kernel handles; so `last` is false.
  u64 x[8];
  if (!INV) {
    // first register pass: stages 0..2, elements e*32 + g straight from global memory
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = src[e * 32 + g];
    fwd_round<3>(x, g, 5, kContigLog, 0, s0, blk, tw, q);
#pragma unroll
    for (int e = 0; e < 8; e++) s[swz((e << 5) | g)] = x[e];
    __syncwarp();
    // second register pass: stages 3..5, elements (g>>2)<<5 | e<<2 | (g&3)
    int base = ((g >> 2) << 5) | (g & 3);
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = s[swz(base | (e << 2))];
    fwd_round<3>(x, base, 2, kContigLog, 3, s0, blk, tw, q);
#pragma unroll
    for (int e = 0; e < 8; e++) s[swz(base | (e << 2))] = x[e];
    __syncwarp();
    // third register pass: stages 6..7, elements g*8 + e
    base = g << 3;
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = s[swz(base | e)];
    fwd_round<2>(x, base, 0, kContigLog, 6, s0, blk, tw, q);
#pragma unroll
    for (int e = 0; e < 8; e++) s[swz(base | e)] = canon4(x[e], q);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) dst[e * 32 + g] = s[swz((e << 5) | g)];
  } else {
    // inverse: stages 7..6, then 5..3, then 2..0 (local numbering)
#pragma unroll
    for (int e = 0; e < 8; e++) s[swz((e << 5) | g)] = src[e * 32 + g];
    __syncwarp();
    int base = g << 3;
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = s[swz(base | e)];
    inv_round<2>(x, base, 0, kContigLog, 6, s0, blk, tw, q, false, nullptr);
#pragma unroll
    for (int e = 0; e < 8; e++) s[swz(base | e)] = x[e];
    __syncwarp();
    base = ((g >> 2) << 5) | (g & 3);
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = s[swz(base | (e << 2))];
    inv_round<3>(x, base, 2, kContigLog, 3, s0, blk, tw, q, false, nullptr);
#pragma unroll
    for (int e = 0; e < 8; e++) s[swz(base | (e << 2))] = x[e];
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = s[swz((e << 5) | g)];
    inv_round<3>(x, g, 5, kContigLog, 0, s0, blk, tw, q, false, nullptr);
#pragma unroll
    for (int e = 0; e < 8; e++) dst[e * 32 + g] = x[e];
  }
}

// ---- strided columns (global stages 0 .. logN-9) ---------------------------

template <bool INV>
__global__ void ntt_strided_kernel(Ptr2 in, Ptr2 out, LimbBatch batch, const Twiddle* __restrict__ tables,
                                   const DevModulus* __restrict__ mods,
                                   const Twiddle* __restrict__ inv_last, uint32_t n,
                                   int logn) {
  extern __shared__ u64 sm_dyn[];
  const int      s1    = logn - kContigLog;       // stages here, rows = 2^s1
  const LimbRef  lr    = batch.limb[blockIdx.y];
  const u64      q     = mods[lr.prime].q;
  const Twiddle* tw    = tables + (size_t)lr.prime * n;
  const Twiddle* fin   = inv_last + (size_t)lr.prime * 2;
  const int      c     = threadIdx.x & (kTileCols - 1);
  const int      g     = threadIdx.x >> 4;        // 0 .. 2^(s1-3)-1
  const size_t   col   = (size_t)blockIdx.x * kTileCols + c;
  const u64*     src   = in.p[lr.sel & 1] + (size_t)lr.a * n + col;
  u64*           dst   = out.p[(lr.sel >> 2) & 1] + (size_t)lr.dst * n + col;
  u64            x[8];

  // rounds cover local stages [l0, l0+R); forward ascending, inverse descending
  if (!INV) {
    int l0 = 0;
    while (l0 < s1) {
      int R      = s1 - l0 < 3 ? s1 - l0 : 3;
      int lowpos = s1 - l0 - R;
      int base   = ((g >> lowpos) << (lowpos + 3)) | (g & ((1 << lowpos) - 1));
      if (l0 == 0) {
#pragma unroll
        for (int e = 0; e < 8; e++)
          x[e] = src[(size_t)(base | (e << lowpos)) << kContigLog];
      } else {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 8; e++) x[e] = sm_dyn[(base | (e << lowpos)) * kTileCols + c];
      }
      if (R == 3) fwd_round<3>(x, base, lowpos, s1, l0, 0, 0, tw, q);
      else if (R == 2) fwd_round<2>(x, base, lowpos, s1, l0, 0, 0, tw, q);
      else fwd_round<1>(x, base, lowpos, s1, l0, 0, 0, tw, q);
      l0 += R;
      if (l0 < s1) {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 8; e++) sm_dyn[(base | (e << lowpos)) * kTileCols + c] = x[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; e++)
          dst[(size_t)(base | (e << lowpos)) << kContigLog] = x[e];
      }
    }
  } else {
    // the first inverse round covers the highest stages [s1-R0, s1), with R0
    // chosen so that the stages left are a multiple of 3; this keeps the
    // 3-bit register field [lowpos, lowpos+3) inside the s1 index bits
    int hi = s1;
    bool first = true;
    while (hi > 0) {
      int R      = (hi % 3 == 0) ? 3 : hi % 3;
      int l0     = hi - R;
      int lowpos = s1 - l0 - R;
      int base = ((g >> lowpos) << (lowpos + 3)) | (g & ((1 << lowpos) - 1));
      if (first) {
#pragma unroll
        for (int e = 0; e < 8; e++)
          x[e] = src[(size_t)(base | (e << lowpos)) << kContigLog];
        first = false;
      } else {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 8; e++) x[e] = sm_dyn[(base | (e << lowpos)) * kTileCols + c];
      }
      if (R == 3) inv_round<3>(x, base, lowpos, s1, l0, 0, 0, tw, q, true, fin);
      else if (R == 2) inv_round<2>(x, base, lowpos, s1, l0, 0, 0, tw, q, true, fin);
      else inv_round<1>(x, base, lowpos, s1, l0, 0, 0, tw, q, true, fin);
      hi = l0;
      if (hi > 0) {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 8; e++) sm_dyn[(base | (e << lowpos)) * kTileCols + c] = x[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; e++)
          dst[(size_t)(base | (e << lowpos)) << kContigLog] = x[e];
      }
    }
  }
}

// ---- small transforms: whole limb in shared memory -------------------------

template <bool INV>
__global__ void ntt_small_kernel(Ptr2 in, Ptr2 out, LimbBatch batch, const Twiddle* __restrict__ tables,
                                 const DevModulus* __restrict__ mods,
                                 const Twiddle* __restrict__ inv_last, uint32_t n,
                                 int logn) {
  extern __shared__ u64 sm_dyn[];
  const LimbRef  lr  = batch.limb[blockIdx.x];
  const u64      q   = mods[lr.prime].q;
  const Twiddle* tw  = tables + (size_t)lr.prime * n;
  const Twiddle* fin = inv_last + (size_t)lr.prime * 2;
  const u64*     src = in.p[lr.sel & 1] + (size_t)lr.a * n;
  u64*           dst = out.p[(lr.sel >> 2) & 1] + (size_t)lr.dst * n;
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
        ct_bfly(a, b, t, q);
        sm_dyn[j1]                 = a;
        sm_dyn[j1 + (1u << tlog)] = b;
      }
      __syncthreads();
    }
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = canon4(sm_dyn[i], q);
  } else {
    for (int l = logn - 1; l >= 0; l--) {
      int tlog = logn - 1 - l;
      for (uint32_t bf = threadIdx.x; bf < half; bf += blockDim.x) {
        uint32_t i  = bf >> tlog;
        uint32_t j1 = ((i << (tlog + 1))) | (bf & ((1u << tlog) - 1));
        u64 a = sm_dyn[j1], b = sm_dyn[j1 + (1u << tlog)];
        if (l == 0) {
          Twiddle n_inv = ld_tw(fin), w_n = ld_tw(fin + 1);
          u64     sum = a + b, dif = a - b + (q << 1);
          a = mul_shoup(sum, n_inv.w, n_inv.wp, q);
          b = mul_shoup(dif, w_n.w, w_n.wp, q);
        } else {
          Twiddle t = ld_tw(tw + (1u << l) + i);
          gs_bfly(a, b, t, q);
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

template <bool INV>
void launch_dir(Ptr2 in, Ptr2 out, const LimbBatch& b) {
  Context*       c   = ctx();
  const Twiddle* tab = INV ? c->d_inv : c->d_fwd;
  const int      logn = (int)c->logN;
  if (logn <= kSmallMaxLog) {
    size_t smem    = (size_t)c->N * sizeof(u64);
    int    threads = c->N / 2 < 512 ? (c->N / 2 < 32 ? 32 : c->N / 2) : 512;
    prof_before(INV ? KID_INTT_SMALL : KID_NTT_SMALL);
    ntt_small_kernel<INV><<<b.count, threads, smem, c->stream>>>(
        in, out, b, tab, c->d_mod, c->d_inv_last, c->N, logn);
    prof_after(INV ? KID_INTT_SMALL : KID_NTT_SMALL, b.count);
    c->launches++;
    CUDA_CHECK(cudaGetLastError());
    return;
  }
  const int s1      = logn - kContigLog;
  dim3      grid_c(c->N / (kContigBlock * kBlocksPerCta), b.count);
  dim3      grid_s((c->N >> s1) / kTileCols, b.count);
  int       threads_s = kTileCols << (s1 - 3);
  size_t    smem_s    = ((size_t)kTileCols << s1) * sizeof(u64);
  static bool attr_done = false;
  if (!attr_done) {
    CUDA_CHECK(cudaFuncSetAttribute(ntt_strided_kernel<false>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
    CUDA_CHECK(cudaFuncSetAttribute(ntt_strided_kernel<true>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
    attr_done = true;
  }
  if (!INV) {
    prof_before(KID_NTT_STRIDED);
    ntt_strided_kernel<false><<<grid_s, threads_s, smem_s, c->stream>>>(
        in, out, b, tab, c->d_mod, c->d_inv_last, c->N, logn);
    prof_after(KID_NTT_STRIDED, b.count);
    // second pass works in place on `out`
    LimbBatch b2 = b;
    for (int i = 0; i < b2.count; i++) {
      b2.limb[i].a   = b2.limb[i].dst;
      b2.limb[i].sel = (uint8_t)((b2.limb[i].sel & 4) | ((b2.limb[i].sel >> 2) & 1));
    }
    prof_before(KID_NTT_CONTIG);
    ntt_contig_kernel<false><<<grid_c, kBlocksPerCta * 32, 0, c->stream>>>(
        out, out, b2, tab, c->d_mod, c->d_inv_last, c->N, logn);
    prof_after(KID_NTT_CONTIG, b.count);
  } else {
    prof_before(KID_INTT_CONTIG);
    ntt_contig_kernel<true><<<grid_c, kBlocksPerCta * 32, 0, c->stream>>>(
        in, out, b, tab, c->d_mod, c->d_inv_last, c->N, logn);
    prof_after(KID_INTT_CONTIG, b.count);
    LimbBatch b2 = b;
    for (int i = 0; i < b2.count; i++) {
      b2.limb[i].a   = b2.limb[i].dst;
      b2.limb[i].sel = (uint8_t)((b2.limb[i].sel & 4) | ((b2.limb[i].sel >> 2) & 1));
    }
    prof_before(KID_INTT_STRIDED);
    ntt_strided_kernel<true><<<grid_s, threads_s, smem_s, c->stream>>>(
        out, out, b2, tab, c->d_mod, c->d_inv_last, c->N, logn);
    prof_after(KID_INTT_STRIDED, b.count);
  }
  c->launches += 2;
  CUDA_CHECK(cudaGetLastError());
}

}  // namespace

void launch_ntt(Ptr2 in, Ptr2 out, const LimbBatch& b, bool inverse) {
  if (b.count == 0) return;
  if (inverse)
    launch_dir<true>(in, out, b);
  else
    launch_dir<false>(in, out, b);
}

}  // namespace fhert
