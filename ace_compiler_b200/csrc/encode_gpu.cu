// The encoder's inverse canonical embedding on the device.
//
// Same arithmetic as the host routine of the CPU runtime (util/src/ntt.c:633-675
// followed by ckks/src/encoder.c:268-292), one IEEE operation at a time: complex
// products as four rounded multiplications and two rounded additions, no fused
// multiply-add anywhere (explicit _rn intrinsics), the roots of unity computed
// by the host's libm and uploaded.  The results are therefore the same doubles
// and the same rounded integers as the host path produces, and a compiled
// program's thousands of weight encodes per image no longer run one after the
// other on a CPU core.
#include <cmath>
#include <complex>
#include <vector>

#include "runtime.h"

namespace fhert {

namespace {

constexpr int     kThreads = 256;
constexpr int64_t kMax64   = (int64_t)(((u64)1 << 63) - ((u64)1 << 9)) - 1;

struct EncodeTables {
  double2*  roots     = nullptr;  // e^(2 pi i k / 2N), k < 2N
  uint32_t* rot_group = nullptr;  // 5^i mod 2N, i < N/2
};

// one Gentleman-Sande stage of the special FFT over `len` points
__global__ void __launch_bounds__(kThreads)
embed_inv_stage(double2* __restrict__ v, const double2* __restrict__ roots,
                const uint32_t* __restrict__ rot_group, uint32_t len, int logm, uint32_t m_order) {
  const uint32_t t = blockIdx.x * kThreads + threadIdx.x;
  if (t >= (len >> 1)) return;
  const uint32_t num2 = 1u << (logm - 1), idx_mod = 1u << (logm + 2), gap = m_order / idx_mod;
  const uint32_t i = t & (num2 - 1), j = (t >> (logm - 1)) << logm;
  const uint32_t e = j + i, o = e + num2;
  const uint32_t r = (idx_mod - (rot_group[i] & (idx_mod - 1))) * gap;
  const double2  a = v[e], b = v[o], w = roots[r];
  double2 plus  = make_double2(__dadd_rn(a.x, b.x), __dadd_rn(a.y, b.y));
  double2 minus = make_double2(__dsub_rn(a.x, b.x), __dsub_rn(a.y, b.y));
  double2 prod;
  prod.x = __dsub_rn(__dmul_rn(minus.x, w.x), __dmul_rn(minus.y, w.y));
  prod.y = __dadd_rn(__dmul_rn(minus.x, w.y), __dmul_rn(minus.y, w.x));
  v[e]   = plus;
  v[o]   = prod;
}

// The last `k` stages (butterfly spans below 2^k) work inside aligned chunks of
// 2^k points: one CTA keeps its chunk in shared memory, runs those stages there
// and finishes with the last step of the encoder for the points it holds: bit
// reversal (point p goes to output index bit_reverse(p)), division by the
// length, scaling by Delta, rounding, and the split into the real / imaginary
// halves of the message polynomial.  The arithmetic per butterfly is the same
// sequence of rounded operations as in the kernel above.
constexpr int kLocalLog = 12;  // 4096 points = 64 KiB of shared memory

__global__ void __launch_bounds__(1024)
embed_inv_local(int64_t* __restrict__ msg, const double2* __restrict__ v,
                const double2* __restrict__ roots, const uint32_t* __restrict__ rot_group,
                uint32_t slots, int log_slots, int k, uint32_t m_order, uint32_t gap, double delta) {
  extern __shared__ double2 chunk[];
  const uint32_t points = 1u << k, base = blockIdx.x * points;
  for (uint32_t p = threadIdx.x; p < points; p += blockDim.x) chunk[p] = v[base + p];
  __syncthreads();
  for (int logm = k; logm > 0; logm--) {
    const uint32_t num2 = 1u << (logm - 1), idx_mod = 1u << (logm + 2), step = m_order / idx_mod;
    for (uint32_t t = threadIdx.x; t < (points >> 1); t += blockDim.x) {
      const uint32_t i = t & (num2 - 1), j = (t >> (logm - 1)) << logm;
      const uint32_t e = j + i, o = e + num2;
      const uint32_t r = (idx_mod - (rot_group[i] & (idx_mod - 1))) * step;
      const double2  a = chunk[e], b = chunk[o], w = roots[r];
      double2 plus  = make_double2(__dadd_rn(a.x, b.x), __dadd_rn(a.y, b.y));
      double2 minus = make_double2(__dsub_rn(a.x, b.x), __dsub_rn(a.y, b.y));
      double2 prod;
      prod.x   = __dsub_rn(__dmul_rn(minus.x, w.x), __dmul_rn(minus.y, w.y));
      prod.y   = __dadd_rn(__dmul_rn(minus.x, w.y), __dmul_rn(minus.y, w.x));
      chunk[e] = plus;
      chunk[o] = prod;
    }
    __syncthreads();
  }
  const double d = (double)slots;
  for (uint32_t p = threadIdx.x; p < points; p += blockDim.x) {
    const uint32_t src = base + p;
    const uint32_t i   = log_slots ? (__brev(src) >> (32 - log_slots)) : 0;
    const double2  x   = chunk[p];
    const double   re  = __dadd_rn(__dmul_rn(__ddiv_rn(x.x, d), delta), 0.5);
    const double   im  = __dadd_rn(__dmul_rn(__ddiv_rn(x.y, d), delta), 0.5);
    const int64_t  r = llround(re), m = llround(im);
    msg[(size_t)i * gap]           = r < 0 ? kMax64 + r : r;
    msg[(size_t)(i + slots) * gap] = m < 0 ? kMax64 + m : m;
  }
}

// real single-precision inputs (a weight vector) widened on the device: point p
// gets (double)in[p] + 0i for p < count and 0 beyond, what the host path builds
__global__ void __launch_bounds__(kThreads)
widen_floats(double2* __restrict__ v, const float* __restrict__ in, uint32_t count, uint32_t slots) {
  const uint32_t p = blockIdx.x * kThreads + threadIdx.x;
  if (p < slots) v[p] = make_double2(p < count ? (double)in[p] : 0.0, 0.0);
}

EncodeTables* tables_of(Context* c) {
  if (c->encode_tables != nullptr) return static_cast<EncodeTables*>(c->encode_tables);
  const size_t m = 2ull * c->N, slots = c->N / 2;
  std::vector<double2>  roots(m);
  std::vector<uint32_t> rot(slots);
  for (size_t i = 0; i < m; i++) {
    double angle = 2 * M_PI * i / m;
    roots[i]     = make_double2(std::cos(angle), std::sin(angle));
  }
  rot[0] = 1;
  for (size_t i = 1; i < slots; i++) rot[i] = (uint32_t)((5ull * rot[i - 1]) % m);
  EncodeTables* t = new EncodeTables();
  if (image_capturing()) image_capture_break("a table built on first use");
  CUDA_CHECK(cudaMalloc(&t->roots, m * sizeof(double2)));
  CUDA_CHECK(cudaMalloc(&t->rot_group, slots * sizeof(uint32_t)));
  CUDA_CHECK(cudaMemcpy(t->roots, roots.data(), m * sizeof(double2), cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(t->rot_group, rot.data(), slots * sizeof(uint32_t), cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaStreamSynchronize(0));  // fully on the device before the library stream reads it
  c->encode_tables = t;
  return t;
}

}  // namespace

void free_encode_tables(Context* c) {
  if (c->encode_tables == nullptr) return;
  EncodeTables* t = static_cast<EncodeTables*>(c->encode_tables);
  cudaFree(t->roots);
  cudaFree(t->rot_group);
  delete t;
  c->encode_tables = nullptr;
}

// values: `count` complex slot values (host); d_msg: N int64 on the device,
// receives the message polynomial (negatives as Max64 + x, zeros between the
// used coefficients when slots < N/2)
void encode_message_on_device(Context* c, const std::complex<double>* values, size_t count,
                              uint32_t slots, int64_t* d_msg, const float* reals) {
  EncodeTables*  t = tables_of(c);
  const uint32_t n = c->N, gap = n / (slots * 2);
  int            lg = 0;
  while ((1u << lg) < slots) lg++;
  double2* v = nullptr;
  CUDA_CHECK(dev_alloc(&v, (size_t)slots * sizeof(double2), c->stream));
  float* d_reals = nullptr;
  if (reals != nullptr) {
    CUDA_CHECK(dev_alloc(&d_reals, count * sizeof(float), c->stream));
    CUDA_CHECK(counted_copy(d_reals, reals, count * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    widen_floats<<<(slots + kThreads - 1) / kThreads, kThreads, 0, c->stream>>>(
        v, d_reals, (uint32_t)count, slots);
    c->launches++;
  } else {
    CUDA_CHECK(cudaMemsetAsync(v, 0, (size_t)slots * sizeof(double2), c->stream));
    // std::complex<double> is two doubles, real part first
    CUDA_CHECK(counted_copy(v, values, count * sizeof(double2), cudaMemcpyHostToDevice, c->stream));
  }
  const uint32_t half_blocks = std::max(1u, ((slots >> 1) + kThreads - 1) / kThreads);
  // stages whose butterflies span 2^kLocalLog points or more run one launch
  // each; the rest, with the rounding, in one launch
  const int    k     = std::min(lg, kLocalLog);
  const size_t smem  = ((size_t)1 << k) * sizeof(double2);
  static bool  attr_done = false;
  if (!attr_done) {
    CUDA_CHECK(cudaFuncSetAttribute(embed_inv_local, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)(((size_t)1 << kLocalLog) * sizeof(double2))));
    attr_done = true;
  }
  prof_before(KID_ENCODE);
  for (int logm = lg; logm > k; logm--)
    embed_inv_stage<<<half_blocks, kThreads, 0, c->stream>>>(v, t->roots, t->rot_group, slots, logm,
                                                             2 * n);
  if (gap > 1) CUDA_CHECK(cudaMemsetAsync(d_msg, 0, (size_t)n * sizeof(int64_t), c->stream));
  const uint32_t threads = std::min(1024u, std::max(32u, 1u << (k > 0 ? k - 1 : 0)));
  embed_inv_local<<<slots >> k, threads, smem, c->stream>>>(
      d_msg, v, t->roots, t->rot_group, slots, lg, k, 2 * n, gap,
      std::pow(2.0, (double)c->sf_bits));
  prof_after(KID_ENCODE, 1);
  c->launches += (lg - k) + 1;
  CUDA_CHECK(cudaGetLastError());
  CUDA_CHECK(dev_free(v, c->stream));
  if (d_reals) CUDA_CHECK(dev_free(d_reals, c->stream));
}

}  // namespace fhert
