// Stand-alone probe (not part of libFHErt_b200.so): what the integer pipes of
// the GPU give the Shoup butterfly of the transforms.
//
//   python -m ace_compiler_b200.build --probes && ace_compiler_b200/probe_butterfly.bin
//
// Part 1: cycles per warp instruction per SM sub-partition for the PTX
// instructions the butterflies are made of (8 independent chains per thread,
// 8 warps per sub-partition).
// Part 2: butterflies per second of register-only loops (8 values per thread,
// three stages = 12 butterflies per round, no memory traffic) for the
// butterfly forms considered for csrc/ntt_kernels.cuh; each form is checked on
// 256 random pairs against 128-bit host arithmetic (same residue class, bound
// of the result).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
typedef unsigned long long u64;
typedef unsigned int u32;
typedef unsigned __int128 u128;
#define CK(x)                                                                         \
  do {                                                                                \
    cudaError_t e = (x);                                                              \
    if (e != cudaSuccess) {                                                           \
      printf("CUDA %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__);        \
      exit(1);                                                                        \
    }                                                                                 \
  } while (0)

// ---- part 1 -----------------------------------------------------------------
constexpr int P_ITERS = 2048, P_ILP = 8;

template <int OP>
__global__ void probe(u64* out, u64 seed, long long* cyc) {
  u64 x[P_ILP];
  u32 a = (u32)seed * (threadIdx.x + 1) | 1, b = (u32)(seed >> 32) + threadIdx.x;
  u64 A = seed * (threadIdx.x + 3);
#pragma unroll
  for (int i = 0; i < P_ILP; i++) x[i] = seed + i * 77 + threadIdx.x;
  __syncthreads();
  long long t0 = clock64();
  for (int it = 0; it < P_ITERS; it++) {
#pragma unroll
    for (int i = 0; i < P_ILP; i++) {
      if (OP == 0) asm volatile("mad.wide.u32 %0, %1, %2, %0;" : "+l"(x[i]) : "r"(a), "r"(b));
      if (OP == 1) { u32 lo = (u32)x[i]; asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(lo) : "r"(a), "r"(b)); x[i] = lo; }
      if (OP == 2) { u32 lo = (u32)x[i]; asm volatile("mul.hi.u32 %0, %0, %1;" : "+r"(lo) : "r"(a)); x[i] = lo | 1; }
      if (OP == 3) asm volatile("add.u64 %0, %0, %1;" : "+l"(x[i]) : "l"(A));
      if (OP == 4) { u32 lo = (u32)x[i]; asm volatile("add.u32 %0, %0, %1;" : "+r"(lo) : "r"(a)); x[i] = lo; }
      if (OP == 5) asm volatile("mul.hi.u64 %0, %0, %1;" : "+l"(x[i]) : "l"(A));
      if (OP == 6) asm volatile("mul.lo.u64 %0, %0, %1;" : "+l"(x[i]) : "l"(A));
    }
  }
  long long t1 = clock64();
  u64 s = 0;
#pragma unroll
  for (int i = 0; i < P_ILP; i++) s ^= x[i];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
  if (threadIdx.x == 0 && blockIdx.x == 0) *cyc = t1 - t0;
}

template <int OP>
void run_probe(const char* name, u64* d_out, long long* d_cyc) {
  const int warps_per_smsp = 8, threads = warps_per_smsp * 4 * 32;
  for (int rep = 0; rep < 2; rep++) {
    probe<OP><<<148, threads>>>(d_out, 0x9e3779b97f4a7c15ull, d_cyc);
    CK(cudaDeviceSynchronize());
  }
  long long c;
  CK(cudaMemcpy(&c, d_cyc, 8, cudaMemcpyDeviceToHost));
  printf("%-14s %6.2f cycles per warp instruction per sub-partition\n", name,
         (double)c / ((double)P_ITERS * P_ILP * warps_per_smsp));
}

// ---- part 2 -----------------------------------------------------------------
struct Tw { u64 w, wp; };
struct Q { u64 q, nq, q2, q4; };
__device__ __forceinline__ u32 lo32(u64 x) { return (u32)x; }
__device__ __forceinline__ u32 hi32(u64 x) { return (u32)(x >> 32); }

__device__ __forceinline__ u64 chain(u64 b, u64 w, u64 h, u64 nq) {  // b*w + h*nq mod 2^64
  u64 t;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(t) : "r"(lo32(b)), "r"(lo32(w)));
  asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(t) : "r"(lo32(h)), "r"(lo32(nq)));
  u32 tl = lo32(t), th = hi32(t);
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(lo32(b)), "r"(hi32(w)));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(hi32(b)), "r"(lo32(w)));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(lo32(h)), "r"(hi32(nq)));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(th) : "r"(hi32(h)), "r"(lo32(nq)));
  return ((u64)th << 32) | tl;
}
__device__ __forceinline__ u64 mulhi_under(u64 b, u64 p) {  // floor(b*p/2^64) - {0,1,2}
  u32 m1 = __umulhi(hi32(b), lo32(p)), m2 = __umulhi(lo32(b), hi32(p));
  u64 t;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(t) : "r"(hi32(b)), "r"(hi32(p)));
  return t + m1 + m2;
}

template <int V>
__device__ __forceinline__ void bf(u64& a, u64& b, const Tw& t, const Q& m) {
  if (V == 0) {  // Harvey, exact quotient, compiler's arithmetic (values in [0, 4q))
    u64 x = a >= m.q2 ? a - m.q2 : a;
    u64 v = b * t.w - __umul64hi(b, t.wp) * m.q;
    a = x + v; b = x - v + m.q2;
  } else if (V == 1) {  // no range correction, exact quotient, accumulate chain
    u64 v = chain(b, t.w, __umul64hi(b, t.wp), m.nq);
    u64 x = a; a = x + v; b = x - v + m.q2;
  } else if (V == 2) {  // no range correction, three-product quotient (the narrow-prime form)
    u64 v = chain(b, t.w, mulhi_under(b, t.wp), m.nq);
    u64 x = a; a = x + v; b = x - v + m.q4;
  } else if (V == 3) {  // correction against 4q, three-product quotient (the wide-prime form)
    u64 x = a >= m.q4 ? a - m.q4 : a;
    u64 v = chain(b, t.w, mulhi_under(b, t.wp), m.nq);
    a = x + v; b = x - v + m.q4;
  } else if (V == 10) {  // inverse, Harvey, compiler's arithmetic
    u64 s = a + b, d = a - b + m.q2;
    a = s >= m.q2 ? s - m.q2 : s;
    b = d * t.w - __umul64hi(d, t.wp) * m.q;
  } else if (V == 11) {  // inverse, no correction, three-product quotient
    u64 s = a + b, d = a - b + m.q4;
    a = s; b = chain(d, t.w, mulhi_under(d, t.wp), m.nq);
  } else {  // inverse, correction against 4q, three-product quotient
    u64 s = a + b, d = a - b + m.q4;
    a = s >= m.q4 ? s - m.q4 : s;
    b = chain(d, t.w, mulhi_under(d, t.wp), m.nq);
  }
}

constexpr int B_ITERS = 512;

template <int V>
__global__ void __launch_bounds__(256) loop(u64* out, const Tw* tw, u64 q) {
  Q m{q, 0 - q, 2 * q, 4 * q};
  u64 x[8];
  Tw t[7];
#pragma unroll
  for (int i = 0; i < 7; i++) t[i] = tw[(threadIdx.x * 7 + i) & 1023];
#pragma unroll
  for (int i = 0; i < 8; i++) x[i] = out[threadIdx.x * 8 + i] % q;
  for (int it = 0; it < B_ITERS; it++) {
#pragma unroll
    for (int j = 0; j < 4; j++) bf<V>(x[j], x[j + 4], t[0], m);
#pragma unroll
    for (int j = 0; j < 2; j++) { bf<V>(x[j], x[j + 2], t[1], m); bf<V>(x[j + 4], x[j + 6], t[2], m); }
#pragma unroll
    for (int j = 0; j < 4; j++) bf<V>(x[2 * j], x[2 * j + 1], t[3 + j], m);
  }
#pragma unroll
  for (int i = 0; i < 8; i++) out[(blockIdx.x * blockDim.x + threadIdx.x) * 8 + i] = x[i];
}

template <int V>
__global__ void one(u64* io, Tw t, u64 q) {
  Q m{q, 0 - q, 2 * q, 4 * q};
  u64 a = io[2 * threadIdx.x], b = io[2 * threadIdx.x + 1];
  bf<V>(a, b, t, m);
  io[2 * threadIdx.x] = a; io[2 * threadIdx.x + 1] = b;
}

static u64 mulmod(u64 a, u64 b, u64 q) { return (u64)((u128)a * b % q); }

template <int V>
void run_bf(const char* name, u64* d_out, Tw* d_tw, u64 q, bool inverse, u64 in_mult) {
  u64 h[512], g[512];
  Tw t; t.w = 0x123456789abcdefull % q; t.wp = (u64)(((u128)t.w << 64) / q);
  srand(V + 1);
  for (int i = 0; i < 512; i++) {
    u64 r = ((u64)rand() << 33) ^ ((u64)rand() << 11) ^ rand();
    h[i] = i < 8 ? q * in_mult - 1 - i : i < 12 ? 0 : r % (q * in_mult);
  }
  u64* d_io; CK(cudaMalloc(&d_io, sizeof(h)));
  CK(cudaMemcpy(d_io, h, sizeof(h), cudaMemcpyHostToDevice));
  one<V><<<1, 256>>>(d_io, t, q);
  CK(cudaMemcpy(g, d_io, sizeof(h), cudaMemcpyDeviceToHost));
  int bad = 0; u64 maxmult = 0;
  for (int i = 0; i < 256; i++) {
    u64 a = h[2 * i] % q, b = h[2 * i + 1] % q, ea, eb;
    if (!inverse) { u64 v = mulmod(b, t.w, q); ea = (a + v) % q; eb = (a + q - v) % q; }
    else { ea = (a + b) % q; eb = mulmod((a + q - b) % q, t.w, q); }
    bad += g[2 * i] % q != ea || g[2 * i + 1] % q != eb;
    maxmult = g[2 * i] / q > maxmult ? g[2 * i] / q : maxmult;
    maxmult = g[2 * i + 1] / q > maxmult ? g[2 * i + 1] / q : maxmult;
  }
  cudaFree(d_io);
  const int ctas = 148 * 2, threads = 256;  // 16 warps per SM
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  loop<V><<<ctas, threads>>>(d_out, d_tw, q);
  cudaEventRecord(e0);
  loop<V><<<ctas, threads>>>(d_out, d_tw, q);
  cudaEventRecord(e1);
  CK(cudaDeviceSynchronize());
  float ms; cudaEventElapsedTime(&ms, e0, e1);
  double gbf = (double)ctas * threads * B_ITERS * 12 / (ms * 1e-3) / 1e9;
  // one limb of N = 2^16 is 16 stages x 32768 butterflies
  printf("%-52s wrong %d  result < %llu q  %7.1f G butterflies/s = %.3f us per 2^16-point limb\n",
         name, bad, maxmult + 1, gbf, 16.0 * 32768 / (gbf * 1e3));
}

int main() {
  u64* d_out; Tw* d_tw; long long* d_cyc;
  size_t n = (size_t)148 * 16 * 512 * 8;
  CK(cudaMalloc(&d_out, n * 8)); CK(cudaMemset(d_out, 0x5a, n * 8));
  CK(cudaMalloc(&d_cyc, 8));
  printf("-- integer pipes\n");
  run_probe<0>("mad.wide.u32", d_out, d_cyc);
  run_probe<1>("mad.lo.u32", d_out, d_cyc);
  run_probe<2>("mul.hi.u32", d_out, d_cyc);
  run_probe<4>("add.u32", d_out, d_cyc);
  run_probe<3>("add.u64", d_out, d_cyc);
  run_probe<6>("mul.lo.u64", d_out, d_cyc);
  run_probe<5>("mul.hi.u64", d_out, d_cyc);
  u64 q = 0x3ffffffffe80001ull;  // an odd 58-bit modulus; primality does not matter here
  Tw h[1024];
  for (int i = 0; i < 1024; i++) { h[i].w = (0x9e3779b97f4a7c15ull * (i + 1)) % q; h[i].wp = (u64)(((u128)h[i].w << 64) / q); }
  CK(cudaMalloc(&d_tw, sizeof(h))); CK(cudaMemcpy(d_tw, h, sizeof(h), cudaMemcpyHostToDevice));
  printf("-- butterflies, registers only\n");
  run_bf<0>("forward, Harvey, exact quotient (compiler arithmetic)", d_out, d_tw, q, false, 4);
  run_bf<1>("forward, no correction, exact quotient, chain", d_out, d_tw, q, false, 8);
  run_bf<2>("forward, no correction, 3-product quotient, chain", d_out, d_tw, q, false, 8);
  run_bf<3>("forward, correction vs 4q, 3-product quotient, chain", d_out, d_tw, q, false, 8);
  run_bf<10>("inverse, Harvey, exact quotient (compiler arithmetic)", d_out, d_tw, q, true, 2);
  run_bf<11>("inverse, no correction, 3-product quotient, chain", d_out, d_tw, q, true, 4);
  run_bf<12>("inverse, correction vs 4q, 3-product quotient, chain", d_out, d_tw, q, true, 4);
  return 0;
}
