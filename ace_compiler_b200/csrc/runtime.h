// Internal declarations shared by the translation units of libFHErt_b200.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <vector>

#include "../../include/fhert_b200.h"
#include "modarith.cuh"

namespace fhert {

typedef unsigned __int128 u128;

#define FHERT_ASSERT(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) {                                                \
      std::fprintf(stderr, "libFHErt_b200: %s:%d: ", __FILE__, __LINE__); \
      std::fprintf(stderr, __VA_ARGS__);                          \
      std::fprintf(stderr, "\n");                                 \
      std::abort();                                               \
    }                                                             \
  } while (0)

#define CUDA_CHECK(call)                                                   \
  do {                                                                     \
    cudaError_t err_ = (call);                                             \
    FHERT_ASSERT(err_ == cudaSuccess, "CUDA error %s at %s",               \
                 cudaGetErrorString(err_), #call);                         \
  } while (0)

// Largest number of limbs (Q plus P) a single launch descriptor can carry.
constexpr int kMaxLimbs = 96;
// Largest digit size alpha, and largest number of special primes K.
constexpr int kMaxDigit = 16;

// One limb of a batched launch: limb offsets (in units of N words) into the
// base pointers of the launch, and the prime it lives under.
struct LimbRef {
  uint16_t a;      // first operand / source
  uint16_t b;      // second operand
  uint16_t dst;    // result
  uint16_t prime;  // index into the context's prime list (Q then P)
};

struct LimbBatch {
  int     count;
  LimbRef limb[kMaxLimbs];
};

// Twiddle entry: root power and its Shoup companion floor(w * 2^64 / q).
struct __align__(16) Twiddle {
  u64 w;
  u64 wp;
};

struct Context {
  uint32_t N     = 0;
  uint32_t logN  = 0;
  int      L     = 0;  // Q primes
  int      K     = 0;  // P primes
  int      dnum  = 0;
  int      alpha = 0;  // primes per digit
  size_t   q0_bits = 0, sf_bits = 0, hamming_weight = 0, input_level = 0;
  std::vector<u64>     primes;   // L + K
  std::vector<u64>     psi;      // 2N-th root per prime
  std::vector<MODULUS> moduli;   // host ABI structs, Q then P, contiguous
  // host twiddle tables (kept for Fhert_get_ntt_tables and host-side NTT)
  std::vector<std::vector<Twiddle>> h_fwd, h_inv;

  // device tables
  DevModulus* d_mod = nullptr;   // [L+K]
  Twiddle*    d_fwd = nullptr;   // [L+K][N], index m+i as in ntt.c:167
  Twiddle*    d_inv = nullptr;   // [L+K][N]
  // last inverse stage with N^-1 folded in: (N^-1, (rou_inv[1] * N^-1))
  Twiddle*    d_inv_last = nullptr;  // [L+K][2]

  // rescale constants for dropping prime l (1 <= l < L), row l, column i < l:
  //   ql_inv[l*L+i]   = q_l^-1 mod q_i                       (crt.c:291-353)
  //   ql_neg[l*L+i]   = floor(Qhat_l * (Qhat_l^-1 mod q_l) / q_l) mod q_i
  //   ql_mod[l*L+i]   = q_l mod q_i
  Twiddle* d_ql_inv = nullptr;
  Twiddle* d_ql_neg = nullptr;
  u64*     d_ql_mod = nullptr;

  // ModDown constants (crt.c:357-414): phat_inv[k] = (P/p_k)^-1 mod p_k,
  // phat_mod_q[i*K+k] = (P/p_k) mod q_i, p_inv[i] = P^-1 mod q_i
  Twiddle* d_phat_inv   = nullptr;
  u64*     d_phat_mod_q = nullptr;
  Twiddle* d_p_inv      = nullptr;
  // Extend: P mod q_i
  Twiddle* d_p_mod_q = nullptr;

  // ModUp constants per (level, digit), built on demand (crt.c:459-566)
  struct ModUpTable {
    int  digit_len = 0;          // limbs of the digit present at this level
    int  out_count = 0;          // complement limbs (other Q limbs + P)
    Twiddle* d_hat_inv = nullptr;  // [digit_len] (Qhat_j,i)^-1 mod q_i
    u64* d_hat_mod = nullptr;    // [digit_len][L+K] indexed by prime
  };
  std::map<std::pair<int, int>, ModUpTable> modup;

  // automorphism index tables by automorphism index k (NTT order)
  std::map<uint32_t, uint32_t*> auto_tables;
  // rotation index -> automorphism index
  std::map<int32_t, uint32_t> auto_idx;
  // keys by automorphism index; 0 = relinearisation key
  std::map<uint32_t, SWITCH_KEY*> keys;

  cudaStream_t stream = nullptr;
  uint64_t     launches = 0;
  // scratch polynomial storage reused by the fused operations
  int64_t* scratch      = nullptr;
  size_t   scratch_words = 0;
};

// Optional per-kernel timing: when enabled every launch is bracketed by CUDA
// events on the library stream and the elapsed times are summed per kernel.
enum KernelId {
  KID_NTT_STRIDED, KID_NTT_CONTIG, KID_NTT_SMALL, KID_INTT_STRIDED, KID_INTT_CONTIG,
  KID_INTT_SMALL, KID_ELEMENTWISE, KID_AUTOMORPHISM, KID_MUL_CONST, KID_RESCALE_LIFT,
  KID_RESCALE_COMBINE, KID_BASE_CONV, KID_MODDOWN_COMBINE, KID_INNER_PRODUCT, KID_MOD_RAISE,
  KID_COUNT
};
extern const char* const kKernelNames[KID_COUNT];
void prof_before(KernelId id);
void prof_after(KernelId id, int limbs);  // limbs = limbs the launch covered

Context* ctx();               // aborts when no context exists
Context* ctx_or_null();
int64_t* scratch(size_t words);  // stream-ordered scratch, grows on demand
void     prof_begin();
size_t   prof_end(char* buf, size_t cap);

// ---- host number theory (context.cu) ----
u64  mulmod(u64 a, u64 b, u64 q);
u64  powmod(u64 a, u64 e, u64 q);
u64  invmod(u64 a, u64 q);
bool is_prime(u64 n);
u64  shoup(u64 w, u64 q);
const Context::ModUpTable& modup_table(Context* c, int level, int digit);
uint32_t* auto_table(Context* c, uint32_t k);

// ---- context.cu ----
Context* create_context(const CKKS_PARAMS* p);
void     destroy_context();
uint32_t auto_index_for(Context* c, int32_t rot_idx);
DevModulus make_dev_modulus(u64 q, uint32_t n);

// ---- kernels (launch wrappers; all queue on ctx()->stream) ----
// in/out are base pointers; limb.a selects the source limb, limb.dst the result
void launch_ntt(const int64_t* in, int64_t* out, const LimbBatch& b, bool inverse);

enum EwOp { EW_ADD, EW_SUB, EW_MUL, EW_MULADD, EW_ADD_SCALAR, EW_MUL_SCALAR };
// res[dst] = a[a] op b[b]   (EW_MULADD: res[dst] += a*b; scalar ops ignore b)
void launch_elementwise(EwOp op, int64_t* res, const int64_t* a, const int64_t* b,
                        int64_t scalar, const LimbBatch& batch);
// res[dst][i] = val[a][table[i]]
void launch_automorphism(int64_t* res, const int64_t* val, const uint32_t* table,
                         const LimbBatch& batch);
// res[dst] = val[a] * c[prime] with per-prime Shoup constants consts[prime]
void launch_mul_const(int64_t* res, const int64_t* val, const Twiddle* consts,
                      const LimbBatch& batch);

// Rescale pieces (rns_poly.c:310-404).  `last` = coefficient form of the limb
// being dropped (prime index l).
//   lift:    tmp[dst] = switch_modulus(last, q_l -> q_i) * ql_neg[l][i]
//   combine: res[dst] = poly[a] * ql_inv[l][i] + tmp[b]
void launch_rescale_lift(int64_t* tmp, const int64_t* last, int l, const LimbBatch& batch);
void launch_rescale_combine(int64_t* res, const int64_t* poly, const int64_t* tmp, int l,
                            const LimbBatch& batch);

// Approximate base conversion (rns_poly.c:218-242, rns_poly_impl.c:287-339):
//   y_i = in[i] * inv[i] mod p_in(i);  out[o] = (sum_i y_i * mat(i,o)) mod p_out(o)
// mat(i,o) = mat[i*in_stride + out.limb[o].b*out_stride]; in.limb[i].a addresses the
// source limb, out.limb[o].dst the result limb.
void launch_base_conv(int64_t* out, const int64_t* in, const LimbBatch& in_limbs,
                      const LimbBatch& out_limbs, const Twiddle* inv, const u64* mat,
                      int in_stride, int out_stride);
// ModDown tail: res[dst] = (x[a] - t[b]) * P^-1 mod q_i
void launch_moddown_combine(int64_t* res, const int64_t* x, const int64_t* t,
                            const LimbBatch& batch);

// Key inner product over `parts` digits: for every limb of the batch
//   acc0[dst] = sum_j ext_j[a] * key0_j[b],  acc1[dst] = sum_j ext_j[a] * key1_j[b]
// acc1/key1 may be null (single product).
constexpr int kMaxParts = 16;
struct InnerArgs {
  int        parts;
  const u64* ext[kMaxParts];
  const u64* key0[kMaxParts];
  const u64* key1[kMaxParts];
};
void launch_inner_product(int64_t* acc0, int64_t* acc1, const InnerArgs& args,
                          const LimbBatch& batch);
// Mod-raise (rns_poly.c:1101-1125): res[dst] = switch_modulus(src, q_0 -> q_i)
void launch_mod_raise(int64_t* res, const int64_t* src, const LimbBatch& batch);

}  // namespace fhert
