// Internal declarations shared by the translation units of libFHErt_b200.
#pragma once
#include <cuda_runtime.h>

#include <complex>
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
constexpr int kMaxLimbs = 192;
// Largest digit size alpha, and largest number of special primes K.
constexpr int kMaxDigit = 16;

// One limb of a batched launch: limb offsets (in units of N words) into the
// base pointers of the launch, the prime it lives under, and which of the two
// base pointers each operand uses (sel bit 0: a, bit 1: b, bit 2: dst), so
// that one launch can cover both polynomials of a ciphertext.
struct LimbRef {
  uint16_t a;      // first operand / source
  uint16_t b;      // second operand
  uint16_t dst;    // result
  uint8_t  prime;  // index into the context's prime list (Q then P)
  uint8_t  sel;
};

struct LimbBatch {
  int     count;
  LimbRef limb[kMaxLimbs];
};

// Up to two base pointers for one operand of a batched launch.
struct Ptr2 {
  u64* p[2];
};
inline Ptr2 ptr2(const void* a, const void* b = nullptr) {
  Ptr2 r;
  r.p[0] = (u64*)a;
  r.p[1] = (u64*)b;
  return r;
}

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
  bool     primes_below_2_60 = false;  // enables the carry-free 32-bit-half accumulators
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
  // secret key in coefficient and NTT form (L Q limbs + K P limbs), public key
  // (L limbs); empty until generate_keys ran
  POLYNOMIAL sk_s{}, sk_ntt{};
  PUBLIC_KEY pk{};
  // encoder tables (util/src/ntt.c:562-590): 2N-th complex roots, powers of 5
  std::vector<double>   fft_rou_re, fft_rou_im;
  std::vector<uint32_t> fft_rot_group;
  // device copies of the encoder's roots of unity, owned by encode_gpu.cu
  void* encode_tables = nullptr;
  // transforms of the monomials the bootstrap multiplies by, owned by bootstrap.cu
  void* monomials = nullptr;
  // bootstrapping precomputation per slot count, owned by bootstrap.cu
  void* bootstrap = nullptr;
  // recorded per-limb vector operations awaiting replay (hw_queue.cu)
  struct HwQueue* hw_queue   = nullptr;
  bool            hw_pending = false;
  bool            draining   = false;  // deferred work is being launched right now
  uint64_t        hw_batched_limbs = 0;
  // a Mod_down / Rescale whose device work waits for its sibling (the second
  // polynomial of the same ciphertext usually follows at once); see api.cu
  struct {
    int            kind = 0;  // 0 none, 1 Mod_down, 2 Rescale
    int64_t*       res  = nullptr;
    const int64_t* src  = nullptr;
    size_t         level = 0;
    int            p_limb = 0;
    bool           is_ntt = true;
  } pair_wait;
  // All digits of the polynomial a program is raising, made at its first
  // Decomp_modup call and handed out by the following ones (api.cu).  The
  // storage belongs to the recorder and is released by the next replay.
  struct {
    bool           valid = false;
    const int64_t* src   = nullptr;  // the polynomial's limbs
    size_t         level = 0;
    bool           is_ntt = true;
    int            parts = 0;
    int64_t*       digits = nullptr;  // [parts][level + K] limbs
  } raised;
  // bytes moved between host and device since the context was made
  uint64_t h2d_bytes = 0, d2h_bytes = 0;

  cudaStream_t stream = nullptr;
  uint64_t     launches = 0;
  // scratch polynomial storage reused by the fused operations
  int64_t* scratch      = nullptr;
  size_t   scratch_words = 0;
  // scratch blocks of a captured run, used in turn: with one block every call
  // that needs scratch would have to wait for the one before it
  static constexpr int kScratchRing = 8;
  int64_t* ring[kScratchRing]       = {};
  size_t   ring_words[kScratchRing] = {};
  unsigned ring_next                = 0;
};

// Optional per-kernel timing: when enabled every launch is bracketed by CUDA
// events on the library stream and the elapsed times are summed per kernel.
enum KernelId {
  KID_NTT_STRIDED, KID_NTT_CONTIG, KID_NTT_SMALL, KID_INTT_STRIDED, KID_INTT_CONTIG,
  KID_INTT_SMALL, KID_ELEMENTWISE, KID_AUTOMORPHISM, KID_MUL_CONST, KID_RESCALE_LIFT,
  KID_RESCALE_COMBINE, KID_BASE_CONV, KID_MODDOWN_COMBINE, KID_INNER_PRODUCT, KID_MOD_RAISE,
  KID_TENSOR, KID_HW_BATCH, KID_ENCODE,
  KID_COUNT
};
extern const char* const kKernelNames[KID_COUNT];
void prof_before(KernelId id);
void prof_after(KernelId id, int limbs);  // limbs = limbs the launch covered

Context* ctx();               // aborts when no context exists; replays recorded Hw_* calls
Context* ctx_noflush();       // same without the replay (accessors, the Hw_* calls themselves)

// cudaMemcpyAsync that also keeps the context's host<->device byte counters
inline cudaError_t counted_copy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind,
                                cudaStream_t stream);
Context* ctx_or_null();
int64_t* scratch(size_t words);  // stream-ordered scratch, grows on demand
void     prof_begin();
bool     prof_running();
size_t   prof_end(char* buf, size_t cap);

// ---- host number theory (context.cu) ----
u64  mulmod(u64 a, u64 b, u64 q);
u64  powmod(u64 a, u64 e, u64 q);
u64  invmod(u64 a, u64 q);
bool is_prime(u64 n);
u64  shoup(u64 w, u64 q);
const Context::ModUpTable& modup_table(Context* c, int level, int digit);
uint32_t* auto_table(Context* c, uint32_t k);

// ---- sampling.cu (host randomness, same generators as the CPU runtime) ----
void seed_prng(const uint32_t seed[16], u64 counter, int64_t fake_time_us);
void release_prng();
void sample_uniform(int64_t* out, size_t n, u64 upper_bound);
void sample_ternary(int64_t* out, size_t n, size_t hamming_weight);
void sample_triangle(int64_t* out, size_t n);

// ---- client.cu ----
void generate_keys(Context* c);
void free_keys(Context* c);
void generate_bootstrap_keys(Context* c, const std::vector<int32_t>& rotations);
SWITCH_KEY* key_slot(Context* c, uint32_t key_id, bool create);
// msg[N] (signed values, negatives stored as Max64 + x) -> residues per limb,
// times scale_pow[prime] when given                       (crt.c:1153-1221)
void launch_encode_split(int64_t* poly, const int64_t* msg, const u64* scale_pow,
                         const LimbBatch& batch);
// small signed samples (-1, 0, 1) -> residues per limb (crt.c:1168-1172)
void launch_small_to_rns(int64_t* poly, const int64_t* vals, const LimbBatch& batch);

// ---- api.cu (batch builders shared with the bootstrapping code) ----
LimbBatch poly_batch(Context* c, POLY res, POLY a, POLY b, size_t level, size_t num_p);
LimbBatch both_polys(const LimbBatch& one);
void      ensure_poly(POLY res, uint32_t degree, size_t num_q, size_t num_p);

// ---- context.cu: device memory of the library stream ----
// All device work of the library runs on one stream, so a block handed back is
// safe to hand out again at once (whatever uses it next is queued behind
// whatever used it last).  Blocks are kept in per-size lists and only a size
// never seen before reaches the driver: the tens of thousands of polynomial
// allocations of a program cost no driver call and no pool bookkeeping.
// FHERT_POOL=0 sends every request to cudaMallocAsync / cudaFreeAsync instead.
cudaError_t dev_alloc(void** ptr, size_t bytes, cudaStream_t stream);
cudaError_t dev_free(void* ptr, cudaStream_t stream);
template <typename T>
inline cudaError_t dev_alloc(T** ptr, size_t bytes, cudaStream_t stream) {
  return dev_alloc(reinterpret_cast<void**>(ptr), bytes, stream);
}
void dev_release_all(cudaStream_t stream);  // gives every kept block back to the driver
// A second set of lists serves the requests made while a whole program run is
// captured for replay (program_api.cu): blocks the captured kernels use must
// never be handed to anybody else between two replays.  While the private mode
// is on, a size the private lists do not hold comes from cudaMalloc (legal
// inside a relaxed capture, unlike a stream-ordered allocation, which would
// become a node of the graph); a block goes back to the lists it came from
// whatever the mode.
void dev_private_mode(bool on);
bool dev_take_private(void* ptr);            // takes one given block out of the private lists
void dev_private_to_common(cudaStream_t s);  // ends the separation: every private block joins the common lists

// ---- capture_dag.cu: data-flow dependences of a captured program run ----
// What one launch (or one group of launches that run one after the other)
// reads and writes, as byte ranges; adjacent ranges are merged.
struct AccessSet {
  std::vector<std::pair<uintptr_t, uintptr_t>> reads, writes;
  static void add(std::vector<std::pair<uintptr_t, uintptr_t>>& v, const void* p, size_t bytes) {
    if (p == nullptr || bytes == 0) return;
    uintptr_t a = (uintptr_t)p, b = a + bytes;
    if (!v.empty() && v.back().second == a) v.back().second = b;
    else v.emplace_back(a, b);
  }
  void read(const void* p, size_t bytes) { add(reads, p, bytes); }
  void write(const void* p, size_t bytes) { add(writes, p, bytes); }
};
void dag_begin();  // at the start of a capture
void dag_end(uint64_t* nodes, uint64_t* edges, uint64_t* barriers, uint64_t* longest_chain = nullptr);
bool dag_active();
// Families of described launches.  Debugging aid: FHERT_DAG_SKIP=<sum of families>
// leaves those launches undescribed (they then order everything around them),
// which tells which description is at fault when a replay differs from a direct run.
enum DagFamily {
  DAG_ELEMENTWISE = 1, DAG_PER_LIMB_CONST = 2, DAG_AUTOMORPHISM = 4, DAG_TENSOR = 8,
  DAG_BASE_CONV = 16, DAG_INNER_PRODUCT = 32, DAG_NTT = 64, DAG_NTT_FUSED = 128,
  DAG_RECORDED_BATCH = 256, DAG_CLEAR = 512, DAG_COPY = 1024
};
bool dag_family_on(int family);
void dag_before(const AccessSet& a);  // sets the dependences of what is launched next
void dag_after();                     // takes note of the node(s) just captured
// Around a launch: fill `set` when `live`, commit(), launch; the destructor
// records the new node.  Launches without such a scope are ordered after all
// earlier and before all later ones.
struct DagScope {
  AccessSet set;
  bool      live;
  explicit DagScope(int family = 0) : live(dag_active() && dag_family_on(family)) {}
  void commit() { if (live) dag_before(set); }
  ~DagScope() { if (live) dag_after(); }
  // limbs of a batch: sel bit 0 picks the base of operand a, bit 1 of b, bit 2 of the result
  void batch(const LimbBatch& b, uint32_t n, const Ptr2* res, const Ptr2* a, const Ptr2* bb,
             bool res_is_read = false) {
    if (!live) return;
    const size_t w = (size_t)n * sizeof(u64);
    for (int i = 0; i < b.count; i++) {
      const LimbRef& lr = b.limb[i];
      if (a) set.read(a->p[lr.sel & 1] + (size_t)lr.a * n, w);
      if (bb) set.read(bb->p[(lr.sel >> 1) & 1] + (size_t)lr.b * n, w);
      if (res) {
        const u64* r = res->p[(lr.sel >> 2) & 1] + (size_t)lr.dst * n;
        set.write(r, w);
        if (res_is_read) set.read(r, w);
      }
    }
  }
};
// cudaMemsetAsync of device memory to zero on the library stream, described
inline cudaError_t zero_async(void* p, size_t bytes, cudaStream_t stream) {
  DagScope dag(DAG_CLEAR);
  if (dag.live) dag.set.write(p, bytes);
  dag.commit();
  return cudaMemsetAsync(p, 0, bytes, stream);
}

// ---- program_api.cu: a captured program run ----
// True while Run_main_graph is capturing the launches of a program run.
bool image_capturing();
// Ends a running capture because `why` cannot be captured (a copy from or to
// host memory, a synchronisation): what was captured so far is launched at
// once, the rest of the run is launched directly and the replay mode goes off.
void image_capture_break(const char* why);
// A copy of host data into pinned memory that lives as long as the captured
// run: a captured host-to-device copy reads the snapshot at every replay (the
// host data of a program run, constants and weights, are the same in every
// run).  nullptr when the budget for such snapshots is used up.
const void* image_capture_stage(const void* src, size_t bytes);
void image_replay_release();  // drops a captured run (context teardown)
// cudaStreamSynchronize that first ends a running capture
inline cudaError_t stream_sync(cudaStream_t stream) {
  if (image_capturing()) image_capture_break("a synchronisation");
  return cudaStreamSynchronize(stream);
}

// ---- encode_gpu.cu ----
// inverse embedding, scaling and rounding of `count` complex slot values (host)
// into the message polynomial d_msg (N int64 on the device)
// (`reals`, when given, replaces `values`: count real single-precision inputs)
void encode_message_on_device(Context* c, const std::complex<double>* values, size_t count,
                              uint32_t slots, int64_t* d_msg, const float* reals = nullptr);
void free_encode_tables(Context* c);

// ---- client_api.cu ----
// encode at sf_degree and level; slots = 0 means N/2, num_p = K also fills
// the special limbs (stored right behind the level Q limbs)
void encode_vector(Context* c, PLAIN plain, std::vector<std::complex<double>>& values,
                   uint32_t sf_degree, uint32_t level, uint32_t slots = 0, uint32_t num_p = 0,
                   const float* reals = nullptr, size_t real_count = 0);
// residues of one real value at the given scale on level Q limbs then num_p
// special limbs
std::vector<int64_t> encode_value(Context* c, double value, uint32_t level, double scale,
                                  uint32_t num_p);

// ---- hw_queue.cu: deferred per-limb vector operations ----
enum HwKind : uint8_t {
  HW_ADD, HW_SUB, HW_MUL, HW_MULADD, HW_ADD_SCALAR, HW_MUL_SCALAR, HW_ROTATE, HW_COPY,
  HW_MAC3  // res = c + a * b, made at replay from a product and the sum that consumes it
};
// records res = a (kind) b on one limb; false = recording is off, launch now
bool hw_record(Context* c, HwKind kind, int64_t* res, const int64_t* a, const int64_t* b,
               const uint32_t* table, int64_t scalar, int prime);
// the newest value of limb dst is the contents of src, private memory that no
// one else writes and that lives until the next replay; false = recording is off
bool hw_alias(Context* c, int64_t* dst, const int64_t* src);
void hw_free_after_replay(Context* c, void* device_memory);
bool hw_recording(Context* c);  // false under FHERT_EAGER_HW=1
void hw_replay(Context* c);   // run everything recorded so far
void pair_flush(Context* c);  // run a waiting Mod_down / Rescale on its own (api.cu)
void hw_release(Context* c);

// ---- program_api.cu ----
// FHERT_TRACE_SUMS=1: prints a checksum of the ciphertext's residues to stderr
void trace_sum(const char* what, CIPHER ciph);

// ---- data_file.cu ----
bool pt_cache_owns(const void* data);  // limb storage lent out by the plaintext cache

// ---- bootstrap.cu ----
// builds the linear-transform plaintexts and the rotation / conjugation keys
// for `slots` (0 = N/2) when the context is deep enough (ckks_context.c:239-262)
void prepare_bootstrap(Context* c, uint32_t slots);
// ciphertext-level pieces shared with ciph_api.cu (evaluator.c:113-286, 401-409)
void mul_const(Context* c, CIPHER res, CIPHER a, double value);
void add_const(Context* c, CIPHER res, CIPHER a, double value);
void mul_integer(Context* c, CIPHER res, CIPHER a, uint64_t power);
void mul_monomial(Context* c, CIPHER res, CIPHER a, uint32_t power);
void mod_switch(CIPHER ct);
void raise_from_level0(Context* c, CIPHER res, CIPHER ciph, uint32_t raise_level);
void shape_like(Context* c, CIPHER res, CIPHER a, double sf, uint32_t sf_degree);
LimbBatch ct_batch(Context* c, CIPHER res, CIPHER a);
void free_bootstrap(Context* c);

// ---- context.cu ----
Context* create_context(const CKKS_PARAMS* p);
void     destroy_context();
uint32_t auto_index_for(Context* c, int32_t rot_idx);
DevModulus make_dev_modulus(u64 q, uint32_t n);

// ---- kernels (launch wrappers; all queue on ctx()->stream) ----
// limb.a selects the source limb of in.p[sel&1], limb.dst the result limb of
// out.p[(sel>>2)&1]
void launch_ntt(Ptr2 in, Ptr2 out, const LimbBatch& b, bool inverse);
// Forward transform with the element-wise passes around it folded in (ring
// degrees above 4096 only: ntt_can_fuse).  The strided pass reads in[a] and
// writes limb k of `mid` (k = position in the batch), the contiguous pass reads
// mid[k] and writes out[dst].
//   prologue (pro_mul set): the source is the coefficient form of a dropped
//     limb modulo q_last; the value transformed under prime i is
//     switch_modulus(v, q_last -> q_i) * pro_mul[i]   (pro_mod[i] = q_last mod q_i)
//   epilogue: kind 1  out = aux[b] * epi_mul[i] + t      (rescale)
//             kind 2  out = (aux[b] - t) * epi_mul[i] (+ add[b])   (ModDown)
//     aux / add use base p[sel bit 1]
struct NttFuse {
  const Twiddle* pro_mul = nullptr;
  const u64*     pro_mod = nullptr;
  u64            q_last  = 0;
  int            epi_kind = 0;
  const Twiddle* epi_mul  = nullptr;
  Ptr2           aux{{nullptr, nullptr}};
  Ptr2           add{{nullptr, nullptr}};
};
bool ntt_can_fuse();
void launch_ntt_fused(Ptr2 in, int64_t* mid, Ptr2 out, const LimbBatch& b, const NttFuse& f);

enum EwOp { EW_ADD, EW_SUB, EW_MUL, EW_MULADD, EW_ADD_SCALAR, EW_MUL_SCALAR, EW_MULADD_SCALAR };
// res[dst] = a[a] op b[b]   (EW_MULADD: res[dst] += a*b; scalar ops ignore b;
// EW_MULADD_SCALAR: res[dst] += a*scalar)
void launch_elementwise(EwOp op, Ptr2 res, Ptr2 a, Ptr2 b, int64_t scalar,
                        const LimbBatch& batch);
// res[dst] = a[a] + per_limb[k] (or * when mul) for the k-th limb of the batch;
// the scalars are residues already reduced modulo the limb's prime
void launch_scalars(bool mul, Ptr2 res, Ptr2 a, const u64* per_limb, const LimbBatch& batch);
// res[dst][i] = val[a][table[i]]
void launch_automorphism(Ptr2 res, Ptr2 val, const uint32_t* table, const LimbBatch& batch);
// res[dst][i] = val[a][table[i]] + add[b][table[i]] on limbs whose sel has bit 1
// set (b indexes limbs of `add`), plain gather on the others
void launch_automorphism_add(Ptr2 res, Ptr2 val, const int64_t* add, const uint32_t* table,
                             const LimbBatch& batch);
// res[dst] = val[a] * consts[prime]
void launch_mul_const(Ptr2 res, Ptr2 val, const Twiddle* consts, const LimbBatch& batch);
// tensor product of two ciphertexts (evaluator.c:137-173), one launch:
// d0 = a0*b0, d1 = a0*b1 + a1*b0, d2 = a1*b1 on `level` limbs
void launch_tensor(int64_t* d0, int64_t* d1, int64_t* d2, const int64_t* a0,
                   const int64_t* a1, const int64_t* b0, const int64_t* b1, int level);
// the same on `count` limbs whose pointers already point at the first of them,
// under primes first_prime, first_prime + 1, ..
void launch_tensor_range(int64_t* d0, int64_t* d1, int64_t* d2, const int64_t* a0,
                         const int64_t* a1, const int64_t* b0, const int64_t* b1, int first_prime,
                         int count);

// Rescale pieces (rns_poly.c:310-404).  `last` holds, per selected base, the
// coefficient form of the limb being dropped (prime index l) at limb.b.
//   lift:    tmp[dst] = switch_modulus(last[b], q_l -> q_i) * ql_neg[l][i]
//   combine: res[dst] = poly[a] * ql_inv[l][i] + tmp[b]
void launch_rescale_lift(Ptr2 tmp, Ptr2 last, int l, const LimbBatch& batch);
void launch_rescale_combine(Ptr2 res, Ptr2 poly, Ptr2 tmp, int l, const LimbBatch& batch);

// Approximate base conversion (rns_poly.c:218-242, rns_poly_impl.c:287-339) of
// up to kMaxParts independent groups in one launch:
//   y_i = in[first_limb+i] * inv[i] mod p(first_prime+i)
//   out[limb(m)] = (sum_i y_i * mat[i*in_stride + prime(m)*out_stride]) mod prime(m)
// for every m in [0, out_total) outside [skip_start, skip_start+skip_len), where
// prime(m) = m < level ? m : L + m - level and limb(m) = m < level ? m : p_limb + m - level.
constexpr int kMaxParts = 16;
struct ConvGroup {
  const u64*     in;
  u64*           out;
  const Twiddle* inv;
  const u64*     mat;
  int            first_limb, first_prime, count;
  int            skip_start, skip_len;
};
struct ConvArgs {
  int       groups, level, out_total, p_limb, in_stride, out_stride;
  // bit m set: output m (index before the skip range is removed: Q limbs then
  // special limbs) is not computed -- it belongs to another GPU
  uint64_t  skip_mask = 0;
  ConvGroup g[kMaxParts];
};
void launch_base_conv(const ConvArgs& args);

// ModDown tail for up to two polynomials:
//   res[g][i] = (x[g][i] - t[g][i]) * P^-1 mod q_i (+ add[g][i] when add[g] is set)
struct ModDownTail {
  int        polys, level;
  uint64_t   skip_mask = 0;  // Q limbs left to another GPU
  u64*       res[2];
  const u64* x[2];
  const u64* t[2];
  const u64* add[2];
};
void launch_moddown_combine(const ModDownTail& args);
// Tail of the fused ModDown + Rescale in coefficient form (rns_poly.c:556-596):
// x = extended polynomial (level Q limbs), t = base conversion of its special
// limbs, both in coefficient form; with l = level - 1
//   last  = (x_l - t_l) * P^-1 mod q_l
//   res_i = ((x_i - t_i) * P^-1 - last) * q_l^-1 mod q_i      for i < l
// where `last` enters the subtraction as the integer in [0, q_l), uncentred,
// and the second step repeats the reference's 128-bit arithmetic on the
// (possibly slightly negative) difference exactly.
void launch_moddown_rescale(int64_t* res, const int64_t* x, const int64_t* t, int level);
// Rescale of `polys` polynomials in coefficient form, without centring the dropped limb
// (rns_poly.c:381-399); res may be x
void launch_rescale_coeff(Ptr2 res, Ptr2 x, int polys, int level);

// Key inner product over `parts` digits for limbs m in [0, level+K):
//   e_j = (in and m < level and m / alpha == j) ? in[m] : ext_ptr[j][m]
//   acc0[m] = sum_j e_j * key0_j[prime(m)],  acc1[m] = sum_j e_j * key1_j[prime(m)]
// acc/ext use level Q limbs followed directly by K P limbs; keys have their P
// limbs at limb index key_p_limb.  in may be null (ext then holds every limb);
// acc1/key1 may be null (single product).
struct InnerArgs {
  int        parts, level, alpha, key_p_limb;
  uint64_t   skip_mask;   // limbs (Q then special) left to another GPU
  const u64* in;
  const u64* ext_ptr[kMaxParts];
  const u64* key0[kMaxParts];
  const u64* key1[kMaxParts];
  u64*       acc0;
  u64*       acc1;
  int        acc_p_limb;  // limb index of the first P limb in acc
  int        ext_p_limb;  // limb index of the first P limb in ext
};
void launch_inner_product(const InnerArgs& args);
// Mod-raise (rns_poly.c:1101-1125): res[dst] = switch_modulus(src, q_0 -> q_i)
void launch_mod_raise(int64_t* res, const int64_t* src, const LimbBatch& batch);

}  // namespace fhert

namespace fhert {
inline cudaError_t counted_copy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind,
                                cudaStream_t stream) {
  Context* c = ctx_or_null();
  if (kind != cudaMemcpyDeviceToDevice && image_capturing()) {
    const void* kept = kind == cudaMemcpyHostToDevice ? image_capture_stage(src, bytes) : nullptr;
    if (kept != nullptr)
      src = kept;
    else
      image_capture_break(kind == cudaMemcpyHostToDevice
                              ? "more host data to copy than the snapshot budget (FHERT_REPLAY_STAGE_MB)"
                              : "a copy to host memory");
  }
  if (c != nullptr) {
    if (kind == cudaMemcpyHostToDevice) c->h2d_bytes += bytes;
    else if (kind == cudaMemcpyDeviceToHost) c->d2h_bytes += bytes;
  }
  DagScope dag(DAG_COPY);
  if (dag.live) {
    if (kind == cudaMemcpyDeviceToDevice) dag.set.read(src, bytes);
    dag.set.write(dst, bytes);
  }
  dag.commit();
  return cudaMemcpyAsync(dst, src, bytes, kind, stream);
}
}  // namespace fhert

// ---- api.cu: multi-polynomial building blocks shared with bootstrap.cu ------
extern "C" {
// ModUp of digits [part_begin, part_end) of a level-`level` polynomial at src:
// digit j lands at ext_base + (j - part_begin) * part_stride limbs, Q limbs at
// limb 0.., special limbs at limb p_limb..; the digit's own limbs are not written
void fhert_raise_parts(fhert::Context* c, const int64_t* src, bool is_ntt, size_t level,
                       int part_begin, int part_end, int64_t* ext_base, size_t part_stride,
                       int p_limb);
// ModDown of one or two extended polynomials (special limbs at ext_p_limb),
// optionally adding add[g] to the result
void fhert_mod_down_polys(fhert::Context* c, int npoly, int64_t* const res[2],
                          const int64_t* const ext[2], int ext_p_limb,
                          const int64_t* const add[2], size_t level, bool is_ntt);
// Rescale of one or two NTT-form polynomials from level to level - 1
void fhert_rescale_polys(fhert::Context* c, int npoly, int64_t* const res[2],
                         const int64_t* const poly[2], size_t level);
}
