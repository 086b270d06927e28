// Limb-sharded ciphertext operations: one ciphertext spread over several GPUs
// for latency (rotation / conjugation, multiplication with relinearisation,
// rescale).
//
// Every rank holds the ciphertext in the usual limb-major layout but only its
// own limbs are valid: Q limbs are dealt out in contiguous blocks of
// qb = ceil(L / world) of the context's L primes (the same owner at every
// level, so results feed the next operation without moving limbs), the special
// limbs in blocks of pb = ceil(K / world).
// All per-limb work (NTT, key inner product, automorphism, the element-wise
// tail of ModDown) stays local.  The two base conversions of a hybrid key
// switch need every limb of their input, so they are preceded by an exchange:
//   1. ModUp: the coefficient form of c1's Q limbs is all-gathered, then each
//      rank converts only into the extended limbs it owns;
//   2. ModDown: the coefficient form of the accumulators' special limbs is
//      all-gathered, then each rank converts only into the Q limbs it owns.
//   3. Rescale: the rank that owns the dropped limb broadcasts its coefficient
//      form; lift, transform and combine are local on the owned limbs.
// The phase functions (Fhert_shard_begin / _mid / _end2, _rescale_begin / _end)
// fill and consume exchange buffers laid out so that each rank's block is
// contiguous (block r = limbs [r*qb, (r+1)*qb)); a host may run the exchange
// itself between them (the one-GPU emulation in ace_compiler_b200/sharded.py
// copies blocks).  Fhert_shard_rotate / _mul_relin / _rescale run whole
// operations with the exchanges issued here as NCCL collectives on the library
// stream (Fhert_shard_comm_init; NCCL is loaded at run time, the library has
// no link-time dependency on it).  Received limbs land in local memory before
// any kernel reads them: no peer loads, no multicast.
//
// Arithmetic per limb is the same as in the single-GPU key switch
// (rns_poly.c:160-308, evaluator.c:411-522 of the CPU runtime), so the owned
// limbs of the result equal the single-GPU result bit for bit.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "runtime.h"

using namespace fhert;

namespace {

struct ShardState {
  int      rank, world;
  size_t   level;
  int      parts, qb, pb;
  int64_t* ext = nullptr;   // [parts][level + K][N] raised digits
  int64_t* acc = nullptr;   // [2][level + K][N] key inner products
  int64_t* conv = nullptr;  // [2][level][N] ModDown conversion results
};

inline int q_begin(const ShardState* s) { return std::min<int>((int)s->level, s->rank * s->qb); }
inline int q_end(const ShardState* s) { return std::min<int>((int)s->level, (s->rank + 1) * s->qb); }
inline int p_begin(const ShardState* s, int K) { return std::min(K, s->rank * s->pb); }
inline int p_end(const ShardState* s, int K) { return std::min(K, (s->rank + 1) * s->pb); }

// bit m set = extended limb m (Q limbs then special limbs) belongs to someone else
uint64_t foreign_mask(const ShardState* s, int K) {
  uint64_t owned = 0;
  for (int i = q_begin(s); i < q_end(s); i++) owned |= 1ull << i;
  for (int k = p_begin(s, K); k < p_end(s, K); k++) owned |= 1ull << (s->level + k);
  return ~owned;
}

void ntt_list(Ptr2 in, Ptr2 out, const std::vector<LimbRef>& limbs, bool inverse) {
  for (size_t off = 0; off < limbs.size(); off += kMaxLimbs) {
    LimbBatch b;
    b.count = (int)std::min((size_t)kMaxLimbs, limbs.size() - off);
    for (int i = 0; i < b.count; i++) b.limb[i] = limbs[off + i];
    launch_ntt(in, out, b, inverse);
  }
}

}  // namespace

extern "C" {

// Exchange geometry for a ciphertext of `level` limbs on `world` ranks:
// limbs per block of the Q exchange and of the special-limb exchange.
void Fhert_shard_blocks(size_t level, int world, int* q_block, int* p_block) {
  Context* c = ctx();
  (void)level;  // ownership does not depend on the level
  if (q_block) *q_block = (c->L + world - 1) / world;
  if (p_block) *p_block = (c->K + world - 1) / world;
}

void* Fhert_shard_begin(const int64_t* c1, size_t level, int rank, int world, int64_t* gather_q) {
  Context* c = ctx();
  FHERT_ASSERT(world >= 1 && rank >= 0 && rank < world, "bad rank %d of %d", rank, world);
  FHERT_ASSERT(level + c->K <= 64, "sharded key switch supports at most 64 extended limbs");
  ShardState* s = new ShardState();
  s->rank  = rank;
  s->world = world;
  s->level = level;
  s->parts = (int)std::min<size_t>((level + c->alpha - 1) / c->alpha, c->dnum);
  s->qb    = (c->L + world - 1) / world;
  s->pb    = (c->K + world - 1) / world;
  const size_t n = c->N, ext = level + c->K;
  CUDA_CHECK(dev_alloc(&s->ext, (size_t)s->parts * ext * n * sizeof(int64_t), c->stream));
  CUDA_CHECK(dev_alloc(&s->acc, 2 * ext * n * sizeof(int64_t), c->stream));
  CUDA_CHECK(dev_alloc(&s->conv, 2 * level * n * sizeof(int64_t), c->stream));
  // own Q limbs of c1 to coefficient form, straight into this rank's block of
  // the exchange buffer (limb i sits at index i of the gathered array)
  std::vector<LimbRef> own;
  for (int i = q_begin(s); i < q_end(s); i++)
    own.push_back(LimbRef{(uint16_t)i, 0, (uint16_t)i, (uint8_t)i, 0});
  ntt_list(ptr2(c1), ptr2(gather_q), own, true);
  return s;
}

// After the Q exchange: raise into the owned extended limbs, multiply with the
// key of rot_idx, and put the coefficient form of the owned special limbs of
// both accumulators into this rank's blocks of gather_p0 / gather_p1.
void Fhert_shard_mid(void* state, const int64_t* c1, const int64_t* gather_q, int32_t rot_idx,
                     int is_conj, int64_t* gather_p0, int64_t* gather_p1) {
  Context*    c = ctx();
  ShardState* s = (ShardState*)state;
  const int    K = c->K, level = (int)s->level;
  const size_t n = c->N, ext = s->level + K;
  const uint64_t foreign = foreign_mask(s, K);

  ConvArgs args;
  args.groups     = s->parts;
  args.level      = level;
  args.out_total  = level + K;
  args.p_limb     = level;
  args.in_stride  = c->L + K;
  args.out_stride = 1;
  args.skip_mask  = foreign;
  std::vector<LimbRef> raised;
  for (int part = 0; part < s->parts; part++) {
    const Context::ModUpTable& t     = modup_table(c, level, part);
    int                        start = c->alpha * part;
    ConvGroup&                 cg    = args.g[part];
    cg.in          = reinterpret_cast<const u64*>(gather_q);
    cg.out         = reinterpret_cast<u64*>(s->ext + (size_t)part * ext * n);
    cg.inv         = t.d_hat_inv;
    cg.mat         = t.d_hat_mod;
    cg.first_limb  = start;
    cg.first_prime = start;
    cg.count       = t.digit_len;
    cg.skip_start  = start;
    cg.skip_len    = t.digit_len;
    for (int m = 0; m < level + K; m++) {
      if ((foreign >> m) & 1) continue;
      if (m >= start && m < start + t.digit_len) continue;
      uint16_t limb  = (uint16_t)(part * ext + m);
      uint8_t  prime = (uint8_t)(m < level ? m : c->L + (m - level));
      raised.push_back(LimbRef{limb, 0, limb, prime, 0});
    }
  }
  launch_base_conv(args);
  ntt_list(ptr2(s->ext), ptr2(s->ext), raised, false);

  // is_conj selects the key: 0 rotation by rot_idx, 1 conjugation, 2 relinearisation
  uint32_t    k   = is_conj == 2 ? 0 : is_conj ? 2 * c->N - 1 : auto_index_for(c, rot_idx);
  SWITCH_KEY* key = key_slot(c, k, false);
  FHERT_ASSERT(key != nullptr, "cannot find the switch key %u", k);
  InnerArgs ia;
  std::memset(&ia, 0, sizeof(ia));
  ia.parts      = s->parts;
  ia.level      = level;
  ia.alpha      = c->alpha;
  ia.key_p_limb = c->L;
  ia.ext_p_limb = level;
  ia.acc_p_limb = level;
  ia.skip_mask  = foreign;
  ia.in         = reinterpret_cast<const u64*>(c1);
  for (int j = 0; j < s->parts; j++) {
    ia.ext_ptr[j] = reinterpret_cast<const u64*>(s->ext + (size_t)j * ext * n);
    ia.key0[j]    = reinterpret_cast<const u64*>(key->_parts[j]._p0._data);
    ia.key1[j]    = reinterpret_cast<const u64*>(key->_parts[j]._p1._data);
  }
  ia.acc0 = reinterpret_cast<u64*>(s->acc);
  ia.acc1 = reinterpret_cast<u64*>(s->acc + ext * n);
  launch_inner_product(ia);

  // own special limbs of both accumulators to coefficient form, into this
  // rank's blocks of the two exchange buffers (special limb k at index k)
  std::vector<LimbRef> sp;
  for (int g = 0; g < 2; g++)
    for (int kk = p_begin(s, K); kk < p_end(s, K); kk++)
      sp.push_back(LimbRef{(uint16_t)(g * ext + level + kk), 0, (uint16_t)kk, (uint8_t)(c->L + kk),
                           (uint8_t)(g ? 4 : 0)});
  ntt_list(ptr2(s->acc), ptr2(gather_p0, gather_p1), sp, true);
}

// After the special-limb exchange: ModDown into the owned Q limbs, add c0,
// apply the automorphism.  out0 / out1 use the full layout; only the owned
// limbs are written.  Releases the state.
void Fhert_shard_end2(void* state, const int64_t* add0, const int64_t* add1,
                      const int64_t* gather_p0, const int64_t* gather_p1, int32_t rot_idx,
                      int is_conj, int64_t* out0, int64_t* out1) {
  Context*    c = ctx();
  ShardState* s = (ShardState*)state;
  const int    K = c->K, level = (int)s->level;
  const size_t n = c->N, ext = s->level + K;
  uint64_t foreign_q = 0;
  for (int i = 0; i < level; i++)
    if (i < q_begin(s) || i >= q_end(s)) foreign_q |= 1ull << i;

  ConvArgs args;
  args.groups     = 2;
  args.level      = level;
  args.out_total  = level;
  args.p_limb     = 0;
  args.in_stride  = 1;
  args.out_stride = K;
  args.skip_mask  = foreign_q;
  for (int g = 0; g < 2; g++) {
    ConvGroup& cg  = args.g[g];
    cg.in          = reinterpret_cast<const u64*>(g ? gather_p1 : gather_p0);
    cg.out         = reinterpret_cast<u64*>(s->conv + (size_t)g * level * n);
    cg.inv         = c->d_phat_inv;
    cg.mat         = c->d_phat_mod_q;
    cg.first_limb  = 0;
    cg.first_prime = c->L;
    cg.count       = K;
    cg.skip_start  = 0;
    cg.skip_len    = 0;
  }
  launch_base_conv(args);
  std::vector<LimbRef> own;
  for (int g = 0; g < 2; g++)
    for (int i = q_begin(s); i < q_end(s); i++) {
      uint16_t t = (uint16_t)(g * level + i);
      own.push_back(LimbRef{t, 0, t, (uint8_t)i, 0});
    }
  ntt_list(ptr2(s->conv), ptr2(s->conv), own, false);

  // (acc - conv) * P^-1 (+ c0) over the owned limbs, in place in conv
  ModDownTail tail;
  tail.polys     = 2;
  tail.level     = level;
  tail.skip_mask = foreign_q;
  for (int g = 0; g < 2; g++) {
    tail.res[g] = reinterpret_cast<u64*>(s->conv + (size_t)g * level * n);
    tail.x[g]   = reinterpret_cast<const u64*>(s->acc + (size_t)g * ext * n);
    tail.t[g]   = reinterpret_cast<const u64*>(s->conv + (size_t)g * level * n);
    tail.add[g] = reinterpret_cast<const u64*>(g == 0 ? add0 : add1);
  }
  if (is_conj == 2) {  // relinearisation: no automorphism, the owned limbs go straight out
    tail.res[0] = reinterpret_cast<u64*>(out0);
    tail.res[1] = reinterpret_cast<u64*>(out1);
  }
  launch_moddown_combine(tail);
  if (is_conj == 2) {
    CUDA_CHECK(dev_free(s->ext, c->stream));
    CUDA_CHECK(dev_free(s->acc, c->stream));
    CUDA_CHECK(dev_free(s->conv, c->stream));
    delete s;
    return;
  }

  uint32_t  k = is_conj ? 2 * c->N - 1 : auto_index_for(c, rot_idx);
  LimbBatch ab;
  ab.count = 0;
  for (int g = 0; g < 2; g++)
    for (int i = q_begin(s); i < q_end(s); i++)
      ab.limb[ab.count++] = LimbRef{(uint16_t)(g * level + i), 0, (uint16_t)i, (uint8_t)i,
                                    (uint8_t)(g ? 4 : 0)};
  launch_automorphism(ptr2(out0, out1), ptr2(s->conv), auto_table(c, k), ab);

  CUDA_CHECK(dev_free(s->ext, c->stream));
  CUDA_CHECK(dev_free(s->acc, c->stream));
  CUDA_CHECK(dev_free(s->conv, c->stream));
  delete s;
}


void Fhert_shard_end(void* state, const int64_t* c0, const int64_t* gather_p0,
                     const int64_t* gather_p1, int32_t rot_idx, int is_conj, int64_t* out0,
                     int64_t* out1) {
  Fhert_shard_end2(state, c0, nullptr, gather_p0, gather_p1, rot_idx, is_conj, out0, out1);
}

// ---- rescale (rns_poly.c:310-404) on the owned limbs -------------------------

// The owner of limb level-1 puts the coefficient form of that limb of both
// polynomials into bcast[0..2N); returns 1 on the owner, 0 elsewhere.
int Fhert_shard_rescale_begin(const int64_t* c0, const int64_t* c1, size_t level, int rank,
                              int world, int64_t* bcast) {
  Context*  c  = ctx();
  const int l  = (int)level - 1;
  const int qb = (c->L + world - 1) / world;
  if (l / qb != rank) return 0;
  LimbBatch lb;
  lb.count = 2;
  for (int g = 0; g < 2; g++)
    lb.limb[g] = LimbRef{(uint16_t)l, 0, (uint16_t)g, (uint8_t)l, (uint8_t)g};
  launch_ntt(ptr2(c0, c1), ptr2(bcast), lb, true);
  return 1;
}

// After the broadcast: res_i = c_i * q_l^-1 + NTT_i(lift(last)) on the owned limbs i < level-1.
void Fhert_shard_rescale_end(const int64_t* c0, const int64_t* c1, size_t level, int rank,
                             int world, const int64_t* bcast, int64_t* res0, int64_t* res1) {
  Context*  c  = ctx();
  const int l  = (int)level - 1;
  const int qb = (c->L + world - 1) / world;
  const int lo = std::min(l, rank * qb), hi = std::min(l, (rank + 1) * qb);
  if (hi <= lo) return;
  const size_t n   = c->N;
  int64_t*     mid = nullptr;
  CUDA_CHECK(dev_alloc(&mid, (size_t)2 * (hi - lo) * n * sizeof(int64_t), c->stream));
  LimbBatch bt;
  bt.count = 0;
  for (int g = 0; g < 2; g++)
    for (int i = lo; i < hi; i++) {
      uint8_t sel = (uint8_t)(g ? (2 | 4) : 0);
      bt.limb[bt.count++] = LimbRef{(uint16_t)g, (uint16_t)i, (uint16_t)i, (uint8_t)i, sel};
    }
  if (ntt_can_fuse()) {
    NttFuse f;
    f.pro_mul  = c->d_ql_neg + (size_t)l * c->L;
    f.pro_mod  = c->d_ql_mod + (size_t)l * c->L;
    f.q_last   = c->primes[l];
    f.epi_kind = 1;
    f.epi_mul  = c->d_ql_inv + (size_t)l * c->L;
    f.aux      = ptr2(c0, c1);
    launch_ntt_fused(ptr2(bcast), mid, ptr2(res0, res1), bt, f);
  } else {
    LimbBatch b2 = bt;
    for (int k = 0; k < bt.count; k++)
      b2.limb[k] = LimbRef{(uint16_t)k, bt.limb[k].a, (uint16_t)k, bt.limb[k].prime, 0};
    launch_rescale_lift(ptr2(mid), ptr2(bcast), l, b2);
    launch_ntt(ptr2(mid), ptr2(mid), b2, false);
    for (int k = 0; k < bt.count; k++)
      b2.limb[k] = LimbRef{bt.limb[k].b, (uint16_t)k, bt.limb[k].dst, bt.limb[k].prime,
                           (uint8_t)((bt.limb[k].sel & 4) ? (1 | 4) : 0)};
    launch_rescale_combine(ptr2(res0, res1), ptr2(c0, c1), ptr2(mid), l, b2);
  }
  CUDA_CHECK(dev_free(mid, c->stream));
}

// Tensor product on the owned limbs (evaluator.c:137-173).
void Fhert_shard_tensor(const int64_t* a0, const int64_t* a1, const int64_t* b0, const int64_t* b1,
                        size_t level, int rank, int world, int64_t* d0, int64_t* d1, int64_t* d2) {
  Context*  c  = ctx();
  const int qb = (c->L + world - 1) / world;
  const int lo = std::min((int)level, rank * qb), hi = std::min((int)level, (rank + 1) * qb);
  if (hi <= lo) return;
  const size_t off = (size_t)lo * c->N;
  launch_tensor_range(d0 + off, d1 + off, d2 + off, a0 + off, a1 + off, b0 + off, b1 + off, lo,
                      hi - lo);
}

// ---- whole operations with the exchanges issued here (NCCL) ------------------

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*)                                     = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int)              = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t)                                        = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t,
                            cudaStream_t)                                        = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t,
                            cudaStream_t)                                        = nullptr;
  ncclResult_t (*GroupStart)()                                                   = nullptr;
  ncclResult_t (*GroupEnd)()                                                     = nullptr;
  const char* (*GetErrorString)(ncclResult_t)                                    = nullptr;
};
NcclApi    g_nccl;
ncclComm_t g_comm  = nullptr;
int        g_rank  = 0;
int        g_world = 1;

bool load_nccl() {
  if (g_nccl.handle != nullptr) return true;
  // a copy already in the process (a host framework's) is reused: same soname
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (h == nullptr) return false;
  g_nccl.GetUniqueId    = (decltype(g_nccl.GetUniqueId))dlsym(h, "ncclGetUniqueId");
  g_nccl.CommInitRank   = (decltype(g_nccl.CommInitRank))dlsym(h, "ncclCommInitRank");
  g_nccl.CommDestroy    = (decltype(g_nccl.CommDestroy))dlsym(h, "ncclCommDestroy");
  g_nccl.AllGather      = (decltype(g_nccl.AllGather))dlsym(h, "ncclAllGather");
  g_nccl.Broadcast      = (decltype(g_nccl.Broadcast))dlsym(h, "ncclBroadcast");
  g_nccl.GroupStart     = (decltype(g_nccl.GroupStart))dlsym(h, "ncclGroupStart");
  g_nccl.GroupEnd       = (decltype(g_nccl.GroupEnd))dlsym(h, "ncclGroupEnd");
  g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(h, "ncclGetErrorString");
  if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllGather ||
      !g_nccl.Broadcast || !g_nccl.GroupStart || !g_nccl.GroupEnd || !g_nccl.GetErrorString)
    return false;
  g_nccl.handle = h;
  return true;
}

#define NCCL_CHECK(call)                                                                  \
  do {                                                                                    \
    ncclResult_t r_ = (call);                                                             \
    FHERT_ASSERT(r_ == ncclSuccess, "NCCL error %s at %s", g_nccl.GetErrorString(r_), #call); \
  } while (0)

// key switch of `poly` on the owned limbs: out_g = ks_g (+ add_g), permuted by the key's
// automorphism unless key_sel is 2 (relinearisation)
void shard_key_switch(Context* c, const int64_t* poly, size_t level, int32_t rot_idx, int key_sel,
                      const int64_t* add0, const int64_t* add1, int64_t* out0, int64_t* out1) {
  const size_t n  = c->N;
  const int    qb = (c->L + g_world - 1) / g_world, pb = (c->K + g_world - 1) / g_world;
  int64_t *gq = nullptr, *gp = nullptr;
  CUDA_CHECK(dev_alloc(&gq, (size_t)g_world * qb * n * sizeof(int64_t), c->stream));
  CUDA_CHECK(dev_alloc(&gp, (size_t)2 * g_world * pb * n * sizeof(int64_t), c->stream));
  int64_t* gp1 = gp + (size_t)g_world * pb * n;
  void*    st  = Fhert_shard_begin(poly, level, g_rank, g_world, gq);
  if (g_world > 1)
    NCCL_CHECK(g_nccl.AllGather(gq + (size_t)g_rank * qb * n, gq, (size_t)qb * n, ncclInt64, g_comm,
                                c->stream));
  Fhert_shard_mid(st, poly, gq, rot_idx, key_sel, gp, gp1);
  if (g_world > 1) {
    // both accumulators' special limbs in one collective launch
    NCCL_CHECK(g_nccl.GroupStart());
    NCCL_CHECK(g_nccl.AllGather(gp + (size_t)g_rank * pb * n, gp, (size_t)pb * n, ncclInt64, g_comm,
                                c->stream));
    NCCL_CHECK(g_nccl.AllGather(gp1 + (size_t)g_rank * pb * n, gp1, (size_t)pb * n, ncclInt64, g_comm,
                                c->stream));
    NCCL_CHECK(g_nccl.GroupEnd());
  }
  Fhert_shard_end2(st, add0, add1, gp, gp1, rot_idx, key_sel, out0, out1);
  CUDA_CHECK(dev_free(gq, c->stream));
  CUDA_CHECK(dev_free(gp, c->stream));
}

void shape_result(Context* c, CIPHER res, size_t level, double sf, uint32_t sf_degree, uint32_t slots) {
  ensure_poly(&res->_c0_poly, c->N, level, 0);
  ensure_poly(&res->_c1_poly, c->N, level, 0);
  res->_c0_poly._is_ntt = res->_c1_poly._is_ntt = true;
  res->_scaling_factor = sf;
  res->_sf_degree      = sf_degree;
  res->_slots          = slots;
}

}  // namespace

// The 128-byte identifier rank 0 makes and hands to the other ranks (by any
// means the host has: a file, a socket, its own process group).
int Fhert_shard_comm_id(void* id128) {
  if (!load_nccl()) return 1;
  ncclUniqueId id;
  if (g_nccl.GetUniqueId(&id) != ncclSuccess) return 2;
  std::memcpy(id128, &id, sizeof(id));
  return 0;
}

// Joins the communicator of `world` ranks (one process per GPU, the context's
// device current).  world = 1 needs no identifier and no NCCL.
int Fhert_shard_comm_init(const void* id128, int rank, int world) {
  ctx();
  if (g_comm != nullptr) {
    g_nccl.CommDestroy(g_comm);
    g_comm = nullptr;
  }
  g_rank  = rank;
  g_world = world;
  if (world == 1) return 0;
  if (!load_nccl()) return 1;
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  ncclResult_t r = g_nccl.CommInitRank(&g_comm, world, id, rank);
  if (r != ncclSuccess) {
    std::fprintf(stderr, "libFHErt_b200: ncclCommInitRank: %s\n", g_nccl.GetErrorString(r));
    g_comm = nullptr;
    return 2;
  }
  return 0;
}

void Fhert_shard_comm_destroy(void) {
  if (g_comm != nullptr) {
    Fhert_sync();
    g_nccl.CommDestroy(g_comm);
    g_comm = nullptr;
  }
  g_rank  = 0;
  g_world = 1;
}

// Rotation (is_conj = 0) or conjugation (1) of a sharded ciphertext
// (evaluator.c:503-594): every rank passes its copy, only owned limbs are read
// and written.
CIPHER Fhert_shard_rotate(CIPHER res, CIPHER ct, int32_t rot_idx, int is_conj) {
  Context*     c     = ctx();
  const size_t level = ct->_c0_poly._num_primes;
  FHERT_ASSERT(g_world == 1 || g_comm != nullptr, "Fhert_shard_comm_init has not run");
  FHERT_ASSERT(res != ct, "sharded rotation cannot work in place");
  shape_result(c, res, level, ct->_scaling_factor, ct->_sf_degree, ct->_slots);
  shard_key_switch(c, ct->_c1_poly._data, level, rot_idx, is_conj ? 1 : 0, ct->_c0_poly._data,
                   nullptr, res->_c0_poly._data, res->_c1_poly._data);
  return res;
}

// Multiplication with relinearisation (evaluator.c:137-173, 288-305).
CIPHER Fhert_shard_mul_relin(CIPHER res, CIPHER a, CIPHER b) {
  Context*     c     = ctx();
  const size_t level = std::min(a->_c0_poly._num_primes, b->_c0_poly._num_primes), n = c->N;
  FHERT_ASSERT(g_world == 1 || g_comm != nullptr, "Fhert_shard_comm_init has not run");
  int64_t* d = nullptr;
  CUDA_CHECK(dev_alloc(&d, 3 * level * n * sizeof(int64_t), c->stream));
  int64_t *d0 = d, *d1 = d + level * n, *d2 = d + 2 * level * n;
  Fhert_shard_tensor(a->_c0_poly._data, a->_c1_poly._data, b->_c0_poly._data, b->_c1_poly._data,
                     level, g_rank, g_world, d0, d1, d2);
  shape_result(c, res, level, a->_scaling_factor * b->_scaling_factor,
               a->_sf_degree + b->_sf_degree, a->_slots);
  shard_key_switch(c, d2, level, 0, 2, d0, d1, res->_c0_poly._data, res->_c1_poly._data);
  CUDA_CHECK(dev_free(d, c->stream));
  return res;
}

// Rescale (evaluator.c:344-363): the owner of the dropped limb broadcasts it.
CIPHER Fhert_shard_rescale(CIPHER res, CIPHER ct) {
  Context*     c     = ctx();
  const size_t level = ct->_c0_poly._num_primes, n = c->N;
  FHERT_ASSERT(level > 1, "rescale: multiply level is not big enough");
  FHERT_ASSERT(g_world == 1 || g_comm != nullptr, "Fhert_shard_comm_init has not run");
  int64_t* bc = nullptr;
  CUDA_CHECK(dev_alloc(&bc, 2 * n * sizeof(int64_t), c->stream));
  Fhert_shard_rescale_begin(ct->_c0_poly._data, ct->_c1_poly._data, level, g_rank, g_world, bc);
  if (g_world > 1) {
    const int qb = (c->L + g_world - 1) / g_world;
    NCCL_CHECK(g_nccl.Broadcast(bc, bc, 2 * n, ncclInt64, (int)((level - 1) / qb), g_comm, c->stream));
  }
  if (res != ct)
    shape_result(c, res, level, ct->_scaling_factor / Get_default_sc(), ct->_sf_degree - 1,
                 ct->_slots);
  else {
    res->_scaling_factor = ct->_scaling_factor / Get_default_sc();
    res->_sf_degree      = ct->_sf_degree - 1;
  }
  Fhert_shard_rescale_end(ct->_c0_poly._data, ct->_c1_poly._data, level, g_rank, g_world, bc,
                          res->_c0_poly._data, res->_c1_poly._data);
  res->_c0_poly._num_primes = res->_c1_poly._num_primes = level - 1;
  CUDA_CHECK(dev_free(bc, c->stream));
  return res;
}

}  // extern "C"
