// Limb-sharded rotation: one ciphertext spread over several GPUs for latency.
//
// Every rank holds the ciphertext in the usual limb-major layout but only its
// own limbs are valid: Q limbs are dealt out in contiguous blocks of
// qb = ceil(level / world), the special limbs in blocks of pb = ceil(K / world).
// All per-limb work (NTT, key inner product, automorphism, the element-wise
// tail of ModDown) stays local.  The two base conversions of a hybrid key
// switch need every limb of their input, so they are preceded by an exchange:
//   1. ModUp: the coefficient form of c1's Q limbs is all-gathered, then each
//      rank converts only into the extended limbs it owns;
//   2. ModDown: the coefficient form of the accumulators' special limbs is
//      all-gathered, then each rank converts only into the Q limbs it owns.
// The exchanges themselves are done by the host (torch.distributed / NCCL
// all_gather on the library stream, see ace_compiler_b200/sharded.py); the
// phases below fill and consume the exchange buffers, which are laid out so
// that each rank's block is contiguous (block r = limbs [r*qb, (r+1)*qb)).
// Received limbs land in local memory before any kernel reads them.
//
// Arithmetic per limb is the same as in the single-GPU key switch
// (rns_poly.c:160-308, evaluator.c:411-522 of the CPU runtime), so the owned
// limbs of the result equal the single-GPU result bit for bit.
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
  if (q_block) *q_block = (int)((level + world - 1) / world);
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
  s->qb    = (int)((level + world - 1) / world);
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

  uint32_t    k   = is_conj ? 2 * c->N - 1 : auto_index_for(c, rot_idx);
  SWITCH_KEY* key = key_slot(c, k, false);
  FHERT_ASSERT(key != nullptr, "cannot find the rotation key of automorphism %u", k);
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
void Fhert_shard_end(void* state, const int64_t* c0, const int64_t* gather_p0,
                     const int64_t* gather_p1, int32_t rot_idx, int is_conj, int64_t* out0,
                     int64_t* out1) {
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
    tail.add[g] = g == 0 ? reinterpret_cast<const u64*>(c0) : nullptr;
  }
  launch_moddown_combine(tail);

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

}  // extern "C"
