// Deferred execution of the per-limb vector entry points (Hw_modadd,
// Hw_modmul, Hw_rotate ...).
//
// A compiled program calls these once per RNS limb from inside its own loops
// (hal/src/hal.c:15-138 are the CPU versions), tens of thousands of times per
// operator.  Launching one kernel per call would leave the GPU idle between
// half-megabyte launches, so the calls are only recorded.  Every other entry
// point of the library reaches the context through ctx(), which first replays
// what was recorded: the recorded operations are ordered by data dependence
// into waves, and each wave runs as one launch covering up to kHwItems limbs
// (operations of different kinds share the launch).
//
// All operations but the rotation work coefficient by coefficient, so a run of
// dependent operations on one limb ("acc += a_i * b_i" over hundreds of i) does
// not need one wave per step: the run becomes a chain inside one wave.  A chain
// is executed by the same blocks item after item; every thread keeps the
// coefficients it owns, so the value it wrote for one item is the value it
// reads for the next (it stays in a register, and is not stored at all when
// nothing else reads it).  Only a rotation's source, which is read through a
// permutation, has to come from an earlier wave.
//
// Dependences are tracked per limb address (operands are whole limbs, either
// identical or disjoint).  A scratch limb that a program reuses for every
// limb of a loop (the "tmp = key * digit; acc += tmp" idiom) would chain all
// iterations together, so a value written over a limb that still has readers
// waiting is given a fresh scratch limb instead (renaming); the last value of
// such a limb is copied to its real address at the end of the replay.
#include <algorithm>
#include <vector>

#include "runtime.h"

namespace fhert {

namespace {

constexpr int kThreads  = 256;
constexpr int kHwItems  = 384;   // limb operations per launch (21 KiB of kernel parameters)
constexpr int kArena    = 64;    // scratch limbs per allocation
constexpr int kMaxNodes = 8192;  // replay at the latest after this many calls

struct HwItem {
  u64*            dst;
  const u64*      a;
  const u64*      b;
  const u64*      c;
  const uint32_t* table;
  u64             scalar;  // already reduced modulo the limb's prime
  uint32_t        prime;
  uint32_t        kind;  // HwKind of this limb operation, kNoStore or-ed in
};

constexpr uint32_t kNoStore  = 0x100;  // the next item of the chain is the only reader
constexpr uint32_t kKindMask = 0xff;

struct HwLaunch {
  int      chains;
  uint16_t first[kHwItems + 1];  // chain y owns item[first[y] .. first[y + 1])
  HwItem   item[kHwItems];
};

// One launch covers one wave, whatever the kinds of its operations: blockIdx.y
// picks a chain, whose items run one after the other on the coefficients this
// thread owns (two per thread).  The result of an item is carried in registers
// to the next one.
__global__ void __launch_bounds__(kThreads)
hw_batch_kernel(const __grid_constant__ HwLaunch launch, const DevModulus* __restrict__ mods,
                uint32_t n) {
  const uint32_t i0 = blockIdx.x * kThreads + threadIdx.x, i1 = i0 + gridDim.x * kThreads;
  const bool     in0 = i0 < n, in1 = i1 < n;
  const u64*     carried = nullptr;
  u64            r0 = 0, r1 = 0;
  auto fetch = [&](const u64* p, u64& x0, u64& x1) {
    if (p == carried) {
      x0 = r0;
      x1 = r1;
    } else {
      x0 = in0 ? p[i0] : 0;
      x1 = in1 ? p[i1] : 0;
    }
  };
  for (int k = launch.first[blockIdx.y], end = launch.first[blockIdx.y + 1]; k < end; k++) {
    const HwItem&    it   = launch.item[k];
    const uint32_t   kind = it.kind & kKindMask;
    const DevModulus m    = mods[it.prime];
    u64              a0, a1, b0 = 0, b1 = 0, t0, t1;
    if (kind == HW_ROTATE) {
      a0 = in0 ? it.a[__ldg(it.table + i0)] : 0;
      a1 = in1 ? it.a[__ldg(it.table + i1)] : 0;
    } else {
      fetch(it.a, a0, a1);
    }
    if (kind == HW_ADD || kind == HW_SUB || kind == HW_MUL || kind == HW_MAC3) fetch(it.b, b0, b1);
    switch (kind) {
      case HW_ADD: t0 = add_mod(a0, b0, m.q); t1 = add_mod(a1, b1, m.q); break;
      case HW_SUB: t0 = sub_mod(a0, b0, m.q); t1 = sub_mod(a1, b1, m.q); break;
      case HW_MUL: t0 = mul_mod(a0, b0, m); t1 = mul_mod(a1, b1, m); break;
      case HW_MAC3: {
        u64 c0, c1;
        fetch(it.c, c0, c1);
        t0 = add_mod(c0, mul_mod(a0, b0, m), m.q);
        t1 = add_mod(c1, mul_mod(a1, b1, m), m.q);
        break;
      }
      case HW_ADD_SCALAR: t0 = add_mod(a0, it.scalar, m.q); t1 = add_mod(a1, it.scalar, m.q); break;
      case HW_MUL_SCALAR: t0 = mul_mod(a0, it.scalar, m); t1 = mul_mod(a1, it.scalar, m); break;
      default: t0 = a0; t1 = a1; break;  // rotation (already permuted) and copy
    }
    r0      = t0;
    r1      = t1;
    carried = it.dst;
    if (!(it.kind & kNoStore)) {
      if (in0) it.dst[i0] = r0;
      if (in1) it.dst[i1] = r1;
    }
  }
}

struct Node {
  HwKind kind;
  HwItem item;
  int    level;
  int    chain;          // nodes of one chain share a wave and run in recording order
  bool   dead;
  int    src_writer[3];  // node that produced each operand, -1 = memory
  u64*   src_addr[3];    // the operands' own addresses
  int    readers;        // recorded operations that read this node's value
  bool   superseded;     // a later recorded call overwrote the same address
};

constexpr int kMixed = -2;  // read by several chains, or through a permutation

// One slot per limb address seen in the current recording.  As a program
// address it tracks the newest value of that limb (Version part); as a place
// in memory it tracks the latest waves that touch it (Usage part).  Slots are
// stamped with the recording's epoch, so starting a new recording costs nothing.
struct Slot {
  u64*     key;
  uint32_t epoch;
  // Version part
  u64* phys;          // where the newest value lives (the address itself or a scratch limb)
  int  writer;        // node that produces it, -1 = already in memory
  int  writer_level;
  int  readers;       // recorded operations that read it
  bool written;       // some recorded operation wrote this address (sticky)
  // Usage part
  int read_level;     // latest wave that reads this memory, and the chain that does
  int read_chain;     // (kMixed = more than one, or a rotation's source)
  int write_level;
  int write_chain;
};
typedef Slot Version;
typedef Slot Usage;

constexpr int kTableLog = 16;

}  // namespace

struct HwQueue {
  std::vector<Node>  nodes;
  std::vector<Slot>  table = std::vector<Slot>((size_t)1 << kTableLog);
  uint32_t           epoch = 1;
  int                used  = 0;
  std::vector<u64*>  renamed;   // addresses whose value went to scratch
  std::vector<u64*>  arenas;
  std::vector<void*> borrowed;  // device memory to release after the next replay
  int                arena_used = kArena;
  int                max_level  = 0;
  std::vector<int>   chain_level;  // wave of every chain
  bool               replaying  = false;
  bool               eager      = false;
  // replay scratch
  std::vector<int>   chain_first, level_first, chain_order, flat;
};

namespace {

HwQueue* queue_of(Context* c) {
  if (c->hw_queue == nullptr) {
    HwQueue* q = new HwQueue();
    const char* e = std::getenv("FHERT_EAGER_HW");
    q->eager      = e != nullptr && e[0] != '\0' && e[0] != '0';
    c->hw_queue   = q;
  }
  return c->hw_queue;
}

u64* scratch_limb(Context* c, HwQueue* q) {
  if (q->arena_used == kArena) {
    u64* p = nullptr;
    CUDA_CHECK(dev_alloc(&p, (size_t)kArena * c->N * sizeof(u64), c->stream));
    q->arenas.push_back(p);
    q->arena_used = 0;
  }
  return q->arenas.back() + (size_t)(q->arena_used++) * c->N;
}

Slot* find_slot(HwQueue* q, const u64* addr, bool create) {
  const size_t mask = ((size_t)1 << kTableLog) - 1;
  size_t h = (size_t)(((uintptr_t)addr >> 6) * 0x9E3779B97F4A7C15ull >> (64 - kTableLog));
  for (;;) {
    Slot& s = q->table[h];
    if (s.epoch != q->epoch) {
      if (!create) return nullptr;
      s = Slot{const_cast<u64*>(addr), q->epoch, const_cast<u64*>(addr), -1, 0, 0, false, 0,
               kMixed, 0, kMixed};
      q->used++;
      return &s;
    }
    if (s.key == addr) return &s;
    h = (h + 1) & mask;
  }
}

Version& version_of(HwQueue* q, u64* addr) { return *find_slot(q, addr, true); }
Usage&   usage_of(HwQueue* q, const u64* addr) { return *find_slot(q, addr, true); }

// Packs chains into launches of at most kHwItems items.  A chain that does not
// fit continues in the next launch, which the stream runs afterwards.
struct Packer {
  Context* c;
  HwLaunch l;
  int      used = 0;
  explicit Packer(Context* ctx) : c(ctx) { l.chains = 0; }
  void flush() {
    if (l.chains == 0) return;
    l.first[l.chains] = (uint16_t)used;
    dim3 grid((c->N + kThreads * 2 - 1) / (kThreads * 2), l.chains);
    DagScope dag(DAG_RECORDED_BATCH);
    if (dag.live) {
      const size_t w = (size_t)c->N * sizeof(u64);
      for (int k = 0; k < used; k++) {
        const HwItem&  it   = l.item[k];
        const uint32_t kind = it.kind & kKindMask;
        dag.set.read(it.a, w);
        if (kind == HW_ADD || kind == HW_SUB || kind == HW_MUL || kind == HW_MAC3) dag.set.read(it.b, w);
        if (kind == HW_MAC3) dag.set.read(it.c, w);
        if (!(it.kind & kNoStore)) dag.set.write(it.dst, w);
      }
    }
    dag.commit();
    prof_before(KID_HW_BATCH);
    hw_batch_kernel<<<grid, kThreads, 0, c->stream>>>(l, c->d_mod, c->N);
    prof_after(KID_HW_BATCH, used);
    c->launches++;
    c->hw_batched_limbs += used;
    CUDA_CHECK(cudaGetLastError());
    l.chains = 0;
    used     = 0;
  }
  // the value of nodes[k] is needed by nobody but the next item of the piece
  static bool only_feeds(const Node* base, const Node& nd, const Node& next) {
    if (!nd.superseded || nd.readers == 0) return false;
    const int self = (int)(&nd - base);
    int       uses = 0;
    for (int j = 0; j < 3; j++) uses += next.src_writer[j] == self;
    return uses == nd.readers;
  }
  void add_chain(const Node* base, const int* member, int size) {
    int pos = 0;
    while (pos < size) {
      if (used == kHwItems) flush();
      int take = std::min(size - pos, kHwItems - used);
      if (take < size - pos && size - pos <= kHwItems && used > 0) {
        flush();  // fits a launch of its own: do not split it
        continue;
      }
      l.first[l.chains++] = (uint16_t)used;
      for (int i = 0; i < take; i++) {
        const Node& nd = base[member[pos + i]];
        HwItem&     it = l.item[used + i];
        it             = nd.item;
        it.kind        = (uint32_t)nd.kind;
        if (i + 1 < take && only_feeds(base, nd, base[member[pos + i + 1]])) it.kind |= kNoStore;
      }
      used += take;
      pos += take;
      if (pos < size) flush();  // the rest of the chain has to run after this piece
    }
  }
};

}  // namespace

void hw_replay(Context* c) {
  HwQueue* q = c->hw_queue;
  if (q == nullptr || q->replaying) return;
  if (q->nodes.empty() && q->renamed.empty() && q->borrowed.empty()) return;
  q->replaying = true;
  // "tmp = a * b; d = x + tmp" with tmp read once, a and b untouched by the
  // recording: one multiply-add; a product overwritten later in the same
  // recording never goes to memory
  auto untouched = [&](const Node& p, int t) {
    if (p.src_writer[t] != -1) return false;
    Slot* sl = find_slot(q, p.src_addr[t], false);
    return sl == nullptr || !sl->written;
  };
  for (Node& sum : q->nodes) {
    if (sum.dead || sum.kind != HW_ADD) continue;
    for (int s = 0; s < 2; s++) {
      int w = sum.src_writer[s];
      if (w < 0) continue;
      Node& prod = q->nodes[w];
      if (prod.dead || prod.kind != HW_MUL || prod.readers != 1 ||
          prod.item.prime != sum.item.prime || !untouched(prod, 0) || !untouched(prod, 1))
        continue;
      sum.kind   = HW_MAC3;
      sum.item.c = s == 0 ? sum.item.b : sum.item.a;
      sum.item.a = prod.item.a;
      sum.item.b = prod.item.b;
      // a product that is still the last value of its address stays, for
      // whoever reads that address after the replay
      if (prod.superseded) prod.dead = true;
      break;
    }
  }
  // live nodes grouped by chain (recording order inside a chain), chains by wave
  const int chains = (int)q->chain_level.size(), nodes = (int)q->nodes.size();
  q->chain_first.assign(chains + 1, 0);
  for (const Node& nd : q->nodes)
    if (!nd.dead) q->chain_first[nd.chain + 1]++;
  for (int i = 0; i < chains; i++) q->chain_first[i + 1] += q->chain_first[i];
  q->flat.resize(q->chain_first[chains]);
  {
    std::vector<int>& fill = q->chain_order;  // borrowed as the per-chain cursor
    fill.assign(q->chain_first.begin(), q->chain_first.end() - 1);
    for (int i = 0; i < nodes; i++)
      if (!q->nodes[i].dead) q->flat[fill[q->nodes[i].chain]++] = i;
  }
  q->level_first.assign(q->max_level + 2, 0);
  for (int ch = 0; ch < chains; ch++) q->level_first[q->chain_level[ch] + 1]++;
  for (int lv = 0; lv <= q->max_level; lv++) q->level_first[lv + 1] += q->level_first[lv];
  q->chain_order.resize(chains);
  {
    std::vector<int> fill(q->level_first.begin(), q->level_first.end() - 1);
    for (int ch = 0; ch < chains; ch++) q->chain_order[fill[q->chain_level[ch]]++] = ch;
  }
  Packer pack(c);
  for (int lv = 1; lv <= q->max_level; lv++) {
    for (int k = q->level_first[lv]; k < q->level_first[lv + 1]; k++) {
      const int ch = q->chain_order[k], size = q->chain_first[ch + 1] - q->chain_first[ch];
      if (size > 0) pack.add_chain(q->nodes.data(), q->flat.data() + q->chain_first[ch], size);
    }
    pack.flush();  // the next wave reads what this one wrote
  }
  // values that ended up in scratch limbs go home
  std::vector<Node> home;
  for (u64* addr : q->renamed) {
    Slot* sl = find_slot(q, addr, false);
    if (sl == nullptr || sl->phys == addr) continue;
    Node nd{};
    nd.kind       = HW_COPY;
    nd.item.dst   = addr;
    nd.item.a     = sl->phys;
    nd.item.prime = 0;
    home.push_back(nd);
    sl->phys = addr;  // listed once even if renamed several times
  }
  for (size_t i = 0; i < home.size(); i++) {
    const int self = (int)i;
    pack.add_chain(home.data(), &self, 1);
  }
  pack.flush();
  for (u64* p : q->arenas) CUDA_CHECK(dev_free(p, c->stream));
  q->arenas.clear();
  for (void* p : q->borrowed) CUDA_CHECK(dev_free(p, c->stream));
  q->borrowed.clear();
  c->raised.valid = false;  // its digits were among the borrowed memory
  q->arena_used = kArena;
  q->nodes.clear();
  q->renamed.clear();
  q->chain_level.clear();
  q->epoch++;
  q->used = 0;
  q->max_level = 0;
  q->replaying = false;
  c->hw_pending = false;
}

void hw_release(Context* c) {
  if (c->hw_queue == nullptr) return;
  hw_replay(c);
  delete c->hw_queue;
  c->hw_queue = nullptr;
}

bool hw_alias(Context* c, int64_t* dst_, const int64_t* src_) {
  HwQueue* q = queue_of(c);
  if (q->eager) return false;
  u64*     dst = reinterpret_cast<u64*>(dst_);
  Version& dv  = version_of(q, dst);
  if (dv.writer >= 0) {
    q->nodes[dv.writer].superseded = true;
    if (dv.readers == 0) q->nodes[dv.writer].dead = true;  // overwritten unread
  }
  dv.phys         = reinterpret_cast<u64*>(const_cast<int64_t*>(src_));
  dv.writer       = -1;
  dv.writer_level = 0;
  dv.readers      = 0;  // `written` stays: only recorded operations count as writes
  q->renamed.push_back(dst);  // the value goes to its real address at the end of the replay
  c->hw_pending = true;
  return true;
}

bool hw_recording(Context* c) { return !queue_of(c)->eager; }

void hw_free_after_replay(Context* c, void* device_memory) {
  queue_of(c)->borrowed.push_back(device_memory);
  c->hw_pending = true;
}

// Records res = a (kind) b.  Returns false when recording is switched off
// (FHERT_EAGER_HW=1) and the caller has to launch the operation itself.
bool hw_record(Context* c, HwKind kind, int64_t* res, const int64_t* a, const int64_t* b,
               const uint32_t* table, int64_t scalar, int prime) {
  HwQueue* q = queue_of(c);
  if (q->eager) return false;
  u64* dst   = reinterpret_cast<u64*>(res);
  u64* src[3] = {reinterpret_cast<u64*>(const_cast<int64_t*>(a)),
                 kind <= HW_MULADD ? reinterpret_cast<u64*>(const_cast<int64_t*>(b)) : nullptr,
                 kind == HW_MULADD ? dst : nullptr};
  Node nd{};
  nd.kind        = kind == HW_MULADD ? HW_MAC3 : kind;
  nd.item.table  = table;
  nd.item.prime  = (uint32_t)prime;
  nd.dead        = false;
  if (kind == HW_ADD_SCALAR || kind == HW_MUL_SCALAR) {
    const int64_t qv = (int64_t)c->primes[prime], sv = scalar % qv;
    nd.item.scalar   = (u64)(sv < 0 ? sv + qv : sv);
  }
  // What this operation has to wait for.  `hard`: the latest wave that must be
  // complete before it starts.  soft: waves it may share, provided it runs in
  // the same chain after the operation it depends on (same coefficient, same
  // thread).
  int hard = 0, soft_level = 0, soft_chain = -1;
  bool soft_clash = false;
  auto depend = [&](int level, int chain, bool permuted) {
    if (level <= 0) return;
    if (permuted || chain < 0) {
      hard = std::max(hard, level);
    } else if (level > soft_level) {
      soft_level = level;
      soft_chain = chain;
      soft_clash = false;
    } else if (level == soft_level && chain != soft_chain) {
      soft_clash = true;
    }
  };
  bool in_place  = false;
  const u64* phys[3] = {nullptr, nullptr, nullptr};
  Slot*      seen[3] = {nullptr, nullptr, nullptr};
  for (int i = 0; i < 3; i++) {
    nd.src_writer[i] = -1;
    nd.src_addr[i]   = src[i];
    if (src[i] == nullptr) continue;
    Version& v = version_of(q, src[i]);
    seen[i]    = &v;
    phys[i]    = v.phys;
    depend(v.writer_level, v.writer >= 0 ? q->nodes[v.writer].chain : kMixed,
           kind == HW_ROTATE && i == 0);
    nd.src_writer[i] = v.writer;
    if (src[i] == dst) in_place = true;
  }
  nd.readers    = 0;
  nd.superseded = false;
  Version& dv = version_of(q, dst);
  u64*     out;
  dv.written = true;
  if (c->raised.valid && res >= c->raised.src && res < c->raised.src + c->raised.level * c->N)
    c->raised.valid = false;  // the polynomial being raised changes: later digits start afresh
  if (dv.writer >= 0) q->nodes[dv.writer].superseded = true;
  if (!in_place && dv.readers > 0) {
    out = scratch_limb(c, q);  // earlier readers keep the old value
  } else {
    out = dv.phys;
    if (!in_place && dv.readers == 0 && dv.writer >= 0) q->nodes[dv.writer].dead = true;
    Usage& u = out == dst ? dv : usage_of(q, out);
    depend(u.read_level, u.read_chain, false);
    depend(u.write_level, u.write_chain, false);
  }
  // a write that lands in the kept digits themselves (a result limb of Decomp_modup
  // is an alias of them until something overwrites it): what is kept no longer
  // equals the raised polynomial, later Decomp_modup calls must raise afresh
  if (c->raised.valid && out >= reinterpret_cast<u64*>(c->raised.digits) &&
      out < reinterpret_cast<u64*>(c->raised.digits) +
                (size_t)c->raised.parts * (c->raised.level + c->K) * c->N)
    c->raised.valid = false;
  int level = std::max(hard + 1, soft_level), chain;
  if (soft_level == level && !soft_clash) {
    chain = soft_chain;  // continues the chain of what it depends on
  } else {
    if (soft_level == level) level++;  // depends on two chains of that wave
    chain = (int)q->chain_level.size();
    q->chain_level.push_back(level);
  }
  for (int i = 0; i < 3; i++) {
    if (src[i] == nullptr) continue;
    Version& v = *seen[i];
    v.readers++;
    if (v.writer >= 0) q->nodes[v.writer].readers++;
    Usage&     u        = v.phys == v.key ? v : usage_of(q, v.phys);
    const bool permuted = kind == HW_ROTATE && i == 0;
    if (level > u.read_level) {
      u.read_level = level;
      u.read_chain = permuted ? kMixed : chain;
    } else if (level == u.read_level && (permuted || u.read_chain != chain)) {
      u.read_chain = kMixed;
    }
  }
  nd.item.dst = out;
  nd.item.a   = phys[0];
  nd.item.b   = phys[1];
  nd.item.c   = phys[2];
  nd.level    = level;
  nd.chain    = chain;
  {
    Usage& u      = out == dst ? dv : usage_of(q, out);
    u.write_level = level;
    u.write_chain = chain;
  }
  if (out != dst) q->renamed.push_back(dst);
  Version& fresh    = dv;
  fresh.phys        = out;
  fresh.writer      = (int)q->nodes.size();
  fresh.writer_level = level;
  fresh.readers     = 0;
  if (q->nodes.capacity() == 0) q->nodes.reserve(kMaxNodes + 8);
  q->nodes.push_back(nd);
  q->max_level  = std::max(q->max_level, level);
  c->hw_pending = true;
  if ((int)q->nodes.size() >= kMaxNodes || q->used > (1 << (kTableLog - 1)))
    ctx();  // runs a waiting Mod_down / Rescale (older) and then the recording
  return true;
}

}  // namespace fhert
