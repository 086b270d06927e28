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
constexpr int kHwItems  = 256;   // limbs per launch
constexpr int kArena    = 64;    // scratch limbs per allocation
constexpr int kMaxNodes = 8192;  // replay at the latest after this many calls

struct HwItem {
  u64*            dst;
  const u64*      a;
  const u64*      b;
  const u64*      c;
  const uint32_t* table;
  int64_t         scalar;
  uint32_t        prime;
  uint32_t        kind;  // HwKind of this limb operation
};

struct HwLaunch {
  int    count;
  HwItem item[kHwItems];
};

// One launch covers the limb operations of one wave, whatever their kinds: the
// kind is uniform per block (blockIdx.y picks the item), so the switch costs no
// divergence.
__global__ void __launch_bounds__(kThreads)
hw_batch_kernel(const __grid_constant__ HwLaunch launch, const DevModulus* __restrict__ mods,
                uint32_t n) {
  const HwItem&    it   = launch.item[blockIdx.y];
  const DevModulus m    = mods[it.prime];
  const uint32_t   kind = it.kind;
  u64              sc   = 0;
  if (kind == HW_ADD_SCALAR || kind == HW_MUL_SCALAR) {
    int64_t s = it.scalar % (int64_t)m.q;
    sc        = s < 0 ? (u64)(s + (int64_t)m.q) : (u64)s;
  }
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
    u64 r;
    switch (kind) {
      case HW_ADD: r = add_mod(it.a[i], it.b[i], m.q); break;
      case HW_SUB: r = sub_mod(it.a[i], it.b[i], m.q); break;
      case HW_MUL: r = mul_mod(it.a[i], it.b[i], m); break;
      case HW_MULADD: r = add_mod(it.dst[i], mul_mod(it.a[i], it.b[i], m), m.q); break;
      case HW_ADD_SCALAR: r = add_mod(it.a[i], sc, m.q); break;
      case HW_MUL_SCALAR: r = mul_mod(it.a[i], sc, m); break;
      case HW_ROTATE: r = it.a[__ldg(it.table + i)]; break;
      case HW_MAC3: r = add_mod(it.c[i], mul_mod(it.a[i], it.b[i], m), m.q); break;
      default: r = it.a[i]; break;
    }
    it.dst[i] = r;
  }
}

struct Node {
  HwKind kind;
  HwItem item;
  int    level;
  bool   dead;
  int    src_writer[3];  // node that produced each operand, -1 = memory
  u64*   src_addr[3];    // the operands' own addresses
  int    readers;        // recorded operations that read this node's value
  bool   superseded;     // a later recorded call overwrote the same address
};

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
  // Usage part
  int read_level;
  int write_level;
};
typedef Slot Version;
typedef Slot Usage;

constexpr int kTableLog = 16;

}  // namespace

struct HwQueue {
  std::vector<Node>                   nodes;
  std::vector<Slot>                   table = std::vector<Slot>((size_t)1 << kTableLog);
  uint32_t                            epoch = 1;
  int                                 used  = 0;
  std::vector<u64*>                   renamed;   // addresses whose value went to scratch
  std::vector<u64*>                   arenas;
  int                                 arena_used = kArena;
  int                                 max_level  = 0;
  bool                                replaying  = false;
  bool                                eager      = false;
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
    CUDA_CHECK(cudaMallocAsync(&p, (size_t)kArena * c->N * sizeof(u64), c->stream));
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
      s = Slot{const_cast<u64*>(addr), q->epoch, const_cast<u64*>(addr), -1, 0, 0, 0, 0};
      q->used++;
      return &s;
    }
    if (s.key == addr) return &s;
    h = (h + 1) & mask;
  }
}

Version& version_of(HwQueue* q, u64* addr) { return *find_slot(q, addr, true); }
Usage&   usage_of(HwQueue* q, const u64* addr) { return *find_slot(q, addr, true); }

void run_wave(Context* c, const std::vector<const Node*>& wave) {
  for (size_t off = 0; off < wave.size(); off += kHwItems) {
    HwLaunch l;
    l.count = (int)std::min<size_t>(kHwItems, wave.size() - off);
    for (int i = 0; i < l.count; i++) {
      l.item[i]      = wave[off + i]->item;
      l.item[i].kind = (uint32_t)wave[off + i]->kind;
    }
    dim3 grid((c->N + kThreads * 2 - 1) / (kThreads * 2), l.count);
    prof_before(KID_HW_BATCH);
    hw_batch_kernel<<<grid, kThreads, 0, c->stream>>>(l, c->d_mod, c->N);
    prof_after(KID_HW_BATCH, l.count);
    c->launches++;
    c->hw_batched_limbs += l.count;
    CUDA_CHECK(cudaGetLastError());
  }
}

}  // namespace

void hw_replay(Context* c) {
  HwQueue* q = c->hw_queue;
  if (q == nullptr || q->nodes.empty() || q->replaying) return;
  q->replaying = true;
  // "tmp = a * b; d = x + tmp" with tmp read once, a and b untouched by the
  // recording: one multiply-add; a product overwritten later in the same
  // recording never goes to memory
  auto untouched = [&](const Node& p, int t) {
    if (p.src_writer[t] != -1) return false;
    Slot* sl = find_slot(q, p.src_addr[t], false);
    return sl == nullptr || sl->writer == -1;
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
  std::vector<const Node*> wave;
  std::vector<std::vector<const Node*>> by_level(q->max_level + 1);
  for (const Node& nd : q->nodes)
    if (!nd.dead) by_level[nd.level].push_back(&nd);
  for (int level = 1; level <= q->max_level; level++)
    if (!by_level[level].empty()) run_wave(c, by_level[level]);
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
  if (!home.empty()) {
    wave.clear();
    for (const Node& nd : home) wave.push_back(&nd);
    run_wave(c, wave);
  }
  for (u64* p : q->arenas) CUDA_CHECK(cudaFreeAsync(p, c->stream));
  q->arenas.clear();
  q->arena_used = kArena;
  q->nodes.clear();
  q->renamed.clear();
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
  nd.kind        = kind;
  nd.item.table  = table;
  nd.item.scalar = scalar;
  nd.item.prime  = (uint32_t)prime;
  nd.dead        = false;
  int  level     = 0;
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
    level      = std::max(level, v.writer_level);
    nd.src_writer[i] = v.writer;
    if (src[i] == dst) in_place = true;
  }
  nd.readers    = 0;
  nd.superseded = false;
  level += 1;
  Version& dv = version_of(q, dst);
  u64*     out;
  if (dv.writer >= 0) q->nodes[dv.writer].superseded = true;
  if (!in_place && dv.readers > 0) {
    out = scratch_limb(c, q);  // earlier readers keep the old value
  } else {
    out = dv.phys;
    if (!in_place && dv.readers == 0 && dv.writer >= 0) q->nodes[dv.writer].dead = true;
    Usage& u = out == dst ? dv : usage_of(q, out);
    level    = std::max(level, std::max(u.read_level, u.write_level) + 1);
  }
  for (int i = 0; i < 3; i++) {
    if (src[i] == nullptr) continue;
    Version& v = *seen[i];
    v.readers++;
    if (v.writer >= 0) q->nodes[v.writer].readers++;
    Usage& u     = v.phys == v.key ? v : usage_of(q, v.phys);
    u.read_level = std::max(u.read_level, level);
  }
  nd.item.dst = out;
  nd.item.a   = phys[0];
  nd.item.b   = phys[1];
  nd.level    = level;
  (out == dst ? dv : usage_of(q, out)).write_level = level;
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
