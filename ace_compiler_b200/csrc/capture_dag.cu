// Dependences of a captured program run taken from the memory its launches
// touch, not from their order in the stream.
//
// A program run is captured from one stream, which would make its graph one
// chain of tens of thousands of short kernels.  Many of them are independent
// (the rotations of one convolution, the two halves of a residual block, the
// branches of a polynomial evaluation), and a short kernel leaves most of the
// GPU idle.  While a run is captured, every launch site that knows what its
// launch reads and writes says so first (DagScope below); the capture
// dependencies of the stream are then set to exactly the nodes that last wrote
// what it reads and that last wrote or read what it writes, so the captured
// graph is the data-flow graph and independent branches run side by side.
//
// Safety does not depend on every launch being described.  After each
// described launch the stream is left depending on all leaves of the graph, so
// a launch nobody described comes after everything captured before it; when
// the next described launch finds that the stream's dependences are no longer
// the ones left there, whatever was captured in between becomes a barrier that
// every later node depends on, and the memory map starts afresh.  Memory that
// the pool hands out again is covered too: the map is by address, so the new
// user of a block waits for the last kernels of its former user.
//
// Read-only tables (twiddles, keys, cached plaintexts, conversion matrices)
// are never written during a run and are left out of the descriptions.
#include <algorithm>
#include <map>
#include <unordered_map>
#include <vector>

#include "access_map.h"
#include "runtime.h"

namespace fhert {

namespace {

struct DagState {
  bool                           on = false;
  AccessMap<cudaGraphNode_t>     map;      // who wrote and read what since the last barrier
  std::vector<cudaGraphNode_t>   leaves;   // nodes nothing depends on yet (sorted)
  std::vector<cudaGraphNode_t>   barrier;  // every new node depends on these
  std::vector<cudaGraphNode_t>   deps;     // of the launch being described (sorted, unique)
  const AccessSet*               pending = nullptr;
  uint64_t                       nodes = 0, edges = 0, barriers = 0, joins = 0;
  size_t                         max_deps = 0;
  std::unordered_map<cudaGraphNode_t, uint32_t> depth;  // longest chain ending at a node
  uint32_t                       max_depth = 0;
};
DagState g_dag;

// An empty node that depends on all current leaves: it takes their place, so
// that the set the stream is left depending on stays small.  Later nodes depend
// on it only if nobody described them, so it orders nothing by itself.
__global__ void dag_join_kernel() {}
constexpr size_t kMaxLeaves = 48;

void sort_unique(std::vector<cudaGraphNode_t>& v) {
  std::sort(v.begin(), v.end());
  v.erase(std::unique(v.begin(), v.end()), v.end());
}

std::vector<cudaGraphNode_t> stream_deps(cudaStream_t stream) {
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  const cudaGraphNode_t*  d      = nullptr;
  size_t                  n      = 0;
  CUDA_CHECK(cudaStreamGetCaptureInfo(stream, &status, nullptr, nullptr, &d, &n));
  FHERT_ASSERT(status == cudaStreamCaptureStatusActive, "the capture of the program run was lost");
  std::vector<cudaGraphNode_t> v(d, d + n);
  std::sort(v.begin(), v.end());
  return v;
}

void set_stream_deps(cudaStream_t stream, std::vector<cudaGraphNode_t>& v) {
  CUDA_CHECK(cudaStreamUpdateCaptureDependencies(stream, v.empty() ? nullptr : v.data(), v.size(),
                                                 cudaStreamSetCaptureDependencies));
}

}  // namespace

void dag_begin() {
  static const bool off = [] {
    const char* e = std::getenv("FHERT_REPLAY_DAG");
    return e != nullptr && e[0] == '0';
  }();
  g_dag    = DagState();
  g_dag.on = !off;
}

void dag_end(uint64_t* nodes, uint64_t* edges, uint64_t* barriers, uint64_t* longest_chain) {
  if (longest_chain) *longest_chain = g_dag.max_depth;
  if (nodes) *nodes = g_dag.nodes;
  if (edges) *edges = g_dag.edges;
  if (barriers) *barriers = g_dag.barriers + (g_dag.joins << 32);
  if (const char* e = std::getenv("FHERT_REPLAY_STATS"))
    if (e[0] == '1' && g_dag.nodes)
      std::fprintf(stderr, "[FHERT_REPLAY] largest dependence set of a node: %zu; longest chain of "
                   "described nodes: %u of %llu\n", g_dag.max_deps, g_dag.max_depth,
                   (unsigned long long)g_dag.nodes);
  g_dag = DagState();
}

bool dag_active() { return g_dag.on && image_capturing(); }
bool dag_family_on(int family) {
  const char* e = std::getenv("FHERT_DAG_SKIP");
  return e == nullptr || !(std::atoi(e) & family);
}

void dag_before(const AccessSet& a) {
  if (!dag_active()) return;
  Context*     c      = ctx_noflush();
  cudaStream_t stream = c->stream;
  std::vector<cudaGraphNode_t> cur = stream_deps(stream);
  if (cur != g_dag.leaves) {
    // launches nobody described were captured since: they come after all that
    // went before (they depended on every leaf) and before all that follows
    g_dag.barrier = cur;
    g_dag.leaves  = cur;
    g_dag.map.clear();
    g_dag.barriers++;
  }
  g_dag.deps = g_dag.barrier;
  g_dag.map.dependences(a.reads, a.writes, g_dag.deps);
  sort_unique(g_dag.deps);
  g_dag.max_deps = std::max(g_dag.max_deps, g_dag.deps.size());
  set_stream_deps(stream, g_dag.deps);
  g_dag.pending = &a;
}

void dag_after() {
  if (!dag_active() || g_dag.pending == nullptr) return;
  Context*     c      = ctx_noflush();
  cudaStream_t stream = c->stream;
  std::vector<cudaGraphNode_t> cur = stream_deps(stream);
  const AccessSet& a = *g_dag.pending;
  g_dag.pending      = nullptr;
  if (cur == g_dag.deps) {
    // nothing was captured (an empty copy or clear): back to "after all leaves"
    set_stream_deps(stream, g_dag.leaves);
    return;
  }
  // one launch, or several that ran one after the other: the stream now depends
  // on the last of them alone
  FHERT_ASSERT(cur.size() == 1 && !std::binary_search(g_dag.deps.begin(), g_dag.deps.end(), cur[0]),
               "capture: unexpected dependences after a described launch");
  cudaGraphNode_t node = cur[0];
  {
    uint32_t d = 0;
    for (cudaGraphNode_t p : g_dag.deps) {
      auto it = g_dag.depth.find(p);
      if (it != g_dag.depth.end()) d = std::max(d, it->second);
    }
    g_dag.depth[node] = d + 1;
    g_dag.max_depth   = std::max(g_dag.max_depth, d + 1);
  }
  g_dag.nodes++;
  g_dag.edges += g_dag.deps.size();
  g_dag.map.record(a.reads, a.writes, node);
  // leaves: the new node replaces the ones it depends on
  std::vector<cudaGraphNode_t> next;
  std::set_difference(g_dag.leaves.begin(), g_dag.leaves.end(), g_dag.deps.begin(), g_dag.deps.end(),
                      std::back_inserter(next));
  next.insert(std::upper_bound(next.begin(), next.end(), node), node);
  g_dag.leaves.swap(next);
  if (g_dag.leaves.size() > kMaxLeaves) {
    set_stream_deps(stream, g_dag.leaves);
    dag_join_kernel<<<1, 1, 0, stream>>>();
    CUDA_CHECK(cudaGetLastError());
    g_dag.leaves = stream_deps(stream);
    FHERT_ASSERT(g_dag.leaves.size() == 1, "capture: the join node did not take the leaves' place");
    g_dag.joins++;
  }
  set_stream_deps(stream, g_dag.leaves);
}

}  // namespace fhert
