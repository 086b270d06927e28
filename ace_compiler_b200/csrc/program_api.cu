// Entry points a compiled program and its driver use around the arithmetic:
// ciphertext metadata initialisers, accessors, tensors, program input/output
// and the per-operator timer.  Semantics follow the CPU runtime function of
// the same name; citations name files inside fhe-cmplr/rtlib/.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <ctime>
#include <map>
#include <string>
#include <vector>

#include "runtime.h"

using namespace fhert;

namespace {

// ant/poly/src/rns_poly.c:18-37: shape res like poly; reuse res's storage when
// large enough (cleared), else allocate zero-filled storage
void init_poly_like(POLY res, POLY poly) {
  if (poly == res) return;
  uint32_t n   = poly->_ring_degree;
  size_t   q   = poly->_num_primes, p = poly->_num_primes_p;
  if (res->_data == nullptr) {
    Alloc_poly_data(res, n, q, p);
  } else if (res->_num_alloc_primes < q + p) {
    Free_poly_data(res);
    Alloc_poly_data(res, n, q, p);
  } else {
    CUDA_CHECK(zero_async(res->_data, res->_num_alloc_primes * (size_t)n * sizeof(int64_t),
                          ctx()->stream));
    res->_ring_degree  = n;
    res->_num_primes   = q;
    res->_num_primes_p = p;
  }
  res->_is_ntt = poly->_is_ntt;
}

void set_level(POLY p, size_t level) {
  FHERT_ASSERT(p->_num_alloc_primes >= level + p->_num_primes_p, "raised level exceed alloc_size");
  p->_num_primes = level;
}

// ant/include/ckks/ciphertext.h:109-135: contents are kept when storage exists
void init_ciphertext(CIPHER res, uint32_t n, size_t level, size_t num_p, double sf,
                     uint32_t sf_degree, uint32_t slots) {
  res->_scaling_factor = sf;
  res->_sf_degree      = sf_degree;
  res->_slots          = slots;
  for (POLY p : {&res->_c0_poly, &res->_c1_poly}) {
    if (p->_data == nullptr) {
      Alloc_poly_data(p, n, level, num_p);
    } else {
      FHERT_ASSERT(p->_ring_degree == n, "unmatched ciphertxt");
      set_level(p, level);
    }
  }
}

// ciphertext.h:137-147
void init_from_ciph(CIPHER res, CIPHER ciph, double sf, uint32_t sf_degree) {
  res->_scaling_factor = sf;
  res->_sf_degree      = sf_degree;
  res->_slots          = ciph->_slots;
  if (res == ciph) return;
  init_poly_like(&res->_c0_poly, &ciph->_c0_poly);
  init_poly_like(&res->_c1_poly, &ciph->_c1_poly);
}

// ciphertext.h:203-238 without resizing: the operand of lower level
CIPHER lower_level(CIPHER a, CIPHER b) {
  if (a->_c0_poly._data == nullptr) return b;
  FHERT_ASSERT(b->_c0_poly._data != nullptr, "poly coeffs of input ciph is invalid");
  return a->_c0_poly._num_primes > b->_c0_poly._num_primes ? b : a;
}

CIPHER3 lower_level3(CIPHER3 a, CIPHER3 b) {
  if (a->_c0_poly._data == nullptr) return b;
  FHERT_ASSERT(b->_c0_poly._data != nullptr, "poly coeffs of input ciph is invalid");
  return a->_c0_poly._num_primes > b->_c0_poly._num_primes ? b : a;
}

// ant/ckks/src/cipher.c:27-34
void init_cipher(CIPHER res, CIPHER ciph, double sf, uint32_t sf_degree) {
  init_from_ciph(res, ciph, sf, sf_degree);
  res->_c0_poly._is_ntt = res->_c1_poly._is_ntt = true;
  set_level(&res->_c0_poly, ciph->_c0_poly._num_primes);
  set_level(&res->_c1_poly, ciph->_c0_poly._num_primes);
}

void init_ciph3_from(CIPHER3 res, POLY c0, POLY c1, POLY c2, double sf, uint32_t sf_degree,
                     uint32_t slots) {
  res->_scaling_factor = sf;
  res->_sf_degree      = sf_degree;
  res->_slots          = slots;
  init_poly_like(&res->_c0_poly, c0);
  init_poly_like(&res->_c1_poly, c1);
  init_poly_like(&res->_c2_poly, c2);
  for (POLY p : {&res->_c0_poly, &res->_c1_poly, &res->_c2_poly}) p->_is_ntt = true;
}

struct IoTable {
  std::map<std::string, std::vector<CIPHERTEXT*>> inputs, outputs;
};
IoTable g_io;

CIPHERTEXT* new_ciph() { return (CIPHERTEXT*)std::calloc(1, sizeof(CIPHERTEXT)); }

// ---- replay of a program run -------------------------------------------------
// A program run is a fixed sequence of launches: the program cannot branch on
// encrypted data, and levels, scales and slot counts are the same for every
// input.  With the replay mode on, the second Run_main_graph captures its
// launches into one CUDA graph (while the host code of the program runs as
// usual), and every later call copies the waiting inputs into the captured
// input blocks, launches the graph and hands out the captured output blocks:
// the host issues one launch per run instead of tens of thousands.
struct PinnedCiph {
  std::string name;
  size_t      idx;
  CIPHERTEXT  meta;  // host fields and device addresses at capture time
};
struct ImageReplay {
  int                     mode        = -1;  // -1: FHERT_REPLAY not read yet, 0 off, 1 on
  int                     direct_runs = 0;   // runs launched directly since the mode went on
  bool                    capturing   = false;
  cudaGraphExec_t         exec        = nullptr;
  uint64_t                launches    = 0;  // launches of this library one replay stands for
  uint64_t                replays     = 0;
  uint64_t                dag_nodes = 0, dag_edges = 0, dag_barriers = 0, dag_chain = 0;  // of the captured graph
  std::vector<PinnedCiph> inputs, outputs;
  std::string             why_off;
  // pinned snapshots of the host data the captured run copies to the device
  std::vector<char*>      stage_chunks;
  size_t                  stage_used = 0, stage_total = 0;  // bytes used in the last chunk / overall
};
constexpr size_t kStageChunk = (size_t)32 << 20;
ImageReplay g_replay;

bool replay_on() {
  if (g_replay.mode < 0) {
    const char* e = std::getenv("FHERT_REPLAY");
    g_replay.mode = e != nullptr && e[0] != '\0' && e[0] != '0';
  }
  return g_replay.mode == 1;
}

void replay_drop(const char* why) {
  Context* c = ctx_noflush();
  if (g_replay.exec != nullptr) {
    CUDA_CHECK(cudaGraphExecDestroy(g_replay.exec));  // a launch in flight still completes
    g_replay.exec = nullptr;
  }
  g_replay.inputs.clear();
  g_replay.outputs.clear();
  if (!g_replay.stage_chunks.empty()) {
    CUDA_CHECK(cudaStreamSynchronize(c->stream));  // a launch in flight may still read them
    for (char* p : g_replay.stage_chunks) CUDA_CHECK(cudaFreeHost(p));
    g_replay.stage_chunks.clear();
    g_replay.stage_used = g_replay.stage_total = 0;
  }
  g_replay.mode        = 0;
  g_replay.direct_runs = 0;
  if (why != nullptr) g_replay.why_off = why;
  dev_private_mode(false);
  dev_private_to_common(c->stream);
}

void launch_captured(Context* c, cudaGraph_t graph, bool keep) {
  cudaGraphExec_t exec = nullptr;
  CUDA_CHECK(cudaGraphInstantiate(&exec, graph, 0));
  CUDA_CHECK(cudaGraphDestroy(graph));
  CUDA_CHECK(cudaGraphLaunch(exec, c->stream));
  if (keep)
    g_replay.exec = exec;
  else
    CUDA_CHECK(cudaGraphExecDestroy(exec));
}

bool same_shape(const POLYNOMIAL& a, const POLYNOMIAL& b) {
  return a._ring_degree == b._ring_degree && a._num_alloc_primes == b._num_alloc_primes &&
         a._num_primes == b._num_primes && a._num_primes_p == b._num_primes_p &&
         a._is_ntt == b._is_ntt;
}

double g_tm_stamp = 0;

double wall_seconds() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

}  // namespace

namespace fhert {
bool image_capturing() { return g_replay.capturing; }

const void* image_capture_stage(const void* src, size_t bytes) {
  static size_t budget = [] {
    const char* e = std::getenv("FHERT_REPLAY_STAGE_MB");
    return (e != nullptr ? (size_t)std::strtoull(e, nullptr, 10) : (size_t)4096) << 20;
  }();
  const size_t need = (bytes + 255) & ~(size_t)255;
  if (g_replay.stage_total + need > budget) return nullptr;
  if (g_replay.stage_chunks.empty() || g_replay.stage_used + need > std::max(kStageChunk, need)) {
    char* chunk = nullptr;
    if (cudaMallocHost(&chunk, std::max(kStageChunk, need)) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    g_replay.stage_chunks.push_back(chunk);
    g_replay.stage_used = 0;
  }
  char* at = g_replay.stage_chunks.back() + g_replay.stage_used;
  std::memcpy(at, src, bytes);
  g_replay.stage_used += need;
  g_replay.stage_total += need;
  return at;
}

void image_capture_break(const char* why) {
  if (!g_replay.capturing) return;
  dag_end(nullptr, nullptr, nullptr);
  g_replay.capturing = false;  // first: the calls below pass the same guards
  Context*    c     = ctx_noflush();
  cudaGraph_t graph = nullptr;
  CUDA_CHECK(cudaStreamEndCapture(c->stream, &graph));
  FHERT_ASSERT(graph != nullptr, "Run_main_graph: the capture of the program run was lost");
  launch_captured(c, graph, false);
  dev_private_mode(false);
  g_replay.mode    = 0;
  g_replay.why_off = std::string("the run cannot be captured: ") + why;
}

void image_replay_release() {
  if (g_replay.mode == 1 || g_replay.exec != nullptr) replay_drop("the context was released");
  g_replay = ImageReplay();
}
}  // namespace fhert

extern "C" {

// ---- program-supplied hooks (include/common/rt_api.h:48-80), weak so that a
// host without a compiled program still links
__attribute__((weak)) DATA_SCHEME* Get_encode_scheme(int) { return nullptr; }
__attribute__((weak)) DATA_SCHEME* Get_decode_scheme(int) { return nullptr; }
__attribute__((weak)) RT_DATA_INFO* Get_rt_data_info(void) { return nullptr; }
__attribute__((weak)) int           Get_input_count(void) { return 0; }
__attribute__((weak)) int           Get_output_count(void) { return 0; }
__attribute__((weak)) bool          Main_graph(void) { return false; }

// ---- accessors (ant/include/poly/rns_poly.h:41-66, ant/ckks/src/cipher.c:164-170)
size_t   Poly_level(POLY poly) { return poly->_num_primes; }
size_t   Num_p(POLY poly) { return poly->_num_primes_p; }
size_t   Num_alloc(POLY poly) { return poly->_num_alloc_primes; }
uint32_t Sc_degree(CIPHER ciph) { return ciph->_sf_degree; }
uint32_t Get_slots(CIPHER ciph) { return ciph->_slots; }
void     Set_slots(CIPHER ciph, uint32_t slots) { ciph->_slots = slots; }

// ---- metadata initialisers (ant/ckks/src/cipher.c:36-156)
void Init_ciph_same_scale(CIPHER res, CIPHER ciph1, CIPHER ciph2) {
  CIPHER ciph = ciph2 != nullptr ? lower_level(ciph1, ciph2) : ciph1;
  if (ciph == ciph2 && ciph1->_c0_poly._data == nullptr) {
    init_from_ciph(ciph1, ciph2, ciph2->_scaling_factor, ciph2->_sf_degree);
  } else if (ciph->_c0_poly._data == nullptr) {
    std::memset(res, 0, sizeof(CIPHERTEXT));
    return;
  }
  init_ciphertext(res, ciph->_c0_poly._ring_degree, ciph->_c0_poly._num_primes,
                  ciph->_c0_poly._num_primes_p, ciph->_scaling_factor, ciph->_sf_degree,
                  ciph->_slots);
  res->_c0_poly._is_ntt = res->_c1_poly._is_ntt = true;
}

void Init_ciph_same_scale_plain(CIPHER res, CIPHER ciph, PLAIN plain) {
  init_cipher(res, ciph, ciph->_scaling_factor, ciph->_sf_degree);
  size_t pl = plain->_poly._num_primes;
  if (ciph->_c0_poly._num_primes > pl) {
    set_level(&res->_c0_poly, pl);
    set_level(&res->_c1_poly, pl);
  }
}

void Init_ciph_up_scale(CIPHER res, CIPHER ciph1, CIPHER ciph2) {
  CIPHER ciph = lower_level(ciph1, ciph2);
  init_cipher(res, ciph, ciph1->_scaling_factor * ciph2->_scaling_factor,
              ciph1->_sf_degree + ciph2->_sf_degree);
}

void Init_ciph_up_scale_plain(CIPHER res, CIPHER ciph, PLAIN plain) {
  init_cipher(res, ciph, ciph->_scaling_factor * plain->_scaling_factor,
              ciph->_sf_degree + plain->_sf_degree);
  size_t pl = plain->_poly._num_primes;
  if (ciph->_c0_poly._num_primes > pl) {
    set_level(&res->_c0_poly, pl);
    set_level(&res->_c1_poly, pl);
  }
}

void Init_ciph_down_scale(CIPHER res, CIPHER ciph) {
  FHERT_ASSERT(ciph->_sf_degree >= 2, "Scale degree of result dec to zero");
  init_cipher(res, ciph, ciph->_scaling_factor / Get_default_sc(), ciph->_sf_degree - 1);
}

void Init_ciph3_down_scale(CIPHER3 res, CIPHER3 ciph) {
  FHERT_ASSERT(ciph->_sf_degree >= 2, "Scale degree of result dec to zero");
  res->_scaling_factor = ciph->_scaling_factor / Get_default_sc();
  res->_sf_degree      = ciph->_sf_degree - 1;
  res->_slots          = ciph->_slots;
  init_poly_like(&res->_c0_poly, &ciph->_c0_poly);
  init_poly_like(&res->_c1_poly, &ciph->_c1_poly);
  init_poly_like(&res->_c2_poly, &ciph->_c2_poly);
}

void Init_ciph_same_scale_ciph3(CIPHER res, CIPHER3 ciph) {
  res->_scaling_factor = ciph->_scaling_factor;
  res->_sf_degree      = ciph->_sf_degree;
  res->_slots          = ciph->_slots;
  init_poly_like(&res->_c0_poly, &ciph->_c0_poly);
  init_poly_like(&res->_c1_poly, &ciph->_c1_poly);
  res->_c0_poly._is_ntt = res->_c1_poly._is_ntt = true;
  set_level(&res->_c0_poly, ciph->_c0_poly._num_primes);
  set_level(&res->_c1_poly, ciph->_c0_poly._num_primes);
}

void Init_ciph3_same_scale_ciph3(CIPHER3 res, CIPHER3 ciph1, CIPHER3 ciph2) {
  CIPHER3 ciph = ciph2 != nullptr ? lower_level3(ciph1, ciph2) : ciph1;
  init_ciph3_from(res, &ciph->_c0_poly, &ciph->_c1_poly, &ciph->_c2_poly,
                  ciph->_scaling_factor, ciph->_sf_degree, ciph->_slots);
}

void Init_ciph3_same_scale(CIPHER3 res, CIPHER3 ciph1, CIPHER3 ciph2) {
  Init_ciph3_same_scale_ciph3(res, ciph1, ciph2);
}

void Init_ciph3_up_scale(CIPHER3 res, CIPHER ciph1, CIPHER ciph2) {
  CIPHER ciph = lower_level(ciph1, ciph2);
  FHERT_ASSERT(ciph->_c0_poly._num_primes_p == 0, "invalid num of p primes");
  init_ciph3_from(res, &ciph->_c0_poly, &ciph->_c0_poly, &ciph->_c0_poly,
                  ciph1->_scaling_factor * ciph2->_scaling_factor,
                  ciph1->_sf_degree + ciph2->_sf_degree, ciph->_slots);
}

// FHERT_TRACE_SUMS=1: every Copy_ciph prints a checksum of the residues it
// copies (a debugging aid for comparing two runs operator by operator, in the
// spirit of the reference's trace file; drains the device each time)
}  // extern "C"
namespace fhert {
void trace_sum(const char* what, CIPHER ciph) {
  static int on = -1, serial = 0;
  if (on < 0) {
    const char* e = std::getenv("FHERT_TRACE_SUMS");
    on            = e != nullptr && e[0] != '\0' && e[0] != '0';
  }
  if (!on) return;
  size_t level = ciph->_c0_poly._num_primes, n = ciph->_c0_poly._ring_degree;
  std::vector<int64_t> host(level * n);
  uint64_t sum[2] = {0, 0};
  int      k      = 0;
  for (POLY p : {&ciph->_c0_poly, &ciph->_c1_poly}) {
    Fhert_download(p, 0, level, host.data());
    for (size_t i = 0; i < host.size(); i++) sum[k] = sum[k] * 1099511628211ull + (uint64_t)host[i];
    k++;
  }
  std::fprintf(stderr, "[FHERT_SUM] %d %s level %zu deg %u %016llx %016llx\n", serial++, what, level,
               ciph->_sf_degree, (unsigned long long)sum[0], (unsigned long long)sum[1]);
}
}  // namespace fhert
extern "C" {

void Copy_ciph(CIPHER res, CIPHER ciph) {
  trace_sum("copy", ciph);
  init_from_ciph(res, ciph, ciph->_scaling_factor, ciph->_sf_degree);
  Copy_poly(&res->_c0_poly, &ciph->_c0_poly);
  Copy_poly(&res->_c1_poly, &ciph->_c1_poly);
}

void Zero_ciph(CIPHER ciph) {
  Free_poly_data(&ciph->_c0_poly);
  Free_poly_data(&ciph->_c1_poly);
  std::memset(ciph, 0, sizeof(*ciph));
}

// ---- tensors (common/src/tensor.c)
TENSOR* Alloc_tensor(size_t n, size_t c, size_t h, size_t w, const double* vals) {
  size_t  bytes = n * c * h * w * sizeof(double);
  TENSOR* t     = (TENSOR*)std::malloc(sizeof(TENSOR) + bytes);
  t->_shape._n  = n;
  t->_shape._c  = c;
  t->_shape._h  = h;
  t->_shape._w  = w;
  if (vals) std::memcpy(t->_vals, vals, bytes);
  else std::memset(t->_vals, 0, bytes);
  return t;
}

void Free_tensor(TENSOR* tensor) { std::free(tensor); }

void Print_tensor(FILE* fp, TENSOR* t) {
  std::fprintf(fp, "(tensor): [\n");
  for (size_t n = 0; n < t->_shape._n; n++) {
    if (n) std::fprintf(fp, "\n");
    for (size_t c = 0; c < t->_shape._c; c++) {
      if (c) std::fprintf(fp, "\n");
      for (size_t h = 0; h < t->_shape._h; h++) {
        if (h) std::fprintf(fp, "\n");
        for (size_t w = 0; w < t->_shape._w; w++)
          std::fprintf(fp, " %f",
                       t->_vals[w + t->_shape._w * (h + t->_shape._h * (c + t->_shape._c * n))]);
      }
    }
  }
  std::fprintf(fp, "\n]\n");
  std::fflush(stdout);
}

// ---- result checks a program compiled with run-time validation calls
// (common/src/rt_validate.c:16-57)
void Validate_impl(double* res, double* msg, uint32_t len, int32_t epsilon) {
  double   error = std::pow(10, epsilon);
  uint32_t bad   = len;
  for (uint32_t i = 0; i < len; i++)
    if (std::fabs(res[i] - msg[i]) > error) {
      bad = i;
      break;
    }
  if (bad < len) {
    std::fprintf(stderr, "ERROR: validation failed at %d. %f != %f\n", bad, res[bad], msg[bad]);
    uint32_t start = bad > 4 ? bad - 4 : 0, end = std::min(start + 8, len);
    for (const char* row : {"idx", "res", "std"}) {
      std::fprintf(stderr, "%s: ", row);
      for (uint32_t j = start; j < end; j++) {
        if (row[0] == 'i') std::fprintf(stderr, "%7d%c ", j, j == bad ? '*' : ' ');
        else std::fprintf(stderr, "%8.4f ", row[0] == 'r' ? res[j] : msg[j]);
      }
      std::fprintf(stderr, "\n");
    }
  }
  std::fprintf(stdout, "%s: internal validation %s.\n", bad < len ? "ERROR" : "INFO",
               bad < len ? "fail" : "pass");
  std::fflush(stdout);
}

void Validate_value_range(bool within_range) {
  if (!within_range)
    std::fprintf(stdout,
                 "Please set a higher level or increase the difference between q0 and sf.\n");
}

// ---- event timers of newer generated programs (common/linux/rtlib_timing.c)
namespace {
struct TmEvent {
  uint64_t count = 0;
  double   total = 0;
};
std::map<std::pair<uint32_t, uint32_t>, TmEvent>            g_tm_events;
std::vector<std::pair<std::pair<uint32_t, uint32_t>, double>> g_tm_stack;
const char* tm_target() {
  static const char* t    = std::getenv("RTLIB_TIMING_OUTPUT");
  return t != nullptr && t[0] != '\0' ? t : nullptr;
}
}  // namespace

void Fhert_tm_event(uint32_t id, uint32_t sub, int end) {
  if (tm_target() == nullptr) return;
  Fhert_sync();
  double now = wall_seconds();
  if (!end) {
    g_tm_stack.push_back({{id, sub}, now});
    return;
  }
  FHERT_ASSERT(!g_tm_stack.empty() && g_tm_stack.back().first == std::make_pair(id, sub),
               "FATAL: RTM stack mismatch");
  TmEvent& e = g_tm_events[{id, sub}];
  e.count++;
  e.total += now - g_tm_stack.back().second;
  g_tm_stack.pop_back();
}

void Fhert_tm_report(void) {
  const char* t = tm_target();
  if (t == nullptr || g_tm_events.empty()) return;
  FILE* fp = !std::strcmp(t, "stdout") ? stdout : (!std::strcmp(t, "stderr") ? stderr : std::fopen(t, "w"));
  if (fp == nullptr) return;
  std::fprintf(fp, "%-12s %-6s %10s %14s\n", "event", "sub", "count", "seconds");
  for (auto& kv : g_tm_events)
    std::fprintf(fp, "%-12u %-6u %10llu %14.6f\n", kv.first.first, kv.first.second,
                 (unsigned long long)kv.second.count, kv.second.total);
  if (fp != stdout && fp != stderr) std::fclose(fp);
  else std::fflush(fp);
  g_tm_events.clear();
}

// ---- timer (common/src/rt_stat.c:23-31); scripts parse this line format
// FHERT_RT_STAT=0 silences the lines and skips the device drain they need
static bool tm_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = std::getenv("FHERT_RT_STAT");
    on            = !(e != nullptr && e[0] == '0');
  }
  // a timer line needs the device drained, which a captured run cannot do
  return on != 0 && !replay_on();
}

void Tm_start(const char*) {
  if (!tm_enabled()) return;
  Fhert_sync();
  g_tm_stamp = wall_seconds();
}

void Tm_taken(const char* msg) {
  if (!tm_enabled()) return;
  Fhert_sync();  // the queued kernels belong to the operator being timed
  double now = wall_seconds();
  std::fprintf(stdout, "[RT_STAT] %s takes %.3f seconds.\n", msg, now - g_tm_stamp);
  g_tm_stamp = now;
  std::fflush(stdout);
}

// ---- program input / output (ant/ckks/src/rtlib.c:164-244)
void Prepare_input(TENSOR* input, const char* name) {
  Context*     c      = ctx();
  DATA_SCHEME* scheme = nullptr;
  for (int i = 0; i < Get_input_count(); i++) {
    DATA_SCHEME* s = Get_encode_scheme(i);
    FHERT_ASSERT(s != nullptr, "invalid encode scheme");
    if (std::strcmp(s->_name, name) == 0) {
      scheme = s;
      break;
    }
  }
  FHERT_ASSERT(scheme != nullptr && scheme->_count > 0, "not find the input");
  size_t total = input->_shape._n * input->_shape._c * input->_shape._h * input->_shape._w;
  size_t hw    = input->_shape._h * input->_shape._w;
  for (int i = 0; i < scheme->_count; i++) {
    const MAP_DESC*     d = &scheme->_desc[i];
    std::vector<double> vec;
    if (d->_count == 0) {
      vec.assign(input->_vals, input->_vals + total);
    } else {
      FHERT_ASSERT(d->_kind == NORMAL && d->_stride == 1, "TODO: other kind");
      size_t loc   = d->_start;
      bool   begin = (loc % hw) == 0, end = ((loc + (size_t)d->_count * d->_stride) % hw) == 0;
      vec.resize(d->_count + 2 * d->_pad);
      for (int k = 0; k < d->_pad; k++)
        vec[k] = begin ? 0 : input->_vals[loc - (size_t)(d->_pad - k) * d->_stride];
      for (int k = 0; k < d->_count; k++, loc += d->_stride) vec[k + d->_pad] = input->_vals[loc];
      for (int k = 0; k < d->_pad; k++)
        vec[k + d->_pad + d->_count] = end ? 0 : input->_vals[loc + (size_t)k * d->_stride];
    }
    PLAINTEXT plain;
    std::memset(&plain, 0, sizeof(plain));
    // a one-element tensor still goes through the vector encoder here
    // (rtlib.c:181 calls the encoder directly, not Encode_double)
    std::vector<double> pairs(2 * vec.size(), 0.0);
    for (size_t k = 0; k < vec.size(); k++) pairs[2 * k] = vec[k];
    Encode_dcmplx(&plain, pairs.data(), vec.size(), 1, (uint32_t)c->input_level);
    CIPHERTEXT* ciph = new_ciph();
    Encrypt(ciph, &plain);
    Free_plain_data(&plain);
    auto& slot = g_io.inputs[name];
    if (slot.size() <= (size_t)i) slot.resize(i + 1, nullptr);
    slot[i] = ciph;
  }
}

CIPHERTEXT Get_input_data(const char* name, size_t idx) {
  auto it = g_io.inputs.find(name);
  FHERT_ASSERT(it != g_io.inputs.end() && idx < it->second.size() && it->second[idx],
               "not find data");
  CIPHERTEXT ret  = *it->second[idx];
  std::free(it->second[idx]);  // the polynomials now belong to the caller
  it->second[idx] = nullptr;
  return ret;
}

void Set_output_data(const char* name, size_t idx, CIPHER data) {
  CIPHERTEXT* out = new_ciph();
  Copy_ciph(out, data);
  Free_ciph_poly(data, 1);
  auto& slot = g_io.outputs[name];
  if (slot.size() <= idx) slot.resize(idx + 1, nullptr);
  slot[idx] = out;
}

// Launches the captured run on the inputs now waiting in the input table.
static bool replay_run() {
  Context* c = ctx();
  for (const PinnedCiph& in : g_replay.inputs) {
    auto it = g_io.inputs.find(in.name);
    if (it == g_io.inputs.end() || in.idx >= it->second.size() || !it->second[in.idx]) return false;
    const CIPHERTEXT* x = it->second[in.idx];
    if (!same_shape(x->_c0_poly, in.meta._c0_poly) || !same_shape(x->_c1_poly, in.meta._c1_poly) ||
        x->_slots != in.meta._slots || x->_sf_degree != in.meta._sf_degree ||
        x->_scaling_factor != in.meta._scaling_factor)
      return false;
  }
  for (const PinnedCiph& in : g_replay.inputs) {
    CIPHERTEXT*& x = g_io.inputs[in.name][in.idx];
    const POLYNOMIAL* src[2] = {&x->_c0_poly, &x->_c1_poly};
    const POLYNOMIAL* dst[2] = {&in.meta._c0_poly, &in.meta._c1_poly};
    for (int k = 0; k < 2; k++)
      CUDA_CHECK(counted_copy(dst[k]->_data, src[k]->_data,
                              src[k]->_num_alloc_primes * (size_t)c->N * sizeof(int64_t),
                              cudaMemcpyDeviceToDevice, c->stream));
    Free_ciph_poly(x, 1);  // the program would have taken and freed it
    std::free(x);
    x = nullptr;
  }
  CUDA_CHECK(cudaGraphLaunch(g_replay.exec, c->stream));
  c->launches += g_replay.launches;
  g_replay.replays++;
  for (const PinnedCiph& out : g_replay.outputs) {
    auto& slot = g_io.outputs[out.name];
    if (slot.size() <= out.idx) slot.resize(out.idx + 1, nullptr);
    if (slot[out.idx] != nullptr) {  // the result of the run before was never fetched
      Free_ciph_poly(slot[out.idx], 1);
      std::free(slot[out.idx]);
    }
    CIPHERTEXT* o = new_ciph();
    *o            = out.meta;
    dev_take_private(o->_c0_poly._data);
    dev_take_private(o->_c1_poly._data);
    slot[out.idx] = o;
  }
  return true;
}

// Runs the program once with its launches captured, then launches the capture.
static void capture_run() {
  Context* c = ctx();
  c->raised.valid = false;
  if (c->scratch) {  // so that the scratch the captured kernels use is a private block
    CUDA_CHECK(dev_free(c->scratch, c->stream));
    c->scratch       = nullptr;
    c->scratch_words = 0;
  }
  // idle blocks of the common lists go back to the driver: the capture needs the room
  dev_release_all(c->stream);
  CUDA_CHECK(cudaStreamSynchronize(c->stream));
  {
    int           dev  = 0;
    cudaMemPool_t pool = nullptr;
    CUDA_CHECK(cudaGetDevice(&dev));
    if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess && pool != nullptr)
      cudaMemPoolTrimTo(pool, 0);
    cudaGetLastError();
  }
  dev_private_mode(true);
  g_replay.inputs.clear();
  g_replay.outputs.clear();
  for (auto& kv : g_io.inputs)
    for (size_t i = 0; i < kv.second.size(); i++) {
      if (kv.second[i] == nullptr) continue;
      CIPHERTEXT* pinned = new_ciph();  // a private copy: replays write the next input here
      Copy_ciph(pinned, kv.second[i]);
      Free_ciph_poly(kv.second[i], 1);
      std::free(kv.second[i]);
      kv.second[i] = pinned;
      g_replay.inputs.push_back(PinnedCiph{kv.first, i, *pinned});
    }
  for (auto& kv : g_io.outputs)
    for (CIPHERTEXT*& o : kv.second)
      if (o != nullptr) {  // left over from a run nobody fetched
        Free_ciph_poly(o, 1);
        std::free(o);
        o = nullptr;
      }
  c = ctx();
  const uint64_t launches0 = c->launches;
  CUDA_CHECK(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeRelaxed));
  g_replay.capturing = true;
  dag_begin();
  bool ok = Main_graph();
  c       = ctx();  // work still deferred belongs to this run
  c->raised.valid = false;
  if (g_replay.capturing) {
    dag_end(&g_replay.dag_nodes, &g_replay.dag_edges, &g_replay.dag_barriers, &g_replay.dag_chain);
    g_replay.capturing = false;
    cudaGraph_t graph  = nullptr;
    CUDA_CHECK(cudaStreamEndCapture(c->stream, &graph));
    FHERT_ASSERT(graph != nullptr, "Run_main_graph: the capture of the program run was lost");
    launch_captured(c, graph, true);
    g_replay.launches = c->launches - launches0;
    if (const char* e = std::getenv("FHERT_REPLAY_STATS"))
      if (e[0] == '1')
        std::fprintf(stderr, "[FHERT_REPLAY] %llu launches captured; %llu described nodes, %llu "
                     "dependences among them, %llu barriers, %llu joins\n",
                     (unsigned long long)g_replay.launches, (unsigned long long)g_replay.dag_nodes,
                     (unsigned long long)g_replay.dag_edges,
                     (unsigned long long)(g_replay.dag_barriers & 0xffffffffu),
                     (unsigned long long)(g_replay.dag_barriers >> 32));
    for (auto& kv : g_io.outputs)
      for (size_t i = 0; i < kv.second.size(); i++)
        if (kv.second[i] != nullptr) g_replay.outputs.push_back(PinnedCiph{kv.first, i, *kv.second[i]});
    dev_private_mode(false);
  } else {
    replay_drop(nullptr);  // the capture was ended on the way; the reason is already noted
  }
  FHERT_ASSERT(ok, "run Main_graph failed");
}

void Run_main_graph(void) {
  if (replay_on() && !prof_running()) {
    if (g_replay.exec != nullptr) {
      if (replay_run()) return;
      replay_drop("the waiting inputs do not match the captured ones");
    } else if (g_replay.direct_runs >= 1) {
      // the first run filled the caches and built the tables made on first use
      capture_run();
      return;
    }
  }
  if (g_replay.mode == 1) g_replay.direct_runs++;
  bool ok = Main_graph();
  FHERT_ASSERT(ok, "run Main_graph failed");
}

// No counterpart in the CPU runtime.  on != 0: the next but one Run_main_graph
// is captured and later ones replay it (see the comment on ImageReplay);
// on == 0: the capture is dropped and runs are launched directly again.
// FHERT_REPLAY=1 in the environment switches the mode on at the first run.
void Fhert_replay_mode(int on) {
  ctx();
  if (on) {
    if (g_replay.mode != 1) {
      g_replay.mode        = 1;
      g_replay.direct_runs = 0;
      g_replay.why_off.clear();
    }
  } else if (g_replay.mode == 1 || g_replay.exec != nullptr) {
    replay_drop("switched off");
  } else {
    g_replay.mode = 0;
  }
}

// Shape of the captured graph: launches of this library in it, launches (or
// groups of launches) whose memory accesses were described, dependences among
// those, launches nobody described (each orders everything around it), and the
// longest chain of described launches.  Zeros when nothing is captured.
void Fhert_replay_graph(uint64_t* launches, uint64_t* described, uint64_t* dependences,
                        uint64_t* undescribed_barriers, uint64_t* longest_chain) {
  const bool have = g_replay.exec != nullptr;
  if (launches) *launches = have ? g_replay.launches : 0;
  if (described) *described = have ? g_replay.dag_nodes : 0;
  if (dependences) *dependences = have ? g_replay.dag_edges : 0;
  if (undescribed_barriers) *undescribed_barriers = have ? (g_replay.dag_barriers & 0xffffffffu) : 0;
  if (longest_chain) *longest_chain = have ? g_replay.dag_chain : 0;
}

// 0: off (why, when given, receives the reason the mode went off by itself),
// 1: on, nothing captured yet, 2: a captured run is being replayed.
int Fhert_replay_state(char* why, size_t cap, uint64_t* replays) {
  if (why != nullptr && cap > 0) std::snprintf(why, cap, "%s", g_replay.why_off.c_str());
  if (replays != nullptr) *replays = g_replay.replays;
  if (!replay_on()) return 0;
  return g_replay.exec != nullptr ? 2 : 1;
}

double* Handle_output(const char* name) {
  Context*     c      = ctx();
  DATA_SCHEME* scheme = nullptr;
  for (int i = 0; i < Get_output_count(); i++) {
    DATA_SCHEME* s = Get_decode_scheme(i);
    FHERT_ASSERT(s != nullptr, "invalid encode scheme");
    if (std::strcmp(s->_name, name) == 0) {
      scheme = s;
      break;
    }
  }
  FHERT_ASSERT(scheme != nullptr && scheme->_count > 0, "not find the output");
  size_t len = scheme->_shape._n * scheme->_shape._c * scheme->_shape._h * scheme->_shape._w;
  if (len == 0) len = c->N / 2;
  double* ret = (double*)std::calloc(len, sizeof(double));
  auto    it  = g_io.outputs.find(name);
  FHERT_ASSERT(it != g_io.outputs.end(), "not find data");
  for (int i = 0; i < scheme->_count; i++) {
    FHERT_ASSERT((size_t)i < it->second.size() && it->second[i], "not find data");
    CIPHERTEXT* ciph = it->second[i];
    PLAINTEXT   plain;
    std::memset(&plain, 0, sizeof(plain));
    Fhert_decrypt(&plain, ciph);
    size_t              slots = plain._slots;
    std::vector<double> vals(2 * slots);
    Fhert_decode(&plain, vals.data(), slots);
    const MAP_DESC* d = &scheme->_desc[i];
    if (d->_count == 0) {
      size_t out_len = slots < len ? slots : len;
      for (size_t k = 0; k < out_len; k++) ret[k] = vals[2 * k];
    } else {
      FHERT_ASSERT((size_t)d->_count <= len && d->_kind == NORMAL, "chunk out of image bound");
      size_t loc = d->_start;
      for (int k = 0; k < d->_count; k++, loc += d->_stride) ret[loc] = vals[2 * k];
    }
    Free_plain_data(&plain);
    Free_ciph_poly(ciph, 1);
    std::free(ciph);
    it->second[i] = nullptr;
  }
  return ret;
}

}  // extern "C"
