// Rescale for callers that must not allocate.
//
// Rescale (api.cu) borrows its working storage -- the coefficient form of the
// limb being dropped plus one lifted copy per remaining limb -- from a
// stream-ordered allocation that grows on demand.  Some hosts cannot tolerate
// that: serving loops that have pinned down their device-memory budget at
// start-up and must not see it move, embedders whose policy forbids the driver
// allocator once the process is running, and callers sharing the GPU with
// another tenant whose allocations they must not disturb.
// Fhert_rescale_static does the same arithmetic with working storage that is
// part of the library image: a file-scope device array of fixed size that
// every GPU loading the library carries until the process exits.
//
// The guarantee "no allocator is called" holds for the call itself.  Work that
// earlier entry points deferred (a Rescale / Mod_down waiting for its sibling,
// recorded Hw_* calls) would run first and does allocate, so the call refuses
// with FHERT_STATIC_PENDING_WORK while such work is waiting: finish it with
// Fhert_sync (or any other entry point) before the phase that must not
// allocate.  With Fhert_profile_begin active every launch also records two
// CUDA events, created on first use.  A CUDA launch error still aborts.
#include "runtime.h"

namespace fhert {

// 40 limbs of 65536 words (20 MiB): enough for a polynomial of up to 40 limbs
// at ring degree 2^16, or proportionally more limbs at smaller degrees.
constexpr size_t kStaticScratchWords = 40ull * 65536ull;

static __device__ __align__(256) unsigned long long g_static_scratch[kStaticScratchWords];

namespace {

constexpr int kMaxDevices = 64;
// Device address of g_static_scratch for each device ordinal.  In host code the
// array's name is only a handle for the symbol look-up below; the address a
// kernel can use has to be asked from the runtime, once per device, while that
// device is current.
int64_t* g_scratch_addr[kMaxDevices] = {nullptr};

int64_t* static_scratch_for_current_device(int* status) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *status = FHERT_STATIC_NO_DEVICE;
    return nullptr;
  }
  if (g_scratch_addr[dev] == nullptr) {
    void*       p   = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&p, g_static_scratch);
    if (err != cudaSuccess || p == nullptr) {
      std::fprintf(stderr, "libFHErt_b200: cannot resolve the static scratch array: %s\n",
                   cudaGetErrorString(err));
      *status = FHERT_STATIC_NO_DEVICE;
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<int64_t*>(p);
  }
  return g_scratch_addr[dev];
}

}  // namespace
}  // namespace fhert

using namespace fhert;

extern "C" int Fhert_rescale_static(int64_t* res, const int64_t* poly, size_t level) {
  Context* c = ctx_or_null();
  if (c == nullptr) {
    std::fprintf(stderr, "libFHErt_b200: Fhert_rescale_static needs a prepared context\n");
    return FHERT_STATIC_NO_CONTEXT;
  }
  if (res == nullptr || poly == nullptr || level < 2 || level > (size_t)c->L) {
    std::fprintf(stderr,
                 "libFHErt_b200: Fhert_rescale_static: level %zu outside [2, %d] or null buffer\n",
                 level, c->L);
    return FHERT_STATIC_BAD_ARGUMENT;
  }
  const size_t n = c->N;
  if (level * n > kStaticScratchWords) {
    std::fprintf(stderr,
                 "libFHErt_b200: Fhert_rescale_static: %zu limbs of %zu words need %zu words of "
                 "working storage, the built-in array holds %zu; use Rescale instead\n",
                 level, n, level * n, (size_t)kStaticScratchWords);
    return FHERT_STATIC_TOO_LARGE;
  }
  if (c->pair_wait.kind != 0 || c->hw_pending) {
    std::fprintf(stderr,
                 "libFHErt_b200: Fhert_rescale_static: deferred work of earlier calls is waiting "
                 "and would allocate; call Fhert_sync first\n");
    return FHERT_STATIC_PENDING_WORK;
  }
  int      status = FHERT_STATIC_OK;
  int64_t* sc     = static_scratch_for_current_device(&status);
  if (sc == nullptr) return status;

  // Same sequence as Rescale in api.cu (rns_poly.c:310-404 of the CPU runtime):
  // inverse NTT of the last limb into slot 0, centred lift and scaling into
  // slots 1.., forward NTT of those, combine with the remaining limbs.  Every
  // slot is written before it is read, so nothing has to be cleared between
  // calls.
  const int l = (int)level - 1;
  LimbBatch lb;
  lb.count   = 1;
  lb.limb[0] = LimbRef{(uint16_t)l, 0, 0, (uint8_t)l, 0};
  launch_ntt(ptr2(poly), ptr2(sc), lb, true);
  LimbBatch bt;
  bt.count = l;
  for (int i = 0; i < l; i++)
    bt.limb[i] = LimbRef{(uint16_t)(1 + i), 0, (uint16_t)(1 + i), (uint8_t)i, 0};
  launch_rescale_lift(ptr2(sc), ptr2(sc), l, bt);
  launch_ntt(ptr2(sc), ptr2(sc), bt, false);
  for (int i = 0; i < l; i++)
    bt.limb[i] = LimbRef{(uint16_t)i, (uint16_t)(1 + i), (uint16_t)i, (uint8_t)i, 0};
  launch_rescale_combine(ptr2(res), ptr2(poly), ptr2(sc), l, bt);
  return FHERT_STATIC_OK;
}

extern "C" size_t Fhert_rescale_static_capacity(void) { return kStaticScratchWords; }
