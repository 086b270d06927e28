// Weight data files and the plaintexts made from them.
//
// A compiled program keeps its constants in a ".msg" file written by the
// compiler (layout: fhe-cmplr/include/fhe/core/rt_data_def.h:91-112): a 4 KiB
// header page, the float payload, then a lookup table of 32-byte entries at
// _lut_ofst.  The program asks for "entry index, len floats, at this scale
// degree and level" and gets an encoded plaintext (rtlib/ant/porting/
// pt_mgr.c:179-214).  Every call site asks for the same (entry, offset, len,
// scale, level) each time it runs, so an optional device-resident cache keeps
// the encoded limbs in HBM and hands out borrowed views.
//
// A file of the other entry type, DE_PLAINTEXT, holds plaintexts the offline
// encoder of the CPU runtime already encoded (one PLAINTEXT_BUFFER per entry:
// fhe-cmplr/include/fhe/core/rt_encode_api.h:22-27, written by
// Encode_plain_buffer, rtlib/ant/ckks/src/plain.c:196-217; read by
// pt_mgr.c:128-159): 8 bytes "ANTPLAIN", version, size, then the host
// PLAINTEXT struct with a null data pointer followed by level * N residues in
// NTT form.  Such an entry is uploaded the first time it is asked for and stays
// on the device; the caller's struct is filled with a borrowed view, which is
// what Free_data leaves alone for this file type (pt_mgr.c:179-183).
#include <cstring>
#include <ctime>
#include <map>
#include <set>
#include <tuple>
#include <vector>

#include "runtime.h"

using namespace fhert;

namespace {

constexpr uint64_t kPage = 4096;

struct FileHeader {  // rt_data_def.h:91-103
  char            magic[8];
  uint32_t        rt_ver;
  uint16_t        flag;
  uint8_t         ent_type;
  uint8_t         ent_align;
  uint64_t        ent_count;
  uint64_t        lut_ofst;
  struct timespec ctime;
  char            model[48];
  char            uuid[40];
};

struct LutEntry {  // rt_data_def.h:105-112
  char     name[16];
  uint32_t index;
  uint32_t size;
  uint64_t scale : 8;
  uint64_t level : 8;
  uint64_t ent_ofst : 48;
};
static_assert(sizeof(LutEntry) == 32, "lookup entry layout");

struct DataFile {
  bool                  open = false;
  FileHeader            hdr;
  std::vector<LutEntry> lut;
  std::vector<char>     payload;  // bytes [4096, lut_ofst) of the file
};
DataFile g_file;

using CacheKey = std::tuple<uint32_t, size_t, size_t, uint32_t, uint32_t>;
struct CacheState {
  std::map<CacheKey, PLAINTEXT> entries;
  std::set<const void*>         owned;  // limb storage held by the cache
  bool                          bypass = false;  // encode every request, keep the cache as it is
  size_t                        bytes = 0, budget = 0, hits = 0, misses = 0;
};
CacheState g_cache;

bool cache_owns(const void* data) { return g_cache.owned.count(data) != 0; }

const float* entry_floats(uint32_t index, size_t ofst, size_t len) {
  FHERT_ASSERT(g_file.open, "no data file is open (Get_rt_data_info returned none)");
  FHERT_ASSERT(g_file.hdr.ent_type != DE_PLAINTEXT, "bad entry type");
  FHERT_ASSERT(index < g_file.hdr.ent_count, "index out of entry range");
  const LutEntry& e = g_file.lut[index];
  FHERT_ASSERT(e.size >= len * sizeof(float), "entry size too small");
  FHERT_ASSERT(e.ent_ofst >= kPage, "entry offset too small");
  uint64_t at = e.ent_ofst - kPage;
  FHERT_ASSERT(at + (ofst + len) * sizeof(float) <= g_file.payload.size(),
               "entry offset too large");
  return reinterpret_cast<const float*>(g_file.payload.data() + at) + ofst;
}

struct PlainBufferHead {  // rt_encode_api.h:22-27
  char     magic[8];
  uint32_t version;
  uint32_t size;
};

// entry `index` of a DE_PLAINTEXT file as a device-resident plaintext
void* plain_from_encoded_entry(void* pt, uint32_t index, uint32_t level) {
  PLAIN plain = (PLAIN)pt;
  FHERT_ASSERT(index < g_file.hdr.ent_count, "index out of entry range");
  CacheKey key{index, 0, 0, 0, 0};
  auto     it = g_cache.entries.find(key);
  if (it == g_cache.entries.end()) {
    const LutEntry& e = g_file.lut[index];
    FHERT_ASSERT(e.ent_ofst >= kPage && e.ent_ofst - kPage + e.size <= g_file.payload.size(),
                 "entry outside the file");
    const char* at = g_file.payload.data() + (e.ent_ofst - kPage);
    PlainBufferHead head;
    std::memcpy(&head, at, sizeof(head));
    FHERT_ASSERT(std::memcmp(head.magic, "ANTPLAIN", 8) == 0 &&
                     sizeof(head) + head.size <= e.size && head.size >= sizeof(PLAINTEXT),
                 "entry %u is not an encoded plaintext", index);
    PLAINTEXT fresh;
    std::memcpy(&fresh, at + sizeof(head), sizeof(PLAINTEXT));
    Context*     c      = ctx();
    const size_t limbs  = fresh._poly._num_primes + fresh._poly._num_primes_p;
    const size_t words  = limbs * (size_t)fresh._poly._ring_degree;
    FHERT_ASSERT(fresh._poly._ring_degree == c->N && limbs > 0 &&
                     sizeof(PLAINTEXT) + words * sizeof(int64_t) <= head.size,
                 "encoded plaintext %u does not fit this context", index);
    fresh._poly._num_alloc_primes = limbs;
    fresh._poly._data             = nullptr;
    CUDA_CHECK(dev_alloc(&fresh._poly._data, words * sizeof(int64_t), c->stream));
    CUDA_CHECK(counted_copy(fresh._poly._data, at + sizeof(head) + sizeof(PLAINTEXT),
                            words * sizeof(int64_t), cudaMemcpyHostToDevice, c->stream));
    g_cache.bytes += words * sizeof(int64_t);
    g_cache.misses++;
    it = g_cache.entries.emplace(key, fresh).first;
    g_cache.owned.insert(fresh._poly._data);
  } else {
    g_cache.hits++;
  }
  FHERT_ASSERT(level == 0 || level == it->second._poly._num_primes,
               "plaintext %u was encoded at level %zu, asked for at level %u", index,
               it->second._poly._num_primes, level);
  if (plain->_poly._data && !cache_owns(plain->_poly._data)) Free_poly_data(&plain->_poly);
  *plain = it->second;
  return pt;
}

void* plain_from_entry(void* pt, uint32_t index, size_t ofst, size_t len, uint32_t scale,
                       uint32_t level) {
  PLAIN        plain = (PLAIN)pt;
  if (g_file.open && g_file.hdr.ent_type == DE_PLAINTEXT) {
    FHERT_ASSERT(ofst == 0, "bad entry type");  // pt_mgr.c:204
    return plain_from_encoded_entry(pt, index, level);
  }
  const float* data  = entry_floats(index, ofst, len);
  if (g_cache.budget == 0 || g_cache.bypass) {
    if (plain->_poly._data && cache_owns(plain->_poly._data)) {  // a borrowed view: drop it
      plain->_poly._data             = nullptr;
      plain->_poly._num_alloc_primes = 0;
    }
    Encode_float(plain, const_cast<float*>(data), len, scale, level);
    return pt;
  }
  CacheKey key{index, ofst, len, scale, level};
  auto     it = g_cache.entries.find(key);
  if (it == g_cache.entries.end()) {
    PLAINTEXT fresh;
    std::memset(&fresh, 0, sizeof(fresh));
    Encode_float(&fresh, const_cast<float*>(data), len, scale, level);
    size_t bytes = fresh._poly._num_alloc_primes * (size_t)fresh._poly._ring_degree * 8;
    if (g_cache.bytes + bytes > g_cache.budget) {  // over budget: hand it over uncached
      if (plain->_poly._data && !cache_owns(plain->_poly._data)) Free_poly_data(&plain->_poly);
      *plain = fresh;
      g_cache.misses++;
      return pt;
    }
    g_cache.bytes += bytes;
    g_cache.misses++;
    it = g_cache.entries.emplace(key, fresh).first;
    g_cache.owned.insert(fresh._poly._data);
  } else {
    g_cache.hits++;
  }
  if (plain->_poly._data && !cache_owns(plain->_poly._data)) Free_poly_data(&plain->_poly);
  *plain = it->second;  // borrowed view; Free_data leaves cache-owned limbs alone
  return pt;
}

}  // namespace

namespace fhert {
// programs of the older generation release plaintexts with Free_poly_data;
// limbs lent out by the cache must survive that
bool pt_cache_owns(const void* data) {
  return (g_cache.budget != 0 || (g_file.open && g_file.hdr.ent_type == DE_PLAINTEXT)) &&
         cache_owns(data);
}
}  // namespace fhert

extern "C" {

bool Pt_mgr_init(const char* fname) {
  FILE* f = std::fopen(fname, "rb");
  if (f == nullptr) return false;
  DataFile df;
  bool     ok = std::fread(&df.hdr, sizeof(FileHeader), 1, f) == 1 &&
            std::memcmp(df.hdr.magic, "!ANTFHE", 8) == 0 && df.hdr.lut_ofst >= kPage;
  if (ok) {
    df.lut.resize(df.hdr.ent_count);
    df.payload.resize(df.hdr.lut_ofst - kPage);
    ok = std::fseek(f, (long)df.hdr.lut_ofst, SEEK_SET) == 0 &&
         (df.lut.empty() ||
          std::fread(df.lut.data(), sizeof(LutEntry), df.lut.size(), f) == df.lut.size()) &&
         std::fseek(f, (long)kPage, SEEK_SET) == 0 &&
         (df.payload.empty() ||
          std::fread(df.payload.data(), 1, df.payload.size(), f) == df.payload.size());
  }
  std::fclose(f);
  FHERT_ASSERT(ok, "failed to read rt data file %s", fname);
  df.open = true;
  g_file  = std::move(df);
  const char* mb = std::getenv("FHERT_PT_CACHE_MB");
  g_cache.budget = mb ? (size_t)std::strtoull(mb, nullptr, 10) << 20 : 0;
  return true;
}

void Pt_mgr_fini(void) {
  for (auto& kv : g_cache.entries) Free_poly_data(&kv.second._poly);
  g_cache = CacheState();
  g_file  = DataFile();
}

void Fhert_pt_cache_bypass(int on) { g_cache.bypass = on != 0; }

void Fhert_pt_cache_stats(size_t* entries, size_t* bytes, size_t* hits, size_t* misses) {
  if (entries) *entries = g_cache.entries.size();
  if (bytes) *bytes = g_cache.bytes;
  if (hits) *hits = g_cache.hits;
  if (misses) *misses = g_cache.misses;
}

void* Pt_from_msg(void* pt, uint32_t index, size_t len, uint32_t scale, uint32_t level) {
  return plain_from_entry(pt, index, 0, len, scale, level);
}

void* Pt_from_msg_ofst(void* pt, uint32_t index, size_t ofst, size_t len, uint32_t scale,
                       uint32_t level) {
  return plain_from_entry(pt, index, ofst, len, scale, level);
}

// pt_mgr.c:179-183: plaintexts made from a message file own their limbs
void Free_data(void* poly) {
  POLY p = (POLY)poly;
  if (!g_file.open || p->_data == nullptr) return;
  if (cache_owns(p->_data)) {
    p->_data             = nullptr;
    p->_num_alloc_primes = 0;
    return;
  }
  Free_poly_data(p);
}

}  // extern "C"
