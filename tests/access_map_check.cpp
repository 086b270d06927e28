// Brute-force check of ace_compiler_b200/csrc/access_map.h: random launches over a
// small address space; the dependences the map reports must equal those of a
// per-byte record of last writer and readers.  Prints "ok <launches>" or the
// first mismatches.
#include <cstdio>
#include <cstdlib>
#include <set>

#include "access_map.h"

int main() {
  const int M = 240;
  fhert::AccessMap<int> map;
  std::vector<int>           writer(M, 0);
  std::vector<std::set<int>> readers(M);
  srand(12345);
  int bad = 0;
  const int launches = 30000;
  for (int node = 1; node <= launches; node++) {
    fhert::ByteRanges reads, writes;
    auto some = [&](fhert::ByteRanges& v, int count) {
      for (int i = 0; i < count; i++) {
        uintptr_t a = rand() % M, b = a + 1 + rand() % 40;
        if (b > (uintptr_t)M) b = M;
        v.emplace_back(a, b);
      }
    };
    some(reads, rand() % 4);
    some(writes, rand() % 3);
    if (rand() % 7 == 0 && !writes.empty()) reads.push_back(writes[0]);  // in place
    std::set<int> want;
    for (auto& r : reads)
      for (uintptr_t c = r.first; c < r.second; c++)
        if (writer[c]) want.insert(writer[c]);
    for (auto& w : writes)
      for (uintptr_t c = w.first; c < w.second; c++) {
        if (writer[c]) want.insert(writer[c]);
        want.insert(readers[c].begin(), readers[c].end());
      }
    std::vector<int> got;
    map.dependences(reads, writes, got);
    if (std::set<int>(got.begin(), got.end()) != want && bad++ < 5)
      printf("launch %d: %zu dependences reported, %zu expected\n", node, got.size(), want.size());
    map.record(reads, writes, node);
    std::set<uintptr_t> written;
    for (auto& w : writes)
      for (uintptr_t c = w.first; c < w.second; c++) {
        writer[c] = node;
        readers[c].clear();
        written.insert(c);
      }
    for (auto& r : reads)
      for (uintptr_t c = r.first; c < r.second; c++)
        if (!written.count(c)) readers[c].insert(node);
    if (node % 5000 == 0) {  // a barrier: everything before is ordered before everything after
      map.clear();
      std::fill(writer.begin(), writer.end(), 0);
      for (auto& s : readers) s.clear();
    }
  }
  if (bad) return 1;
  printf("ok %d\n", launches);
  return 0;
}
