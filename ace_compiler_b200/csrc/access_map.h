// Who last wrote and who has read each piece of memory since: the bookkeeping
// behind the data-flow dependences of a captured program run (capture_dag.cu).
// Plain C++, no CUDA: Node is any value type with an "empty" value Node().
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <utility>
#include <vector>

namespace fhert {

typedef std::vector<std::pair<uintptr_t, uintptr_t>> ByteRanges;  // half-open [first, second)

template <typename Node>
class AccessMap {
 public:
  // Nodes a launch has to wait for: the last writer of everything it reads,
  // the last writer and all readers since of everything it writes.  Appended
  // to deps, which the caller sorts and de-duplicates.
  void dependences(const ByteRanges& reads, const ByteRanges& writes, std::vector<Node>& deps) {
    for (const auto& r : reads)
      for_each(r.first, r.second, [&](Seg& s) {
        if (s.writer != Node()) deps.push_back(s.writer);
      });
    for (const auto& w : writes)
      for_each(w.first, w.second, [&](Seg& s) {
        if (s.writer != Node()) deps.push_back(s.writer);
        deps.insert(deps.end(), s.readers.begin(), s.readers.end());
      });
  }

  // The launch has become `node`: written pieces have one writer and no
  // readers, read pieces one more reader.
  void record(const ByteRanges& reads, const ByteRanges& writes, Node node) {
    for (const auto& w : writes) {
      split_at(w.first);
      split_at(w.second);
      segs_.erase(segs_.lower_bound(w.first), segs_.lower_bound(w.second));
      segs_[w.first] = Seg{w.second, node, {}};
    }
    for (const auto& r : reads) {
      // pieces of the range never touched before get a segment without writer
      split_at(r.first);
      split_at(r.second);
      uintptr_t  at = r.first;
      ByteRanges gaps;
      for (auto it = segs_.lower_bound(r.first); it != segs_.end() && it->first < r.second; ++it) {
        if (it->first > at) gaps.emplace_back(at, it->first);
        at = it->second.end;
      }
      if (at < r.second) gaps.emplace_back(at, r.second);
      for (auto& g : gaps) segs_[g.first] = Seg{g.second, Node(), {}};
      for_each(r.first, r.second, [&](Seg& s) {
        if (s.writer != node) s.readers.push_back(node);
      });
    }
  }

  void   clear() { segs_.clear(); }
  size_t pieces() const { return segs_.size(); }

 private:
  struct Seg {
    uintptr_t         end;
    Node              writer;  // Node(): not written since the map was cleared
    std::vector<Node> readers;
  };
  std::map<uintptr_t, Seg> segs_;  // disjoint pieces of touched memory by start address

  // makes `at` a piece boundary if it falls inside a piece
  void split_at(uintptr_t at) {
    auto it = segs_.upper_bound(at);
    if (it == segs_.begin()) return;
    --it;
    if (it->first < at && at < it->second.end) {
      Seg right      = it->second;
      it->second.end = at;
      segs_[at]      = right;
    }
  }
  template <typename F>
  void for_each(uintptr_t a, uintptr_t b, F&& f) {
    split_at(a);
    split_at(b);
    for (auto it = segs_.lower_bound(a); it != segs_.end() && it->first < b; ++it) f(it->second);
  }
};

}  // namespace fhert
