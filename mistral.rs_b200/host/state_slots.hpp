// Fixed pool of recurrent-state slots, the counterpart of the block pool for layers whose memory of a sequence is
// a constant-size state (linear attention, state-space layers, carried convolution inputs) instead of pages:
// a request takes one slot at admission and gives it back when it ends.  Slots are handed out lowest-free-first so
// a trace of admissions and releases always yields the same slot numbers.  Host-only.
#pragma once
#include <cstdint>
#include <set>
#include <unordered_map>

namespace mrs {

class StateSlotPool {
 public:
  explicit StateSlotPool(size_t n) : n_(n) {
    for (size_t i = 0; i < n; i++) free_.insert(i);
  }
  size_t capacity() const { return n_; }
  size_t num_free() const { return free_.size(); }
  // slot of the request (taking a new one for an unknown request), or -1 when none is free
  int64_t acquire(uint64_t req) {
    auto it = owner_.find(req);
    if (it != owner_.end()) return (int64_t)it->second;
    if (free_.empty()) return -1;
    const size_t s = *free_.begin();
    free_.erase(free_.begin());
    owner_.emplace(req, s);
    return (int64_t)s;
  }
  int64_t slot_of(uint64_t req) const {
    auto it = owner_.find(req);
    return it == owner_.end() ? -1 : (int64_t)it->second;
  }
  bool release(uint64_t req) {
    auto it = owner_.find(req);
    if (it == owner_.end()) return false;
    free_.insert(it->second);
    owner_.erase(it);
    return true;
  }

 private:
  size_t n_;
  std::set<size_t> free_;
  std::unordered_map<uint64_t, size_t> owner_;
};

}  // namespace mrs
