// Best-fit allocator with immediate coalescing over a range of byte offsets.
//
// Takes over the job of gorgonia's bfc (cuda/bfc.go:298-463): host-side bookkeeping for one
// slab of device memory. Contract kept from the reference: alloc(size <= 0) fails, every
// returned offset is a multiple of the alignment, freeing an unknown offset does nothing,
// running out of room is reported with the amount asked for and the amount in use.
// The structure is different: free blocks sit in a size-ordered set (best fit in O(log n))
// and an offset-ordered map, and a freed block is merged with its neighbours at once, so
// there is no separate coalescing pass and no fragmentation ratio to watch.
#pragma once
#include <cstdint>
#include <map>
#include <set>
#include <utility>

namespace b200 {

class Bfc {
 public:
  Bfc() = default;
  Bfc(int64_t bytes, int64_t align) { reserve(bytes, align); }

  void reserve(int64_t bytes, int64_t align) {
    align_ = align > 0 ? align : 1;
    size_ = bytes - bytes % align_;
    reset();
  }

  void reset() {
    by_off_.clear();
    by_size_.clear();
    used_.clear();
    used_bytes_ = 0;
    if (size_ > 0) insert_free(0, size_);
  }

  // Returns 0 and the offset, or -1 (bad size) / -2 (out of memory).
  int alloc(int64_t bytes, int64_t *offset) {
    if (bytes <= 0) return -1;
    int64_t need = (bytes + align_ - 1) / align_ * align_;
    auto it = by_size_.lower_bound({need, -1});
    if (it == by_size_.end()) return -2;
    int64_t sz = it->first, off = it->second;
    erase_free(off, sz);
    if (sz > need) insert_free(off + need, sz - need);
    used_[off] = need;
    used_bytes_ += need;
    *offset = off;
    return 0;
  }

  // Returns 0 if the offset was live, 1 if it was unknown (nothing happens).
  int free(int64_t off) {
    auto u = used_.find(off);
    if (u == used_.end()) return 1;
    int64_t sz = u->second;
    used_.erase(u);
    used_bytes_ -= sz;
    // merge with the free block that starts where this one ends
    auto next = by_off_.find(off + sz);
    if (next != by_off_.end()) {
      int64_t nsz = next->second;
      erase_free(off + sz, nsz);
      sz += nsz;
    }
    // merge with the free block that ends where this one starts
    auto prev = by_off_.lower_bound(off);
    if (prev != by_off_.begin()) {
      --prev;
      if (prev->first + prev->second == off) {
        int64_t poff = prev->first, psz = prev->second;
        erase_free(poff, psz);
        off = poff;
        sz += psz;
      }
    }
    insert_free(off, sz);
    return 0;
  }

  bool is_live(int64_t off) const { return used_.count(off) != 0; }
  int64_t live_size(int64_t off) const {
    auto u = used_.find(off);
    return u == used_.end() ? 0 : u->second;
  }
  int64_t used() const { return used_bytes_; }
  int64_t capacity() const { return size_; }
  int64_t free_blocks() const { return (int64_t)by_off_.size(); }
  int64_t live_blocks() const { return (int64_t)used_.size(); }
  int64_t largest_free() const { return by_size_.empty() ? 0 : by_size_.rbegin()->first; }
  int64_t align() const { return align_; }

 private:
  void insert_free(int64_t off, int64_t sz) {
    by_off_[off] = sz;
    by_size_.insert({sz, off});
  }
  void erase_free(int64_t off, int64_t sz) {
    by_off_.erase(off);
    by_size_.erase({sz, off});
  }
  int64_t align_ = 256, size_ = 0, used_bytes_ = 0;
  std::map<int64_t, int64_t> by_off_;              // free: offset -> size
  std::set<std::pair<int64_t, int64_t>> by_size_;  // free: (size, offset)
  std::map<int64_t, int64_t> used_;                // live: offset -> size
};

}  // namespace b200
