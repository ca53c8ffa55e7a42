// Caching block pool behind tvb_malloc / tvb_free.
//
// The reference gives every tensor its own cudaMalloc and cudaFree
// (include/backend/cuda/cuda_tensor.cpp:14-33, cuda_tensor.h:14-32), so each
// ops::Mul pays a device allocation for its result.  This pool keeps freed
// blocks and hands them out again: the steady state of a loop of matmuls makes
// no driver call at all.
//
// The pool is host code with the backing allocator injected, so its logic is
// tested on a machine without a GPU (malloc as backing, or a backing that fails
// on demand).  It is not stream-aware: a block must not be freed while work that
// uses it is still queued on a stream other than the one its next user runs on;
// the C ABI frees its own scratch only after ordering that with an event.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <unordered_map>

namespace tvb {

struct PoolStats {
  uint64_t bytes_in_use = 0;
  uint64_t bytes_cached = 0;
  uint64_t backing_allocs = 0;
  uint64_t backing_frees = 0;
  uint64_t reuse_hits = 0;
  uint64_t peak_bytes_in_use = 0;
};

class BlockPool {
 public:
  // return 0 on success; *p must be at least 256-byte aligned
  using BackingAlloc = int (*)(void** p, size_t bytes, void* user);
  using BackingFree = int (*)(void* p, void* user);

  BlockPool(BackingAlloc a, BackingFree f, void* user) : alloc_(a), free_(f), user_(user) {}
  BlockPool(const BlockPool&) = delete;
  BlockPool& operator=(const BlockPool&) = delete;
  ~BlockPool() { release_all(); }

  // Size classes: multiples of 512 B below 1 MiB, multiples of 2 MiB above, so that
  // the slightly different sizes of successive results still land on the same block.
  static size_t round_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    const size_t small = 512, large = size_t(2) << 20;
    if (bytes < (size_t(1) << 20)) return (bytes + small - 1) / small * small;
    return (bytes + large - 1) / large * large;
  }

  // 0 = ok, 1 = backing allocator failed even after the cache was emptied
  int allocate(size_t bytes, void** out) {
    const size_t want = round_size(bytes);
    std::lock_guard<std::mutex> g(mu_);
    // best fit among cached blocks, but never waste more than 1/8 of the block
    auto it = cached_.lower_bound(want);
    if (it != cached_.end() && it->first - want <= it->first / 8) {
      void* p = it->second;
      const size_t sz = it->first;
      cached_.erase(it);
      stats_.bytes_cached -= sz;
      live_[p] = sz;
      note_in_use(sz);
      stats_.reuse_hits++;
      *out = p;
      return 0;
    }
    void* p = nullptr;
    int rc = alloc_(&p, want, user_);
    if (rc != 0 || p == nullptr) {
      // out of memory: return everything cached to the driver and try once more
      trim_locked();
      p = nullptr;
      rc = alloc_(&p, want, user_);
      if (rc != 0 || p == nullptr) return 1;
    }
    stats_.backing_allocs++;
    live_[p] = want;
    note_in_use(want);
    *out = p;
    return 0;
  }

  // 0 = ok, 1 = pointer was not handed out by this pool (or freed twice)
  int release(void* p) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find(p);
    if (it == live_.end()) return 1;
    const size_t sz = it->second;
    live_.erase(it);
    stats_.bytes_in_use -= sz;
    cached_.emplace(sz, p);
    stats_.bytes_cached += sz;
    return 0;
  }

  bool owns(const void* p) {
    std::lock_guard<std::mutex> g(mu_);
    return live_.count(const_cast<void*>(p)) != 0;
  }

  void trim() {
    std::lock_guard<std::mutex> g(mu_);
    trim_locked();
  }

  // Frees cached AND live blocks (context teardown).
  void release_all() {
    std::lock_guard<std::mutex> g(mu_);
    trim_locked();
    for (auto& kv : live_) {
      free_(kv.first, user_);
      stats_.backing_frees++;
    }
    live_.clear();
    stats_.bytes_in_use = 0;
  }

  PoolStats stats() {
    std::lock_guard<std::mutex> g(mu_);
    return stats_;
  }

 private:
  void note_in_use(size_t sz) {
    stats_.bytes_in_use += sz;
    if (stats_.bytes_in_use > stats_.peak_bytes_in_use) stats_.peak_bytes_in_use = stats_.bytes_in_use;
  }
  void trim_locked() {
    for (auto& kv : cached_) {
      free_(kv.second, user_);
      stats_.backing_frees++;
    }
    cached_.clear();
    stats_.bytes_cached = 0;
  }

  BackingAlloc alloc_;
  BackingFree free_;
  void* user_;
  std::mutex mu_;
  std::multimap<size_t, void*> cached_;
  std::unordered_map<void*, size_t> live_;
  PoolStats stats_;
};

}  // namespace tvb
