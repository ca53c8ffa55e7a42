// Host-only unit test of the caching block pool (tensorvia_b200/csrc/block_pool.h) with
// malloc as the backing allocator and a switch that makes the backing allocator fail.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "block_pool.h"

static int g_allocs = 0, g_frees = 0;
static bool g_fail = false;
static size_t g_budget = ~size_t(0), g_used = 0;

static int fake_alloc(void** p, size_t bytes, void*) {
  if (g_fail || g_used + bytes > g_budget) return 1;
  *p = aligned_alloc(256, bytes);
  if (!*p) return 1;
  g_used += bytes;
  ++g_allocs;
  // remember the size in a side table through the pointer value itself
  return 0;
}
static std::vector<std::pair<void*, size_t>> g_sizes;
static int fake_alloc_tracked(void** p, size_t bytes, void* u) {
  int rc = fake_alloc(p, bytes, u);
  if (rc == 0) g_sizes.emplace_back(*p, bytes);
  return rc;
}
static int fake_free(void* p, void*) {
  for (auto& kv : g_sizes)
    if (kv.first == p) { g_used -= kv.second; kv.first = nullptr; }
  free(p);
  ++g_frees;
  return 0;
}

#define CHECK(c) do { if (!(c)) { printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); return 1; } } while (0)

int main() {
  using tvb::BlockPool;
  CHECK(BlockPool::round_size(1) == 512);
  CHECK(BlockPool::round_size(513) == 1024);
  CHECK(BlockPool::round_size((1u << 20) + 1) == (size_t(2) << 20));
  CHECK(BlockPool::round_size(size_t(33) << 20) == (size_t(34) << 20));
  {
    BlockPool pool(fake_alloc_tracked, fake_free, nullptr);
    void *a = nullptr, *b = nullptr, *c = nullptr;
    CHECK(pool.allocate(1000, &a) == 0 && a);
    CHECK((reinterpret_cast<uintptr_t>(a) & 255) == 0);
    CHECK(pool.allocate(1000, &b) == 0 && b != a);
    CHECK(pool.stats().bytes_in_use == 2048 && pool.stats().backing_allocs == 2);
    CHECK(pool.release(a) == 0);
    CHECK(pool.release(a) == 1);                 // double free is refused
    int dummy;
    CHECK(pool.release(&dummy) == 1);            // foreign pointer is refused
    CHECK(pool.stats().bytes_cached == 1024);
    CHECK(pool.allocate(900, &c) == 0 && c == a);  // same size class: served from the cache
    CHECK(pool.stats().reuse_hits == 1 && pool.stats().backing_allocs == 2);
    // a much smaller request must not burn a large cached block
    void* big = nullptr;
    CHECK(pool.allocate(size_t(64) << 20, &big) == 0);
    CHECK(pool.release(big) == 0);
    void* small = nullptr;
    CHECK(pool.allocate(size_t(4) << 20, &small) == 0 && small != big);
    // a result that is a little smaller reuses the block (within 1/8)
    void* again = nullptr;
    CHECK(pool.allocate(size_t(60) << 20, &again) == 0 && again == big);
    CHECK(pool.stats().peak_bytes_in_use >= (size_t(64) << 20));
    // steady state of a loop: no backing allocation after the first round
    const auto before = pool.stats().backing_allocs;
    for (int i = 0; i < 100; ++i) {
      void* r = nullptr;
      CHECK(pool.allocate(size_t(42) << 20, &r) == 0);
      CHECK(pool.release(r) == 0);
    }
    CHECK(pool.stats().backing_allocs == before + 1);
    pool.trim();
    CHECK(pool.stats().bytes_cached == 0);
    // injected allocation failure
    g_fail = true;
    void* f = nullptr;
    CHECK(pool.allocate(123456, &f) == 1);
    g_fail = false;
    // out of memory with a full cache: the pool empties its cache and retries
    g_budget = g_used + (size_t(16) << 20);
    void* x = nullptr;
    CHECK(pool.allocate(size_t(12) << 20, &x) == 0);
    CHECK(pool.release(x) == 0);                 // 12 MiB now cached, 4 MiB of budget left
    void* y = nullptr;
    CHECK(pool.allocate(size_t(14) << 20, &y) == 0);  // only fits after the cached block is returned
    CHECK(pool.stats().bytes_cached == 0);
    g_budget = ~size_t(0);
  }
  CHECK(g_allocs == g_frees);  // the destructor gave everything back, live blocks included
  printf("block pool: all checks passed (%d backing allocations)\n", g_allocs);
  return 0;
}
