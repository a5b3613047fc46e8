// Page-id allocator of the paged cache (control plane only: it owns no memory).
//
// Same surface and behaviour as the reference's pool
// (core/include/distie/block_pool.h:16-44, core/src/block_pool.cpp:25-114):
// ids 0..n-1, the first allocations return 0, 1, 2, ...; freed ids are handed out
// again last-in-first-out; Allocate and Free are all-or-nothing; a bad id, a
// duplicate inside one call or a double free throws std::invalid_argument before
// anything changes; every call takes the mutex.  With DISTIE_MEMORY_LOG=1 events
// go to stderr.
#pragma once

#include <cstddef>
#include <cstdint>
#include <mutex>
#include <vector>

namespace distie_b200 {

using PageId = std::int32_t;

class BlockPool {
 public:
  explicit BlockPool(std::size_t num_blocks);
  ~BlockPool();
  BlockPool(const BlockPool&) = delete;
  BlockPool& operator=(const BlockPool&) = delete;

  std::vector<PageId> Allocate(std::size_t count);
  void Free(const std::vector<PageId>& ids);

  std::size_t num_blocks() const noexcept { return held_.size(); }
  std::size_t num_free() const;
  std::size_t num_used() const;
  double utilization() const;

 private:
  mutable std::mutex mutex_;
  std::vector<PageId> stack_;          // free ids; back() is handed out next
  std::vector<std::uint8_t> held_;     // 1 while an id is out
  std::vector<std::uint32_t> marked_;  // call number that last named the id (duplicate check)
  std::uint32_t call_ = 0;
};

}  // namespace distie_b200
