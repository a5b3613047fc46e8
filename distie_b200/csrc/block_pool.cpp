#include "block_pool.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <string>

namespace distie_b200 {
namespace {

bool LogOn() {
  const char* flag = std::getenv("DISTIE_MEMORY_LOG");
  return flag != nullptr && std::strcmp(flag, "1") == 0;
}

void Log(const std::string& text) {
  if (LogOn()) std::fprintf(stderr, "[distie.memory] %s\n", text.c_str());
}

}  // namespace

BlockPool::BlockPool(std::size_t num_blocks) {
  if (num_blocks == 0) throw std::invalid_argument("num_blocks must be > 0");
  if (num_blocks > static_cast<std::size_t>(std::numeric_limits<PageId>::max()))
    throw std::invalid_argument("num_blocks exceeds the page id range");
  held_.assign(num_blocks, 0);
  marked_.assign(num_blocks, 0);
  stack_.resize(num_blocks);
  // Highest id at the bottom so that the first allocations come out as 0, 1, 2, ...
  for (std::size_t i = 0; i < num_blocks; ++i) stack_[i] = static_cast<PageId>(num_blocks - 1 - i);
  Log("pool constructed num_blocks=" + std::to_string(num_blocks));
}

BlockPool::~BlockPool() { Log("pool destroyed used=" + std::to_string(held_.size() - stack_.size())); }

std::vector<PageId> BlockPool::Allocate(std::size_t count) {
  std::vector<PageId> out;
  if (count == 0) return out;
  std::lock_guard<std::mutex> guard(mutex_);
  if (count > stack_.size()) {
    Log("allocate failed requested=" + std::to_string(count) + " free=" + std::to_string(stack_.size()));
    throw std::runtime_error("out of blocks: requested " + std::to_string(count) + ", free " +
                             std::to_string(stack_.size()));
  }
  out.assign(stack_.rbegin(), stack_.rbegin() + static_cast<std::ptrdiff_t>(count));
  stack_.resize(stack_.size() - count);
  for (PageId id : out) held_[static_cast<std::size_t>(id)] = 1;
  return out;
}

void BlockPool::Free(const std::vector<PageId>& ids) {
  if (ids.empty()) return;
  std::lock_guard<std::mutex> guard(mutex_);
  if (++call_ == 0) {  // the counter wrapped: forget old marks
    std::fill(marked_.begin(), marked_.end(), 0u);
    call_ = 1;
  }
  for (PageId id : ids) {  // check everything before anything changes
    if (id < 0 || static_cast<std::size_t>(id) >= held_.size())
      throw std::invalid_argument("block id out of range: " + std::to_string(id));
    const std::size_t at = static_cast<std::size_t>(id);
    if (marked_[at] == call_) throw std::invalid_argument("duplicate block id in free(): " + std::to_string(id));
    marked_[at] = call_;
    if (!held_[at]) throw std::invalid_argument("double free of block " + std::to_string(id));
  }
  for (PageId id : ids) {
    held_[static_cast<std::size_t>(id)] = 0;
    stack_.push_back(id);
  }
}

std::size_t BlockPool::num_free() const {
  std::lock_guard<std::mutex> guard(mutex_);
  return stack_.size();
}

std::size_t BlockPool::num_used() const {
  std::lock_guard<std::mutex> guard(mutex_);
  return held_.size() - stack_.size();
}

double BlockPool::utilization() const {
  std::lock_guard<std::mutex> guard(mutex_);
  return static_cast<double>(held_.size() - stack_.size()) / static_cast<double>(held_.size());
}

}  // namespace distie_b200
