// General-purpose offset allocator over one caller-owned range (pinned host slabs of the offload engine, long-lived device
// reservations): allocate and free in any order, best fit, neighbouring free blocks coalesce.
//
// The reference's CPUOffloadEngine keeps an 8 GB pool and hands regions of it to a worker thread
// (src/zero_optimizer_core.cpp:357-564). Pinning memory is the expensive part on a GPU host (a driver call that takes
// milliseconds per allocation), so the pool pins ONE slab and this allocator carves it; like the arenas of this library it
// never touches the memory itself, it only does the bookkeeping of [0, capacity).
#include <cstdint>
#include <map>
#include <mutex>

namespace {
struct OffsetPool {
  uint64_t capacity = 0, used = 0, peak = 0, allocations = 0, failures = 0;
  std::map<uint64_t, uint64_t> free_by_offset;  // offset -> size
  std::map<uint64_t, uint64_t> live;            // offset -> size
  std::mutex m;
};
inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }
}  // namespace

extern "C" {

void* inv_pool_create(uint64_t capacity) {
  OffsetPool* p = new OffsetPool();
  p->capacity = capacity;
  if (capacity) p->free_by_offset[0] = capacity;
  return p;
}

void inv_pool_destroy(void* h) { delete static_cast<OffsetPool*>(h); }

// Best fit: the smallest free block that holds `bytes` at `alignment` (a power of two, at least 256). The head and tail
// of the chosen block that are not used go back to the free list. Returns UINT64_MAX when nothing fits.
uint64_t inv_pool_alloc(void* h, uint64_t bytes, uint64_t alignment) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  if (alignment < 256) alignment = 256;
  if (bytes == 0) bytes = 1;
  std::lock_guard<std::mutex> g(p->m);
  auto best = p->free_by_offset.end();
  uint64_t best_size = UINT64_MAX;
  for (auto it = p->free_by_offset.begin(); it != p->free_by_offset.end(); ++it) {
    const uint64_t start = align_up(it->first, alignment);
    if (start + bytes > it->first + it->second || start + bytes < start) continue;
    if (it->second < best_size) {
      best = it;
      best_size = it->second;
    }
  }
  if (best == p->free_by_offset.end()) {
    p->failures++;
    return UINT64_MAX;
  }
  const uint64_t off = best->first, size = best->second, start = align_up(off, alignment), end = start + bytes;
  p->free_by_offset.erase(best);
  if (start > off) p->free_by_offset[off] = start - off;
  if (off + size > end) p->free_by_offset[end] = off + size - end;
  p->live[start] = bytes;
  p->used += bytes;
  if (p->used > p->peak) p->peak = p->used;
  p->allocations++;
  return start;
}

// Returns the bytes released, or -1 when `offset` is not a live allocation.
int64_t inv_pool_free(void* h, uint64_t offset) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  std::lock_guard<std::mutex> g(p->m);
  auto it = p->live.find(offset);
  if (it == p->live.end()) return -1;
  uint64_t off = offset, size = it->second;
  const uint64_t released = size;
  p->live.erase(it);
  p->used -= released;
  auto next = p->free_by_offset.lower_bound(off);
  if (next != p->free_by_offset.end() && off + size == next->first) {  // merge with the block after
    size += next->second;
    next = p->free_by_offset.erase(next);
  }
  if (next != p->free_by_offset.begin()) {  // merge with the block before
    auto prev = std::prev(next);
    if (prev->first + prev->second == off) {
      off = prev->first;
      size += prev->second;
      p->free_by_offset.erase(prev);
    }
  }
  p->free_by_offset[off] = size;
  return (int64_t)released;
}

uint64_t inv_pool_used(void* h) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  std::lock_guard<std::mutex> g(p->m);
  return p->used;
}
uint64_t inv_pool_peak(void* h) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  std::lock_guard<std::mutex> g(p->m);
  return p->peak;
}
uint64_t inv_pool_capacity(void* h) { return static_cast<OffsetPool*>(h)->capacity; }
uint64_t inv_pool_largest_free(void* h) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  std::lock_guard<std::mutex> g(p->m);
  uint64_t best = 0;
  for (auto& kv : p->free_by_offset) best = kv.second > best ? kv.second : best;
  return best;
}
uint64_t inv_pool_free_blocks(void* h) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  std::lock_guard<std::mutex> g(p->m);
  return p->free_by_offset.size();
}
uint64_t inv_pool_live_blocks(void* h) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  std::lock_guard<std::mutex> g(p->m);
  return p->live.size();
}
uint64_t inv_pool_failures(void* h) {
  OffsetPool* p = static_cast<OffsetPool*>(h);
  std::lock_guard<std::mutex> g(p->m);
  return p->failures;
}

}  // extern "C"
