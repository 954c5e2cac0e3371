// Address-space arenas for device and pinned-host memory (the reference's Buffer / MemoryPool / StackAllocator,
// include/oil/memory.h:17-291, restated for one large range that lives in HBM or pinned memory).
//
// An arena never touches the memory it manages: it hands out offsets inside [0, capacity) of a range the caller
// allocated once (a 180 GB device lets a training job take its activations, staging buffers and KV pages from one
// reservation instead of going through the driver's allocator at every step). Two disciplines:
//   * bump:  lock-free fetch-add allocation, freed all at once by reset() (per-step scratch);
//   * stack: push a marker, allocate, pop back to the marker (nested scopes such as one transformer block).
// Offsets are aligned to at least 256 bytes (TMA descriptors want 16, coalesced access 128, 256 keeps tiles whole).
#include <atomic>
#include <cstdint>
#include <mutex>
#include <vector>

namespace {
struct Arena {
  uint64_t capacity;
  std::atomic<uint64_t> offset{0};
  std::atomic<uint64_t> peak{0};
  std::atomic<uint64_t> allocations{0};
  std::atomic<uint64_t> failures{0};
  std::mutex marker_mutex;
  std::vector<uint64_t> markers;
};
inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }
}  // namespace

extern "C" {

void* inv_arena_create(uint64_t capacity) {
  Arena* a = new Arena();
  a->capacity = capacity;
  return a;
}

void inv_arena_destroy(void* h) { delete static_cast<Arena*>(h); }

// Returns the offset of the new block, or UINT64_MAX when the arena is full (nothing is reserved then).
uint64_t inv_arena_alloc(void* h, uint64_t bytes, uint64_t alignment) {
  Arena* a = static_cast<Arena*>(h);
  if (alignment < 256) alignment = 256;
  uint64_t old = a->offset.load(std::memory_order_relaxed);
  for (;;) {
    const uint64_t start = align_up(old, alignment);
    const uint64_t end = start + bytes;
    if (end > a->capacity || end < start) {
      a->failures.fetch_add(1, std::memory_order_relaxed);
      return UINT64_MAX;
    }
    if (a->offset.compare_exchange_weak(old, end, std::memory_order_acq_rel, std::memory_order_relaxed)) {
      uint64_t p = a->peak.load(std::memory_order_relaxed);
      while (end > p && !a->peak.compare_exchange_weak(p, end, std::memory_order_relaxed)) {
      }
      a->allocations.fetch_add(1, std::memory_order_relaxed);
      return start;
    }
  }
}

void inv_arena_reset(void* h) {
  Arena* a = static_cast<Arena*>(h);
  std::lock_guard<std::mutex> g(a->marker_mutex);
  a->markers.clear();
  a->offset.store(0, std::memory_order_release);
}

// Stack discipline: returns the depth after the push.
int64_t inv_arena_push(void* h) {
  Arena* a = static_cast<Arena*>(h);
  std::lock_guard<std::mutex> g(a->marker_mutex);
  a->markers.push_back(a->offset.load(std::memory_order_acquire));
  return (int64_t)a->markers.size();
}

// Rewinds to the last marker; returns the bytes released, or -1 without a marker.
int64_t inv_arena_pop(void* h) {
  Arena* a = static_cast<Arena*>(h);
  std::lock_guard<std::mutex> g(a->marker_mutex);
  if (a->markers.empty()) return -1;
  const uint64_t m = a->markers.back();
  a->markers.pop_back();
  const uint64_t cur = a->offset.exchange(m, std::memory_order_acq_rel);
  return (int64_t)(cur - m);
}

uint64_t inv_arena_used(void* h) { return static_cast<Arena*>(h)->offset.load(std::memory_order_acquire); }
uint64_t inv_arena_peak(void* h) { return static_cast<Arena*>(h)->peak.load(std::memory_order_acquire); }
uint64_t inv_arena_capacity(void* h) { return static_cast<Arena*>(h)->capacity; }
uint64_t inv_arena_allocations(void* h) { return static_cast<Arena*>(h)->allocations.load(std::memory_order_acquire); }
uint64_t inv_arena_failures(void* h) { return static_cast<Arena*>(h)->failures.load(std::memory_order_acquire); }

}  // extern "C"
