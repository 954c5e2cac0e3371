// Hierarchical page tables for long-context KV caches, with a physical-block budget and LRU eviction.
//
// Reference: PagedKVCacheBase / PagedKVCache4M (2-level, 4096 x 4096 entries of 16-token blocks = 268M tokens)
// / PagedKVCache1T (3-level) with a physical memory cap, LRU eviction to per-block disk files and reload on
// touch (include/oil/kv_cache.h:73-238, src/kv_cache.cpp:286-815). This file owns the bookkeeping only: it maps
// (sequence, logical block) -> physical slot, decides which slot to evict, and tells the caller which logical
// block's bytes must be written out / read back; the bytes themselves live in device or host tensors that the
// Python layer (inference/kv_cache_ext.py) moves with ordinary copies.
#include <cstdint>
#include <list>
#include <memory>
#include <unordered_map>
#include <vector>

namespace {

constexpr int kFan = 4096;  // entries per table level

struct Leaf {
  std::vector<int32_t> slot;  // physical slot or -1 (not resident) per logical block
  std::vector<uint8_t> spilled;
  Leaf() : slot(kFan, -1), spilled(kFan, 0) {}
};
struct Mid {
  std::vector<std::unique_ptr<Leaf>> leaf;
  Mid() : leaf(kFan) {}
};

struct Table {
  int levels;           // 2 or 3
  int64_t num_slots;    // physical blocks that fit the memory cap
  std::vector<std::unique_ptr<Mid>> top;            // 3-level: top[kFan] -> Mid -> Leaf
  std::unique_ptr<Mid> root;                        // 2-level: root -> Leaf
  std::vector<int64_t> slot_owner;                  // logical block id held by each slot, -1 free
  std::vector<int32_t> free_slots;
  std::list<int32_t> lru;                           // front = most recent
  std::unordered_map<int32_t, std::list<int32_t>::iterator> lru_pos;
  int64_t evictions = 0, reloads = 0, touches = 0;

  Leaf* leaf_for(int64_t block, bool create) {
    const int64_t li = block / kFan;
    Mid* mid;
    if (levels == 2) {
      if (li >= kFan) return nullptr;
      mid = root.get();
    } else {
      const int64_t ti = li / kFan;
      if (ti >= kFan) return nullptr;
      if (!top[ti]) {
        if (!create) return nullptr;
        top[ti] = std::make_unique<Mid>();
      }
      mid = top[ti].get();
    }
    auto& lf = mid->leaf[li % kFan];
    if (!lf) {
      if (!create) return nullptr;
      lf = std::make_unique<Leaf>();
    }
    return lf.get();
  }
  void touch(int32_t slot) {
    auto it = lru_pos.find(slot);
    if (it != lru_pos.end()) lru.erase(it->second);
    lru.push_front(slot);
    lru_pos[slot] = lru.begin();
  }
};

}  // namespace

extern "C" {

void* pt_create(int levels, int64_t num_slots) {
  if ((levels != 2 && levels != 3) || num_slots < 1) return nullptr;
  auto* t = new Table();
  t->levels = levels;
  t->num_slots = num_slots;
  if (levels == 2) t->root = std::make_unique<Mid>();
  else t->top.resize(kFan);
  t->slot_owner.assign((size_t)num_slots, -1);
  for (int64_t s = num_slots - 1; s >= 0; --s) t->free_slots.push_back((int32_t)s);
  return t;
}
void pt_destroy(void* h) { delete static_cast<Table*>(h); }
int64_t pt_max_blocks(void* h) {
  auto* t = static_cast<Table*>(h);
  return t->levels == 2 ? (int64_t)kFan * kFan : (int64_t)kFan * kFan * kFan;
}

// Makes `block` resident and most-recently used. Returns its slot. *evicted_block receives the logical block that
// had to leave that slot (caller writes its bytes out first) or -1; *needs_reload is 1 when `block` was spilled
// earlier (caller reads its bytes back into the slot).
int32_t pt_acquire(void* h, int64_t block, int64_t* evicted_block, int* needs_reload) {
  auto* t = static_cast<Table*>(h);
  *evicted_block = -1;
  *needs_reload = 0;
  Leaf* lf = t->leaf_for(block, true);
  if (!lf) return -1;
  const int i = (int)(block % kFan);
  ++t->touches;
  if (lf->slot[i] >= 0) {
    t->touch(lf->slot[i]);
    return lf->slot[i];
  }
  int32_t slot;
  if (!t->free_slots.empty()) {
    slot = t->free_slots.back();
    t->free_slots.pop_back();
  } else {
    slot = t->lru.back();  // least recently used
    const int64_t victim = t->slot_owner[(size_t)slot];
    Leaf* vl = t->leaf_for(victim, false);
    if (vl) {
      vl->slot[victim % kFan] = -1;
      vl->spilled[victim % kFan] = 1;
    }
    *evicted_block = victim;
    ++t->evictions;
  }
  if (lf->spilled[i]) {
    *needs_reload = 1;
    ++t->reloads;
  }
  lf->slot[i] = slot;
  t->slot_owner[(size_t)slot] = block;
  t->touch(slot);
  return slot;
}
// Slot of a resident block, -1 otherwise (no LRU update).
int32_t pt_lookup(void* h, int64_t block) {
  auto* t = static_cast<Table*>(h);
  Leaf* lf = t->leaf_for(block, false);
  return lf ? lf->slot[block % kFan] : -1;
}
int pt_is_spilled(void* h, int64_t block) {
  auto* t = static_cast<Table*>(h);
  Leaf* lf = t->leaf_for(block, false);
  return lf ? lf->spilled[block % kFan] : 0;
}
void pt_release(void* h, int64_t block) {
  auto* t = static_cast<Table*>(h);
  Leaf* lf = t->leaf_for(block, false);
  if (!lf) return;
  const int i = (int)(block % kFan);
  const int32_t slot = lf->slot[i];
  lf->spilled[i] = 0;
  if (slot < 0) return;
  lf->slot[i] = -1;
  t->slot_owner[(size_t)slot] = -1;
  auto it = t->lru_pos.find(slot);
  if (it != t->lru_pos.end()) {
    t->lru.erase(it->second);
    t->lru_pos.erase(it);
  }
  t->free_slots.push_back(slot);
}
void pt_stats(void* h, int64_t out[4]) {
  auto* t = static_cast<Table*>(h);
  out[0] = t->touches;
  out[1] = t->evictions;
  out[2] = t->reloads;
  out[3] = t->num_slots - (int64_t)t->free_slots.size();
}

}  // extern "C"
