// Logical VRAM tier: which experts are admitted to the GPU, in which region, under which generation.
// Host-only bookkeeping (no CUDA call in this file); the physical slots live in mer_abi.cu and follow
// the decisions made here through mer_expert_demand_admit / mer_expert_hot_promote.
//
// Semantics follow the reference's GpuExpertCache (expert_cache.rs:734-1350):
//   * two byte budgets cut from one capacity by anchor_ratio: the Anchor Core (never evicted) and the
//     LRU Edge (foreground demand, evicts least recently used);
//   * generations start at 1, grow monotonically, are allocated BEFORE any eviction, never reused;
//   * get() is the only call that counts hits / misses and refreshes LRU recency;
//   * a threshold-driven promotion can be claimed once per edge (ram_hits == promote_after_hits) and once
//     more after every logical eviction of the id (re-arm), never twice while one is pending;
//   * speculative admission (try_promote_lru_no_evict) never evicts and never uses the Anchor Core.
// One mutex guards all state; the critical sections are map / list manipulation only.
#include <cstdint>
#include <cstring>
#include <list>
#include <mutex>
#include <new>
#include <unordered_map>
#include <unordered_set>

#include "../../include/mer_b200.h"

#define MER_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct Admission {
  uint64_t generation = 0, bytes = 0, tag = 0;
};

struct LruEdge {
  // most recently used at the front
  std::list<uint32_t> order;
  struct Node {
    Admission adm;
    std::list<uint32_t>::iterator pos;
  };
  std::unordered_map<uint32_t, Node> map;

  const Admission *peek(uint32_t id) const {
    auto it = map.find(id);
    return it == map.end() ? nullptr : &it->second.adm;
  }
  const Admission *touch(uint32_t id) {
    auto it = map.find(id);
    if (it == map.end()) return nullptr;
    order.splice(order.begin(), order, it->second.pos);
    return &it->second.adm;
  }
  void put_new(uint32_t id, const Admission &a) {
    order.push_front(id);
    map[id] = Node{a, order.begin()};
  }
  bool pop(uint32_t id, Admission *out) {
    auto it = map.find(id);
    if (it == map.end()) return false;
    if (out) *out = it->second.adm;
    order.erase(it->second.pos);
    map.erase(it);
    return true;
  }
  bool pop_lru(uint32_t *id, Admission *out) {
    if (order.empty()) return false;
    *id = order.back();
    return pop(*id, out);
  }
};

bool fits(uint64_t used, uint64_t bytes, uint64_t cap) { return bytes <= cap && used <= cap - bytes; }

}  // namespace

struct mer_gpu_cache {
  std::mutex mu;
  uint64_t anchor_cap = 0, lru_cap = 0, promote_after_hits = 0;
  std::unordered_map<uint32_t, Admission> anchor;
  uint64_t anchor_used = 0;
  LruEdge lru;
  uint64_t lru_used = 0;
  uint64_t next_generation = 1;
  std::unordered_set<uint32_t> pending, rearm;
  uint64_t promotions = 0, hits = 0, misses = 0;

  bool alloc_generation(uint64_t *g) {
    if (next_generation == UINT64_MAX) return false;  // the last value is never handed out: exhaustion refuses cleanly
    *g = next_generation++;
    return true;
  }
  void clear_markers(uint32_t id) {
    pending.erase(id);
    rearm.erase(id);
  }
  // Evicts least-recently-used dynamic entries until `bytes` more fit; every victim may claim one new promotion.
  void make_room(uint64_t bytes, uint32_t *evicted, size_t max_evicted, size_t *n_evicted) {
    while (!fits(lru_used, bytes, lru_cap)) {
      uint32_t vid;
      Admission v;
      if (!lru.pop_lru(&vid, &v)) break;
      lru_used = lru_used >= v.bytes ? lru_used - v.bytes : 0;
      rearm.insert(vid);
      if (evicted && n_evicted && *n_evicted < max_evicted) evicted[*n_evicted] = vid;
      if (n_evicted) (*n_evicted)++;
    }
  }
  // An id that is already admitted and threshold-hot: Anchor stays, LRU graduates when the Anchor Core has room.
  // Returns -1 when the id is absent (a payload is required).
  int resolve_existing_hot(uint32_t id) {
    if (anchor.count(id)) {
      clear_markers(id);
      return MER_HOT_ALREADY_ANCHOR;
    }
    const Admission *p = lru.peek(id);
    if (!p) return -1;
    const uint64_t bytes = p->bytes;
    if (!fits(anchor_used, bytes, anchor_cap)) {
      clear_markers(id);
      return MER_HOT_ALREADY_LRU_ANCHOR_FULL;
    }
    Admission a;
    lru.pop(id, &a);  // only this id leaves the list: no other entry's recency moves
    lru_used -= bytes;
    anchor[id] = a;
    anchor_used += bytes;
    clear_markers(id);
    return MER_HOT_MOVED_LRU_TO_ANCHOR;
  }
  static bool is_transition(int outcome) {
    return outcome == MER_HOT_MOVED_LRU_TO_ANCHOR || outcome == MER_HOT_INSTALLED_ANCHOR || outcome == MER_HOT_INSTALLED_LRU;
  }
};

namespace {
void fill(mer_gpu_admission *out, uint32_t id, int region, const Admission *a) {
  if (!out) return;
  out->expert_id = id;
  out->region = (uint32_t)region;
  out->generation = a ? a->generation : 0;
  out->bytes = a ? a->bytes : 0;
  out->payload_tag = a ? a->tag : 0;
}
}  // namespace

MER_EXPORT int mer_gpu_cache_create(uint64_t capacity_bytes, float anchor_ratio, uint64_t promote_after_hits, mer_gpu_cache **out) {
  if (!out) return MER_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  mer_gpu_cache *c = new (std::nothrow) mer_gpu_cache();
  if (!c) return MER_ERR_PHYSICAL_CAPACITY;
  float ratio = anchor_ratio;
  if (!(ratio >= 0.0f)) ratio = 0.0f;  // NaN clamps to 0 as well
  if (ratio > 1.0f) ratio = 1.0f;
  // the anchor share is computed in single precision and truncated, like the reference's `(capacity as f32 * ratio) as usize`
  uint64_t a = (uint64_t)((float)capacity_bytes * ratio);
  if (a > capacity_bytes) a = capacity_bytes;
  c->anchor_cap = a;
  c->lru_cap = capacity_bytes - a;
  c->promote_after_hits = promote_after_hits;
  *out = c;
  return MER_OK;
}

MER_EXPORT void mer_gpu_cache_destroy(mer_gpu_cache *c) { delete c; }

MER_EXPORT int mer_gpu_cache_get(mer_gpu_cache *c, uint32_t id, mer_gpu_admission *out) {
  if (!c) return MER_LOOKUP_MISS;
  std::lock_guard<std::mutex> lock(c->mu);
  auto it = c->anchor.find(id);
  if (it != c->anchor.end()) {
    c->hits++;
    fill(out, id, MER_REGION_ANCHOR, &it->second);
    return MER_LOOKUP_ANCHOR_HIT;
  }
  if (const Admission *a = c->lru.touch(id)) {
    c->hits++;
    fill(out, id, MER_REGION_LRU, a);
    return MER_LOOKUP_LRU_HIT;
  }
  c->misses++;
  fill(out, id, MER_REGION_NONE, nullptr);
  return MER_LOOKUP_MISS;
}

MER_EXPORT int mer_gpu_cache_current_admission(mer_gpu_cache *c, uint32_t id, mer_gpu_admission *out) {
  if (!c) return 0;
  std::lock_guard<std::mutex> lock(c->mu);
  auto it = c->anchor.find(id);
  if (it != c->anchor.end()) {
    fill(out, id, MER_REGION_ANCHOR, &it->second);
    return 1;
  }
  if (const Admission *a = c->lru.peek(id)) {
    fill(out, id, MER_REGION_LRU, a);
    return 1;
  }
  fill(out, id, MER_REGION_NONE, nullptr);
  return 0;
}

MER_EXPORT int mer_gpu_cache_contains(mer_gpu_cache *c, uint32_t id) { return mer_gpu_cache_current_admission(c, id, nullptr); }

MER_EXPORT int mer_gpu_cache_contains_generation(mer_gpu_cache *c, uint32_t id, uint64_t generation) {
  mer_gpu_admission a;
  return mer_gpu_cache_current_admission(c, id, &a) && a.generation == generation;
}

MER_EXPORT int mer_gpu_cache_should_promote(mer_gpu_cache *c, uint64_t ram_hits) {
  return c && c->promote_after_hits > 0 && ram_hits >= c->promote_after_hits;
}

MER_EXPORT int mer_gpu_cache_claim_promotion(mer_gpu_cache *c, uint32_t id, uint64_t ram_hits) {
  if (!mer_gpu_cache_should_promote(c, ram_hits)) return 0;
  std::lock_guard<std::mutex> lock(c->mu);
  // LRU residency does not refuse a claim: the entry may still graduate into the Anchor Core
  if (c->anchor.count(id) || c->pending.count(id)) return 0;
  const bool edge = ram_hits == c->promote_after_hits;
  const bool rearmed = c->rearm.erase(id) > 0;
  if (!edge && !rearmed) return 0;
  return c->pending.insert(id).second ? 1 : 0;
}

MER_EXPORT void mer_gpu_cache_cancel_promotion(mer_gpu_cache *c, uint32_t id) {
  if (!c) return;
  std::lock_guard<std::mutex> lock(c->mu);
  if (c->pending.erase(id)) c->rearm.insert(id);
}

MER_EXPORT int mer_gpu_cache_promote_hot_existing(mer_gpu_cache *c, uint32_t id) {
  if (!c) return MER_HOT_NO_CAPACITY;
  std::lock_guard<std::mutex> lock(c->mu);
  const int o = c->resolve_existing_hot(id);
  if (o < 0) return MER_HOT_PAYLOAD_REQUIRED;
  if (mer_gpu_cache::is_transition(o)) c->promotions++;
  return o;
}

MER_EXPORT int mer_gpu_cache_promote_hot_sync(mer_gpu_cache *c, uint32_t id, uint64_t bytes, uint64_t payload_tag, uint32_t *evicted,
                                              size_t max_evicted, size_t *n_evicted, uint64_t *generation) {
  if (n_evicted) *n_evicted = 0;
  if (!c) return MER_HOT_NO_CAPACITY;
  std::lock_guard<std::mutex> lock(c->mu);
  int o = c->resolve_existing_hot(id);
  if (o >= 0) {
    if (mer_gpu_cache::is_transition(o)) c->promotions++;
    if (generation) {
      auto it = c->anchor.find(id);
      const Admission *a = it != c->anchor.end() ? &it->second : c->lru.peek(id);
      *generation = a ? a->generation : 0;
    }
    return o;
  }
  if (bytes == 0) {
    c->clear_markers(id);
    return MER_HOT_NO_CAPACITY;
  }
  const bool use_anchor = fits(c->anchor_used, bytes, c->anchor_cap);
  if (!use_anchor && bytes > c->lru_cap) {
    c->clear_markers(id);
    return MER_HOT_NO_CAPACITY;
  }
  uint64_t g;
  if (!c->alloc_generation(&g)) {
    c->clear_markers(id);
    return MER_HOT_GENERATION_EXHAUSTED;
  }
  c->clear_markers(id);
  const Admission a{g, bytes, payload_tag};
  if (use_anchor) {
    c->anchor[id] = a;
    c->anchor_used += bytes;
    o = MER_HOT_INSTALLED_ANCHOR;
  } else {
    c->make_room(bytes, evicted, max_evicted, n_evicted);
    c->lru.put_new(id, a);
    c->lru_used += bytes;
    o = MER_HOT_INSTALLED_LRU;
  }
  c->promotions++;
  if (generation) *generation = g;
  return o;
}

MER_EXPORT int mer_gpu_cache_promote_sync(mer_gpu_cache *c, uint32_t id, uint64_t bytes, uint64_t payload_tag, uint32_t *evicted,
                                          size_t max_evicted, size_t *n_evicted, uint64_t *generation) {
  if (n_evicted) *n_evicted = 0;
  if (!c) return 0;
  std::lock_guard<std::mutex> lock(c->mu);
  c->clear_markers(id);
  if (bytes == 0) return 0;
  auto it = c->anchor.find(id);
  if (it != c->anchor.end()) {
    if (generation) *generation = it->second.generation;
    return 1;
  }
  if (const Admission *a = c->lru.touch(id)) {  // already resident: becomes most recently used, nothing is re-counted
    if (generation) *generation = a->generation;
    return 1;
  }
  const bool use_anchor = fits(c->anchor_used, bytes, c->anchor_cap);
  if (!use_anchor && bytes > c->lru_cap) return 0;
  uint64_t g;
  if (!c->alloc_generation(&g)) return 0;
  const Admission a{g, bytes, payload_tag};
  if (use_anchor) {
    c->anchor[id] = a;
    c->anchor_used += bytes;
  } else {
    c->make_room(bytes, evicted, max_evicted, n_evicted);
    c->lru.put_new(id, a);
    c->lru_used += bytes;
  }
  c->promotions++;
  if (generation) *generation = g;
  return 1;
}

MER_EXPORT int mer_gpu_cache_try_promote_lru_no_evict(mer_gpu_cache *c, uint32_t id, uint64_t bytes, uint64_t payload_tag,
                                                      uint64_t *generation) {
  if (!c) return 0;
  std::lock_guard<std::mutex> lock(c->mu);
  if (bytes == 0) return 0;
  if (c->anchor.count(id) || c->lru.peek(id)) {
    c->clear_markers(id);  // already satisfied: stale markers go, recency stays (a warm-up path is not an access)
    return 0;
  }
  if (!fits(c->lru_used, bytes, c->lru_cap)) return 0;  // strictly non-evicting; markers are left as they are
  uint64_t g;
  if (!c->alloc_generation(&g)) return 0;
  c->clear_markers(id);
  c->lru.put_new(id, Admission{g, bytes, payload_tag});
  c->lru_used += bytes;
  c->promotions++;
  if (generation) *generation = g;
  return 1;
}

MER_EXPORT int mer_gpu_cache_demand_admission_preflight(mer_gpu_cache *c, uint32_t id, uint64_t payload_bytes) {
  if (!c) return MER_DEMAND_ERR_EMPTY_PAYLOAD;
  std::lock_guard<std::mutex> lock(c->mu);
  if (c->anchor.count(id) || c->lru.peek(id)) return MER_DEMAND_ALREADY_ADMITTED;
  if (payload_bytes == 0) return MER_DEMAND_ERR_EMPTY_PAYLOAD;
  if (payload_bytes > c->lru_cap) return MER_DEMAND_ERR_EXCEEDS_LRU_CAPACITY;
  return MER_DEMAND_NEEDS_PAYLOAD;
}

MER_EXPORT int mer_gpu_cache_demand_admit_lru(mer_gpu_cache *c, uint32_t id, uint64_t bytes, uint64_t payload_tag, uint32_t *evicted,
                                              size_t max_evicted, size_t *n_evicted, uint64_t *generation) {
  if (n_evicted) *n_evicted = 0;
  if (!c || bytes == 0) return MER_DEMAND_ERR_EMPTY_PAYLOAD;
  std::lock_guard<std::mutex> lock(c->mu);
  if (c->anchor.count(id) || c->lru.peek(id)) return MER_DEMAND_ALREADY_ADMITTED;  // nothing changes, not even recency
  if (bytes > c->lru_cap) return MER_DEMAND_ERR_EXCEEDS_LRU_CAPACITY;
  uint64_t g;
  if (!c->alloc_generation(&g)) return MER_DEMAND_ERR_GENERATION_EXHAUSTED;  // before any eviction
  c->make_room(bytes, evicted, max_evicted, n_evicted);
  c->clear_markers(id);
  c->lru.put_new(id, Admission{g, bytes, payload_tag});
  c->lru_used += bytes;
  c->promotions++;
  if (generation) *generation = g;
  return MER_DEMAND_ADMITTED;
}

MER_EXPORT int mer_gpu_cache_remove(mer_gpu_cache *c, uint32_t id, uint64_t generation) {
  if (!c) return 0;
  std::lock_guard<std::mutex> lock(c->mu);
  auto it = c->anchor.find(id);
  if (it != c->anchor.end()) {
    if (it->second.generation != generation) return 0;
    c->anchor_used -= it->second.bytes;
    c->anchor.erase(it);
    return 1;
  }
  const Admission *a = c->lru.peek(id);
  if (!a || a->generation != generation) return 0;
  c->lru_used -= a->bytes;
  c->lru.pop(id, nullptr);
  return 1;
}

MER_EXPORT int mer_gpu_cache_stats_read(mer_gpu_cache *c, mer_gpu_cache_stats *out) {
  if (!c || !out) return MER_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(c->mu);
  out->anchor_capacity_bytes = c->anchor_cap;
  out->lru_capacity_bytes = c->lru_cap;
  out->anchor_used_bytes = c->anchor_used;
  out->lru_used_bytes = c->lru_used;
  out->used_bytes = c->anchor_used + c->lru_used;
  out->anchor_len = c->anchor.size();
  out->lru_len = c->lru.map.size();
  out->promotions = c->promotions;
  out->hits = c->hits;
  out->misses = c->misses;
  out->next_generation = c->next_generation;
  out->promote_after_hits = c->promote_after_hits;
  out->pending_promotions = c->pending.size();
  out->rearmed_promotions = c->rearm.size();
  return MER_OK;
}

MER_EXPORT int mer_gpu_cache_set_next_generation(mer_gpu_cache *c, uint64_t next_generation) {
  if (!c || next_generation == 0) return MER_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(c->mu);
  if (next_generation < c->next_generation) return MER_ERR_INVALID_ARGUMENT;  // generations never go back
  c->next_generation = next_generation;
  return MER_OK;
}

MER_EXPORT int mer_gpu_cache_marker_state(mer_gpu_cache *c, uint32_t id) {
  if (!c) return 0;
  std::lock_guard<std::mutex> lock(c->mu);
  return (c->pending.count(id) ? 1 : 0) | (c->rearm.count(id) ? 2 : 0);
}
