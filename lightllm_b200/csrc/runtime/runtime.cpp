// Host-side runtime pieces with a C ABI (loaded through ctypes):
//   * atomics on words that live in POSIX shared memory (cross-process locks, counters, the
//     router -> rank mailbox generation counter); replaces the `atomics` cffi package the
//     reference depends on (lightllm/server/core/objs/atomic_lock.py)
//   * KV slot allocator (LIFO stack of free slot ids)   (reference: kv_cache_mem_manager/allocator.py)
//   * radix prefix tree over token ids with slot-index values, reference counts and LRU leaf
//     eviction                                         (reference: router/dynamic_prompt/radix_cache.py)
// No CUDA here; everything is plain C++17.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <queue>
#include <thread>
#include <unordered_map>
#include <vector>

#define LLB_EXPORT extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------------------------------
// atomics on shared-memory words
// ------------------------------------------------------------------------------------------
static inline std::atomic<int32_t>* a32(void* p) { return reinterpret_cast<std::atomic<int32_t>*>(p); }
static inline std::atomic<int64_t>* a64(void* p) { return reinterpret_cast<std::atomic<int64_t>*>(p); }
static_assert(sizeof(std::atomic<int32_t>) == 4 && sizeof(std::atomic<int64_t>) == 8, "lock-free layout expected");

LLB_EXPORT int32_t llb_atomic_load_i32(void* p) { return a32(p)->load(std::memory_order_acquire); }
LLB_EXPORT void llb_atomic_store_i32(void* p, int32_t v) { a32(p)->store(v, std::memory_order_release); }
LLB_EXPORT int32_t llb_atomic_add_i32(void* p, int32_t v) { return a32(p)->fetch_add(v, std::memory_order_acq_rel); }
LLB_EXPORT int32_t llb_atomic_cas_i32(void* p, int32_t expected, int32_t desired) {
  return a32(p)->compare_exchange_strong(expected, desired, std::memory_order_acq_rel) ? 1 : 0;
}
LLB_EXPORT int64_t llb_atomic_load_i64(void* p) { return a64(p)->load(std::memory_order_acquire); }
LLB_EXPORT void llb_atomic_store_i64(void* p, int64_t v) { a64(p)->store(v, std::memory_order_release); }
LLB_EXPORT int64_t llb_atomic_add_i64(void* p, int64_t v) { return a64(p)->fetch_add(v, std::memory_order_acq_rel); }

// Spin lock on a shm word (0 = free, 1 = held).  Bounded: returns 0 if `timeout_ns` elapsed.
LLB_EXPORT int32_t llb_spin_lock(void* p, int64_t timeout_ns) {
  auto t0 = std::chrono::steady_clock::now();
  int spins = 0;
  for (;;) {
    int32_t exp = 0;
    if (a32(p)->compare_exchange_weak(exp, 1, std::memory_order_acquire)) return 1;
    if (++spins > 64) {
      std::this_thread::yield();
      if ((spins & 1023) == 0 && timeout_ns >= 0) {
        auto dt = std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
        if (dt > timeout_ns) return 0;
      }
    }
  }
}
LLB_EXPORT void llb_spin_unlock(void* p) { a32(p)->store(0, std::memory_order_release); }

// ------------------------------------------------------------------------------------------
// slot allocator
// ------------------------------------------------------------------------------------------
struct SlotAlloc {
  std::vector<int32_t> stack;
  int64_t top = 0;  // stack[top..) are free
};

LLB_EXPORT void* llb_slots_create(int64_t size) {
  auto* s = new SlotAlloc();
  s->stack.resize(size);
  for (int64_t i = 0; i < size; ++i) s->stack[i] = (int32_t)i;
  return s;
}
LLB_EXPORT void llb_slots_destroy(void* h) { delete reinterpret_cast<SlotAlloc*>(h); }
LLB_EXPORT int64_t llb_slots_free_count(void* h) {
  auto* s = reinterpret_cast<SlotAlloc*>(h);
  return (int64_t)s->stack.size() - s->top;
}
LLB_EXPORT int32_t llb_slots_alloc(void* h, int64_t n, int32_t* out) {
  auto* s = reinterpret_cast<SlotAlloc*>(h);
  if (n > (int64_t)s->stack.size() - s->top) return -1;
  std::memcpy(out, s->stack.data() + s->top, n * sizeof(int32_t));
  s->top += n;
  return 0;
}
LLB_EXPORT int32_t llb_slots_free(void* h, const int32_t* idx, int64_t n) {
  auto* s = reinterpret_cast<SlotAlloc*>(h);
  if (n > s->top) return -1;  // more frees than allocations
  s->top -= n;
  std::memcpy(s->stack.data() + s->top, idx, n * sizeof(int32_t));
  return 0;
}
LLB_EXPORT void llb_slots_reset(void* h) {
  auto* s = reinterpret_cast<SlotAlloc*>(h);
  for (size_t i = 0; i < s->stack.size(); ++i) s->stack[i] = (int32_t)i;
  s->top = 0;
}

// ------------------------------------------------------------------------------------------
// radix tree
// ------------------------------------------------------------------------------------------
struct RNode {
  std::unordered_map<int64_t, RNode*> children;
  RNode* parent = nullptr;
  std::vector<int64_t> key;
  std::vector<int32_t> value;
  int64_t ref = 0;
  int64_t time_id = 0;
  bool alive = true;
  bool leaf() const { return children.empty(); }
};

struct HeapItem {
  int64_t time_id;
  RNode* node;
  bool operator>(const HeapItem& o) const { return time_id > o.time_id; }
};

struct RTree {
  RNode* root;
  int64_t tick = 0;
  int64_t total_tokens = 0;
  int64_t refed_tokens = 0;
  std::priority_queue<HeapItem, std::vector<HeapItem>, std::greater<HeapItem>> heap;
  std::vector<RNode*> graveyard;  // dead nodes stay allocated while heap entries may point at them

  RTree() {
    root = new RNode();
    root->ref = 1;
  }
  ~RTree() {
    std::vector<RNode*> st{root};
    while (!st.empty()) {
      RNode* n = st.back();
      st.pop_back();
      for (auto& kv : n->children) st.push_back(kv.second);
      delete n;
    }
    for (RNode* n : graveyard) delete n;
  }
  void touch(RNode* n) { n->time_id = ++tick; }
  void maybe_evictable(RNode* n) {
    if (n != root && n->ref == 0 && n->leaf() && n->alive) heap.push({n->time_id, n});
  }
  static int64_t match_len(const std::vector<int64_t>& a, const int64_t* b, int64_t nb) {
    int64_t n = std::min<int64_t>((int64_t)a.size(), nb), i = 0;
    while (i < n && a[i] == b[i]) ++i;
    return i;
  }
  RNode* split(RNode* node, int64_t at) {
    RNode* head = new RNode();
    head->key.assign(node->key.begin(), node->key.begin() + at);
    head->value.assign(node->value.begin(), node->value.begin() + at);
    head->parent = node->parent;
    head->ref = node->ref;
    head->time_id = node->time_id;
    node->parent->children[head->key[0]] = head;
    node->key.erase(node->key.begin(), node->key.begin() + at);
    node->value.erase(node->value.begin(), node->value.begin() + at);
    node->parent = head;
    head->children[node->key[0]] = node;
    return head;
  }
};

LLB_EXPORT void* llb_radix_create() { return new RTree(); }
LLB_EXPORT void llb_radix_destroy(void* h) { delete reinterpret_cast<RTree*>(h); }
LLB_EXPORT int64_t llb_radix_total_tokens(void* h) { return reinterpret_cast<RTree*>(h)->total_tokens; }
LLB_EXPORT int64_t llb_radix_refed_tokens(void* h) { return reinterpret_cast<RTree*>(h)->refed_tokens; }

// returns the number of leading tokens that were already present
LLB_EXPORT int64_t llb_radix_insert(void* h, const int64_t* key, const int32_t* value, int64_t n) {
  auto* t = reinterpret_cast<RTree*>(h);
  RNode* node = t->root;
  int64_t pos = 0;
  t->touch(node);
  while (pos < n) {
    auto it = node->children.find(key[pos]);
    if (it == node->children.end()) {
      RNode* nn = new RNode();
      nn->key.assign(key + pos, key + n);
      nn->value.assign(value + pos, value + n);
      nn->parent = node;
      node->children[key[pos]] = nn;
      t->touch(nn);
      t->total_tokens += n - pos;
      t->maybe_evictable(nn);
      return pos;
    }
    RNode* child = it->second;
    int64_t m = RTree::match_len(child->key, key + pos, n - pos);
    if (m < (int64_t)child->key.size()) child = t->split(child, m);
    t->touch(child);
    pos += m;
    node = child;
  }
  return pos;
}

// Longest cached prefix. Writes slot ids to out_values (capacity >= n); *out_node gets the last node.
LLB_EXPORT int64_t llb_radix_match(void* h, const int64_t* key, int64_t n, int32_t update_refs, int32_t* out_values,
                                   void** out_node) {
  auto* t = reinterpret_cast<RTree*>(h);
  RNode* node = t->root;
  int64_t pos = 0;
  while (pos < n) {
    auto it = node->children.find(key[pos]);
    if (it == node->children.end()) break;
    RNode* child = it->second;
    int64_t m = RTree::match_len(child->key, key + pos, n - pos);
    if (m == 0) break;
    if (m < (int64_t)child->key.size()) child = t->split(child, m);
    std::memcpy(out_values + pos, child->value.data(), m * sizeof(int32_t));
    t->touch(child);
    pos += m;
    node = child;
  }
  *out_node = pos > 0 ? node : nullptr;
  if (pos > 0 && update_refs) {
    for (RNode* p = node; p && p != t->root; p = p->parent) {
      if (p->ref == 0) t->refed_tokens += (int64_t)p->key.size();
      p->ref += 1;
    }
  }
  return pos;
}

LLB_EXPORT void llb_radix_add_ref(void* h, void* node) {
  auto* t = reinterpret_cast<RTree*>(h);
  for (RNode* p = reinterpret_cast<RNode*>(node); p && p != t->root; p = p->parent) {
    if (p->ref == 0) t->refed_tokens += (int64_t)p->key.size();
    p->ref += 1;
  }
}
LLB_EXPORT int32_t llb_radix_dec_ref(void* h, void* node) {
  auto* t = reinterpret_cast<RTree*>(h);
  for (RNode* p = reinterpret_cast<RNode*>(node); p && p != t->root; p = p->parent) {
    if (p->ref <= 0) return -1;
    p->ref -= 1;
    if (p->ref == 0) {
      t->refed_tokens -= (int64_t)p->key.size();
      t->maybe_evictable(p);
    }
  }
  return 0;
}

// Evicts unreferenced leaves, least recently used first, until `need` tokens were released or
// `cap` output slots are used up. Returns the number of slot ids written to `out`.
LLB_EXPORT int64_t llb_radix_evict(void* h, int64_t need, int32_t* out, int64_t cap) {
  auto* t = reinterpret_cast<RTree*>(h);
  int64_t released = 0;
  while (released < need && !t->heap.empty()) {
    HeapItem it = t->heap.top();
    RNode* n = it.node;
    if (!n->alive || n->ref != 0 || !n->leaf()) {
      t->heap.pop();
      continue;
    }
    if (it.time_id != n->time_id) {  // stale timestamp: requeue with the current one
      t->heap.pop();
      t->heap.push({n->time_id, n});
      continue;
    }
    int64_t len = (int64_t)n->key.size();
    if (released + len > cap) break;
    t->heap.pop();
    std::memcpy(out + released, n->value.data(), len * sizeof(int32_t));
    released += len;
    t->total_tokens -= len;
    RNode* parent = n->parent;
    parent->children.erase(n->key[0]);
    n->alive = false;
    t->graveyard.push_back(n);
    t->maybe_evictable(parent);
  }
  if (t->heap.empty() && !t->graveyard.empty()) {
    for (RNode* n : t->graveyard) delete n;
    t->graveyard.clear();
  }
  return released;
}

// Compaction: a node that nobody references and that has exactly one child, also unreferenced, absorbs that
// child (keys and slots appended, grandchildren adopted).  Chains like that are left behind when a sibling
// branch is evicted or when a sequence was inserted piece by piece.  Node handles held by callers always have a
// reference count above zero, so no handle is invalidated.  Returns the number of nodes merged away.
LLB_EXPORT int64_t llb_radix_merge(void* h) {
  auto* t = reinterpret_cast<RTree*>(h);
  int64_t merged = 0;
  std::vector<RNode*> st;
  for (auto& kv : t->root->children) st.push_back(kv.second);
  while (!st.empty()) {
    RNode* n = st.back();
    st.pop_back();
    bool changed = false;
    while (n->ref == 0 && n->children.size() == 1) {
      RNode* c = n->children.begin()->second;
      if (c->ref != 0) break;
      n->key.insert(n->key.end(), c->key.begin(), c->key.end());
      n->value.insert(n->value.end(), c->value.begin(), c->value.end());
      n->time_id = std::max(n->time_id, c->time_id);
      std::unordered_map<int64_t, RNode*> kids = std::move(c->children);
      c->children.clear();
      n->children = std::move(kids);
      for (auto& kv : n->children) kv.second->parent = n;
      c->parent = nullptr;
      c->alive = false;
      t->graveyard.push_back(c);
      ++merged;
      changed = true;
    }
    if (changed) t->maybe_evictable(n);
    for (auto& kv : n->children) st.push_back(kv.second);
  }
  return merged;
}

LLB_EXPORT int64_t llb_radix_node_count(void* h) {
  auto* t = reinterpret_cast<RTree*>(h);
  int64_t c = 0;
  std::vector<RNode*> st{t->root};
  while (!st.empty()) {
    RNode* n = st.back();
    st.pop_back();
    ++c;
    for (auto& kv : n->children) st.push_back(kv.second);
  }
  return c;
}
