// H1: host-side core of the hybrid KV cache -- a reference-counted block pool (PagedAttention
// level) and a path-compressed radix tree over token blocks (RadixAttention level), behind a
// plain C ABI that the Python package binds with ctypes.
//
// Differences from the reference's design, on purpose:
//  * crates/kv/src/lib.rs:207-403 (PagedKvAllocator) reserves ceil(max_len / page) pages up
//    front and has no sharing; here blocks are allocated as a sequence grows and carry reference
//    counts, so a prefix block can be shared by many sequences and by the radix tree.
//  * crates/kv/src/hybrid_cache.rs:137-338 (RadixCache) is a one-node-per-token trie whose
//    eviction loop does not terminate once over capacity (leaves keep ref 1 forever); here an edge
//    holds a run of whole blocks, nodes are split on partial matches, sequences lock the path they
//    use, and eviction pops unlocked leaves in LRU order from a heap.
// Thread safety: each object has its own mutex; calls on one object serialise.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct BlockPool {
  int num_blocks;
  std::vector<int> ref;
  std::deque<int> free_list;
  std::mutex mu;
  uint64_t allocs = 0, frees = 0, failed = 0;
  explicit BlockPool(int n) : num_blocks(n), ref(n, 0) {
    for (int i = 0; i < n; ++i) free_list.push_back(i);
  }
  int alloc(int n, int* out) {
    std::lock_guard<std::mutex> g(mu);
    if ((int)free_list.size() < n) {
      ++failed;
      return -1;
    }
    for (int i = 0; i < n; ++i) {
      int b = free_list.front();
      free_list.pop_front();
      ref[b] = 1;
      out[i] = b;
    }
    allocs += n;
    return 0;
  }
  int incref(int b) {
    std::lock_guard<std::mutex> g(mu);
    if (b < 0 || b >= num_blocks || ref[b] <= 0) return -1;
    return ++ref[b];
  }
  int decref(int b) {
    std::lock_guard<std::mutex> g(mu);
    if (b < 0 || b >= num_blocks || ref[b] <= 0) return -1;
    if (--ref[b] == 0) {
      free_list.push_back(b);
      ++frees;
    }
    return ref[b];
  }
  int refcount(int b) {
    std::lock_guard<std::mutex> g(mu);
    return (b < 0 || b >= num_blocks) ? -1 : ref[b];
  }
};

struct Node {
  int id;
  int parent;
  std::vector<int32_t> tokens;  // length = blocks.size() * block_size
  std::vector<int> blocks;
  std::unordered_map<std::string, int> children;  // key = bytes of the child's first block of tokens
  int lock = 0;                                   // number of live sequences using this node or a descendant
  uint64_t last_access = 0;
  bool alive = true;
};

struct RadixTree {
  int block_size;
  BlockPool* pool;
  std::vector<Node> nodes;
  std::vector<int> free_nodes;
  uint64_t clock = 0;
  uint64_t hits = 0, misses = 0, hit_tokens = 0, query_tokens = 0, evicted_blocks = 0, inserted_blocks = 0;
  int cached_blocks = 0;
  std::mutex mu;

  RadixTree(int bs, BlockPool* p) : block_size(bs), pool(p) {
    nodes.emplace_back();
    nodes[0].id = 0;
    nodes[0].parent = -1;
  }
  std::string key_of(const int32_t* t) const {
    return std::string(reinterpret_cast<const char*>(t), sizeof(int32_t) * block_size);
  }
  int new_node() {
    if (!free_nodes.empty()) {
      int id = free_nodes.back();
      free_nodes.pop_back();
      nodes[id] = Node();
      nodes[id].id = id;
      return id;
    }
    nodes.emplace_back();
    nodes.back().id = (int)nodes.size() - 1;
    return nodes.back().id;
  }
  // Split `child` so that its first `keep` blocks stay in a new intermediate node; returns that node.
  int split(int child, int keep) {
    const int mid = new_node();
    Node& c = nodes[child];
    Node& m = nodes[mid];
    m.parent = c.parent;
    m.tokens.assign(c.tokens.begin(), c.tokens.begin() + (size_t)keep * block_size);
    m.blocks.assign(c.blocks.begin(), c.blocks.begin() + keep);
    m.lock = c.lock;
    m.last_access = c.last_access;
    nodes[m.parent].children[key_of(m.tokens.data())] = mid;
    c.tokens.erase(c.tokens.begin(), c.tokens.begin() + (size_t)keep * block_size);
    c.blocks.erase(c.blocks.begin(), c.blocks.begin() + keep);
    c.parent = mid;
    m.children[key_of(c.tokens.data())] = child;
    return mid;
  }
  // Longest cached prefix in whole blocks.  Writes block ids, returns their count; *last_node is the
  // deepest node fully matched (after a split if the match ended inside an edge).
  int match(const int32_t* toks, int n, int* out_blocks, int max_out, int* last_node, bool touch) {
    int cur = 0, matched = 0;
    const int nb = n / block_size;
    ++clock;
    while (matched < nb) {
      auto it = nodes[cur].children.find(key_of(toks + (size_t)matched * block_size));
      if (it == nodes[cur].children.end()) break;
      int ch = it->second;
      const int cb = (int)nodes[ch].blocks.size();
      int k = 1;  // first block matched by key
      while (k < cb && matched + k < nb &&
             std::memcmp(nodes[ch].tokens.data() + (size_t)k * block_size, toks + (size_t)(matched + k) * block_size,
                         sizeof(int32_t) * block_size) == 0)
        ++k;
      if (k < cb) ch = split(ch, k);
      for (int j = 0; j < k && matched + j < max_out; ++j) out_blocks[matched + j] = nodes[ch].blocks[j];
      matched += k;
      cur = ch;
      if (touch) nodes[cur].last_access = clock;
      if (k < cb) break;
    }
    if (touch) {
      query_tokens += n;
      hit_tokens += (uint64_t)matched * block_size;
      if (matched > 0) ++hits; else ++misses;
    }
    *last_node = cur;
    return matched;
  }
  // Insert the whole-block prefix of toks; blocks[i] backs block i.  Blocks already cached keep the
  // cached id (the caller's duplicate is not referenced).  Returns the number of NEW blocks adopted.
  int insert(const int32_t* toks, int n, const int* blocks, int* last_node) {
    const int nb = n / block_size;
    std::vector<int> tmp(std::max(nb, 1));
    int node = 0;
    const int matched = match(toks, nb * block_size, tmp.data(), nb, &node, false);
    int adopted = 0;
    if (matched < nb) {
      const int id = new_node();
      Node& c = nodes[id];
      c.parent = node;
      c.tokens.assign(toks + (size_t)matched * block_size, toks + (size_t)nb * block_size);
      c.blocks.assign(blocks + matched, blocks + nb);
      c.last_access = ++clock;
      for (int b : c.blocks) pool->incref(b);
      nodes[node].children[key_of(c.tokens.data())] = id;
      adopted = nb - matched;
      cached_blocks += adopted;
      inserted_blocks += adopted;
      node = id;
    }
    *last_node = node;
    return adopted;
  }
  void lock_path(int node, int delta) {
    while (node > 0) {
      nodes[node].lock += delta;
      if (nodes[node].lock < 0) nodes[node].lock = 0;
      node = nodes[node].parent;
    }
  }
  // Evict unlocked leaves, least recently used first, until `want` blocks went back to the pool's free list.
  // A leaf whose blocks are all still referenced by somebody else (a running sequence publishes its blocks while
  // it holds them) would free nothing: it stays cached and is not counted.
  int evict(int want) {
    typedef std::pair<uint64_t, int> E;
    std::priority_queue<E, std::vector<E>, std::greater<E>> heap;
    for (auto& nd : nodes)
      if (nd.alive && nd.id != 0 && nd.children.empty() && nd.lock == 0 && nd.parent >= 0 && !nd.blocks.empty())
        heap.push({nd.last_access, nd.id});
    int released = 0;
    while (released < want && !heap.empty()) {
      const int id = heap.top().second;
      heap.pop();
      Node& nd = nodes[id];
      if (!nd.alive || !nd.children.empty() || nd.lock != 0) continue;
      int freeable = 0;
      for (int b : nd.blocks) freeable += pool->refcount(b) == 1 ? 1 : 0;
      if (freeable == 0) continue;
      for (int b : nd.blocks) pool->decref(b);
      released += freeable;
      cached_blocks -= (int)nd.blocks.size();
      evicted_blocks += nd.blocks.size();
      const int par = nd.parent;
      nodes[par].children.erase(key_of(nd.tokens.data()));
      nd.alive = false;
      nd.blocks.clear();
      nd.tokens.clear();
      free_nodes.push_back(id);
      Node& p = nodes[par];
      if (par != 0 && p.children.empty() && p.lock == 0) heap.push({p.last_access, par});
    }
    return released;
  }
  int evictable() {
    // blocks held only by unlocked nodes (a node is unlocked iff no descendant is locked)
    int n = 0;
    for (auto& nd : nodes)
      if (nd.alive && nd.id != 0 && nd.lock == 0) n += (int)nd.blocks.size();
    return n;
  }
};

}  // namespace

extern "C" {

void* ubkv_pool_create(int num_blocks) { return new BlockPool(num_blocks); }
void ubkv_pool_destroy(void* p) { delete static_cast<BlockPool*>(p); }
int ubkv_pool_alloc(void* p, int n, int* out) { return static_cast<BlockPool*>(p)->alloc(n, out); }
int ubkv_pool_incref(void* p, int b) { return static_cast<BlockPool*>(p)->incref(b); }
int ubkv_pool_decref(void* p, int b) { return static_cast<BlockPool*>(p)->decref(b); }
int ubkv_pool_num_free(void* p) {
  BlockPool* bp = static_cast<BlockPool*>(p);
  std::lock_guard<std::mutex> g(bp->mu);
  return (int)bp->free_list.size();
}
int ubkv_pool_refcount(void* p, int b) {
  BlockPool* bp = static_cast<BlockPool*>(p);
  std::lock_guard<std::mutex> g(bp->mu);
  return (b < 0 || b >= bp->num_blocks) ? -1 : bp->ref[b];
}
void ubkv_pool_stats(void* p, uint64_t* out4) {
  BlockPool* bp = static_cast<BlockPool*>(p);
  std::lock_guard<std::mutex> g(bp->mu);
  out4[0] = bp->allocs; out4[1] = bp->frees; out4[2] = bp->failed; out4[3] = bp->free_list.size();
}

void* ubkv_radix_create(int block_size, void* pool) { return new RadixTree(block_size, static_cast<BlockPool*>(pool)); }
void ubkv_radix_destroy(void* t) { delete static_cast<RadixTree*>(t); }
int ubkv_radix_match(void* t, const int32_t* toks, int n, int* out_blocks, int max_out, int* last_node) {
  RadixTree* r = static_cast<RadixTree*>(t);
  std::lock_guard<std::mutex> g(r->mu);
  return r->match(toks, n, out_blocks, max_out, last_node, true);
}
// match + lock the matched path + one reference per matched block, as one step with respect to eviction: between a
// plain match and the caller's own incref / lock another thread could evict the leaf and hand its blocks out again
int ubkv_radix_acquire(void* t, const int32_t* toks, int n, int* out_blocks, int max_out, int* last_node) {
  RadixTree* r = static_cast<RadixTree*>(t);
  std::lock_guard<std::mutex> g(r->mu);
  const int m = r->match(toks, n, out_blocks, max_out, last_node, true);
  if (m > 0) {
    r->lock_path(*last_node, 1);
    for (int i = 0; i < m && i < max_out; ++i) r->pool->incref(out_blocks[i]);
  }
  return m;
}
int ubkv_radix_insert(void* t, const int32_t* toks, int n, const int* blocks, int* last_node) {
  RadixTree* r = static_cast<RadixTree*>(t);
  std::lock_guard<std::mutex> g(r->mu);
  return r->insert(toks, n, blocks, last_node);
}
void ubkv_radix_lock(void* t, int node, int delta) {
  RadixTree* r = static_cast<RadixTree*>(t);
  std::lock_guard<std::mutex> g(r->mu);
  r->lock_path(node, delta);
}
int ubkv_radix_evict(void* t, int want_blocks) {
  RadixTree* r = static_cast<RadixTree*>(t);
  std::lock_guard<std::mutex> g(r->mu);
  return r->evict(want_blocks);
}
int ubkv_radix_evictable(void* t) {
  RadixTree* r = static_cast<RadixTree*>(t);
  std::lock_guard<std::mutex> g(r->mu);
  return r->evictable();
}
void ubkv_radix_stats(void* t, uint64_t* out8) {
  RadixTree* r = static_cast<RadixTree*>(t);
  std::lock_guard<std::mutex> g(r->mu);
  out8[0] = r->hits; out8[1] = r->misses; out8[2] = r->hit_tokens; out8[3] = r->query_tokens;
  out8[4] = r->evicted_blocks; out8[5] = r->inserted_blocks; out8[6] = (uint64_t)r->cached_blocks;
  uint64_t live = 0;
  for (auto& nd : r->nodes) live += nd.alive ? 1 : 0;
  out8[7] = live;
}

}  // extern "C"
