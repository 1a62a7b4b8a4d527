// Multi-threaded stress driver for the host KV core (block pool + radix tree), meant to be built together with
// kv_core.cpp under -fsanitize=thread and -fsanitize=address,undefined (tests/test_sanitizers.py does that).
// Eight threads admit, extend, publish and release sequences that share a few prompt prefixes, and evict when the pool
// runs dry -- the same call pattern as the serving engine, but concurrent.  At the end everything is evicted and the
// pool must be whole again.  Exit code 0 = invariants hold; the sanitizer runtime reports races and memory errors.
//
// Not part of the shared library (the ".cc" suffix keeps it out of the library's source list).
#include <cstdint>
#include <cstdio>
#include <random>
#include <thread>
#include <vector>

extern "C" {
void* ubkv_pool_create(int num_blocks);
void ubkv_pool_destroy(void* p);
int ubkv_pool_alloc(void* p, int n, int* out);
int ubkv_pool_decref(void* p, int b);
int ubkv_pool_num_free(void* p);
void* ubkv_radix_create(int block_size, void* pool);
void ubkv_radix_destroy(void* t);
int ubkv_radix_acquire(void* t, const int32_t* toks, int n, int* out_blocks, int max_out, int* last_node);
int ubkv_radix_insert(void* t, const int32_t* toks, int n, const int* blocks, int* last_node);
void ubkv_radix_lock(void* t, int node, int delta);
int ubkv_radix_evict(void* t, int want_blocks);
void ubkv_radix_stats(void* t, uint64_t* out8);
}

int main(int argc, char** argv) {
  const int kBlocks = 192, kBs = 16, kThreads = 8;
  const int iters = argc > 1 ? std::atoi(argv[1]) : 400;
  void* pool = ubkv_pool_create(kBlocks);
  void* tree = ubkv_radix_create(kBs, pool);
  std::vector<std::thread> th;
  std::vector<int> bad(kThreads, 0);
  for (int w = 0; w < kThreads; ++w) {
    th.emplace_back([&, w] {
      std::mt19937 rng(1234 + w);
      for (int it = 0; it < iters; ++it) {
        const int family = rng() % 4, len = kBs * (2 + rng() % 5);
        std::vector<int32_t> toks(len);
        for (int i = 0; i < len; ++i) toks[i] = i < 2 * kBs ? family * 1000 + i : int32_t(rng() % 50000);
        const int nb = len / kBs;
        std::vector<int> blocks(nb);
        int node = 0;
        const int hit = ubkv_radix_acquire(tree, toks.data(), len, blocks.data(), nb, &node);
        const int need = nb - hit;
        bool ok = true;
        if (need > 0 && ubkv_pool_alloc(pool, need, blocks.data() + hit) != 0) {
          ubkv_radix_evict(tree, need);
          ok = ubkv_pool_alloc(pool, need, blocks.data() + hit) == 0;
        }
        if (ok) {
          int last = 0;
          ubkv_radix_insert(tree, toks.data(), len, blocks.data(), &last);
        }
        // release: the references this sequence holds (matched + own), then the path lock
        const int held = ok ? nb : hit;
        for (int i = 0; i < held; ++i)
          if (ubkv_pool_decref(pool, blocks[i]) < 0) ++bad[w];
        if (hit > 0) ubkv_radix_lock(tree, node, -1);
      }
    });
  }
  for (auto& t : th) t.join();
  int errors = 0;
  for (int b : bad) errors += b;
  ubkv_radix_evict(tree, 1 << 30);
  uint64_t st[8];
  ubkv_radix_stats(tree, st);
  const int free_now = ubkv_pool_num_free(pool);
  std::printf("free %d of %d, cached %llu, hits %llu, evicted %llu, bad decrefs %d\n", free_now, kBlocks,
              (unsigned long long)st[6], (unsigned long long)st[0], (unsigned long long)st[4], errors);
  ubkv_radix_destroy(tree);
  ubkv_pool_destroy(pool);
  return (free_now == kBlocks && st[6] == 0 && errors == 0) ? 0 : 1;
}
