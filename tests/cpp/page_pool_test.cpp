// The page pool through its C++ class (unholy_b200/csrc/page_pool.hpp), the way a C++ engine would hold it in place of
// the reference's free_pages_ / evictable_ / page_by_hash_ / page_info_ / tables_ members (src/engine/engine.hpp:258-306).
// Standalone like the reference's tests (tools/sched_test/main.cpp): prints, returns non-zero on failure. CPU only.
#include <cstdio>
#include <numeric>
#include <vector>

#include "../../unholy_b200/csrc/page_pool.hpp"

static int fails = 0;
#define EXPECT(cond)                                              \
  do {                                                            \
    if (!(cond)) {                                                \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++fails;                                                    \
    }                                                             \
  } while (0)

int main() {
  using pkv::PagePool;
  PagePool pool(/*pages*/ 32, /*page_tokens*/ 4, /*slots*/ 4, /*pages per seq*/ 8, /*prefix cache*/ true);
  std::vector<int32_t> prompt(15);
  std::iota(prompt.begin(), prompt.end(), 100);
  // admission: slot 0, pages 0..3 in order (src/engine/engine.cpp:95-96,437-444)
  const int a = pool.open();
  EXPECT(pool.match_prefix(a, prompt.data(), int(prompt.size()), nullptr) == 0);
  EXPECT(pool.assign_slot(a) == 0);
  EXPECT(pool.alloc(a, 15));
  EXPECT((pool.pages(a) == std::vector<int32_t>{0, 1, 2, 3}));
  EXPECT(pool.take_dirty());
  EXPECT(pool.tables()[0] == 0 && pool.tables()[3] == 3);
  pool.register_pages(a, prompt.data(), int(prompt.size()), 15);  // three full pages get names
  EXPECT(pool.cached_count() == 3);
  pool.close(a);                                                  // tail first: evictable = [2, 1, 0]; page 3 is free
  EXPECT((pool.evictable_list() == std::vector<int32_t>{2, 1, 0}));
  EXPECT(pool.free_list().back() == 3);
  // a second request with the same prompt shares the three named pages and computes from token 12
  const int b = pool.open();
  EXPECT(pool.match_prefix(b, prompt.data(), int(prompt.size()), nullptr) == 12);
  EXPECT((pool.pages(b) == std::vector<int32_t>{0, 1, 2}));
  EXPECT(pool.evictable_count() == 0 && pool.refs(1) == 1);
  EXPECT(pool.assign_slot(b) == 0);
  EXPECT(pool.alloc(b, 15) && pool.pages(b).back() == 3);
  // a boundary without a saved state cannot be resumed from (the engine's snapshot condition)
  const int c = pool.open();
  const uint8_t ok[3] = {1, 0, 0};
  EXPECT(pool.match_prefix(c, prompt.data(), int(prompt.size()), ok) == 4);
  EXPECT(pool.refs(0) == 2 && pool.refs(1) == 1);
  // fork + copy-on-write: the child shares b's pages; its first write into the shared last page takes a fresh one
  const int d = pool.fork(b, 15);
  EXPECT(pool.refs(3) == 2);
  std::vector<std::pair<int32_t, int32_t>> moves;
  EXPECT(pool.alloc(d, 16) && pool.cow(d, 15, 1, moves) == 1);
  EXPECT(moves.size() == 1 && moves[0].first == 3 && moves[0].second == 4 && pool.refs(3) == 1 && pool.refs(4) == 1);
  // compaction after releases: live ids >= W move into the holes below W
  pool.close(c);
  pool.close(b);
  std::vector<int32_t> freed;
  pool.free_lru(32, freed);
  moves.clear();
  const int W = pool.num_pages() - pool.free_count();
  pool.compact(moves);
  for (const int32_t p : pool.pages(d)) EXPECT(p < W);
  EXPECT(pool.available() == 32 - int(pool.pages(d).size()));
  std::printf(fails ? "FAILED\n" : "all ok\n");
  return fails ? 1 : 0;
}
