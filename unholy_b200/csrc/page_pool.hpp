// Host-side page pool: block allocator, prefix-cache bookkeeping and block tables of the paged KV cache.
//
// Observable behaviour (which physical page id is handed out when, which pages are shared, the block-table contents)
// follows ewtodd/unholy's engine: src/engine/engine.cpp:87-98 (initial free list descending, so page 0 is taken
// first), :234-248 (take_page: free list back, else evict the least recently used cached page), :437-444 (alloc_pages),
// :208-217 (unref tail first; a cached page becomes evictable, others go back to the free list), :257-280 (chained
// splitmix page names), :284-336 (match_prefix), :340-353 (register_pages), :250-254 (write_table leaves stale tails).
// The data structures are this library's own: the LRU is an intrusive doubly linked list over page ids held in two
// flat arrays, sequences are small integer handles.
//
// Three operations have no counterpart in the reference and fix their own rule here: copy-on-write of shared pages
// (fork + cow), freeing pages from the LRU front without handing them out (free_lru), and hole-filling compaction
// (compact); migrate moves a sequence between two pools (shards). Each emits (source page, destination page) pairs for
// the device-side page copy.
//
// Single-threaded, like the engine thread that owns the reference's allocator.
#pragma once

#include <cstdint>
#include <unordered_map>
#include <utility>
#include <vector>

namespace pkv {

uint64_t mix64(uint64_t x);
// Name of page `index` given the previous page's name (or the chain seed for index 0) and the page's tokens.
uint64_t chain_page_hash(uint64_t prev, const int32_t* tokens, int page_tokens);
uint64_t chain_page_hash_keys(uint64_t prev, const uint64_t* keys, int page_tokens);
// token_key of src/engine/engine.cpp:264-270 for every position of a sequence: uint32(token), or for positions inside
// image block i (starts[i] <= p < starts[i] + lens[i]) mix64(hashes[i] + (p - starts[i])); the first block that holds
// the position wins, as in the reference's loop.
void token_keys(const int32_t* tokens, int n, const int32_t* starts, const int32_t* lens, const uint64_t* hashes, int nimages,
                uint64_t* keys_out);
constexpr uint64_t kHashSeed = 0x243f6a8885a308d3ull;

class PagePool {
 public:
  PagePool(int num_pages, int page_tokens, int max_slots, int max_pages_per_seq, bool prefix_cache);

  int num_pages() const { return int(info_.size()); }
  int page_tokens() const { return page_tokens_; }
  int max_slots() const { return max_slots_; }
  int max_pages_per_seq() const { return width_; }
  int available() const { return int(free_.size()) + lru_count_; }
  int free_count() const { return int(free_.size()); }
  int evictable_count() const { return lru_count_; }
  int cached_count() const { return int(by_hash_.size()); }

  int open();
  void close(int seq);
  bool valid(int seq) const { return seq >= 0 && seq < int(seqs_.size()) && seqs_[size_t(seq)].open; }
  // A sequence's positions are named either by token ids (key = uint32(token), the text rule) or by 64-bit keys the
  // caller computed (token_keys(): image positions are named by the image's hash and the offset in the block,
  // src/engine/engine.cpp:264-270). Exactly one of the two pointers is non-null.
  struct Keys {
    const int32_t* tokens = nullptr;
    const uint64_t* keys = nullptr;
    uint64_t at(size_t i) const { return keys ? keys[i] : uint64_t(uint32_t(tokens[i])); }
  };
  int match_prefix(int seq, Keys k, int ntokens, const uint8_t* boundary_ok);
  int match_prefix(int seq, const int32_t* tokens, int ntokens, const uint8_t* boundary_ok) {
    return match_prefix(seq, Keys{tokens, nullptr}, ntokens, boundary_ok);
  }
  // How many leading full pages of the positions (at most (ntokens - 1) / page_tokens, as match_prefix) the prefix
  // cache names right now; nothing changes. The walk match_prefix does before it looks for a resumable boundary
  // (src/engine/engine.cpp:289-291).
  int cached_prefix(Keys k, int ntokens) const;
  int assign_slot(int seq);
  bool alloc(int seq, int upto);
  void register_pages(int seq, Keys k, int ntokens, int done_pos);
  void register_pages(int seq, const int32_t* tokens, int ntokens, int done_pos) {
    register_pages(seq, Keys{tokens, nullptr}, ntokens, done_pos);
  }
  void release(int seq);
  // The page half of drop_prefix (src/engine/engine.cpp:419-425): a matched prefix whose snapshot could not be read is
  // given back, tail first; the sequence keeps its slot and starts over from position 0.
  void drop_prefix(int seq);

  int fork(int from, int ntokens);
  // cow_pairs / compact_pairs: how many (source, destination) pairs the call would emit now; nothing changes.
  int cow_pairs(int seq, int s0, int n) const;
  int cow(int seq, int s0, int n, std::vector<std::pair<int32_t, int32_t>>& moves);
  int free_lru(int count, std::vector<int32_t>& freed);
  int compact_pairs() const;
  int compact(std::vector<std::pair<int32_t, int32_t>>& moves);
  static int migrate(PagePool& src, int seq, PagePool& dst, std::vector<std::pair<int32_t, int32_t>>& moves);

  const std::vector<int32_t>& pages(int seq) const { return seqs_[size_t(seq)].pages; }
  int slot(int seq) const { return seqs_[size_t(seq)].slot; }
  int refs(int page) const { return info_[size_t(page)].refs; }
  uint64_t hash(int page) const { return info_[size_t(page)].cached ? info_[size_t(page)].hash : 0; }
  const std::vector<int32_t>& free_list() const { return free_; }
  std::vector<int32_t> evictable_list() const;
  const std::vector<int32_t>& tables() const { return tables_; }
  bool take_dirty() {
    const bool d = dirty_;
    dirty_ = false;
    return d;
  }
  bool dirty() const { return dirty_; }

 private:
  struct Page {
    uint64_t hash = 0;
    int refs = 0;
    bool cached = false;
    int32_t prev = -1, next = -1;  // LRU links (valid while the page is evictable)
    bool in_lru = false;
  };
  struct Seq {
    bool open = false;
    int slot = -1;
    int registered = 0;
    std::vector<int32_t> pages;
    std::vector<uint64_t> hashes;
  };
  int32_t take_page();
  void write_table(const Seq& s);
  void hash_upto(Seq& s, Keys k, int npages);
  void unname(Page& pg);
  void lru_push_back(int32_t p);
  void lru_unlink(int32_t p);
  void unref(Seq& s);

  int page_tokens_, max_slots_, width_;
  bool cache_on_;
  std::vector<Page> info_;
  std::vector<int32_t> free_, free_slots_;
  int32_t lru_head_ = -1, lru_tail_ = -1;
  int lru_count_ = 0;
  std::unordered_map<uint64_t, int32_t> by_hash_;
  std::vector<Seq> seqs_;
  std::vector<int> free_handles_;
  std::vector<int32_t> tables_;
  bool dirty_ = true;
};

}  // namespace pkv
