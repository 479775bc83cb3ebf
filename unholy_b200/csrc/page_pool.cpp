// PagePool implementation and its C ABI (pkv_pool_* in include/unholy_pkv.h). See page_pool.hpp for the contract and
// the reference lines each rule follows.
#include "page_pool.hpp"

#include <algorithm>
#include <cstring>
#include <new>

#include "../../include/unholy_pkv.h"

namespace pkv {

// splitmix64 finaliser (src/engine/engine.cpp:257-261).
uint64_t mix64(uint64_t x) {
  x ^= x >> 30;
  x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27;
  x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

// src/engine/engine.cpp:272-280: every token of the page is folded in as h = mix64(h + golden + uint32(token)).
uint64_t chain_page_hash(uint64_t prev, const int32_t* tokens, int page_tokens) {
  uint64_t h = prev;
  for (int i = 0; i < page_tokens; ++i) h = mix64(h + 0x9e3779b97f4a7c15ull + uint64_t(uint32_t(tokens[i])));
  return h;
}

uint64_t chain_page_hash_keys(uint64_t prev, const uint64_t* keys, int page_tokens) {
  uint64_t h = prev;
  for (int i = 0; i < page_tokens; ++i) h = mix64(h + 0x9e3779b97f4a7c15ull + keys[i]);
  return h;
}

void token_keys(const int32_t* tokens, int n, const int32_t* starts, const int32_t* lens, const uint64_t* hashes, int nimages,
                uint64_t* keys_out) {
  for (int p = 0; p < n; ++p) keys_out[p] = uint64_t(uint32_t(tokens[p]));
  for (int i = nimages - 1; i >= 0; --i)  // earlier blocks overwrite later ones: the first match wins
    for (int p = std::max(starts[i], 0); p < starts[i] + lens[i] && p < n; ++p) keys_out[p] = mix64(hashes[i] + uint64_t(p - starts[i]));
}

PagePool::PagePool(int num_pages, int page_tokens, int max_slots, int max_pages_per_seq, bool prefix_cache)
    : page_tokens_(page_tokens), max_slots_(max_slots), width_(max_pages_per_seq), cache_on_(prefix_cache) {
  info_.resize(size_t(num_pages));
  free_.reserve(size_t(num_pages));
  for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);
  for (int s = max_slots - 1; s >= 0; --s) free_slots_.push_back(s);
  tables_.assign(size_t(max_slots) * size_t(max_pages_per_seq), 0);
}

void PagePool::lru_push_back(int32_t p) {
  Page& pg = info_[size_t(p)];
  pg.prev = lru_tail_;
  pg.next = -1;
  pg.in_lru = true;
  if (lru_tail_ >= 0) info_[size_t(lru_tail_)].next = p;
  else lru_head_ = p;
  lru_tail_ = p;
  ++lru_count_;
}

void PagePool::lru_unlink(int32_t p) {
  Page& pg = info_[size_t(p)];
  if (!pg.in_lru) return;
  if (pg.prev >= 0) info_[size_t(pg.prev)].next = pg.next;
  else lru_head_ = pg.next;
  if (pg.next >= 0) info_[size_t(pg.next)].prev = pg.prev;
  else lru_tail_ = pg.prev;
  pg.prev = pg.next = -1;
  pg.in_lru = false;
  --lru_count_;
}

std::vector<int32_t> PagePool::evictable_list() const {
  std::vector<int32_t> out;
  out.reserve(size_t(lru_count_));
  for (int32_t p = lru_head_; p >= 0; p = info_[size_t(p)].next) out.push_back(p);
  return out;
}

int32_t PagePool::take_page() {
  int32_t p;
  if (!free_.empty()) {
    p = free_.back();
    free_.pop_back();
  } else {
    p = lru_head_;
    lru_unlink(p);
    Page& pg = info_[size_t(p)];
    by_hash_.erase(pg.hash);
    pg.cached = false;
  }
  info_[size_t(p)].refs = 1;
  return p;
}

void PagePool::write_table(const Seq& s) {
  if (s.slot < 0) return;
  std::copy(s.pages.begin(), s.pages.end(), tables_.begin() + ptrdiff_t(size_t(s.slot) * size_t(width_)));
  dirty_ = true;
}

int PagePool::open() {
  int h;
  if (!free_handles_.empty()) {
    h = free_handles_.back();
    free_handles_.pop_back();
  } else {
    h = int(seqs_.size());
    seqs_.emplace_back();
  }
  seqs_[size_t(h)] = Seq{};
  seqs_[size_t(h)].open = true;
  return h;
}

void PagePool::close(int seq) {
  release(seq);
  seqs_[size_t(seq)] = Seq{};
  free_handles_.push_back(seq);
}

void PagePool::hash_upto(Seq& s, Keys k, int npages) {
  while (int(s.hashes.size()) < npages) {
    const size_t i = s.hashes.size(), at = i * size_t(page_tokens_);
    const uint64_t prev = i ? s.hashes.back() : kHashSeed;
    s.hashes.push_back(k.keys ? chain_page_hash_keys(prev, k.keys + at, page_tokens_) : chain_page_hash(prev, k.tokens + at, page_tokens_));
  }
}

int PagePool::match_prefix(int seq, Keys tokens, int ntokens, const uint8_t* boundary_ok) {
  Seq& s = seqs_[size_t(seq)];
  const int limit = (ntokens - 1) / page_tokens_;  // the last token is always computed
  if (!cache_on_ || limit <= 0 || !s.pages.empty()) return 0;
  hash_upto(s, tokens, limit);
  int best = 0;
  for (int i = 0; i < limit; ++i) {
    if (!by_hash_.count(s.hashes[size_t(i)])) break;
    if (!boundary_ok || boundary_ok[i]) best = i + 1;
  }
  for (int i = 0; i < best; ++i) {
    const int32_t p = by_hash_.at(s.hashes[size_t(i)]);
    Page& pg = info_[size_t(p)];
    if (pg.refs++ == 0) lru_unlink(p);
    s.pages.push_back(p);
  }
  s.registered = best;
  return best * page_tokens_;
}

int PagePool::cached_prefix(Keys k, int ntokens) const {
  const int limit = (ntokens - 1) / page_tokens_;
  if (!cache_on_ || limit <= 0) return 0;
  uint64_t h = kHashSeed;
  for (int i = 0; i < limit; ++i) {
    const size_t at = size_t(i) * size_t(page_tokens_);
    h = k.keys ? chain_page_hash_keys(h, k.keys + at, page_tokens_) : chain_page_hash(h, k.tokens + at, page_tokens_);
    if (!by_hash_.count(h)) return i;
  }
  return limit;
}

int PagePool::assign_slot(int seq) {
  Seq& s = seqs_[size_t(seq)];
  if (s.slot >= 0) return s.slot;
  if (free_slots_.empty()) return -1;
  s.slot = free_slots_.back();
  free_slots_.pop_back();
  write_table(s);
  dirty_ = true;
  return s.slot;
}

bool PagePool::alloc(int seq, int upto) {
  Seq& s = seqs_[size_t(seq)];
  const size_t need = size_t((upto + page_tokens_ - 1) / page_tokens_);
  if (need <= s.pages.size()) return true;
  if (need > size_t(width_) || need - s.pages.size() > size_t(available())) return false;
  while (s.pages.size() < need) s.pages.push_back(take_page());
  write_table(s);
  return true;
}

void PagePool::register_pages(int seq, Keys tokens, int ntokens, int done_pos) {
  Seq& s = seqs_[size_t(seq)];
  if (!cache_on_) return;
  const int full = std::min({done_pos / page_tokens_, int(s.pages.size()), ntokens / page_tokens_});
  if (full <= s.registered) return;
  hash_upto(s, tokens, full);
  for (int i = s.registered; i < full; ++i) {
    const int32_t p = s.pages[size_t(i)];
    Page& pg = info_[size_t(p)];
    if (!pg.cached && by_hash_.emplace(s.hashes[size_t(i)], p).second) {
      pg.hash = s.hashes[size_t(i)];
      pg.cached = true;
    }
  }
  s.registered = full;
}

void PagePool::unref(Seq& s) {
  for (auto it = s.pages.rbegin(); it != s.pages.rend(); ++it) {
    Page& pg = info_[size_t(*it)];
    if (--pg.refs > 0) continue;
    if (pg.cached) lru_push_back(*it);
    else free_.push_back(*it);
  }
  s.pages.clear();
}

void PagePool::release(int seq) {
  Seq& s = seqs_[size_t(seq)];
  unref(s);
  if (s.slot >= 0) free_slots_.push_back(s.slot);
  s.slot = -1;
  s.registered = 0;
}

void PagePool::drop_prefix(int seq) {
  Seq& s = seqs_[size_t(seq)];
  unref(s);
  s.registered = 0;
}

// Fork: the child shares every page holding positions [0, ntokens) of the parent, a partial last page included.
int PagePool::fork(int from, int ntokens) {
  const int npages = std::min((ntokens + page_tokens_ - 1) / page_tokens_, int(seqs_[size_t(from)].pages.size()));
  const int child = open();
  const Seq& parent = seqs_[size_t(from)];  // (after open(): the vector may have grown)
  Seq& c = seqs_[size_t(child)];
  c.pages.assign(parent.pages.begin(), parent.pages.begin() + npages);
  const int full = std::min(ntokens / page_tokens_, npages);
  c.hashes.assign(parent.hashes.begin(), parent.hashes.begin() + std::min<size_t>(parent.hashes.size(), size_t(full)));
  c.registered = std::min(parent.registered, full);
  for (const int32_t p : c.pages) ++info_[size_t(p)].refs;
  return child;
}

void PagePool::unname(Page& pg) {
  by_hash_.erase(pg.hash);
  pg.cached = false;
  pg.hash = 0;
}

// Copy-on-write: a page of `seq` that rows [s0, s0 + n) touch is not privately writable when another sequence also
// references it (refs > 1) or when the prefix cache names it (a later match_prefix would share the modified page under
// the old name). Such a page is replaced by a fresh one and the caller copies the payload of each (old, fresh) pair
// before writing; the old page keeps its name and, when this was its last reference, becomes evictable. A named page
// held only by this sequence is written in place after losing its name when the pool has no page to spare.
int PagePool::cow_pairs(int seq, int s0, int n) const {
  const Seq& s = seqs_[size_t(seq)];
  if (n <= 0) return 0;
  const int first = s0 / page_tokens_, last = std::min((s0 + n - 1) / page_tokens_, int(s.pages.size()) - 1);
  int avail = available(), pairs = 0;
  for (int i = first; i <= last; ++i) {
    const Page& pg = info_[size_t(s.pages[size_t(i)])];
    if (pg.refs > 1) {
      if (avail-- <= 0) return -1;
      ++pairs;
    } else if (pg.cached && avail > 0) {
      ++pairs;  // takes one page and makes one evictable
    }
  }
  return pairs;
}

int PagePool::cow(int seq, int s0, int n, std::vector<std::pair<int32_t, int32_t>>& moves) {
  if (n <= 0) return 0;
  if (cow_pairs(seq, s0, n) < 0) return -1;
  Seq& s = seqs_[size_t(seq)];
  const int first = s0 / page_tokens_, last = std::min((s0 + n - 1) / page_tokens_, int(s.pages.size()) - 1);
  bool touched = false;
  for (int i = first; i <= last; ++i) {
    const int32_t old = s.pages[size_t(i)];
    Page& pg = info_[size_t(old)];
    if (pg.refs <= 1 && !pg.cached) continue;
    if (i < s.registered) s.registered = i;  // the private page is unnamed until registered again
    if (pg.refs <= 1 && available() <= 0) {
      unname(pg);
      continue;
    }
    const int32_t fresh = take_page();
    if (--info_[size_t(old)].refs == 0) lru_push_back(old);  // (only a named page gets here with one reference)
    s.pages[size_t(i)] = fresh;
    moves.emplace_back(old, fresh);
    touched = true;
  }
  if (touched) write_table(s);
  return int(moves.size());
}

// The evict branch of take_page applied `count` times, with the page going to the free list instead of to a caller.
int PagePool::free_lru(int count, std::vector<int32_t>& freed) {
  int done = 0;
  while (done < count && lru_head_ >= 0) {
    const int32_t p = lru_head_;
    lru_unlink(p);
    unname(info_[size_t(p)]);
    free_.push_back(p);
    freed.push_back(p);
    ++done;
  }
  return done;
}

int PagePool::compact_pairs() const {
  const int N = num_pages(), W = N - int(free_.size());
  int holes = 0;
  for (const int32_t p : free_) holes += p < W;
  return holes;  // every hole below W is filled by exactly one live page at or above W
}

// Hole filling: with W live pages, every live id >= W moves into a free id < W (both ascending, paired in order).
int PagePool::compact(std::vector<std::pair<int32_t, int32_t>>& moves) {
  const int N = num_pages();
  std::vector<uint8_t> is_free(size_t(N), 0);
  for (const int32_t p : free_) is_free[size_t(p)] = 1;
  const int W = N - int(free_.size());
  std::vector<int32_t> holes, sources;
  for (int p = 0; p < W; ++p)
    if (is_free[size_t(p)]) holes.push_back(p);
  for (int p = W; p < N; ++p)
    if (!is_free[size_t(p)]) sources.push_back(p);
  std::vector<int32_t> remap(size_t(N), -1);
  for (size_t i = 0; i < sources.size(); ++i) {
    const int32_t from = sources[i], to = holes[i];
    remap[size_t(from)] = to;
    moves.emplace_back(from, to);
    Page& a = info_[size_t(from)];
    Page& b = info_[size_t(to)];
    b = a;
    a = Page{};
    if (b.in_lru) {  // relink the neighbours (and the ends) to the new id
      if (b.prev >= 0) info_[size_t(b.prev)].next = to;
      else lru_head_ = to;
      if (b.next >= 0) info_[size_t(b.next)].prev = to;
      else lru_tail_ = to;
    }
    if (b.cached) by_hash_[b.hash] = to;
  }
  if (!sources.empty()) {
    for (Seq& s : seqs_) {
      if (!s.open) continue;
      bool touched = false;
      for (int32_t& p : s.pages)
        if (remap[size_t(p)] >= 0) {
          p = remap[size_t(p)];
          touched = true;
        }
      if (touched) write_table(s);
    }
  }
  free_.clear();
  for (int p = N - 1; p >= W; --p) free_.push_back(p);
  return int(sources.size());
}

// The sequence leaves `src` (pages unreferenced tail first, slot returned) and gets fresh pages of `dst` in logical
// order; returns the new handle in dst, or -1 when dst cannot hold it (nothing changes then).
int PagePool::migrate(PagePool& src, int seq, PagePool& dst, std::vector<std::pair<int32_t, int32_t>>& moves) {
  const std::vector<int32_t> old = src.seqs_[size_t(seq)].pages;
  if (int(old.size()) > dst.available() || int(old.size()) > dst.width_) return -1;
  const int h = dst.open();
  Seq& d = dst.seqs_[size_t(h)];
  for (const int32_t p : old) {
    const int32_t q = dst.take_page();
    d.pages.push_back(q);
    moves.emplace_back(p, q);
  }
  src.close(seq);
  return h;
}

}  // namespace pkv

// ---------------------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------------------
struct pkv_pool {
  pkv::PagePool impl;
  pkv_pool(int a, int b, int c, int d, bool e) : impl(a, b, c, d, e) {}
};

namespace {
// Every caller has checked `cap` and the pointers against the pair count BEFORE changing the pool.
int emit(const std::vector<std::pair<int32_t, int32_t>>& moves, int32_t* src_out, int32_t* dst_out, int cap) {
  if (int(moves.size()) > cap || ((!src_out || !dst_out) && !moves.empty())) return -2;
  for (size_t i = 0; i < moves.size(); ++i) {
    src_out[i] = moves[i].first;
    dst_out[i] = moves[i].second;
  }
  return int(moves.size());
}
int copy_out(const std::vector<int32_t>& v, int32_t* out, int cap) {
  if (out)
    for (int i = 0; i < int(v.size()) && i < cap; ++i) out[i] = v[size_t(i)];
  return int(v.size());
}
}  // namespace

extern "C" {

pkv_pool* pkv_pool_create(int num_pages, int page_tokens, int max_slots, int max_pages_per_seq, int prefix_cache) {
  if (num_pages <= 0 || page_tokens <= 0 || max_slots <= 0 || max_pages_per_seq <= 0) return nullptr;
  return new (std::nothrow) pkv_pool(num_pages, page_tokens, max_slots, max_pages_per_seq, prefix_cache != 0);
}
void pkv_pool_destroy(pkv_pool* p) { delete p; }

int pkv_pool_seq_open(pkv_pool* p) { return p ? p->impl.open() : -1; }
int pkv_pool_seq_close(pkv_pool* p, int seq) {
  if (!p || !p->impl.valid(seq)) return PKV_ERR_ARG;
  p->impl.close(seq);
  return PKV_OK;
}
int pkv_pool_match_prefix(pkv_pool* p, int seq, const int32_t* tokens, int ntokens, const uint8_t* boundary_ok) {
  if (!p || !p->impl.valid(seq) || (!tokens && ntokens > 0)) return -1;
  return p->impl.match_prefix(seq, tokens, ntokens, boundary_ok);
}
int pkv_pool_match_prefix_keys(pkv_pool* p, int seq, const uint64_t* keys, int nkeys, const uint8_t* boundary_ok) {
  if (!p || !p->impl.valid(seq) || (!keys && nkeys > 0)) return -1;
  return p->impl.match_prefix(seq, pkv::PagePool::Keys{nullptr, keys}, nkeys, boundary_ok);
}
int pkv_pool_cached_prefix_keys(const pkv_pool* p, const uint64_t* keys, int nkeys) {
  if (!p || (!keys && nkeys > 0)) return -1;
  return p->impl.cached_prefix(pkv::PagePool::Keys{nullptr, keys}, nkeys);
}
int pkv_pool_register_keys(pkv_pool* p, int seq, const uint64_t* keys, int nkeys, int done_pos) {
  if (!p || !p->impl.valid(seq) || (!keys && nkeys > 0)) return PKV_ERR_ARG;
  p->impl.register_pages(seq, pkv::PagePool::Keys{nullptr, keys}, nkeys, done_pos);
  return PKV_OK;
}
int pkv_token_keys(const int32_t* tokens, int n, const int32_t* starts, const int32_t* lens, const uint64_t* hashes, int nimages,
                   uint64_t* keys_out) {
  if (n < 0 || nimages < 0 || (n > 0 && (!tokens || !keys_out)) || (nimages > 0 && (!starts || !lens || !hashes))) return PKV_ERR_ARG;
  pkv::token_keys(tokens, n, starts, lens, hashes, nimages, keys_out);
  return PKV_OK;
}
uint64_t pkv_page_hash_keys(const uint64_t* keys, int page_tokens, int page_index) {
  uint64_t h = pkv::kHashSeed;
  for (int i = 0; i <= page_index; ++i) h = pkv::chain_page_hash_keys(h, keys + size_t(i) * size_t(page_tokens), page_tokens);
  return h;
}
int pkv_pool_assign_slot(pkv_pool* p, int seq) { return p && p->impl.valid(seq) ? p->impl.assign_slot(seq) : -1; }
int pkv_pool_alloc(pkv_pool* p, int seq, int upto) { return p && p->impl.valid(seq) && p->impl.alloc(seq, upto) ? 1 : 0; }
int pkv_pool_register(pkv_pool* p, int seq, const int32_t* tokens, int ntokens, int done_pos) {
  if (!p || !p->impl.valid(seq) || (!tokens && ntokens > 0)) return PKV_ERR_ARG;
  p->impl.register_pages(seq, tokens, ntokens, done_pos);
  return PKV_OK;
}
int pkv_pool_release(pkv_pool* p, int seq) {
  if (!p || !p->impl.valid(seq)) return PKV_ERR_ARG;
  p->impl.release(seq);
  return PKV_OK;
}
int pkv_pool_drop_prefix(pkv_pool* p, int seq) {
  if (!p || !p->impl.valid(seq)) return PKV_ERR_ARG;
  p->impl.drop_prefix(seq);
  return PKV_OK;
}
int pkv_pool_fork(pkv_pool* p, int from, int ntokens) {
  if (!p || !p->impl.valid(from) || ntokens < 0) return -1;
  return p->impl.fork(from, ntokens);
}
int pkv_pool_cow(pkv_pool* p, int seq, int s0, int n, int32_t* src_out, int32_t* dst_out, int cap) {
  if (!p || !p->impl.valid(seq) || s0 < 0) return -1;
  const int pairs = p->impl.cow_pairs(seq, s0, n);
  if (pairs < 0) return -1;
  if (pairs > cap || (pairs > 0 && (!src_out || !dst_out))) return -2;  // nothing has changed
  std::vector<std::pair<int32_t, int32_t>> moves;
  if (p->impl.cow(seq, s0, n, moves) < 0) return -1;
  return emit(moves, src_out, dst_out, cap);
}
int pkv_pool_cow_pairs(const pkv_pool* p, int seq, int s0, int n) {
  return p && p->impl.valid(seq) && s0 >= 0 ? p->impl.cow_pairs(seq, s0, n) : -1;
}
int pkv_pool_compact_pairs(const pkv_pool* p) { return p ? p->impl.compact_pairs() : -1; }
int pkv_pool_free_lru(pkv_pool* p, int count, int32_t* freed_out, int cap) {
  if (!p) return -1;
  std::vector<int32_t> freed;
  p->impl.free_lru(count, freed);
  copy_out(freed, freed_out, cap);
  return int(freed.size());
}
int pkv_pool_compact(pkv_pool* p, int32_t* src_out, int32_t* dst_out, int cap) {
  if (!p) return -1;
  const int pairs = p->impl.compact_pairs();
  if (pairs > cap || (pairs > 0 && (!src_out || !dst_out))) return -2;  // nothing has changed
  std::vector<std::pair<int32_t, int32_t>> moves;
  p->impl.compact(moves);
  return emit(moves, src_out, dst_out, cap);
}
int pkv_pool_migrate(pkv_pool* src, int seq, pkv_pool* dst, int* seq_out, int32_t* src_out, int32_t* dst_out, int cap) {
  if (!src || !dst || !seq_out || !src->impl.valid(seq)) return -1;
  const int pairs = int(src->impl.pages(seq).size());
  if (pairs > cap || (pairs > 0 && (!src_out || !dst_out))) return -2;  // nothing has changed
  std::vector<std::pair<int32_t, int32_t>> moves;
  const int h = pkv::PagePool::migrate(src->impl, seq, dst->impl, moves);
  if (h < 0) return -1;
  *seq_out = h;
  return emit(moves, src_out, dst_out, cap);
}

int pkv_pool_available(const pkv_pool* p) { return p ? p->impl.available() : -1; }
int pkv_pool_free_count(const pkv_pool* p) { return p ? p->impl.free_count() : -1; }
int pkv_pool_evictable_count(const pkv_pool* p) { return p ? p->impl.evictable_count() : -1; }
int pkv_pool_cached_count(const pkv_pool* p) { return p ? p->impl.cached_count() : -1; }
int pkv_pool_seq_pages(const pkv_pool* p, int seq, int32_t* out, int cap) {
  return p && p->impl.valid(seq) ? copy_out(p->impl.pages(seq), out, cap) : -1;
}
int pkv_pool_seq_slot(const pkv_pool* p, int seq) { return p && p->impl.valid(seq) ? p->impl.slot(seq) : -1; }
int pkv_pool_page_refs(const pkv_pool* p, int page) {
  return p && page >= 0 && page < p->impl.num_pages() ? p->impl.refs(page) : -1;
}
uint64_t pkv_pool_page_hash(const pkv_pool* p, int page) {
  return p && page >= 0 && page < p->impl.num_pages() ? p->impl.hash(page) : 0;
}
int pkv_pool_dirty(pkv_pool* p) { return p && p->impl.dirty() ? 1 : 0; }
const int32_t* pkv_pool_tables(pkv_pool* p) {
  if (!p) return nullptr;
  p->impl.take_dirty();
  return p->impl.tables().data();
}
int pkv_pool_free_list(const pkv_pool* p, int32_t* out, int cap) { return p ? copy_out(p->impl.free_list(), out, cap) : -1; }
int pkv_pool_evictable_list(const pkv_pool* p, int32_t* out, int cap) {
  return p ? copy_out(p->impl.evictable_list(), out, cap) : -1;
}
uint64_t pkv_page_hash(const int32_t* tokens, int page_tokens, int page_index) {
  uint64_t h = pkv::kHashSeed;
  for (int i = 0; i <= page_index; ++i) h = pkv::chain_page_hash(h, tokens + size_t(i) * size_t(page_tokens), page_tokens);
  return h;
}

}  // extern "C"
