// SnapshotStore implementation and its C ABI (pkv_snap_* in include/unholy_pkv.h). See snapshot_store.hpp for the
// contract and the reference lines each rule follows.
#include "snapshot_store.hpp"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <memory>
#include <new>

#include "../../include/unholy_pkv.h"

namespace pkv {

namespace {
uint64_t scramble(uint64_t x) {
  x ^= x >> 29;
  x *= 0x9fb21c651e98df25ull;
  x ^= x >> 32;
  x *= 0xd6e8feb86659fd93ull;
  return x ^ (x >> 31);
}
// 64 bits over a buffer, four independent lanes over 32-byte strides (what was written is checked when it is read back;
// the sum never leaves the process, so it need not be the reference's).
uint64_t checksum(const uint8_t* p, size_t n) {
  uint64_t lane[4] = {0x1d8e4e27c47d124full, 0x3c6ef372fe94f82bull, 0x5be0cd19137e2179ull, 0x7f4a7c159e3779b9ull};
  size_t i = 0;
  for (; i + 32 <= n; i += 32)
    for (int l = 0; l < 4; ++l) {
      uint64_t w;
      std::memcpy(&w, p + i + size_t(l) * 8, 8);
      lane[l] = (lane[l] + w) * 0x9e3779b97f4a7c15ull;
      lane[l] ^= lane[l] >> 29;
    }
  uint64_t t = scramble(uint64_t(n));
  for (int l = 0; l < 4; ++l) t = scramble(t ^ lane[l]);
  for (; i < n; ++i) t = scramble(t + p[i]);
  return t;
}
}  // namespace

template <class T>
void SnapshotStore::Lru<T>::push_back(std::vector<T>& v, int i) {
  T& e = v[size_t(i)];
  e.prev = tail;
  e.next = -1;
  e.in_lru = true;
  if (tail >= 0) v[size_t(tail)].next = i;
  else head = i;
  tail = i;
  ++count;
}
template <class T>
void SnapshotStore::Lru<T>::push_front(std::vector<T>& v, int i) {
  T& e = v[size_t(i)];
  e.prev = -1;
  e.next = head;
  e.in_lru = true;
  if (head >= 0) v[size_t(head)].prev = i;
  else tail = i;
  head = i;
  ++count;
}
template <class T>
void SnapshotStore::Lru<T>::unlink(std::vector<T>& v, int i) {
  T& e = v[size_t(i)];
  if (!e.in_lru) return;
  if (e.prev >= 0) v[size_t(e.prev)].next = e.next;
  else head = e.next;
  if (e.next >= 0) v[size_t(e.next)].prev = e.prev;
  else tail = e.prev;
  e.prev = e.next = -1;
  e.in_lru = false;
  --count;
}

SnapshotStore::SnapshotStore(int ram_slots, HostSegments host, Disk disk) : host_(std::move(host)), cfg_(std::move(disk)) {
  snaps_.resize(size_t(std::max(ram_slots, 0)));
  for (int s = ram_slots - 1; s >= 0; --s) free_.push_back(s);
  if (ram_slots > 0) open_file();
}

SnapshotStore::~SnapshotStore() {
  if (io_thread_.joinable()) {
    {
      std::lock_guard<std::mutex> lk(io_mu_);
      io_stop_ = true;
    }
    io_cv_.notify_all();
    io_thread_.join();
  }
  if (fd_ >= 0) {
    ::close(fd_);
    ::unlink(path_.c_str());  // disk entries do not outlive the store
  }
}

void SnapshotStore::fail_disk(const std::string& why) {
  if (!disk_on_) return;
  disk_on_ = false;
  std::fprintf(stderr, "snapshot store: disk tier off: %s\n", why.c_str());
}

// The preallocated snapshot file and the I/O thread. Any failure leaves the tier off.
void SnapshotStore::open_file() {
  if (cfg_.slots <= 0 || cfg_.dir.empty()) return;
  disk_on_ = true;
  Segments segs;
  host_(0, segs);
  size_t bytes = 0;
  bool aligned = true;
  for (const auto& s : segs) {
    bytes += s.second;
    aligned = aligned && reinterpret_cast<uintptr_t>(s.first) % 4096 == 0 && s.second % 4096 == 0;
  }
  if (bytes == 0) return fail_disk("the snapshots are not in host memory");
  slot_bytes_ = bytes;
  ::mkdir(cfg_.dir.c_str(), 0700);
  path_ = cfg_.dir + "/snapshots.bin";
  direct_ = aligned;
  fd_ = ::open(path_.c_str(), O_RDWR | O_CREAT | O_TRUNC | (direct_ ? O_DIRECT : 0), 0600);
  if (fd_ < 0 && direct_ && errno == EINVAL) {  // a filesystem without O_DIRECT (tmpfs)
    direct_ = false;
    fd_ = ::open(path_.c_str(), O_RDWR | O_CREAT | O_TRUNC, 0600);
  }
  if (fd_ < 0) return fail_disk("open " + path_ + ": " + std::strerror(errno));
  const off_t total = off_t(slot_bytes_) * cfg_.slots;
  const int e = ::posix_fallocate(fd_, 0, total);
  if (e == EOPNOTSUPP || e == EINVAL) {
    if (::ftruncate(fd_, total) != 0) return fail_disk(std::string("ftruncate: ") + std::strerror(errno));
  } else if (e != 0) {
    return fail_disk("allocating " + std::to_string(total >> 20) + " MiB in " + path_ + ": " + std::strerror(e));
  }
  disk_.assign(size_t(cfg_.slots), Slot{});
  for (int d = cfg_.slots - 1; d >= 0; --d) free_disk_.push_back(d);
  reserve_ = std::min(std::max(int(snaps_.size()) - 1, 1), 2);
  io_thread_ = std::thread([this] { io_loop(); });
}

// One operation at a time, in queue order.
void SnapshotStore::io_loop() {
  for (;;) {
    Op op;
    {
      std::unique_lock<std::mutex> lk(io_mu_);
      io_cv_.wait(lk, [&] { return io_stop_ || !io_q_.empty(); });
      if (io_stop_) return;
      op = std::move(io_q_.front());
      io_q_.pop_front();
      io_busy_ = true;
    }
    if (cfg_.io_hook) cfg_.io_hook(op.write);
    op.ok = true;
    const off_t base = off_t(op.slot) * off_t(slot_bytes_);
    off_t off = base;
    uint64_t sum = 0;
    for (const auto& seg : op.segs) {
      uint8_t* p = seg.first;
      const size_t n = seg.second;
      size_t done = 0;
      while (done < n) {
        const ssize_t r = op.write ? ::pwrite(fd_, p + done, n - done, off + off_t(done)) : ::pread(fd_, p + done, n - done, off + off_t(done));
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) {
          op.ok = false;
          op.err = std::string(op.write ? "write" : "read") + " of snapshot slot " + std::to_string(op.slot) + ": " +
                   (r < 0 ? std::strerror(errno) : "end of file");
          break;
        }
        done += size_t(r);
      }
      if (!op.ok) break;
      off += off_t(n);
      sum = scramble(sum ^ checksum(p, n));
    }
    if (!direct_) ::posix_fadvise(fd_, base, off_t(slot_bytes_), POSIX_FADV_DONTNEED);
    if (op.ok && op.write) op.sum = sum;
    if (op.ok && !op.write && sum != op.sum) {
      op.ok = false;
      op.err = "snapshot slot " + std::to_string(op.slot) + " read back differently from what was written";
    }
    {
      std::lock_guard<std::mutex> lk(io_mu_);
      io_done_.push_back(std::move(op));
      io_busy_ = false;
    }
    idle_cv_.notify_all();
  }
}

void SnapshotStore::wait_idle() {
  std::unique_lock<std::mutex> lk(io_mu_);
  idle_cv_.wait(lk, [&] { return io_q_.empty() && !io_busy_; });
}

void SnapshotStore::queue(bool write, int snap, int slot, uint64_t id, uint64_t sum) {
  Op op;
  op.write = write;
  op.snap = snap;
  op.slot = slot;
  op.id = id;
  op.sum = sum;
  host_(snap, op.segs);
  ++io_pending_;
  {
    std::lock_guard<std::mutex> lk(io_mu_);
    io_q_.push_back(std::move(op));
  }
  io_cv_.notify_one();
}

bool SnapshotStore::droppable(int id) const {
  const Snap& s = snaps_[size_t(id)];
  return s.stale || disk_by_hash_.count(s.hash) > 0;
}

void SnapshotStore::forget_name(Snap& s, int) {
  by_hash_.erase(s.hash);
  s.cached = s.stale = false;
}

SnapshotStore::Hit SnapshotStore::match(const uint64_t* page_hashes, int npages, const uint8_t* allow) {
  Hit ram, disk;
  for (int i = 0; i < npages; ++i) {
    if (allow && !allow[i]) continue;
    const uint64_t h = page_hashes[i];
    const auto it = by_hash_.find(h);
    if (it != by_hash_.end()) {
      ram = Hit{i + 1, it->second, -1, h};
    } else if (disk_on_) {
      const auto dt = disk_by_hash_.find(h);
      if (dt != disk_by_hash_.end()) disk = Hit{i + 1, -1, dt->second, h};
    }
  }
  // A disk hit deeper than the RAM ones is read into a free RAM slot (none free: the RAM hit, if any, is used).
  if (disk.pages > ram.pages && !free_.empty()) {
    disk.snap = free_.back();
    free_.pop_back();
    Snap& s = snaps_[size_t(disk.snap)];
    s.refs = 1;
    s.cached = s.stale = false;
    Slot& d = disk_[size_t(disk.disk_slot)];
    if (d.refs++ == 0) disk_lru_.unlink(disk_, disk.disk_slot);
    return disk;
  }
  if (ram.pages == 0) return Hit{};
  Snap& s = snaps_[size_t(ram.snap)];
  if (s.refs++ == 0 && !s.io) lru_.unlink(snaps_, ram.snap);  // (one being spilled is not in the list)
  s.stale = false;
  return ram;
}

uint64_t SnapshotStore::start_load(const Hit& h) {
  Snap& s = snaps_[size_t(h.snap)];
  s.io = true;
  s.hash = h.hash;
  const uint64_t id = ++load_ids_;
  queue(false, h.snap, h.disk_slot, id, disk_[size_t(h.disk_slot)].sum);
  ++totals_.disk_hits;
  return id;
}

void SnapshotStore::cancel_load(const Hit& h) {
  if (h.disk_slot >= 0) put_disk(h.disk_slot);
}

int SnapshotStore::take() {
  int id = -1;
  if (!free_.empty()) {
    id = free_.back();
    free_.pop_back();
  } else if (disk_on_) {  // only a cached snapshot that loses nothing: superseded, or already on disk
    for (int i = lru_.head; i >= 0; i = snaps_[size_t(i)].next)
      if (droppable(i)) {
        id = i;
        break;
      }
    if (id < 0) return -1;
    lru_.unlink(snaps_, id);
    forget_name(snaps_[size_t(id)], id);
  } else if (lru_.head >= 0) {
    id = lru_.head;
    lru_.unlink(snaps_, id);
    forget_name(snaps_[size_t(id)], id);
  } else {
    return -1;
  }
  snaps_[size_t(id)].refs = 1;
  return id;
}

void SnapshotStore::put(int id) {
  Snap& s = snaps_[size_t(id)];
  if (--s.refs > 0 || s.io) return;  // an I/O in flight settles it when it completes
  settle(id);
}

void SnapshotStore::settle(int id) {
  if (snaps_[size_t(id)].cached) lru_.push_back(snaps_, id);
  else free_.push_back(id);
}

void SnapshotStore::commit(int id, uint64_t hash, bool past_prompt, Rolling& rolling) {
  Snap& s = snaps_[size_t(id)];
  if (by_hash_.emplace(hash, id).second) {
    s.hash = hash;
    s.cached = true;
  }
  put(id);
  if (!s.cached || !past_prompt) return;
  if (rolling.id >= 0 && rolling.id != id) {  // the save it supersedes goes to the front of the eviction order
    const auto f = by_hash_.find(rolling.hash);
    Snap& old = snaps_[size_t(rolling.id)];
    if (f != by_hash_.end() && f->second == rolling.id && old.refs == 0 && !old.io) {
      lru_.unlink(snaps_, rolling.id);
      lru_.push_front(snaps_, rolling.id);
      old.stale = true;
    }
  }
  rolling.id = id;
  rolling.hash = hash;
}

int SnapshotStore::spare() const {
  int n = int(free_.size());
  for (int i = lru_.head; i >= 0; i = snaps_[size_t(i)].next) n += droppable(i);
  return n;
}

int SnapshotStore::take_disk_slot() {
  if (!free_disk_.empty()) {
    const int d = free_disk_.back();
    free_disk_.pop_back();
    return d;
  }
  if (disk_lru_.head >= 0) {  // (slots being read are not in the list)
    const int d = disk_lru_.head;
    disk_lru_.unlink(disk_, d);
    disk_by_hash_.erase(disk_[size_t(d)].hash);
    disk_[size_t(d)].valid = false;
    return d;
  }
  return -1;
}

void SnapshotStore::put_disk(int slot) {
  Slot& d = disk_[size_t(slot)];
  if (--d.refs == 0 && d.valid) disk_lru_.push_back(disk_, slot);
}

// Keeps `reserve_` RAM slots free: the least recently used cached snapshots are written to disk (their RAM slots go
// free when the write completes), or dropped when a later one superseded them or the disk has them already.
void SnapshotStore::spill() {
  if (!disk_on_) return;
  while (int(free_.size()) + spills_out_ < reserve_ && lru_.head >= 0) {
    const int id = lru_.head;
    Snap& s = snaps_[size_t(id)];
    const auto dt = disk_by_hash_.find(s.hash);
    if (s.stale || dt != disk_by_hash_.end()) {
      if (dt != disk_by_hash_.end() && disk_[size_t(dt->second)].refs == 0) {  // used again: so is the disk copy
        disk_lru_.unlink(disk_, dt->second);
        disk_lru_.push_back(disk_, dt->second);
      }
      lru_.unlink(snaps_, id);
      forget_name(s, id);
      free_.push_back(id);
      continue;
    }
    const int d = take_disk_slot();
    if (d < 0) break;  // every disk slot is being read
    lru_.unlink(snaps_, id);
    s.io = true;
    ++spills_out_;
    queue(true, id, d, 0, 0);
  }
}

bool SnapshotStore::poll(std::vector<Done>* out) {
  if (io_pending_ == 0) return false;
  std::deque<Op> done;
  {
    std::lock_guard<std::mutex> lk(io_mu_);
    done.swap(io_done_);
  }
  for (Op& op : done) {
    --io_pending_;
    Snap& s = snaps_[size_t(op.snap)];
    s.io = false;
    if (!op.ok) fail_disk(op.err);
    if (!op.write) {
      const uint64_t h = disk_[size_t(op.slot)].hash;
      put_disk(op.slot);
      if (op.ok) {
        s.hash = h;
        if (by_hash_.emplace(h, op.snap).second) s.cached = true;  // the RAM copy is cached too
        totals_.disk_read_bytes += slot_bytes_;
      }
      if (s.refs == 0) settle(op.snap);  // whoever wanted it is gone (else the waiting sequence holds the reference)
    } else {
      --spills_out_;
      Slot& d = disk_[size_t(op.slot)];
      const bool stored = op.ok && disk_on_ && disk_by_hash_.emplace(s.hash, op.slot).second;
      if (stored) {
        d.hash = s.hash;
        d.sum = op.sum;
        d.valid = true;
        d.refs = 0;
        disk_lru_.push_back(disk_, op.slot);
        ++totals_.spills;
        totals_.disk_write_bytes += slot_bytes_;
      } else {
        free_disk_.push_back(op.slot);
      }
      if (s.refs == 0) {  // (a request that hit it meanwhile keeps the RAM copy; it is cached again when released)
        if (stored) {
          const auto f = by_hash_.find(s.hash);
          if (f != by_hash_.end() && f->second == op.snap) by_hash_.erase(f);
          s.cached = false;
          free_.push_back(op.snap);
        } else {
          settle(op.snap);
        }
      }
    }
    if (out) out->push_back(Done{op.write, op.ok, op.id, op.snap});
  }
  return !done.empty();
}

void SnapshotStore::clear() {
  disk_by_hash_.clear();
  disk_lru_ = Lru<Slot>{};
  free_disk_.clear();
  for (size_t i = disk_.size(); i-- > 0;) {
    disk_[i] = Slot{};
    free_disk_.push_back(int(i));
  }
  by_hash_.clear();
  lru_ = Lru<Snap>{};
  free_.clear();
  for (size_t i = snaps_.size(); i-- > 0;) {
    const bool io = snaps_[i].io;
    snaps_[i] = Snap{};
    snaps_[i].io = io;  // an operation in flight still completes
    if (!io) free_.push_back(int(i));
  }
}

SnapshotStore::Counters SnapshotStore::counters() const {
  Counters c = totals_;
  c.cached = int(by_hash_.size());
  c.free_or_evictable = int(free_.size()) + lru_.count;
  c.on_disk = int(disk_by_hash_.size());
  c.io_pending = io_pending_;
  return c;
}

}  // namespace pkv

// ---------------------------------------------------------------------------------------------------------------------
// C ABI: snapshots of one contiguous host region each (snapshot id at host_base + id * snap_bytes).
// ---------------------------------------------------------------------------------------------------------------------
struct pkv_snap {
  std::unique_ptr<pkv::SnapshotStore> impl;
  void (*hook)(int, void*) = nullptr;
  void* hook_user = nullptr;
};

extern "C" {

pkv_snap* pkv_snap_create(int ram_slots, uint8_t* host_base, size_t snap_bytes, const char* dir, int disk_slots,
                          void (*io_hook)(int write, void* user), void* hook_user) {
  if (ram_slots < 0) return nullptr;
  auto* s = new (std::nothrow) pkv_snap;
  if (!s) return nullptr;
  s->hook = io_hook;
  s->hook_user = hook_user;
  pkv::SnapshotStore::Disk disk;
  if (dir && *dir && disk_slots > 0) {
    disk.dir = dir;
    disk.slots = disk_slots;
  }
  if (io_hook) disk.io_hook = [s](bool write) { s->hook(write ? 1 : 0, s->hook_user); };
  s->impl = std::make_unique<pkv::SnapshotStore>(
      ram_slots,
      [host_base, snap_bytes](int id, pkv::SnapshotStore::Segments& out) {
        if (host_base && snap_bytes) out.emplace_back(host_base + size_t(id) * snap_bytes, snap_bytes);
      },
      std::move(disk));
  return s;
}
void pkv_snap_destroy(pkv_snap* s) { delete s; }
int pkv_snap_disk_on(const pkv_snap* s) { return s && s->impl->disk_on() ? 1 : 0; }
int pkv_snap_match(pkv_snap* s, const uint64_t* page_hashes, int npages, const uint8_t* allow, pkv_snap_hit* hit_out) {
  if (!s || !hit_out || npages < 0 || (npages > 0 && !page_hashes)) return PKV_ERR_ARG;
  const pkv::SnapshotStore::Hit h = s->impl->match(page_hashes, npages, allow);
  *hit_out = pkv_snap_hit{h.pages, h.snap, h.disk_slot, 0, h.hash};
  return PKV_OK;
}
uint64_t pkv_snap_start_load(pkv_snap* s, const pkv_snap_hit* hit) {
  if (!s || !hit || hit->disk_slot < 0 || hit->snap < 0) return 0;
  return s->impl->start_load(pkv::SnapshotStore::Hit{hit->pages, hit->snap, hit->disk_slot, hit->hash});
}
void pkv_snap_cancel_load(pkv_snap* s, const pkv_snap_hit* hit) {
  if (s && hit) s->impl->cancel_load(pkv::SnapshotStore::Hit{hit->pages, hit->snap, hit->disk_slot, hit->hash});
}
int pkv_snap_take(pkv_snap* s) { return s ? s->impl->take() : -1; }
void pkv_snap_put(pkv_snap* s, int id) {
  if (s && id >= 0) s->impl->put(id);
}
void pkv_snap_commit(pkv_snap* s, int id, uint64_t hash, int past_prompt, int* rolling_id, uint64_t* rolling_hash) {
  if (!s || id < 0 || !rolling_id || !rolling_hash) return;
  pkv::SnapshotStore::Rolling r{*rolling_id, *rolling_hash};
  s->impl->commit(id, hash, past_prompt != 0, r);
  *rolling_id = r.id;
  *rolling_hash = r.hash;
}
int pkv_snap_spare(const pkv_snap* s) { return s ? s->impl->spare() : -1; }
void pkv_snap_spill(pkv_snap* s) {
  if (s) s->impl->spill();
}
int pkv_snap_poll(pkv_snap* s, pkv_snap_done* done_out, int cap) {
  if (!s) return -1;
  std::vector<pkv::SnapshotStore::Done> done;
  s->impl->poll(&done);
  for (int i = 0; done_out && i < int(done.size()) && i < cap; ++i)
    done_out[i] = pkv_snap_done{done[size_t(i)].write ? 1 : 0, done[size_t(i)].ok ? 1 : 0, done[size_t(i)].snap, 0, done[size_t(i)].load_id};
  return int(done.size());
}
void pkv_snap_clear(pkv_snap* s) {
  if (s) s->impl->clear();
}
void pkv_snap_wait_idle(pkv_snap* s) {
  if (s) s->impl->wait_idle();
}
int pkv_snap_counters(const pkv_snap* s, pkv_snap_counters_t* out) {
  if (!s || !out) return PKV_ERR_ARG;
  const pkv::SnapshotStore::Counters c = s->impl->counters();
  *out = pkv_snap_counters_t{c.cached, c.free_or_evictable, c.on_disk, c.io_pending, c.spills, c.disk_hits, c.disk_read_bytes, c.disk_write_bytes};
  return PKV_OK;
}

}  // extern "C"
