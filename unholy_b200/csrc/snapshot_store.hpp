// Bookkeeping of slot-state snapshots and their disk tier: which snapshot slot a save goes into, which one a prefix hit
// restores, what is evicted when, what is written to the snapshot file and read back. The copies between a slot's
// device state and a snapshot are pkv_state_copies; this is the storage side around them. Host only.
//
// Observable behaviour (which snapshot id is handed out when, what a prefix hit finds, what the counters say) follows
// ewtodd/unholy's engine: src/engine/engine.cpp:87-92 (free list descending, so snapshot 0 is taken first), :284-336
// (the deepest boundary with a RAM snapshot, or a deeper one that only the disk has when a RAM slot is free), :361-397
// (take / put / settle; with the disk tier only a snapshot that loses nothing is taken over), :949-970 (commit; a
// decoding sequence's previous snapshot goes to the front of the eviction order, marked stale), :1018-1058 (the
// preallocated O_DIRECT file), :1061-1109 (the I/O thread: one operation at a time, a 64-bit checksum of what was
// written is checked on read), :1139-1187 (disk slots: free list, then least recently used; spilling keeps a reserve
// of RAM slots free), :1190-1261 (completions), :1011-1015 (any I/O error turns the tier off, once). The data
// structures are this library's own (index-linked lists over flat arrays).
//
// Single-threaded like the engine thread that owns the reference's bookkeeping, plus one I/O thread owned by the store.
#pragma once

#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <utility>
#include <vector>

namespace pkv {

class SnapshotStore {
 public:
  using Segments = std::vector<std::pair<uint8_t*, size_t>>;
  // The host memory of snapshot `id`, in a fixed order (StepModel::snapshot_host, src/engine/step.hpp:88-90).
  using HostSegments = std::function<void(int id, Segments& out)>;
  struct Disk {
    std::string dir;  // empty or slots <= 0: no disk tier
    int slots = 0;
    std::function<void(bool write)> io_hook;  // tests: runs on the I/O thread before each operation
  };
  struct Rolling {  // per sequence: the snapshot its decoding saved last (superseded by the next)
    int id = -1;
    uint64_t hash = 0;
  };
  struct Hit {
    int pages = 0;        // the prefix covers this many full pages (0: no hit)
    int snap = -1;        // RAM snapshot to restore (referenced by the caller from now on)
    int disk_slot = -1;   // >= 0: `snap` is an empty RAM slot that start_load() must fill from this disk slot first
    uint64_t hash = 0;    // name of the boundary
  };
  struct Done {  // a finished disk operation
    bool write = false, ok = false;
    uint64_t load_id = 0;  // reads: what start_load returned
    int snap = -1;
  };
  struct Counters {
    int cached = 0, free_or_evictable = 0, on_disk = 0, io_pending = 0;
    uint64_t spills = 0, disk_hits = 0, disk_read_bytes = 0, disk_write_bytes = 0;
  };

  SnapshotStore(int ram_slots, HostSegments host, Disk disk);
  ~SnapshotStore();
  SnapshotStore(const SnapshotStore&) = delete;
  SnapshotStore& operator=(const SnapshotStore&) = delete;

  bool disk_on() const { return disk_on_; }
  // page_hashes[i] names the boundary at the end of page i; allow[i] == 0 (allow may be null) rules a boundary out.
  Hit match(const uint64_t* page_hashes, int npages, const uint8_t* allow);
  uint64_t start_load(const Hit& h);  // queues the read of h.disk_slot into h.snap; the caller waits for its Done
  void cancel_load(const Hit& h);     // a disk hit that is given up before start_load (the RAM slot goes back with put)
  int take();                         // a slot for a save, or -1
  void put(int id);                   // drops one reference
  void commit(int id, uint64_t hash, bool past_prompt, Rolling& rolling);  // a save into `id` has completed
  int spare() const;                  // slots a save at a prompt's last boundary may take without losing a prefix
  void spill();
  bool poll(std::vector<Done>* out);  // handles finished disk operations; true if there were any
  void clear();                       // forgets everything (after a failed step the contents are unknown)
  Counters counters() const;
  void wait_idle();                   // tests: returns once the I/O thread has nothing queued or running

 private:
  struct Snap {
    uint64_t hash = 0;
    int refs = 0;
    bool cached = false, io = false, stale = false, in_lru = false;
    int prev = -1, next = -1;
  };
  struct Slot {  // a slot of the snapshot file
    uint64_t hash = 0, sum = 0;
    int refs = 0;
    bool valid = false, in_lru = false;
    int prev = -1, next = -1;
  };
  struct Op {
    bool write = false;
    int snap = 0, slot = 0;
    uint64_t id = 0, sum = 0;
    Segments segs;
    bool ok = false;
    std::string err;
  };
  template <class T>
  struct Lru {  // doubly linked by index through the elements' prev / next
    int head = -1, tail = -1, count = 0;
    void push_back(std::vector<T>& v, int i);
    void push_front(std::vector<T>& v, int i);
    void unlink(std::vector<T>& v, int i);
  };
  bool droppable(int id) const;
  void settle(int id);
  void forget_name(Snap& s, int id);
  int take_disk_slot();
  void put_disk(int slot);
  void queue(bool write, int snap, int slot, uint64_t id, uint64_t sum);
  void fail_disk(const std::string& why);
  void open_file();
  void io_loop();

  HostSegments host_;
  Disk cfg_;
  std::vector<Snap> snaps_;
  std::vector<int> free_;
  Lru<Snap> lru_;
  std::unordered_map<uint64_t, int> by_hash_;
  // disk tier
  bool disk_on_ = false, direct_ = false;
  int fd_ = -1, reserve_ = 1, spills_out_ = 0, io_pending_ = 0;
  size_t slot_bytes_ = 0;
  std::string path_;
  std::vector<Slot> disk_;
  std::vector<int> free_disk_;
  Lru<Slot> disk_lru_;
  std::unordered_map<uint64_t, int> disk_by_hash_;
  uint64_t load_ids_ = 0;
  Counters totals_;
  std::thread io_thread_;
  std::mutex io_mu_;
  std::condition_variable io_cv_, idle_cv_;
  std::deque<Op> io_q_, io_done_;
  bool io_stop_ = false, io_busy_ = false;
};

}  // namespace pkv
