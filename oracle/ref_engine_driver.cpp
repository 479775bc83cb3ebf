// Drives the reference's own, unmodified engine (src/engine/engine.cpp + sampler.cpp, compiled where they lie under
// the reference checkout by oracle/build_oracle.py) through a recording StepModel, and exposes what crosses the
// scheduler<->model boundary (src/engine/step.hpp:76-106) behind a C interface: every set_block_tables() call, every
// submitted chunk and state save, every finished request, and the allocator counters after each iterate(). The
// page-pool tests replay that trace into the from-scratch allocator and compare block tables entry for entry.
// TEST INFRASTRUCTURE ONLY; output goes to oracle/_ref/.
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "engine/engine.hpp"

using namespace unholy::engine;

namespace {

uint64_t mix(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  return x;
}

constexpr int kVocab = 512;

// Event log: flat int64 records, first word = kind.
//   1 nchunks {seq slot s0 n}* nsaves {slot snapshot}* nrestores {slot snapshot}*     a submitted step
//   2 table_index                                  set_block_tables (the table itself in tables[table_index])
//   3 seq                                          request finished (its pages were released)
//   4 running waiting free_pages cached_pages preemptions snapshots free_snapshots    after one iterate()
//   5 disk_snapshots snapshot_io spills disk_hits  after one iterate(), only with the disk tier (follows record 4)
struct Trace {
  std::vector<int64_t> ev;
  std::vector<std::vector<int32_t>> tables;
};

class RecordingModel final : public StepModel {
 public:
  RecordingModel(int pages, int page_tokens, int slots, int pps, int max_tokens, int snapshots, Trace& tr)
      : pages_(pages), page_(page_tokens), slots_(slots), pps_(pps), max_tokens_(max_tokens), snaps_(snapshots), tr_(tr) {}
  int vocab() const override { return kVocab; }
  int max_tokens() const override { return max_tokens_; }
  int max_logit_rows() const override { return 256; }
  int max_slots() const override { return slots_; }
  int max_pages_per_seq() const override { return pps_; }
  int num_pages() const override { return pages_; }
  int page_tokens() const override { return page_; }
  int num_snapshots() const override { return snaps_; }
  // One 4096-byte, 4096-aligned region per snapshot once give_host_snapshots() was called (the disk tier needs them).
  void give_host_snapshots() {
    snap_mem_.reset(static_cast<uint8_t*>(std::aligned_alloc(4096, size_t(snaps_ > 0 ? snaps_ : 1) * 4096)));
    std::memset(snap_mem_.get(), 0, size_t(snaps_ > 0 ? snaps_ : 1) * 4096);
  }
  void snapshot_host(int id, std::vector<std::pair<uint8_t*, size_t>>& segs) const override {
    if (snap_mem_) segs.push_back({snap_mem_.get() + size_t(id) * 4096, size_t(4096)});
  }
  void set_block_tables(const std::vector<int32_t>& t) override {
    tr_.ev.push_back(2);
    tr_.ev.push_back(int64_t(tr_.tables.size()));
    tr_.tables.push_back(t);
  }
  uint64_t submit(const StepInput& in) override {
    tr_.ev.push_back(1);
    tr_.ev.push_back(int64_t(in.chunks.size()));
    for (const Chunk& c : in.chunks) {
      tr_.ev.push_back(int64_t(c.seq));
      tr_.ev.push_back(c.slot);
      tr_.ev.push_back(c.s0);
      tr_.ev.push_back(c.n);
    }
    tr_.ev.push_back(int64_t(in.save.size()));
    for (const StateOp& s : in.save) {
      tr_.ev.push_back(s.slot);
      tr_.ev.push_back(s.snapshot);
    }
    tr_.ev.push_back(int64_t(in.restore.size()));
    for (const StateOp& s : in.restore) {
      tr_.ev.push_back(s.slot);
      tr_.ev.push_back(s.snapshot);
    }
    // A save leaves the snapshot's bytes different from whatever the slot held before (the disk tier checksums them).
    if (snap_mem_)
      for (const StateOp& s : in.save) {
        const uint64_t v = mix(++save_counter_);
        for (size_t i = 0; i < 4096; i += 8) std::memcpy(snap_mem_.get() + size_t(s.snapshot) * 4096 + i, &v, 8);
      }
    // Logits: one-hot on a token that depends only on (request, position), never EOS (id 1).
    logits_.assign(in.logit_rows.size() * size_t(kVocab), 0.0f);
    for (size_t r = 0; r < in.logit_rows.size(); ++r) {
      const int row = in.logit_rows[r];
      uint64_t seq = 0;
      for (const Chunk& c : in.chunks)
        if (row >= c.t0 && row < c.t0 + c.n) seq = c.seq;
      const int tok = 2 + int(mix(seq * 1000003ull + uint64_t(in.pos[size_t(row)])) % uint64_t(kVocab - 2));
      logits_[r * size_t(kVocab) + size_t(tok)] = 1.0f;
    }
    return ++ticket_;
  }
  void wait(uint64_t, std::vector<float>& logits) override { logits = logits_; }

 private:
  int pages_, page_, slots_, pps_, max_tokens_, snaps_;
  Trace& tr_;
  std::vector<float> logits_;
  uint64_t ticket_ = 0, save_counter_ = 0;
  struct Free {
    void operator()(uint8_t* p) const { std::free(p); }
  };
  std::unique_ptr<uint8_t, Free> snap_mem_;
};

// Disk operations under the test's control: the I/O thread's hook (EngineConfig::io_hook, src/engine/engine.hpp:131)
// holds operation number i until `released` exceeds i, so the test decides between which two iterate() calls an
// operation completes. Waits are bounded: a forgotten release delays, it does not hang.
struct Gate {
  std::atomic<long> started{0}, released{0}, tid{0};
  std::atomic<bool> in_hook{false};
  void hook() {
    in_hook = true;
    tid = long(::syscall(SYS_gettid));
    const long i = started.fetch_add(1);
    for (int spin = 0; spin < 200000 && released.load() <= i; ++spin) std::this_thread::sleep_for(std::chrono::microseconds(100));
    in_hook = false;
  }
  // Whether the I/O thread sleeps outside the hook: with nothing at the gate that is its wait for the next operation.
  bool idle() const {
    if (in_hook.load() || tid.load() == 0) return false;
    char path[64], buf[256];
    std::snprintf(path, sizeof path, "/proc/self/task/%ld/stat", tid.load());
    std::FILE* f = std::fopen(path, "r");
    if (!f) return false;
    const size_t n = std::fread(buf, 1, sizeof buf - 1, f);
    std::fclose(f);
    buf[n] = 0;
    const char* p = std::strrchr(buf, ')');  // "pid (comm) S ..."
    return p && p[1] == ' ' && p[2] == 'S';
  }
};

struct Driver {
  Trace tr;
  Gate gate;
  bool disk = false;
  std::unique_ptr<RecordingModel> model;
  std::unique_ptr<Engine> engine;
  ~Driver() {
    gate.released = 1l << 40;  // whatever still waits at the gate goes through before the engine joins its I/O thread
    engine.reset();
  }
};

}  // namespace

extern "C" {

void* refeng_create(int num_pages, int page_tokens, int max_slots, int max_pages_per_seq, int max_batch_tokens,
                    int num_snapshots) {
  auto* d = new Driver;
  d->model = std::make_unique<RecordingModel>(num_pages, page_tokens, max_slots, max_pages_per_seq, max_batch_tokens,
                                              num_snapshots, d->tr);
  EngineConfig cfg;
  cfg.max_batch_tokens = max_batch_tokens;
  cfg.prefix_cache = true;
  cfg.on_finish = [d](const RequestLog& l) {
    d->tr.ev.push_back(3);
    d->tr.ev.push_back(int64_t(l.id));
  };
  d->engine = std::make_unique<Engine>(*d->model, cfg, false);
  return d;
}

// The same engine with the snapshot disk tier on: `disk_slots` slots in `dir`/snapshots.bin, host memory for the
// snapshots, disk operations gated (refeng_io_release), and no waiting for a RAM slot by the clock (save_wait_ms = 0:
// a save that finds no slot is skipped at once), so that the trace depends on the order of calls only.
void* refeng_create_disk(int num_pages, int page_tokens, int max_slots, int max_pages_per_seq, int max_batch_tokens,
                         int num_snapshots, const char* dir, int disk_slots) {
  auto* d = new Driver;
  d->disk = true;
  d->model = std::make_unique<RecordingModel>(num_pages, page_tokens, max_slots, max_pages_per_seq, max_batch_tokens,
                                              num_snapshots, d->tr);
  d->model->give_host_snapshots();
  EngineConfig cfg;
  cfg.max_batch_tokens = max_batch_tokens;
  cfg.prefix_cache = true;
  cfg.snapshot_dir = dir;
  cfg.disk_snapshots = disk_slots;
  cfg.save_wait_ms = 0;
  cfg.io_hook = [d](bool) { d->gate.hook(); };
  cfg.on_finish = [d](const RequestLog& l) {
    d->tr.ev.push_back(3);
    d->tr.ev.push_back(int64_t(l.id));
  };
  d->engine = std::make_unique<Engine>(*d->model, cfg, false);
  return d;
}

// Lets the next n gated disk operations run and returns when they have completed. The I/O thread runs one operation
// at a time: with `more` operations queued behind them, the next one reaching the gate means they are done; with none,
// the thread going back to sleep outside the hook does (seen three times in a row, 200 us apart; 5 ms grace where
// /proc cannot tell).
void refeng_io_release(void* h, int n, int more) {
  auto* d = static_cast<Driver*>(h);
  const auto nap = [](int us) { std::this_thread::sleep_for(std::chrono::microseconds(us)); };
  const long target = d->gate.released.fetch_add(n) + n;
  for (int spin = 0; spin < 100000 && d->gate.started.load() < target; ++spin) nap(100);
  if (more) {
    for (int spin = 0; spin < 100000 && d->gate.started.load() <= target; ++spin) nap(100);
    return;
  }
  int seen = 0;
  for (int spin = 0; spin < 10000 && seen < 3; ++spin) {
    seen = d->gate.idle() ? seen + 1 : 0;
    nap(200);
  }
  if (seen < 3) nap(5000);
}

void refeng_destroy(void* h) { delete static_cast<Driver*>(h); }

uint64_t refeng_submit(void* h, const int32_t* prompt, int n, int max_tokens) {
  auto* d = static_cast<Driver*>(h);
  GenRequest r;
  r.prompt.assign(prompt, prompt + n);
  r.max_tokens = max_tokens;
  r.ignore_eos = true;
  r.sampling.temperature = 0.0f;
  return d->engine->submit(std::move(r), [](GenOutput&&) {});
}

// A prompt with image blocks (src/engine/engine.hpp:57-61): block i covers positions [starts[i], starts[i] + lens[i])
// and is named by hashes[i]; the embedding rows the engine hands to the model are zeros of width 4 (the recording
// model ignores them).
uint64_t refeng_submit_images(void* h, const int32_t* prompt, int n, int max_tokens, const int32_t* starts,
                              const int32_t* lens, const uint64_t* hashes, int nimages) {
  auto* d = static_cast<Driver*>(h);
  GenRequest r;
  r.prompt.assign(prompt, prompt + n);
  for (int i = 0; i < nimages; ++i) {
    GenImage im;
    im.start = starts[i];
    im.len = lens[i];
    im.span_start = starts[i];
    im.span_end = starts[i] + lens[i] - 1;
    im.hash = hashes[i];
    im.rows = std::make_shared<const std::vector<uint16_t>>(size_t(lens[i]) * 4, uint16_t(0));
    r.images.push_back(std::move(im));
  }
  r.max_tokens = max_tokens;
  r.ignore_eos = true;
  r.sampling.temperature = 0.0f;
  return d->engine->submit(std::move(r), [](GenOutput&&) {});
}

// Engine::abort (src/engine/engine.hpp:166): takes effect at the start of the next iterate().
void refeng_abort(void* h, uint64_t id) { static_cast<Driver*>(h)->engine->abort(id); }

int refeng_iterate(void* h) {
  auto* d = static_cast<Driver*>(h);
  const bool did = d->engine->iterate();
  const EngineStats s = d->engine->stats();
  for (int64_t v : {int64_t(4), int64_t(s.running), int64_t(s.waiting), int64_t(s.free_pages), int64_t(s.cached_pages),
                    int64_t(s.preemptions), int64_t(s.snapshots), int64_t(s.free_snapshots)})
    d->tr.ev.push_back(v);
  if (d->disk)
    for (int64_t v : {int64_t(5), int64_t(s.disk_snapshots), int64_t(s.snapshot_io), int64_t(s.spills), int64_t(s.disk_hits)})
      d->tr.ev.push_back(v);
  return did ? 1 : 0;
}

long refeng_trace_len(void* h) { return long(static_cast<Driver*>(h)->tr.ev.size()); }
void refeng_trace_copy(void* h, int64_t* out) {
  auto& ev = static_cast<Driver*>(h)->tr.ev;
  std::memcpy(out, ev.data(), ev.size() * sizeof(int64_t));
}
int refeng_num_tables(void* h) { return int(static_cast<Driver*>(h)->tr.tables.size()); }
void refeng_table_copy(void* h, int index, int32_t* out) {
  auto& t = static_cast<Driver*>(h)->tr.tables[size_t(index)];
  std::memcpy(out, t.data(), t.size() * sizeof(int32_t));
}
// The token the recording model makes the engine sample for (request, position): position p's logits give token p + 1.
int refeng_token(uint64_t seq, int pos) { return 2 + int(mix(seq * 1000003ull + uint64_t(pos)) % uint64_t(kVocab - 2)); }

}  // extern "C"
