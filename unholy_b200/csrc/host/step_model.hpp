// PkvStepModel: the reference's scheduler <-> model boundary (class StepModel, src/engine/step.hpp:76-106) implemented
// on the paged KV-cache library, so that the reference's unmodified Engine (src/engine/engine.cpp) drives the GPU path
// through set_block_tables / submit / wait exactly as it drives its resident models.
//
// What it models is the KV path alone — the scheme of the reference's own scheduler test model (FakeModel,
// tools/sched_test/main.cpp:53-260) with the store moved into HBM: the "KV row" a token writes carries the token id, a
// row pool of num_pages() x page_tokens() rows lives on the device and is addressed ONLY through the engine's block
// tables, every chunk of a step is appended by pkv_step_run, and the logits of a row are one-hot on a function of the
// WHOLE sequence gathered back through the slot's block-table row in the same launch (so a wrong page id, a stale
// table, a lost row or a page shared wrongly changes the sampled tokens). The per-slot state that is not paged (here:
// a running hash of the slot's tokens and its length) lives in a device buffer and is saved into / restored from
// pinned-host snapshots by pkv_state_copies, driven by the engine's StateOp lists — the reference's state_copies
// (src/engine/resident.hip:545-557).
//
// Header-only and never compiled into libunholy_pkv.so: it needs the reference's headers on the include path
// (-I<reference>/src) and links with libunholy_pkv.so and the CUDA runtime.
//
// Semantics kept from the reference's resident model: set_block_tables checks the size and takes effect for steps
// submitted afterwards, in-flight steps keep theirs (src/engine/resident.hip:702-707: the upload is stream-ordered);
// submit returns a ticket and enqueues; wait(ticket) must be called in submission order and at most max_inflight()
// steps may be outstanding (src/engine/step.hpp:8-11); errors are std::runtime_error.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <deque>
#include <functional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../../include/unholy_pkv.h"
#include "engine/step.hpp"

namespace unholy::kernels {

class PkvStepModel final : public engine::StepModel {
 public:
  // next_token: the model's "forward": the token that follows a sequence (the test's stand-in for real logits).
  using NextToken = std::function<int32_t(const std::vector<int32_t>&)>;
  static constexpr int kWidth = 8;  // bf16 values per stored row: 16 bytes, the token id in the first two

  PkvStepModel(int vocab, int slots, int pages_per_seq, int pages, int page_tokens, int max_tokens, int max_logit_rows, int inflight,
               int snapshots, NextToken next_token)
      : vocab_(vocab), slots_(slots), ppseq_(pages_per_seq), pages_(pages), page_(page_tokens), max_tokens_(max_tokens),
        max_rows_(max_logit_rows), inflight_(inflight), snapshots_(snapshots), next_token_(std::move(next_token)),
        kmax_(pages_per_seq * page_tokens), state_(size_t(slots)) {
    ck(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "stream");
    ck(cudaMalloc(&d_pool_, size_t(pages) * page_tokens * kWidth * 2), "row pool");
    ck(cudaMemset(d_pool_, 0xff, size_t(pages) * page_tokens * kWidth * 2), "row pool");  // not zero-initialised in the reference either
    ck(cudaMalloc(&d_tables_, size_t(slots) * pages_per_seq * 4), "tables");
    ck(cudaMemset(d_tables_, 0, size_t(slots) * pages_per_seq * 4), "tables");
    ck(cudaMalloc(&d_state_, size_t(slots) * kStateBytes), "slot state");
    ck(cudaMemset(d_state_, 0, size_t(slots) * kStateBytes), "slot state");
    if (snapshots > 0) {
      ck(cudaHostAlloc(reinterpret_cast<void**>(&snap_host_), size_t(snapshots) * kSnapBytes, cudaHostAllocMapped), "snapshots");
      std::memset(snap_host_, 0, size_t(snapshots) * kSnapBytes);
    }
    for (Step& st : ring_) {
      const size_t T = size_t(max_tokens), Q = size_t(max_logit_rows);
      ck(cudaMallocHost(reinterpret_cast<void**>(&st.h_in), in_bytes()), "step staging");
      ck(cudaMalloc(reinterpret_cast<void**>(&st.d_in), in_bytes()), "step inputs");
      ck(cudaMalloc(reinterpret_cast<void**>(&st.d_idx), Q * size_t(kmax_) * 4), "index lists");
      ck(cudaMalloc(reinterpret_cast<void**>(&st.d_out), Q * size_t(kmax_) * kWidth * 2), "gathered rows");
      ck(cudaMallocHost(reinterpret_cast<void**>(&st.h_out), Q * size_t(kmax_) * kWidth * 2), "gathered rows (host)");
      ck(cudaMallocHost(reinterpret_cast<void**>(&st.h_idx), Q * size_t(kmax_) * 4), "index lists (host)");
      ck(cudaEventCreateWithFlags(&st.done, cudaEventDisableTiming), "event");
      (void)T;
    }
  }
  ~PkvStepModel() override {
    cudaStreamSynchronize(stream_);
    for (Step& st : ring_) {
      cudaFreeHost(st.h_in);
      cudaFree(st.d_in);
      cudaFree(st.d_idx);
      cudaFree(st.d_out);
      cudaFreeHost(st.h_out);
      cudaFreeHost(st.h_idx);
      if (st.done) cudaEventDestroy(st.done);
    }
    cudaFree(d_pool_);
    cudaFree(d_tables_);
    cudaFree(d_state_);
    cudaFreeHost(snap_host_);
    cudaStreamDestroy(stream_);
  }

  int vocab() const override { return vocab_; }
  int max_tokens() const override { return max_tokens_; }
  int max_logit_rows() const override { return max_rows_; }
  int max_slots() const override { return slots_; }
  int max_pages_per_seq() const override { return ppseq_; }
  int num_pages() const override { return pages_; }
  int page_tokens() const override { return page_; }
  int max_inflight() const override { return inflight_; }
  int num_snapshots() const override { return snapshots_; }
  void snapshot_host(int id, std::vector<std::pair<uint8_t*, size_t>>& segs) const override {
    segs.emplace_back(snap_host_ + size_t(id) * kSnapBytes, kSnapBytes);
  }

  // src/engine/resident.hip:702-707: size check; the new tables are used by steps submitted from now on.
  void set_block_tables(const std::vector<int32_t>& tables) override {
    if (tables.size() != size_t(slots_) * size_t(ppseq_)) throw std::runtime_error("set_block_tables: size");
    tables_ = tables;
    tables_dirty_ = true;
  }

  uint64_t submit(const engine::StepInput& in) override {
    if (int(pending_.size()) >= inflight_) throw std::runtime_error("submit: too many steps in flight");
    const int T = int(in.ids.size()), Q = int(in.logit_rows.size());
    if (in.ids.size() != in.pos.size() || T > max_tokens_ || Q > max_rows_) throw std::runtime_error("submit: step too large");
    Step& st = ring_[size_t(next_ % kRing)];
    ck(cudaEventSynchronize(st.done), "step buffers still in use");  // (its wait() has long returned: inflight_ < kRing)
    const pkv_stream_t ps = reinterpret_cast<pkv_stream_t>(stream_);
    if (tables_dirty_) {  // stream-ordered: steps already queued keep the tables they were submitted with
      st.tables = tables_;
      ck(cudaMemcpyAsync(d_tables_, st.tables.data(), st.tables.size() * 4, cudaMemcpyHostToDevice, stream_), "tables upload");
      tables_dirty_ = false;
    }
    // restores: snapshot -> the slot's device state (pkv_state_copies), and the host mirror follows the snapshot
    const pkv_state_seg seg{d_state_, kStateBytes, 0};
    if (!in.restore.empty()) {
      std::vector<pkv_state_op> ops;
      for (const engine::StateOp& r : in.restore) ops.push_back({r.slot, r.snapshot});
      throw_rc(pkv_state_copies(&seg, 1, ops.data(), int(ops.size()), snap_host_, kSnapBytes, snapshots_, slots_, 0, ps), "restore");
      for (const engine::StateOp& r : in.restore) {
        const SlotState* sn = reinterpret_cast<const SlotState*>(snap_host_ + size_t(r.snapshot) * kSnapBytes);
        if (sn->magic != kMagic) throw std::runtime_error("submit: restore of an unsaved snapshot");
        state_[size_t(r.slot)] = *sn;
      }
    }
    // the step's rows: one 16-byte row per token, the id in its first four bytes; chunks as the engine planned them
    Layout lay = layout(st.h_in);
    std::vector<int> chunk_of_row(size_t(T), -1);
    int t = 0;
    for (size_t ci = 0; ci < in.chunks.size(); ++ci) {
      const engine::Chunk& c = in.chunks[ci];
      if (c.t0 != t || c.n <= 0 || c.slot < 0 || c.slot >= slots_) throw std::runtime_error("submit: chunk layout");
      SlotState& ss = state_[size_t(c.slot)];
      if (c.s0 != 0 && c.s0 != int(ss.len)) throw std::runtime_error("submit: a chunk does not continue its slot's sequence");
      if (c.s0 == 0) ss = SlotState{kMagic, kBasis, 0, {}};
      lay.chunks[ci] = pkv_chunk{c.slot, c.s0, c.n, c.t0};
      for (int k = 0; k < c.n; ++k) {
        const int32_t id = in.ids[size_t(t + k)];
        if (in.pos[size_t(t + k)] != c.s0 + k) throw std::runtime_error("submit: pos");
        uint16_t* row = lay.rows + size_t(t + k) * kWidth;
        std::memset(row, 0, kWidth * 2);
        std::memcpy(row, &id, 4);
        ss.hash = (ss.hash ^ uint64_t(uint32_t(id))) * 1099511628211ull;
        chunk_of_row[size_t(t + k)] = int(ci);
      }
      ss.len = uint64_t(c.s0 + c.n);
      t += c.n;
    }
    // one query row per wanted logit row: every position of its sequence up to and including the row's own
    st.q_len.assign(size_t(Q), 0);
    for (int r = 0; r < Q; ++r) {
      const int row = in.logit_rows[size_t(r)];
      if (row < 0 || row >= T || chunk_of_row[size_t(row)] < 0) throw std::runtime_error("submit: logit row outside the chunks");
      const engine::Chunk& c = in.chunks[size_t(chunk_of_row[size_t(row)])];
      const int len = c.s0 + (row - c.t0) + 1;
      lay.q_chunk[r] = chunk_of_row[size_t(row)];
      lay.q_visible[r] = len;
      st.q_len[size_t(r)] = len;
      int32_t* idx = st.h_idx + size_t(r) * size_t(kmax_);
      for (int p = 0; p < kmax_; ++p) idx[p] = p < len ? p : -1;
    }
    ck(cudaMemcpyAsync(st.d_in, st.h_in, in_bytes(), cudaMemcpyHostToDevice, stream_), "step upload");
    if (Q) ck(cudaMemcpyAsync(st.d_idx, st.h_idx, size_t(Q) * size_t(kmax_) * 4, cudaMemcpyHostToDevice, stream_), "index upload");
    if (T > 0 || Q > 0) {
      const Layout dl = layout(st.d_in);
      pkv_step step;
      std::memset(&step, 0, sizeof(step));
      step.width = step.row_stride = kWidth;
      step.rows_per_page = page_;
      step.max_pages_per_seq = ppseq_;
      step.num_pages = pages_;
      step.fp8_block = 64;
      step.nchunks = int(in.chunks.size());
      step.T = T;
      step.Q = Q;
      step.k = kmax_;
      step.max_slots = slots_;
      step.tables = d_tables_;
      step.chunks = dl.chunks;
      step.q_chunk = dl.q_chunk;
      step.q_visible = dl.q_visible;
      pkv_layer ly;
      std::memset(&ly, 0, sizeof(ly));
      ly.rows = dl.rows;
      ly.row_pool = static_cast<uint16_t*>(d_pool_);
      ly.idx = st.d_idx;
      ly.gathered = st.d_out;
      throw_rc(pkv_step_run(&step, &ly, 1, PKV_DO_ROWS | PKV_DO_GATHER | (bulk_ ? PKV_VARIANT_BULK : 0), ps), "step");
      if (Q) ck(cudaMemcpyAsync(st.h_out, st.d_out, size_t(Q) * size_t(kmax_) * kWidth * 2, cudaMemcpyDeviceToHost, stream_), "read back");
    }
    // the slots' unpaged state after the step goes to the device, then the saves copy it into their snapshots
    if (!in.save.empty()) {
      st.states = state_;
      ck(cudaMemcpyAsync(d_state_, st.states.data(), st.states.size() * kStateBytes, cudaMemcpyHostToDevice, stream_), "state upload");
      std::vector<pkv_state_op> ops;
      for (const engine::StateOp& sv : in.save) {
        if (state_[size_t(sv.slot)].len % uint64_t(page_) != 0) throw std::runtime_error("submit: save off a page boundary");
        ops.push_back({sv.slot, sv.snapshot});
      }
      throw_rc(pkv_state_copies(&seg, 1, ops.data(), int(ops.size()), snap_host_, kSnapBytes, snapshots_, slots_, 1, ps), "save");
    }
    ck(cudaEventRecord(st.done, stream_), "event");
    st.rows = Q;
    pending_.push_back(next_);
    ++steps;
    return next_++;
  }

  void wait(uint64_t ticket, std::vector<float>& logits) override {
    if (pending_.empty() || pending_.front() != ticket) throw std::runtime_error("wait: out of order");
    pending_.pop_front();
    Step& st = ring_[size_t(ticket % kRing)];
    ck(cudaEventSynchronize(st.done), "step");
    throw_rc(pkv_stream_check(reinterpret_cast<pkv_stream_t>(stream_)), "device-side check");
    logits.assign(size_t(st.rows) * size_t(vocab_), -10.0f);
    std::vector<int32_t> seq;
    for (int r = 0; r < st.rows; ++r) {
      const int len = st.q_len[size_t(r)];
      seq.resize(size_t(len));
      const uint16_t* rows = st.h_out + size_t(r) * size_t(kmax_) * kWidth;
      for (int p = 0; p < len; ++p) std::memcpy(&seq[size_t(p)], rows + size_t(p) * kWidth, 4);
      const int32_t tok = next_token_(seq);
      if (tok < 0 || tok >= vocab_) throw std::runtime_error("wait: next_token outside the vocabulary");
      logits[size_t(r) * size_t(vocab_) + size_t(tok)] = 10.0f;
    }
  }

  void use_bulk_pipeline(bool on) { bulk_ = on; }
  int steps = 0;

 private:
  static constexpr int kRing = 4;  // step buffers (more than max_inflight)
  static constexpr size_t kStateBytes = 64, kSnapBytes = 4096;
  static constexpr uint64_t kMagic = 0x504b565354415445ull, kBasis = 1469598103934665603ull;
  struct SlotState {  // a slot's unpaged state: 64 bytes on the device, 4096-byte snapshots on the host
    uint64_t magic = 0, hash = kBasis, len = 0;
    uint64_t pad[5] = {};
  };
  static_assert(sizeof(SlotState) == kStateBytes, "slot state size");
  struct Layout {  // one step's inputs in one block: rows, chunks, q_chunk, q_visible
    uint16_t* rows;
    pkv_chunk* chunks;
    int32_t *q_chunk, *q_visible;
  };
  struct Step {
    unsigned char *h_in = nullptr, *d_in = nullptr;
    int32_t *h_idx = nullptr, *d_idx = nullptr;
    uint16_t *d_out = nullptr, *h_out = nullptr;
    cudaEvent_t done = nullptr;
    std::vector<int32_t> tables;
    std::vector<SlotState> states;
    std::vector<int> q_len;
    int rows = 0;
  };
  size_t in_bytes() const {
    return size_t(max_tokens_) * kWidth * 2 + size_t(max_tokens_) * sizeof(pkv_chunk) + 2 * size_t(max_rows_) * 4;
  }
  Layout layout(unsigned char* base) const {
    Layout l;
    l.rows = reinterpret_cast<uint16_t*>(base);
    l.chunks = reinterpret_cast<pkv_chunk*>(base + size_t(max_tokens_) * kWidth * 2);
    l.q_chunk = reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(l.chunks) + size_t(max_tokens_) * sizeof(pkv_chunk));
    l.q_visible = l.q_chunk + max_rows_;
    return l;
  }
  static void ck(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("PkvStepModel: ") + what + ": " + cudaGetErrorString(e));
  }
  static void throw_rc(int rc, const char* what) {
    if (rc != PKV_OK) throw std::runtime_error(std::string("PkvStepModel: ") + what + ": " + pkv_last_error());
  }

  int vocab_, slots_, ppseq_, pages_, page_, max_tokens_, max_rows_, inflight_, snapshots_;
  NextToken next_token_;
  int kmax_;
  bool bulk_ = true;
  cudaStream_t stream_ = nullptr;
  void *d_pool_ = nullptr, *d_state_ = nullptr;
  int32_t* d_tables_ = nullptr;
  uint8_t* snap_host_ = nullptr;
  std::vector<int32_t> tables_;
  bool tables_dirty_ = false;
  std::vector<SlotState> state_;
  Step ring_[kRing];
  std::deque<uint64_t> pending_;
  uint64_t next_ = 1;
};

}  // namespace unholy::kernels
