// The page pool sharded over the GPUs of one box by request ownership, and page migration between shards, as a C++
// host behind the C ABI (pkv_shards_* in include/unholy_pkv.h). One process, one host thread and one step stream per
// shard; a request's pages, block-table row and allocator state live on its owner, so a step needs no exchange between
// GPUs. The only inter-GPU operation is migration: the destination shard takes pages from its own allocator and pulls
// the payload of every layer with pkv_copy_pages on a migration stream of its own, reading the source's pools with plain
// 16-byte loads through peer access (no bulk/TMA copy ever reads peer memory here), while both shards go on stepping
// their other requests. Ordering is by CUDA events: the pull waits for the source's queued steps, the destination's
// next step waits for the pull, and the host releases the source's pages only after the pull's event has completed.
// Nothing on the device spins on a flag.
//
// ewtodd/unholy has no sharded pool and pages never move between its cards (the design notes at the root of its
// repository, lines 119-123 and 148-149): parity for this file is unpinned. The nearest pattern in the reference is the pull-kernel + event ordering of
// src/engine/resident.hip:213-232,908-910. The bookkeeping underneath is the pinned allocator (page_pool.hpp).
#include <cuda_runtime.h>

#include <algorithm>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/unholy_pkv.h"
#include "page_pool.hpp"
#include "pkv_internal.hpp"

namespace {

struct DeviceGuard {  // the calling thread's current device is restored on scope exit
  int saved = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&saved);
    cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    if (saved >= 0) cudaSetDevice(saved);
  }
};

// One host thread that runs the tasks posted to it in order (a shard's launches are issued by its own thread, so the
// shards' host work runs in parallel).
class Worker {
 public:
  Worker() : th_([this] { loop(); }) {}
  ~Worker() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    th_.join();
  }
  void post(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      task_ = std::move(fn);
      busy_ = true;
    }
    cv_.notify_all();
  }
  void wait() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [this] { return !busy_; });
  }

 private:
  void loop() {
    for (;;) {
      std::function<void()> fn;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stop_ || task_; });
        if (stop_ && !task_) return;
        fn = std::move(task_);
        task_ = nullptr;
      }
      fn();
      {
        std::lock_guard<std::mutex> lk(mu_);
        busy_ = false;
      }
      cv_.notify_all();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::function<void()> task_;
  bool busy_ = false, stop_ = false;
  std::thread th_;
};

struct Request {
  int shard = -1, seq = -1, length = 0;
  bool active = false;  // takes part in its shard's steps (false while it migrates)
};

constexpr int kStaging = 3;  // pinned staging sets per shard: a set is reused only after its upload has run

struct Shard {
  int device = 0;
  std::unique_ptr<pkv::PagePool> pool;
  std::vector<void*> row_pools, key_pools;  // per layer
  int32_t* d_tables = nullptr;
  // per-step descriptors: chunks [max_slots], q_chunk [max_slots], q_visible [max_slots]
  pkv_chunk* d_chunks = nullptr;
  int32_t *d_qchunk = nullptr, *d_qvis = nullptr;
  struct Staging {
    int32_t* tables = nullptr;
    pkv_chunk* chunks = nullptr;
    int32_t *qchunk = nullptr, *qvis = nullptr;
    cudaEvent_t used = nullptr;
  } staging[kStaging];
  int turn = 0;
  cudaStream_t step_stream = nullptr, mig_stream = nullptr;
  cudaEvent_t mark[2] = {nullptr, nullptr};
  std::unique_ptr<Worker> worker;
  std::string error;
  int rc = PKV_OK;
  // The step's launches, captured once per (number of local requests, io pointers) and replayed: the launch parameters
  // do not change from step to step (positions and block tables are read from device buffers that are refreshed by
  // stream-ordered uploads in front of every replay).
  cudaGraphExec_t graph = nullptr;
  std::vector<const void*> graph_key;
};

struct Migration {
  int request, src, dst, new_seq;
  size_t bytes;
  int32_t *h_ids = nullptr, *d_ids = nullptr;  // [2 * npages]: source ids then destination ids
  cudaEvent_t src_ready = nullptr, start = nullptr, done = nullptr;
};

}  // namespace

struct pkv_shards {
  pkv_shard_config cfg;
  std::vector<Shard> shards;
  std::map<int, Request> requests;
  std::vector<Migration> pending;
  bool use_graphs = true;  // PKV_SHARD_GRAPH=0: issue the launches of every step directly
  double migrated_bytes = 0;
  std::vector<float> mig_kernel_ms;  // per destination shard, summed over completed pulls
};

namespace {

int fail(int code, const std::string& msg) {
  pkv_g_err = msg;
  return code;
}
int fail_cuda(const char* what, cudaError_t e) { return fail(PKV_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e)); }

#define SH_CUDA(call)                                        \
  do {                                                       \
    const cudaError_t e_ = (call);                           \
    if (e_ != cudaSuccess) return fail_cuda(#call, e_);      \
  } while (0)

size_t row_page_bytes(const pkv_shard_config& c) { return size_t(c.rows_per_page) * size_t(c.row_stride) * 2u; }
size_t key_page_bytes(const pkv_shard_config& c) { return size_t(c.rows_per_page) * 68u; }

std::vector<int> local_requests(const pkv_shards& S, int shard) {
  std::vector<int> out;
  for (const auto& kv : S.requests)  // std::map: ascending request id
    if (kv.second.shard == shard && kv.second.active) out.push_back(kv.first);
  return out;
}

int upload_tables(pkv_shards& S, Shard& sh, Shard::Staging& st) {
  const size_t n = size_t(S.cfg.max_slots) * size_t(S.cfg.max_pages_per_seq);
  sh.pool->take_dirty();
  std::memcpy(st.tables, sh.pool->tables().data(), n * sizeof(int32_t));
  SH_CUDA(cudaMemcpyAsync(sh.d_tables, st.tables, n * sizeof(int32_t), cudaMemcpyHostToDevice, sh.step_stream));
  return PKV_OK;
}

// One decode step of a shard, issued by the shard's own thread.
int shard_step(pkv_shards& S, int g, const pkv_shard_io* io) {
  Shard& sh = S.shards[size_t(g)];
  SH_CUDA(cudaSetDevice(sh.device));
  const std::vector<int> order = local_requests(S, g);
  const int Q = int(order.size());
  if (Q == 0) return PKV_OK;
  if (Q > S.cfg.max_slots) return fail(PKV_ERR_LIMIT, "pkv_shards_step: more local requests than slots");
  for (const int r : order) {  // positions advance: a new page now and then (alloc_pages, src/engine/engine.cpp:437-444)
    Request& rq = S.requests.at(r);
    if (!sh.pool->alloc(rq.seq, rq.length + 1)) return fail(PKV_ERR_LIMIT, "pkv_shards_step: a shard's pool is full");
  }
  Shard::Staging& st = sh.staging[sh.turn];
  sh.turn = (sh.turn + 1) % kStaging;
  SH_CUDA(cudaEventSynchronize(st.used));  // the upload that last read this staging set has run
  if (sh.pool->dirty())
    if (const int rc = upload_tables(S, sh, st)) return rc;
  for (int i = 0; i < Q; ++i) {
    const Request& rq = S.requests.at(order[size_t(i)]);
    st.chunks[i] = pkv_chunk{sh.pool->slot(rq.seq), rq.length, 1, i};
    st.qchunk[i] = i;
    st.qvis[i] = rq.length + 1;
  }
  // chunks, q_chunk and q_visible lie in one block on both sides: one upload per step
  SH_CUDA(cudaMemcpyAsync(sh.d_chunks, st.chunks, size_t(S.cfg.max_slots) * (sizeof(pkv_chunk) + 2 * sizeof(int32_t)), cudaMemcpyHostToDevice,
                          sh.step_stream));
  SH_CUDA(cudaEventRecord(st.used, sh.step_stream));
  pkv_step step;
  std::memset(&step, 0, sizeof(step));
  step.width = S.cfg.width;
  step.row_stride = S.cfg.row_stride;
  step.rows_per_page = S.cfg.rows_per_page;
  step.max_pages_per_seq = S.cfg.max_pages_per_seq;
  step.num_pages = S.cfg.num_pages;
  step.fp8_block = 64;
  step.nchunks = step.T = step.Q = Q;
  step.k = S.cfg.k;
  step.max_slots = S.cfg.max_slots;
  step.tables = sh.d_tables;
  step.chunks = sh.d_chunks;
  step.q_chunk = sh.d_qchunk;
  step.q_visible = sh.d_qvis;
  std::vector<const void*> key{reinterpret_cast<const void*>(size_t(Q))};
  for (int l = 0; l < S.cfg.layers; ++l) {
    const pkv_shard_io& x = io[size_t(g) * size_t(S.cfg.layers) + size_t(l)];
    key.insert(key.end(), {x.rows, x.keys, x.idx, x.gathered});
  }
  const bool use_graph = S.use_graphs;
  if (use_graph && sh.graph && key == sh.graph_key) {
    SH_CUDA(cudaGraphLaunch(sh.graph, sh.step_stream));
    for (const int r : order) ++S.requests.at(r).length;
    return PKV_OK;
  }
  if (use_graph) {
    if (sh.graph) cudaGraphExecDestroy(sh.graph);
    sh.graph = nullptr;
    SH_CUDA(cudaStreamBeginCapture(sh.step_stream, cudaStreamCaptureModeThreadLocal));
  }
  int launch_rc = PKV_OK;
  for (int l = 0; l < S.cfg.layers && launch_rc == PKV_OK; ++l) {
    const pkv_shard_io& x = io[size_t(g) * size_t(S.cfg.layers) + size_t(l)];
    pkv_layer ly;
    std::memset(&ly, 0, sizeof(ly));
    ly.rows = x.rows;
    ly.row_pool = static_cast<uint16_t*>(sh.row_pools[size_t(l)]);
    ly.keys = x.keys;
    ly.key_pool_fp4 = x.keys && S.cfg.key_pools ? static_cast<uint8_t*>(sh.key_pools[size_t(l)]) : nullptr;
    ly.idx = x.idx;
    ly.gathered = x.gathered;
    const int flags = PKV_DO_ROWS | PKV_DO_GATHER | PKV_VARIANT_BULK | (ly.key_pool_fp4 ? PKV_DO_KEYS_FP4 : 0);
    launch_rc = pkv_step_run(&step, &ly, 1, flags, reinterpret_cast<pkv_stream_t>(sh.step_stream));
  }
  if (use_graph) {
    cudaGraph_t captured = nullptr;
    const cudaError_t e = cudaStreamEndCapture(sh.step_stream, &captured);  // (always ends the capture, also after a failed launch)
    if (launch_rc != PKV_OK) {
      if (captured) cudaGraphDestroy(captured);
      return launch_rc;
    }
    if (e != cudaSuccess) return fail_cuda("cudaStreamEndCapture", e);
    const cudaError_t ie = cudaGraphInstantiate(&sh.graph, captured, 0);
    cudaGraphDestroy(captured);
    if (ie != cudaSuccess) return fail_cuda("cudaGraphInstantiate", ie);
    sh.graph_key = key;
    SH_CUDA(cudaGraphLaunch(sh.graph, sh.step_stream));
  } else if (launch_rc != PKV_OK) {
    return launch_rc;
  }
  for (const int r : order) ++S.requests.at(r).length;
  return PKV_OK;
}

void free_shard(Shard& sh) {
  cudaSetDevice(sh.device);
  for (void* p : sh.row_pools) cudaFree(p);
  for (void* p : sh.key_pools) cudaFree(p);
  cudaFree(sh.d_tables);
  cudaFree(sh.d_chunks);
  for (auto& st : sh.staging) {
    cudaFreeHost(st.tables);
    cudaFreeHost(st.chunks);
    if (st.used) cudaEventDestroy(st.used);
  }
  if (sh.graph) cudaGraphExecDestroy(sh.graph);
  if (sh.step_stream) cudaStreamDestroy(sh.step_stream);
  if (sh.mig_stream) cudaStreamDestroy(sh.mig_stream);
  for (auto& e : sh.mark)
    if (e) cudaEventDestroy(e);
}

int init_shard(pkv_shards& S, Shard& sh) {
  const pkv_shard_config& c = S.cfg;
  SH_CUDA(cudaSetDevice(sh.device));
  sh.pool = std::make_unique<pkv::PagePool>(c.num_pages, c.rows_per_page, c.max_slots, c.max_pages_per_seq, false);
  for (int l = 0; l < c.layers; ++l) {
    void* p = nullptr;
    SH_CUDA(cudaMalloc(&p, size_t(c.num_pages) * row_page_bytes(c)));
    sh.row_pools.push_back(p);
    if (c.key_pools) {
      SH_CUDA(cudaMalloc(&p, size_t(c.num_pages) * key_page_bytes(c)));
      sh.key_pools.push_back(p);
    }
  }
  const size_t tn = size_t(c.max_slots) * size_t(c.max_pages_per_seq);
  SH_CUDA(cudaMalloc(reinterpret_cast<void**>(&sh.d_tables), tn * sizeof(int32_t)));
  SH_CUDA(cudaMemset(sh.d_tables, 0, tn * sizeof(int32_t)));
  const size_t desc_bytes = size_t(c.max_slots) * (sizeof(pkv_chunk) + 2 * sizeof(int32_t));
  SH_CUDA(cudaMalloc(reinterpret_cast<void**>(&sh.d_chunks), desc_bytes));
  sh.d_qchunk = reinterpret_cast<int32_t*>(sh.d_chunks + c.max_slots);
  sh.d_qvis = sh.d_qchunk + c.max_slots;
  for (auto& st : sh.staging) {
    SH_CUDA(cudaMallocHost(reinterpret_cast<void**>(&st.tables), tn * sizeof(int32_t)));
    SH_CUDA(cudaMallocHost(reinterpret_cast<void**>(&st.chunks), desc_bytes));
    st.qchunk = reinterpret_cast<int32_t*>(st.chunks + c.max_slots);
    st.qvis = st.qchunk + c.max_slots;
    SH_CUDA(cudaEventCreateWithFlags(&st.used, cudaEventDisableTiming));
  }
  SH_CUDA(cudaStreamCreateWithFlags(&sh.step_stream, cudaStreamNonBlocking));
  SH_CUDA(cudaStreamCreateWithFlags(&sh.mig_stream, cudaStreamNonBlocking));
  for (auto& e : sh.mark) SH_CUDA(cudaEventCreate(&e));
  sh.worker = std::make_unique<Worker>();
  return PKV_OK;
}

}  // namespace

extern "C" {

pkv_shards* pkv_shards_create(const pkv_shard_config* cfg, const int* devices) {
  if (!cfg || !devices || cfg->ngpus <= 0 || cfg->ngpus > 64 || cfg->num_pages <= 0 || cfg->rows_per_page <= 0 || cfg->width <= 0 ||
      cfg->width % 8 != 0 || cfg->row_stride < cfg->width || cfg->row_stride % 8 != 0 || cfg->layers <= 0 ||
      cfg->layers * (cfg->key_pools ? 2 : 1) > 128 || cfg->max_slots <= 0 || cfg->max_pages_per_seq <= 0 || cfg->k < 0) {
    fail(PKV_ERR_ARG, "pkv_shards_create: bad configuration (at most 128 pools move in one migration launch)");
    return nullptr;
  }
  int saved = -1;
  cudaGetDevice(&saved);
  auto S = std::make_unique<pkv_shards>();
  S->cfg = *cfg;
  if (const char* v = std::getenv("PKV_SHARD_GRAPH")) S->use_graphs = std::atoi(v) != 0;
  S->shards.resize(size_t(cfg->ngpus));
  S->mig_kernel_ms.assign(size_t(cfg->ngpus), 0.0f);
  bool ok = true;
  for (int g = 0; g < cfg->ngpus && ok; ++g) {
    S->shards[size_t(g)].device = devices[g];
    ok = init_shard(*S, S->shards[size_t(g)]) == PKV_OK;
  }
  // Peer access, once, between every pair of distinct devices (the pull kernel reads a peer's pool directly).
  for (int a = 0; a < cfg->ngpus && ok; ++a)
    for (int b = 0; b < cfg->ngpus && ok; ++b) {
      const int da = devices[a], db = devices[b];
      if (da == db) continue;
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, da, db) != cudaSuccess || !can) {
        fail(PKV_ERR_CUDA, "pkv_shards_create: device " + std::to_string(da) + " cannot access device " + std::to_string(db));
        ok = false;
        break;
      }
      cudaSetDevice(da);
      const cudaError_t e = cudaDeviceEnablePeerAccess(db, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (e != cudaSuccess) {
        fail_cuda("cudaDeviceEnablePeerAccess", e);
        ok = false;
      }
    }
  if (!ok) {
    for (auto& sh : S->shards) free_shard(sh);
    S.reset();
  }
  if (saved >= 0) cudaSetDevice(saved);
  return S.release();
}

void pkv_shards_destroy(pkv_shards* S) {
  if (!S) return;
  int saved = -1;
  cudaGetDevice(&saved);
  for (auto& sh : S->shards) {
    cudaSetDevice(sh.device);
    cudaDeviceSynchronize();
  }
  for (auto& m : S->pending) {
    cudaFreeHost(m.h_ids);
    cudaSetDevice(S->shards[size_t(m.dst)].device);
    cudaFree(m.d_ids);
    for (cudaEvent_t e : {m.src_ready, m.start, m.done})
      if (e) cudaEventDestroy(e);
  }
  for (auto& sh : S->shards) {
    sh.worker.reset();
    free_shard(sh);
  }
  if (saved >= 0) cudaSetDevice(saved);
  delete S;
}

int pkv_shards_add(pkv_shards* S, int request, int shard, int length) {
  if (!S || shard < 0 || shard >= S->cfg.ngpus || length < 0) return fail(PKV_ERR_ARG, "pkv_shards_add: bad argument");
  if (S->requests.count(request)) return fail(PKV_ERR_ARG, "pkv_shards_add: the request exists");
  pkv::PagePool& pool = *S->shards[size_t(shard)].pool;
  const int seq = pool.open();
  if (pool.assign_slot(seq) < 0 || !pool.alloc(seq, length)) {
    pool.close(seq);
    return fail(PKV_ERR_LIMIT, "pkv_shards_add: the shard has no slot or not enough pages");
  }
  S->requests[request] = Request{shard, seq, length, true};
  return PKV_OK;
}

int pkv_shards_remove(pkv_shards* S, int request) {
  if (!S || !S->requests.count(request)) return fail(PKV_ERR_ARG, "pkv_shards_remove: unknown request");
  const Request rq = S->requests[request];
  if (!rq.active) return fail(PKV_ERR_ARG, "pkv_shards_remove: the request is migrating");
  S->shards[size_t(rq.shard)].pool->close(rq.seq);
  S->requests.erase(request);
  return PKV_OK;
}

int pkv_shards_owner(const pkv_shards* S, int request) {
  if (!S) return -1;
  const auto it = S->requests.find(request);
  return it != S->requests.end() ? it->second.shard : -1;
}
int pkv_shards_length(const pkv_shards* S, int request) {
  if (!S) return -1;
  const auto it = S->requests.find(request);
  return it != S->requests.end() ? it->second.length : -1;
}
int pkv_shards_slot(const pkv_shards* S, int request) {
  if (!S) return -1;
  const auto it = S->requests.find(request);
  return it != S->requests.end() ? S->shards[size_t(it->second.shard)].pool->slot(it->second.seq) : -1;
}
int pkv_shards_local(const pkv_shards* S, int shard, int32_t* requests_out, int cap) {
  if (!S || shard < 0 || shard >= S->cfg.ngpus) return -1;
  const std::vector<int> v = local_requests(*S, shard);
  for (int i = 0; requests_out && i < int(v.size()) && i < cap; ++i) requests_out[i] = v[size_t(i)];
  return int(v.size());
}
int pkv_shards_free_pages(const pkv_shards* S, int shard) {
  return S && shard >= 0 && shard < S->cfg.ngpus ? S->shards[size_t(shard)].pool->available() : -1;
}
void* pkv_shards_row_pool(pkv_shards* S, int shard, int layer) {
  if (!S || shard < 0 || shard >= S->cfg.ngpus || layer < 0 || layer >= S->cfg.layers) return nullptr;
  return S->shards[size_t(shard)].row_pools[size_t(layer)];
}
void* pkv_shards_key_pool(pkv_shards* S, int shard, int layer) {
  if (!S || !S->cfg.key_pools || shard < 0 || shard >= S->cfg.ngpus || layer < 0 || layer >= S->cfg.layers) return nullptr;
  return S->shards[size_t(shard)].key_pools[size_t(layer)];
}
void* pkv_shards_stream(pkv_shards* S, int shard) {
  return S && shard >= 0 && shard < S->cfg.ngpus ? S->shards[size_t(shard)].step_stream : nullptr;
}

const int32_t* pkv_shards_tables(pkv_shards* S, int shard) {
  if (!S || shard < 0 || shard >= S->cfg.ngpus) return nullptr;
  Shard& sh = S->shards[size_t(shard)];
  DeviceGuard dg(sh.device);
  if (sh.pool->dirty()) {
    Shard::Staging& st = sh.staging[sh.turn];
    sh.turn = (sh.turn + 1) % kStaging;
    if (cudaEventSynchronize(st.used) != cudaSuccess || upload_tables(*S, sh, st) != PKV_OK ||
        cudaEventRecord(st.used, sh.step_stream) != cudaSuccess)
      return nullptr;
  }
  return sh.d_tables;
}

int pkv_shards_step(pkv_shards* S, const pkv_shard_io* io) {
  if (!S || !io) return fail(PKV_ERR_ARG, "pkv_shards_step: null argument");
  for (int g = 0; g < S->cfg.ngpus; ++g) {
    Shard& sh = S->shards[size_t(g)];
    sh.worker->post([S, g, io, &sh] {
      sh.rc = shard_step(*S, g, io);
      if (sh.rc != PKV_OK) sh.error = pkv_g_err;  // (the worker thread's message)
    });
  }
  int rc = PKV_OK;
  for (auto& sh : S->shards) {
    sh.worker->wait();
    if (sh.rc != PKV_OK && rc == PKV_OK) rc = fail(sh.rc, sh.error);
  }
  return rc;
}

int pkv_shards_mark(pkv_shards* S, int which) {
  if (!S || which < 0 || which > 1) return fail(PKV_ERR_ARG, "pkv_shards_mark: bad argument");
  for (auto& sh : S->shards) {
    DeviceGuard dg(sh.device);
    SH_CUDA(cudaEventRecord(sh.mark[which], sh.step_stream));
  }
  return PKV_OK;
}

int pkv_shards_elapsed_ms(pkv_shards* S, float* ms_out) {
  if (!S || !ms_out) return fail(PKV_ERR_ARG, "pkv_shards_elapsed_ms: null argument");
  for (size_t g = 0; g < S->shards.size(); ++g) {
    Shard& sh = S->shards[g];
    DeviceGuard dg(sh.device);
    SH_CUDA(cudaEventSynchronize(sh.mark[1]));
    SH_CUDA(cudaEventElapsedTime(&ms_out[g], sh.mark[0], sh.mark[1]));
  }
  return PKV_OK;
}

int pkv_shards_sync(pkv_shards* S) {
  if (!S) return fail(PKV_ERR_ARG, "pkv_shards_sync: null argument");
  for (auto& sh : S->shards) {
    DeviceGuard dg(sh.device);
    SH_CUDA(cudaStreamSynchronize(sh.step_stream));
    SH_CUDA(cudaStreamSynchronize(sh.mig_stream));
  }
  return PKV_OK;
}

int pkv_shards_migrate_begin(pkv_shards* S, const int32_t* requests, const int32_t* dst_shards, int n) {
  if (!S || n < 0 || (n > 0 && (!requests || !dst_shards))) return fail(PKV_ERR_ARG, "pkv_shards_migrate_begin: bad argument");
  const pkv_shard_config& c = S->cfg;
  for (int i = 0; i < n; ++i) {
    const auto it = S->requests.find(requests[i]);
    if (it == S->requests.end() || !it->second.active || dst_shards[i] < 0 || dst_shards[i] >= c.ngpus)
      return fail(PKV_ERR_ARG, "pkv_shards_migrate_begin: unknown or already migrating request, or bad destination");
  }
  int begun = 0;
  for (int i = 0; i < n; ++i) {
    Request& rq = S->requests[requests[i]];
    const int a = rq.shard, b = dst_shards[i];
    if (a == b) continue;
    Shard& src = S->shards[size_t(a)];
    Shard& dst = S->shards[size_t(b)];
    // Destination pages, in logical order, exactly as alloc_pages hands them out; nothing changes when it has no room.
    const int h = dst.pool->open();
    if (dst.pool->assign_slot(h) < 0 || !dst.pool->alloc(h, rq.length)) {
      dst.pool->close(h);
      return fail(PKV_ERR_LIMIT, "pkv_shards_migrate_begin: destination shard " + std::to_string(b) + " has no room for request " +
                                     std::to_string(requests[i]) + " (" + std::to_string(begun) + " migrations were begun)");
    }
    const std::vector<int32_t>& sp = src.pool->pages(rq.seq);
    const std::vector<int32_t>& dp = dst.pool->pages(h);
    const int np = int(sp.size());
    Migration m{requests[i], a, b, h, 0, nullptr, nullptr, nullptr, nullptr, nullptr};
    m.bytes = size_t(np) * size_t(c.layers) * (row_page_bytes(c) + (c.key_pools ? key_page_bytes(c) : 0));
    rq.active = false;  // leaves the source's step set now; its pages stay referenced until the pull is complete
    {
      DeviceGuard dg(src.device);
      SH_CUDA(cudaEventCreateWithFlags(&m.src_ready, cudaEventDisableTiming));
      SH_CUDA(cudaEventRecord(m.src_ready, src.step_stream));  // every write the source has queued to these pages
    }
    DeviceGuard dg(dst.device);
    SH_CUDA(cudaEventCreate(&m.start));
    SH_CUDA(cudaEventCreate(&m.done));
    // The destination pages may have belonged to a request whose last step is still queued on the destination.
    SH_CUDA(cudaEventRecord(m.start, dst.step_stream));
    SH_CUDA(cudaStreamWaitEvent(dst.mig_stream, m.start, 0));
    if (np > 0) {
      SH_CUDA(cudaMallocHost(reinterpret_cast<void**>(&m.h_ids), size_t(2 * np) * sizeof(int32_t)));
      SH_CUDA(cudaMalloc(reinterpret_cast<void**>(&m.d_ids), size_t(2 * np) * sizeof(int32_t)));
      std::copy(sp.begin(), sp.end(), m.h_ids);
      std::copy(dp.begin(), dp.end(), m.h_ids + np);
      SH_CUDA(cudaStreamWaitEvent(dst.mig_stream, m.src_ready, 0));
      SH_CUDA(cudaMemcpyAsync(m.d_ids, m.h_ids, size_t(2 * np) * sizeof(int32_t), cudaMemcpyHostToDevice, dst.mig_stream));
      std::vector<pkv_pool_desc> descs;
      for (int l = 0; l < c.layers; ++l) {
        descs.push_back(pkv_pool_desc{src.row_pools[size_t(l)], dst.row_pools[size_t(l)], row_page_bytes(c)});
        if (c.key_pools) descs.push_back(pkv_pool_desc{src.key_pools[size_t(l)], dst.key_pools[size_t(l)], key_page_bytes(c)});
      }
      SH_CUDA(cudaEventRecord(m.start, dst.mig_stream));
      if (const int rc = pkv_copy_pages(descs.data(), int(descs.size()), m.d_ids, m.d_ids + np, np, c.num_pages, c.num_pages,
                                        reinterpret_cast<pkv_stream_t>(dst.mig_stream)))
        return rc;
    } else {
      SH_CUDA(cudaEventRecord(m.start, dst.mig_stream));
    }
    SH_CUDA(cudaEventRecord(m.done, dst.mig_stream));
    S->pending.push_back(m);
    ++begun;
  }
  return PKV_OK;
}

int pkv_shards_migrate_end(pkv_shards* S, int wait) {
  if (!S) return -1;
  int finished = 0;
  for (size_t i = 0; i < S->pending.size();) {
    Migration& m = S->pending[i];
    Shard& src = S->shards[size_t(m.src)];
    Shard& dst = S->shards[size_t(m.dst)];
    DeviceGuard dg(dst.device);
    cudaError_t e = wait ? cudaEventSynchronize(m.done) : cudaEventQuery(m.done);
    if (e == cudaErrorNotReady) {
      ++i;
      continue;
    }
    if (e != cudaSuccess) {
      fail_cuda("pkv_shards_migrate_end", e);
      return -1;
    }
    float ms = 0;
    if (cudaEventElapsedTime(&ms, m.start, m.done) == cudaSuccess) S->mig_kernel_ms[size_t(m.dst)] += ms;
    S->migrated_bytes += double(m.bytes);
    // The payload has landed: the destination's later steps are ordered behind it, the source's pages are released (tail
    // first, as unref_pages does) and the request joins the destination's steps.
    cudaStreamWaitEvent(dst.step_stream, m.done, 0);
    Request& rq = S->requests[m.request];
    src.pool->close(rq.seq);
    rq.shard = m.dst;
    rq.seq = m.new_seq;
    rq.active = true;
    cudaFreeHost(m.h_ids);
    cudaFree(m.d_ids);
    cudaEventDestroy(m.start);
    cudaEventDestroy(m.done);
    {
      DeviceGuard dgs(src.device);
      cudaEventDestroy(m.src_ready);
    }
    S->pending.erase(S->pending.begin() + ptrdiff_t(i));
    ++finished;
  }
  return finished;
}

int pkv_shards_migrate_pending(const pkv_shards* S) { return S ? int(S->pending.size()) : -1; }

int pkv_shards_migrate_landed(pkv_shards* S) {
  if (!S) return -1;
  int landed = 0;
  for (const Migration& m : S->pending) {
    DeviceGuard dg(S->shards[size_t(m.dst)].device);
    landed += cudaEventQuery(m.done) == cudaSuccess;
  }
  return landed;
}

int pkv_shards_migrate_stats(pkv_shards* S, double* bytes_out, float* kernel_ms_out) {
  if (!S) return fail(PKV_ERR_ARG, "pkv_shards_migrate_stats: null argument");
  if (bytes_out) *bytes_out = S->migrated_bytes;
  for (size_t g = 0; kernel_ms_out && g < S->shards.size(); ++g) kernel_ms_out[g] = S->mig_kernel_ms[g];
  return PKV_OK;
}

}  // extern "C"
