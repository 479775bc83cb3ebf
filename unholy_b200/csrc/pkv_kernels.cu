// sm_100a kernels of the paged KV-cache path and their C ABI (declared in include/unholy_pkv.h).
//
// What the kernels replace in ewtodd/unholy: store_rows (src/kernels/ref_attn.hip:88-93), store_rows_fp4 /
// load_rows_fp4 (src/kernels/indexer.hip:43-62), act_quant_fp8 / fake_quant_* (src/kernels/ref_elem.hip:18-59),
// glm_store_latent (src/kernels/glm_fast.hip:37-51), copy_kernel (src/kernels/ref_elem.hip:269-278) and the gather
// loop the attention kernels carry (src/kernels/attn_wmma.hip:75-113). The path is pure data movement plus
// elementwise quantisation, so it is bound by HBM bandwidth: no tensor cores are used. Design rules:
//   * every global access is a 16-byte vector, coalesced along a row (a 576-wide bf16 row is 72 vectors = 9 full
//     128-byte lines when the pool base is 128-byte aligned);
//   * one launch covers all chunks of a step and up to PKV_MAX_LAYERS layers (the reference launches once per
//     chunk, layer and pool), with a grid sized from the SM count;
//   * a step has two implementations: a vector kernel (every load of a tile in flight before the first store), and a
//     bulk-copy pipeline (cp.async.bulk global->shared->global with mbarrier completion) in which single-warp CTAs
//     stream key tiles, append tiles and gather tiles through one ring of shared-memory stages; a gathered tile is
//     contiguous in the output and leaves as a single bulk store, an append tile as one store per page-contiguous run;
//   * quantisation keeps 8 values per thread and reduces the block maximum with warp shuffles;
//   * block-table entries are bounds-checked; a bad entry is skipped and recorded in a status word, never dereferenced;
//     the only device-side wait (an mbarrier) is bounded and records when it gives up.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/unholy_pkv.h"
#include "pkv_numeric.cuh"

// The calling thread's last error message (shared by every translation unit of the library).
thread_local std::string pkv_g_err;
// Which top-k path pkv_topk_bf16 takes: 0 = one cluster launch where the shape allows it, 1 = always the four launches
// with scratch (pkv_tune knob 7; default from PKV_TOPK_PATH).
int pkv_g_topk_path = [] {
  const char* v = std::getenv("PKV_TOPK_PATH");
  return v ? std::atoi(v) : 0;
}();

namespace {

std::string& g_err = pkv_g_err;

int fail(int code, const std::string& msg) {
  g_err = msg;
  return code;
}
int fail_cuda(const char* what, cudaError_t e) {
  g_err = std::string(what) + ": " + cudaGetErrorString(e);
  return PKV_ERR_CUDA;
}
#define PKV_LAUNCH_CHECK(name)                                   \
  do {                                                           \
    const cudaError_t e_ = cudaGetLastError();                   \
    if (e_ != cudaSuccess) return fail_cuda(name " launch", e_); \
  } while (0)

// First failed device-side check (0 = none). Kind in the low byte, an entry index above it.
__device__ int g_status = 0;
__device__ __forceinline__ void report(int kind, int index) { atomicCAS(&g_status, 0, kind | (index << 8)); }

struct DeviceInfo {
  int sms = 0;
  bool ok = false;
};
const DeviceInfo& device_info() {
  thread_local DeviceInfo info[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    static DeviceInfo none;
    return none;
  }
  if (!info[dev].ok) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) {
      info[dev].sms = sms;
      info[dev].ok = true;
    }
  }
  return info[dev];
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------------------------------------------------
// Tuning knobs (environment, read once): grid multipliers and the bulk pipeline's shape.
// ---------------------------------------------------------------------------------------------------------------------
int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  return v && *v ? std::atoi(v) : dflt;
}
struct Tuning {
  int bulk_shape = env_int("PKV_BULK_SHAPE", 0);         // STAGES * 100 + ROWS of the bulk pipeline; 0: by launch size
  int bulk_ctas_per_sm = env_int("PKV_BULK_CTAS_PER_SM", 0);  // 0: as many as shared memory allows
  int pdl = env_int("PKV_PDL", 1);                       // programmatic dependent launch of the bulk kernel
  int vec_ctas_per_sm = env_int("PKV_VEC_CTAS_PER_SM", 5);
  int fuse = env_int("PKV_BULK_FUSE", 1);                // the bulk launch carries the step's appends itself
  int batch = env_int("PKV_BULK_BATCH", -1);             // tiles resolved together (0: a full warp's worth; -1: by launch size)
  int resolve_late = env_int("PKV_BULK_RESOLVE_LATE", 0);
  int pipe = env_int("PKV_PIPE", -1);                    // warp-specialised pipeline: 1 always, 0 never, -1 by launch shape
  int wait_polls = env_int("PKV_WAIT_POLLS", 1 << 21);   // polls (of up to 1 us each) before a device-side wait gives up
  int debug_tile = -1;                                   // test hook: CTA 0 over-states the bytes this tile expects
  int copy_bulk = env_int("PKV_COPY_BULK", 1);           // page moves inside a pool through the bulk-copy ring
};
Tuning& tuning() {
  static Tuning t;
  return t;
}

// ---------------------------------------------------------------------------------------------------------------------
// Streaming 16-byte accesses: the pool rows and the gathered output are touched once per launch, so they bypass L1 and
// are marked evict-first in L2.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4* p, const uint4& v) { __stcs(p, v); }
// 32 bytes at a 32-byte aligned address as one store instruction (sm_100: 256-bit global stores).
__device__ __forceinline__ void st_stream32(void* p, const uint32_t* w) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
               "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// ---------------------------------------------------------------------------------------------------------------------
// Generic quantisers: one thread per 8 consecutive values of a row. rows x cols values; cols % block == 0,
// block in {32, 64, 128}. Row r's input starts at x + r * ldx.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 load8(const uint16_t* p, bool vec) {
  if (vec) return *reinterpret_cast<const uint4*>(p);
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = uint32_t(p[2 * i]) | (uint32_t(p[2 * i + 1]) << 16);
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void store8_bf16(uint16_t* p, const float* v, bool vec) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = uint32_t(pkv::f32_to_bf16_bits(v[2 * i])) | (uint32_t(pkv::f32_to_bf16_bits(v[2 * i + 1])) << 16);
  if (vec) {
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      p[2 * i] = uint16_t(w[i]);
      p[2 * i + 1] = uint16_t(w[i] >> 16);
    }
  }
}

enum QuantMode { kFp8Codes = 0, kFp8Fake = 1, kFp4Fake = 2 };

// fp8 codes + scales into dense arrays q [rows][cols], s [rows][cols/block]; or fake quantisation in place.
template <int MODE>
__global__ void __launch_bounds__(256) quant_rows_kernel(const uint16_t* __restrict__ x, int ldx, uint8_t* __restrict__ q,
                                                         uint8_t* __restrict__ s, int rows, int cols, int block,
                                                         bool vec) {
  const int per_row = cols >> 3, group = block >> 3;
  const long long total = (long long)rows * per_row;
  const long long span = ((total + 31) / 32) * 32;  // whole warps stay in the loop: the shuffles need every lane
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < span; u += (long long)gridDim.x * blockDim.x) {
    const bool live = u < total;
    const int r = live ? int(u / per_row) : 0, j = live ? int(u % per_row) : 0;
    uint16_t* xr = const_cast<uint16_t*>(x) + size_t(r) * ldx + size_t(j) * 8;
    float v[8];
    if (live) pkv::unpack8(load8(xr, vec), v);
    else
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    const float amax = pkv::group_max(pkv::absmax8(v), group);
    if (MODE == kFp4Fake) {
      const float sc = pkv::e8m0_bits_to_f32(pkv::fp4_scale_exp(amax));
      if (live) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = pkv::e2m1_bits_to_f32(pkv::e2m1_nibble(fminf(fmaxf(v[i] / sc, -6.0f), 6.0f))) * sc;
        store8_bf16(xr, o, vec);
      }
    } else {
      const uint32_t se = pkv::fp8_scale_exp(amax);
      const float sc = pkv::e8m0_bits_to_f32(se);
      if (!live) continue;
      const uint2 codes = pkv::fp8_pack8(v, sc);
      if (MODE == kFp8Fake) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = pkv::e4m3_bits_to_f32(((i < 4 ? codes.x : codes.y) >> (8 * (i & 3))) & 0xffu) * sc;
        store8_bf16(xr, o, vec);
      } else {
        uint8_t* qp = q + size_t(r) * cols + size_t(j) * 8;
        if ((reinterpret_cast<uintptr_t>(qp) & 7u) == 0) {
          *reinterpret_cast<uint2*>(qp) = codes;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) qp[i] = uint8_t((i < 4 ? codes.x : codes.y) >> (8 * (i & 3)));
        }
        if (j % group == 0) s[size_t(r) * (cols / block) + j / group] = uint8_t(se);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Step kernels. Parameters travel by value (one struct < 4 KB).
// ---------------------------------------------------------------------------------------------------------------------
struct StepParams {
  pkv_step s;
  int L;
  int flags;
  int append_tiles;  // per layer
  int key_tiles;     // per layer (bulk kernel only)
  int tpq_shift;     // log2(gather tiles per query) when that is a power of two, else -1 (bulk kernel only)
  int rpp_shift;     // log2(rows_per_page) when that is a power of two, else -1
  int resolve_late;  // resolve the next batch when the LAST tile of the current one is issued (else the first)
  int gather_tiles;  // per layer
  int tiles_per_q;
  int wait_polls;    // polls before a bounded wait gives up (pipe kernel)
  int debug_tile;    // >= 0: CTA 0 expects 16 bytes more than this tile brings, so its wait runs out (test hook)
  pkv_layer layers[PKV_MAX_LAYERS];
};

// The chunk holding batch row t (chunks ordered by t0, disjoint); -1 if none.
__device__ __forceinline__ int find_chunk(const pkv_chunk* __restrict__ chunks, int n, int t) {
  if (t < n) {  // a decode step: chunk t is batch row t
    const int t0 = __ldg(&chunks[t].t0);
    if (t0 == t && __ldg(&chunks[t].n) >= 1) return t;
  }
  int lo = 0, hi = n;  // last chunk with t0 <= t
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(&chunks[mid].t0) <= t) lo = mid;
    else hi = mid;
  }
  if (n == 0) return -1;
  const int t0 = __ldg(&chunks[lo].t0), cn = __ldg(&chunks[lo].n);
  return (t >= t0 && t < t0 + cn) ? lo : -1;
}

// Physical row id of logical row `lr` of `slot`, or -1 (recorded) when the table entry is unusable.
__device__ __forceinline__ long long physical_row(const pkv_step& s, int slot, int lr, int tag) {
  const int pg = (s.rows_per_page & (s.rows_per_page - 1)) == 0 ? lr >> (31 - __clz(s.rows_per_page)) : lr / s.rows_per_page;
  if (lr < 0 || pg >= s.max_pages_per_seq || unsigned(slot) >= unsigned(s.max_slots)) {
    report(2, tag);
    return -1;
  }
  const int page = __ldg(&s.tables[size_t(slot) * s.max_pages_per_seq + pg]);
  if (unsigned(page) >= unsigned(s.num_pages)) {
    report(1, tag);
    return -1;
  }
  return (long long)page * s.rows_per_page + (lr - pg * s.rows_per_page);
}

constexpr int kVecThreads = 384;            // 12 warps
constexpr int kAppendRows = kVecThreads / 16;  // batch rows per append tile: 16 threads quantise one 128-wide key row
constexpr int kGatherRows = 32;             // index entries per gather tile
constexpr int kGatherUnroll = 6;            // 32 rows x 72 vectors = 384 threads x 6

// One 128-wide key row held by 16 consecutive lanes (8 values each, lane j of the row in `j`): MXFP4 and / or fp8
// quantisation and the stores into the row's place (physical row `rid`; negative: nothing is stored). Every lane of the
// warp must call it: the block maxima and the row's four MXFP4 scale bytes travel by shuffles.
__device__ __forceinline__ void quantise_key_row(const pkv_step& s, const pkv_layer& ly, float* v, long long rid, int j,
                                                 bool fp4, bool fp8, bool rotate) {
  if (rotate) pkv::hadamard128_lanes(v, j);  // PKV_KEYS_HADAMARD: the reference's hadamard128 in front of store_rows_fp4
  const float a8 = pkv::absmax8(v);
  if (fp4) {
    const uint32_t se = pkv::fp4_scale_exp(pkv::group_max(a8, 4));
    const uint32_t codes = pkv::fp4_pack8(v, pkv::e8m0_bits_to_f32(se));
    const int base = (threadIdx.x & 31) & 16;  // the row's first lane
    const uint32_t s0 = __shfl_sync(0xffffffffu, se, base), s1 = __shfl_sync(0xffffffffu, se, base + 4),
                   s2 = __shfl_sync(0xffffffffu, se, base + 8), s3 = __shfl_sync(0xffffffffu, se, base + 12);
    if (rid >= 0) {
      const long long page = rid / s.rows_per_page;
      const int slot = int(rid - page * s.rows_per_page);
      uint8_t* pg = ly.key_pool_fp4 + size_t(page) * size_t(s.rows_per_page) * 68u;
      *reinterpret_cast<uint32_t*>(pg + size_t(slot) * 64u + j * 4) = codes;
      if (j == 0)
        *reinterpret_cast<uint32_t*>(pg + size_t(s.rows_per_page) * 64u + size_t(slot) * 4u) =
            s0 | (s1 << 8) | (s2 << 16) | (s3 << 24);
    }
  }
  if (fp8) {
    const int group = s.fp8_block >> 3;
    const uint32_t se = pkv::fp8_scale_exp(pkv::group_max(a8, group));
    const uint2 codes = pkv::fp8_pack8(v, pkv::e8m0_bits_to_f32(se));
    if (rid >= 0) {
      *reinterpret_cast<uint2*>(ly.key_fp8_codes + size_t(rid) * PKV_FP4_ROW_DIM + j * 8) = codes;
      if (j % group == 0) ly.key_fp8_scales[size_t(rid) * (PKV_FP4_ROW_DIM / s.fp8_block) + j / group] = uint8_t(se);
    }
  }
}

// One append tile: batch rows [t_first, t_first + kAppendRows) of one layer. Copies the bf16 rows into the pool and
// quantises the keys (MXFP4 and/or fp8) to the same physical rows.
template <int NT>
__device__ void append_tile(const StepParams& P, const pkv_layer& ly, int t_first, long long* s_rid) {
  constexpr int kRows = NT / 16;
  const pkv_step& s = P.s;
  const int tid = threadIdx.x;
  const int nrows = min(kRows, s.T - t_first);
  if (tid < kRows) {
    long long rid = -1;
    if (tid < nrows) {
      const int t = t_first + tid;
      const int c = find_chunk(s.chunks, s.nchunks, t);
      if (c >= 0) {
        const pkv_chunk ch = s.chunks[c];
        rid = physical_row(s, ch.slot, ch.s0 + (t - ch.t0), t);
      }
    }
    s_rid[tid] = rid;
  }
  __syncthreads();
  if ((P.flags & PKV_DO_ROWS) && ly.rows && ly.row_pool) {
    const int vpr = s.width >> 3;
    const int total = nrows * vpr;
    const uint4* src = reinterpret_cast<const uint4*>(ly.rows + size_t(t_first) * s.width);
    for (int base = 0; base < total; base += NT * 5) {  // five loads in flight per thread before the first store
      uint4 v[5];
#pragma unroll
      for (int i = 0; i < 5; ++i) {
        const int u = base + i * NT + tid;
        if (u < total) v[i] = ld_stream(src + u);
      }
#pragma unroll
      for (int i = 0; i < 5; ++i) {
        const int u = base + i * NT + tid;
        if (u < total) {
          const int r = u / vpr, c = u - r * vpr;
          const long long rid = s_rid[r];
          if (rid >= 0) st_stream(reinterpret_cast<uint4*>(ly.row_pool + size_t(rid) * s.row_stride) + c, v[i]);
        }
      }
    }
  }
  const bool fp4 = (P.flags & PKV_DO_KEYS_FP4) && ly.keys && ly.key_pool_fp4;
  const bool fp8 = (P.flags & PKV_DO_KEYS_FP8) && ly.keys && ly.key_fp8_codes && ly.key_fp8_scales;
  if (fp4 || fp8) {
    // 16 threads per key row, 8 values each; every lane runs the shuffles.
    const int r = tid >> 4, j = tid & 15;
    const long long rid = r < nrows ? s_rid[r] : -1;
    float v[8];
    if (rid >= 0) {
      pkv::unpack8(*reinterpret_cast<const uint4*>(ly.keys + size_t(t_first + r) * PKV_FP4_ROW_DIM + j * 8), v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    quantise_key_row(s, ly, v, rid, j, fp4, fp8, (P.flags & PKV_KEYS_HADAMARD) != 0);
  }
  __syncthreads();
}

// Source row of entry `e` of query `q`: the pool row, the row being appended in this launch when the entry falls in
// the query's own chunk and rows are appended by the same launch, or nullptr when masked.
__device__ __forceinline__ const uint4* gather_source(const StepParams& P, const pkv_layer& ly, int q, int e) {
  const pkv_step& s = P.s;
  if (e >= s.k) return nullptr;
  // Three loads that depend on nothing are issued together; the chunk and the block-table entry follow.
  const int row = __ldg(&ly.idx[size_t(q) * s.k + e]);
  const int vis = __ldg(&s.q_visible[q]);
  const int qc = __ldg(&s.q_chunk[q]);
  if (unsigned(qc) >= unsigned(s.nchunks)) {
    report(2, q);
    return nullptr;
  }
  const pkv_chunk ch = s.chunks[qc];
  if (row < 0 || row >= vis) return nullptr;
  if ((P.flags & PKV_DO_ROWS) && ly.rows && row >= ch.s0 && row < ch.s0 + ch.n)
    return reinterpret_cast<const uint4*>(ly.rows + size_t(ch.t0 + (row - ch.s0)) * s.width);
  const long long rid = physical_row(s, ch.slot, row, q);
  if (rid < 0) return nullptr;
  return reinterpret_cast<const uint4*>(ly.row_pool + size_t(rid) * s.row_stride);
}

// Copies one resolved tile (rows s_src[0..nrows), nullptr = zeros) to its contiguous place in the output. All of a
// thread's loads are issued before its first store.
__device__ __forceinline__ void copy_tile_vec(const uint4* const* s_src, uint4* out, int nrows, int vpr) {
  const int tid = threadIdx.x;
  const int total = nrows * vpr;
  for (int base = 0; base < total; base += kVecThreads * kGatherUnroll) {
    uint4 v[kGatherUnroll];
#pragma unroll
    for (int i = 0; i < kGatherUnroll; ++i) {
      const int u = base + i * kVecThreads + tid;
      v[i] = make_uint4(0, 0, 0, 0);
      if (u < total) {
        const int r = u / vpr, c = u - r * vpr;
        const uint4* p = s_src[r];
        if (p) v[i] = ld_stream(p + c);
      }
    }
#pragma unroll
    for (int i = 0; i < kGatherUnroll; ++i) {
      const int u = base + i * kVecThreads + tid;
      if (u < total) st_stream(out + u, v[i]);
    }
  }
}

// One gather tile with vector loads: 32 entries of one query.
__device__ void gather_tile_vec(const StepParams& P, const pkv_layer& ly, int tile, const uint4** s_src) {
  const pkv_step& s = P.s;
  const int q = tile / P.tiles_per_q, e0 = (tile - q * P.tiles_per_q) * kGatherRows;
  if (threadIdx.x < kGatherRows) s_src[threadIdx.x] = gather_source(P, ly, q, e0 + int(threadIdx.x));
  __syncthreads();
  copy_tile_vec(s_src, reinterpret_cast<uint4*>(ly.gathered + (size_t(q) * s.k + e0) * s.width), min(kGatherRows, s.k - e0),
                s.width >> 3);
  __syncthreads();
}

__global__ void __launch_bounds__(kVecThreads, 3) step_vec_kernel(const __grid_constant__ StepParams P) {
  __shared__ long long s_rid[kAppendRows];
  __shared__ const uint4* s_src[kGatherRows];
  const int per_layer = P.append_tiles + P.gather_tiles;
  const long long total = (long long)per_layer * P.L;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (long long w = blockIdx.x; w < total; w += gridDim.x) {
    const int layer = int(w / per_layer), r = int(w - (long long)layer * per_layer);
    const pkv_layer& ly = P.layers[layer];
    if (r < P.append_tiles) append_tile<kVecThreads>(P, ly, r * kAppendRows, s_rid);
    else gather_tile_vec(P, ly, r - P.append_tiles, s_src);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Bulk-copy pipeline: the primitives (mbarrier, cp.async.bulk in both directions, bulk-group waits, the proxy fence)
// and the step kernel built on them. One warp per CTA; STAGES tiles rotate through shared memory, so (STAGES - 2) tiles
// of loads and up to 2 tiles of stores are in flight per warp at any time.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// The same with a time limit (nanoseconds) up to which the hardware may keep the thread suspended: the thread wakes as
// soon as the phase completes, so a loop of these neither spins hot nor oversleeps the way polling with nanosleep does.
__device__ __forceinline__ uint32_t mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok;
}
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// A wait that cannot hang: gives up after ~2^22 polls (seconds), reports, and tells the caller to stop.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int tag) {
  for (int spin = 0; spin < (1 << 22); ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if (spin > 64) __nanosleep(64);
  }
  report(3, tag);
  return false;
}

// Key quantisation of one staged tile: rows of 128 bf16 keys already in shared memory (key_bytes apart), 16 lanes
// per row, two rows per pass of the warp. Same arithmetic and stores as append_tile.
template <int ROWS>
__device__ __forceinline__ void quantise_staged_keys(const StepParams& P, const pkv_layer& ly, const unsigned char* stage,
                                                     const long long* rids, int nrows, bool fp4, bool fp8) {
  const pkv_step& s = P.s;
  const int lane = threadIdx.x, j = lane & 15;
#pragma unroll 1
  for (int r0 = 0; r0 < ROWS; r0 += 2) {
    if (r0 >= nrows) break;
    const int r = r0 + (lane >> 4);
    const long long rid = r < nrows ? rids[r] : -1;
    float v[8];
    pkv::unpack8(*reinterpret_cast<const uint4*>(stage + size_t(r < ROWS ? r : 0) * (PKV_FP4_ROW_DIM * 2) + j * 16), v);
    quantise_key_row(s, ly, v, rid, j, fp4, fp8, (P.flags & PKV_KEYS_HADAMARD) != 0);
  }
}

// The whole step of up to PKV_MAX_LAYERS layers as ONE stream of tiles through one bulk-copy pipeline. Per layer:
//   key tiles    ROWS batch rows of new keys: one bulk load of the contiguous source, quantised from shared memory;
//   append tiles ROWS batch rows of new KV rows: one bulk load of the contiguous source, then one bulk store per run of
//                rows that are contiguous in the pool (a run ends at a page boundary or where the chunk changes);
//   gather tiles ROWS index entries of one query: one bulk load per row, one bulk store of the contiguous tile.
// Tiles are dealt round-robin to single-warp CTAs; each keeps STAGES tiles rotating (loads of STAGES - 2 tiles in
// flight while up to two tiles drain).
template <int STAGES, int ROWS, int BATCH>
__global__ void __launch_bounds__(32) step_bulk_kernel(const __grid_constant__ StepParams P) {
  static_assert(ROWS <= 32 && ROWS % 2 == 0 && 32 % ROWS == 0 && STAGES >= 3, "one lane per row; two stages drain while the others fill");
  static_assert(BATCH >= 1 && BATCH * ROWS <= 32 && (BATCH & (BATCH - 1)) == 0, "a batch is resolved by one warp, one lane per row");
  constexpr int kBatch = BATCH;  // tiles whose addresses are resolved together, one lane per row
  enum Kind { kKeys = 0, kAppend = 1, kGather = 2 };
  struct Tile {  // what issue and drain need to know about a tile
    int layer, kind, a, b;  // gather: a = query, b = first entry; keys / append: a = first batch row
  };
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[STAGES];
  __shared__ long long s_rid[STAGES][ROWS];      // pool rows of a staged key / append tile
  __shared__ Tile s_tile[STAGES];                // the staged tiles
  __shared__ const uint4* s_src[2][32];          // resolved batches: gather source pointers (nullptr: masked) ...
  __shared__ long long s_bat_rid[2][32];         // ... and pool rows of key / append rows
  __shared__ Tile s_bat_tile[2][kBatch];
  const pkv_step& s = P.s;
  const int lane = threadIdx.x;
  const uint32_t row_bytes = uint32_t(s.width) * 2u, key_bytes = PKV_FP4_ROW_DIM * 2u;
  const uint32_t stage_bytes = row_bytes * ROWS;
  // All tile arithmetic is 32-bit and incremental: a single warp runs the whole pipeline, so every long dependent
  // instruction sequence (a 64-bit division is about a hundred) is paid in full on the critical path.
  const unsigned tiles_per_q = unsigned(s.k + ROWS - 1) / ROWS;
  const unsigned key_tiles = unsigned(P.key_tiles), app_tiles = unsigned(P.append_tiles);
  const unsigned per_layer = key_tiles + app_tiles + unsigned(s.Q) * tiles_per_q;
  const unsigned total = per_layer * unsigned(P.L);  // the host keeps this below 2^31
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i) mbar_init(smem_addr(&bars[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  // Programmatic dependent launch: this grid may have been scheduled while the previous kernel of the stream was still
  // draining. Nothing above touches global memory; everything below waits for that kernel's writes to be visible.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned first = blockIdx.x, stride = gridDim.x;
  const int mine = first < total ? int((total - first + stride - 1) / stride) : 0;
  const bool fp4 = (P.flags & PKV_DO_KEYS_FP4) != 0, fp8 = (P.flags & PKV_DO_KEYS_FP8) != 0;

  // Address resolution runs a batch of kBatch tiles at a time, one lane per row of each tile, so the dependent loads
  // (index entry -> chunk -> block-table entry) cost one latency per batch instead of one per tile and overlap the
  // copies of earlier tiles. Two batches rotate: batch b + 1 is resolved when the first tile of batch b is issued.
  // Each lane walks its own tile sequence (this CTA's tiles sub, sub + kBatch, ...) with a (layer, offset) cursor.
  const int sub = lane / ROWS, r_in = lane % ROWS;
  unsigned cur_layer = 0, cur_local = 0;  // position of this lane's next tile to resolve
  {
    const unsigned w = first + unsigned(sub) * stride;  // one division per kernel, not per tile
    cur_layer = w / per_layer;
    cur_local = w - cur_layer * per_layer;
  }
  const unsigned adv = unsigned(kBatch) * stride;
  auto resolve_batch = [&](int b) {
    const int j = b * kBatch + sub;
    const uint4* src = nullptr;
    long long rid = -1;
    if (sub < kBatch && j < mine) {
      const pkv_layer& ly = P.layers[cur_layer];
      Tile t;
      t.layer = int(cur_layer);
      if (cur_local >= key_tiles + app_tiles) {
        const unsigned g = cur_local - key_tiles - app_tiles;
        const unsigned q = P.tpq_shift >= 0 ? g >> P.tpq_shift : g / tiles_per_q;
        const unsigned e0 = (g - q * tiles_per_q) * ROWS;
        t.kind = kGather, t.a = int(q), t.b = int(e0);
        src = gather_source(P, ly, int(q), int(e0) + r_in);
      } else {
        const bool keys = cur_local < key_tiles;
        const int t_first = int(keys ? cur_local : cur_local - key_tiles) * ROWS, row = t_first + r_in;
        t.kind = keys ? kKeys : kAppend, t.a = t_first, t.b = 0;
        if (row < s.T) {
          const int c = find_chunk(s.chunks, s.nchunks, row);
          if (c >= 0) {
            const pkv_chunk ch = s.chunks[c];
            rid = physical_row(s, ch.slot, ch.s0 + (row - ch.t0), row);
          }
        }
      }
      if (r_in == 0) s_bat_tile[b & 1][sub] = t;
      cur_local += adv;
      while (cur_local >= per_layer) {
        cur_local -= per_layer;
        ++cur_layer;
      }
    }
    s_src[b & 1][lane] = src;
    s_bat_rid[b & 1][lane] = rid;
    __syncwarp();
  };

  // Starts the loads of tile j into stage st (its batch is resolved).
  auto issue = [&](int j, int st) {
    const int slot = (j / kBatch) & 1, sub_j = j % kBatch, off = sub_j * ROWS;
    const Tile t = s_bat_tile[slot][sub_j];
    const pkv_layer& ly = P.layers[t.layer];
    unsigned char* stage = smem + size_t(st) * stage_bytes;
    const uint32_t bar = smem_addr(&bars[st]);
    if (lane == 0) s_tile[st] = t;
    if (t.kind == kGather) {
      const uint4* src = lane < ROWS ? s_src[slot][off + lane] : nullptr;
      const unsigned valid = __ballot_sync(0xffffffffu, src != nullptr);
      if (lane == 0) mbar_expect_tx(bar, uint32_t(__popc(valid)) * row_bytes);
      // Masked rows (and rows past k, which are never stored) are zero-filled by the whole warp, one row at a time.
      unsigned masked = ~valid & (ROWS == 32 ? 0xffffffffu : ((1u << ROWS) - 1u));
      while (masked) {
        const int r = __ffs(masked) - 1;
        masked &= masked - 1;
        uint4* z = reinterpret_cast<uint4*>(stage + size_t(r) * row_bytes);
        for (uint32_t i = lane; i < row_bytes / 16; i += 32) z[i] = make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
      if (src) bulk_load(smem_addr(stage + size_t(lane) * row_bytes), src, row_bytes, bar);
    } else {
      // Batch rows [t.a, t.a + nrows): lane 0 loads the contiguous source; the rows' pool ids travel with the stage.
      const int nrows = min(ROWS, s.T - t.a);
      if (lane == 0) {
        const uint32_t each = t.kind == kKeys ? key_bytes : row_bytes;
        const unsigned char* src = t.kind == kKeys ? reinterpret_cast<const unsigned char*>(ly.keys) + size_t(t.a) * key_bytes
                                                   : reinterpret_cast<const unsigned char*>(ly.rows) + size_t(t.a) * row_bytes;
        mbar_expect_tx(bar, uint32_t(nrows) * each);
        bulk_load(smem_addr(stage), src, uint32_t(nrows) * each, bar);
      }
      if (lane < ROWS) s_rid[st][lane] = s_bat_rid[slot][off + lane];
      __syncwarp();
    }
    // The first tile of a batch is on its way: resolve the batch after it while its copies fly.
    if (sub_j == (P.resolve_late ? kBatch - 1 : 0) && (j / kBatch + 1) * kBatch < mine) resolve_batch(j / kBatch + 1);
  };

  constexpr int ahead = STAGES - 2;
  if (mine > 0) resolve_batch(0);
  int st_issue = 0;
  for (int j = 0; j < ahead && j < mine; ++j) {
    issue(j, st_issue);
    st_issue = st_issue + 1 == STAGES ? 0 : st_issue + 1;
  }
  bool alive = true;
  int j_fail = 0, st = 0;
  uint32_t parity = 0;
  for (int j = 0; j < mine; ++j) {
    // The stage tile j + ahead goes into was drained by tile j - 2; its stores must have finished reading shared memory
    // (every lane waits on its own bulk groups: append tiles are stored by several lanes).
    if (j + ahead < mine) {
      bulk_wait_read<1>();
      __syncwarp();
      issue(j + ahead, st_issue);
      st_issue = st_issue + 1 == STAGES ? 0 : st_issue + 1;
    }
    alive = mbar_wait_bounded(smem_addr(&bars[st]), parity, int(blockIdx.x));
    alive = __all_sync(0xffffffffu, alive);
    if (!alive) {
      j_fail = j;
      break;
    }
    const Tile t = s_tile[st];
    const pkv_layer& ly = P.layers[t.layer];
    unsigned char* stage = smem + size_t(st) * stage_bytes;
    if (t.kind == kGather) {
      const int nrows = min(ROWS, s.k - t.b);
      fence_async_smem();  // the zero rows were written through the generic proxy
      __syncwarp();
      if (lane == 0)
        bulk_store(ly.gathered + (size_t(t.a) * s.k + t.b) * s.width, smem_addr(stage), uint32_t(nrows) * row_bytes);
    } else {
      const int nrows = min(ROWS, s.T - t.a);
      if (t.kind == kKeys) {
        quantise_staged_keys<ROWS>(P, ly, stage, s_rid[st], nrows, fp4 && ly.key_pool_fp4, fp8 && ly.key_fp8_codes && ly.key_fp8_scales);
      } else {
        // Runs of rows that are contiguous in the pool leave with one bulk store each.
        const long long rid = lane < nrows ? s_rid[st][lane] : -1;
        const long long prev = __shfl_up_sync(0xffffffffu, rid, 1);
        const bool start = rid >= 0 && (lane == 0 || prev < 0 || rid != prev + 1 || s.row_stride != s.width);
        const unsigned breaks = __ballot_sync(0xffffffffu, start || rid < 0);
        if (start) {
          const unsigned higher = lane == 31 ? 0u : (breaks & ~((2u << lane) - 1u));
          const int next = higher ? __ffs(higher) - 1 : 32;
          bulk_store(ly.row_pool + size_t(rid) * s.row_stride, smem_addr(stage + size_t(lane) * row_bytes),
                     uint32_t(next - lane) * row_bytes);
        }
      }
    }
    bulk_commit();
    __syncwarp();
    if (++st == STAGES) {
      st = 0;
      parity ^= 1u;
    }
  }
  if (!alive) {
    // Gave up on tile j_fail: give the loads of the tiles already started a second, bounded chance to land before the
    // CTA's shared memory is released.
    int st2 = st;
    uint32_t par2 = parity;
    for (int jj = j_fail; jj < mine && jj <= j_fail + ahead; ++jj) {
      const uint32_t bar = smem_addr(&bars[st2]);
      for (int spin = 0; spin < (1 << 18); ++spin) {
        if (mbar_try_wait(bar, par2)) break;
        __nanosleep(256);
      }
      if (++st2 == STAGES) st2 = 0, par2 ^= 1u;
    }
  }
  bulk_wait_all();
  __syncwarp();
}

// ---------------------------------------------------------------------------------------------------------------------
// The bulk pipeline with warp-specialised CTAs. A tile is ROWS rows: an append tile (ROWS batch rows of new KV rows,
// contiguous in the source, one bulk store per page-contiguous run) or a gather tile (ROWS index entries of one query,
// one bulk load per row, one bulk store of the contiguous tile). Tiles are dealt round-robin to CTAs.
//   warp 0, the mover:     streams its CTA's tiles through the ring of STAGES shared-memory stages (loads of
//                          STAGES - 2 tiles in flight while up to two tiles drain). It computes a tile's kind and
//                          position itself (arithmetic only) and never loads an index, a chunk or a table entry;
//   warps 1..kResWarps, the resolvers: run the dependent loads (index entry -> chunk -> block-table entry) for 32 rows
//                          at a time, one lane per row, taking batches in turn and staying up to kResBatches batches
//                          ahead of the mover, into a shared-memory ring (a chain is three memory latencies long: one
//                          warp alone resolves more slowly than the mover moves); the mover picks a row's source
//                          pointer or pool row up when it needs it (a gather tile when its loads are issued, an append
//                          tile only when it is stored);
//   the other warps, key workers (launched only when the step quantises keys): take pairs of key rows grid-wide with plain
//                          16-byte loads, 16 lanes per row, and write codes and scales; independent of the ring.
// Every wait (mbarrier) is bounded: after P.wait_polls polls the waiting warp records kind 3 in the status word, raises
// the CTA's abort flag and the CTA winds down (loads in flight get a second bounded chance to land).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kResWarps = 1;
constexpr int kResBatches = 3;
constexpr int kKeyWarps = 4;
constexpr int kKeyUnroll = 2;  // units (pairs of key rows) a key worker has in flight
constexpr int kFirstKeyWarp = 1 + kResWarps;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int STAGES, int ROWS>
__global__ void __launch_bounds__(32 * (kFirstKeyWarp + kKeyWarps)) step_pipe_kernel(const __grid_constant__ StepParams P) {
  static_assert(ROWS <= 32 && ROWS % 2 == 0 && 32 % ROWS == 0 && STAGES >= 3, "one lane per row; two stages drain while the others fill");
  constexpr int kBatch = 32 / ROWS;  // tiles per resolved batch
  static_assert(STAGES - 2 <= (kResBatches - 1) * kBatch, "the mover may not issue further ahead than the resolver's ring reaches");
  constexpr unsigned long long kNoRow = ~0ull;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[STAGES];
  __shared__ __align__(8) unsigned long long res_full[kResBatches], res_empty[kResBatches];
  __shared__ unsigned long long s_res[kResBatches][32];  // per row: gather source pointer (0: masked) or pool row (kNoRow: none)
  __shared__ int s_abort;
  const pkv_step& s = P.s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row_bytes = uint32_t(s.width) * 2u, stage_bytes = row_bytes * ROWS;
  const unsigned tiles_per_q = unsigned(s.k + ROWS - 1) / ROWS;
  const unsigned app_tiles = unsigned(P.append_tiles);
  const unsigned per_layer = app_tiles + unsigned(s.Q) * tiles_per_q;
  const unsigned total = per_layer * unsigned(P.L);  // the host keeps this below 2^31
  const unsigned first = blockIdx.x, stride = gridDim.x;
  const int mine = first < total ? int((total - first + stride - 1) / stride) : 0;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i) mbar_init(smem_addr(&bars[i]), 1);
#pragma unroll
    for (int i = 0; i < kResBatches; ++i) {
      mbar_init(smem_addr(&res_full[i]), 1);
      mbar_init(smem_addr(&res_empty[i]), 1);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // Programmatic dependent launch: nothing above touches global memory; everything below waits for the previous
  // kernel of the stream to have completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  volatile int* abort_flag = &s_abort;
  auto wait_bounded = [&](uint32_t bar, uint32_t parity, int tag) -> bool {
    for (int spin = 0; spin < P.wait_polls; ++spin) {  // each poll may stay suspended for up to a microsecond
      if (mbar_try_wait_for(bar, parity, 1000u)) return true;
      if ((spin & 255) == 255 && *abort_flag) return false;
    }
    report(3, tag);
    *abort_flag = 1;
    return false;
  };
  // Position of tile w in the launch: (layer, offset in the layer); offsets below app_tiles are append tiles.
  auto advance = [&](unsigned& layer, unsigned& local, unsigned by) {
    local += by;
    while (local >= per_layer) {
      local -= per_layer;
      ++layer;
    }
  };

  if (warp >= kFirstKeyWarp) {
    // ---- key workers ----
    const bool fp4 = (P.flags & PKV_DO_KEYS_FP4) != 0, fp8 = (P.flags & PKV_DO_KEYS_FP8) != 0;
    if (!P.key_tiles || !(fp4 || fp8)) return;
    const bool rotate = (P.flags & PKV_KEYS_HADAMARD) != 0;
    const unsigned upl = unsigned(s.T + 1) / 2, units = upl * unsigned(P.L);  // a unit = two key rows of one layer
    const unsigned nworkers = gridDim.x * unsigned(blockDim.x / 32 - kFirstKeyWarp);
    const int j = lane & 15;
    for (unsigned u0 = blockIdx.x * unsigned(blockDim.x / 32 - kFirstKeyWarp) + unsigned(warp - kFirstKeyWarp); u0 < units;
         u0 += kKeyUnroll * nworkers) {
      // kKeyUnroll units per pass: all their key loads and address chains are in flight before the arithmetic starts
      uint4 raw[kKeyUnroll];
      long long rid[kKeyUnroll];
      unsigned layer[kKeyUnroll];
#pragma unroll
      for (int i = 0; i < kKeyUnroll; ++i) {
        const unsigned u = u0 + unsigned(i) * nworkers;
        rid[i] = -1;
        raw[i] = make_uint4(0, 0, 0, 0);
        layer[i] = 0;
        if (u < units) {
          layer[i] = u / upl;
          const int r = int(u - layer[i] * upl) * 2 + (lane >> 4);
          if (r < s.T) {
            raw[i] = ld_stream(reinterpret_cast<const uint4*>(P.layers[layer[i]].keys + size_t(r) * PKV_FP4_ROW_DIM) + j);
            const int c = find_chunk(s.chunks, s.nchunks, r);
            if (c >= 0) {
              const pkv_chunk ch = s.chunks[c];
              rid[i] = physical_row(s, ch.slot, ch.s0 + (r - ch.t0), r);
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < kKeyUnroll; ++i) {
        if (u0 + unsigned(i) * nworkers >= units) break;  // (uniform across the warp)
        const pkv_layer& ly = P.layers[layer[i]];
        float v[8];
        pkv::unpack8(raw[i], v);
        quantise_key_row(s, ly, v, rid[i], j, fp4 && ly.key_pool_fp4, fp8 && ly.key_fp8_codes && ly.key_fp8_scales, rotate);
      }
    }
    return;
  }

  if (warp >= 1) {
    // ---- resolver `warp - 1`: batches b = warp - 1, warp - 1 + kResWarps, ...; batch b = this CTA's tiles
    //      [b * kBatch, (b + 1) * kBatch), lane = (tile in batch, row in tile) ----
    const int sub = lane / ROWS, r_in = lane % ROWS;
    unsigned cl = 0, cloc = 0;
    if (mine > 0) {
      const unsigned w = first + unsigned((warp - 1) * kBatch + sub) * stride;  // one division per kernel, not per tile
      cl = w / per_layer;
      cloc = w - cl * per_layer;
    }
    const int nb = (mine + kBatch - 1) / kBatch;
    for (int b = warp - 1; b < nb; b += kResWarps) {
      const int slot = b % kResBatches;
      if (b >= kResBatches) {  // the mover has finished with the batch that used this slot
        const bool ok = wait_bounded(smem_addr(&res_empty[slot]), uint32_t((b / kResBatches - 1) & 1), int(blockIdx.x));
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      unsigned long long v = 0;
      if (b * kBatch + sub < mine) {
        const pkv_layer& ly = P.layers[cl];
        if (cloc >= app_tiles) {
          const unsigned g = cloc - app_tiles;
          const unsigned q = P.tpq_shift >= 0 ? g >> P.tpq_shift : g / tiles_per_q;
          const unsigned e0 = (g - q * tiles_per_q) * ROWS;
          v = reinterpret_cast<unsigned long long>(gather_source(P, ly, int(q), int(e0) + r_in));
        } else {
          const int row = int(cloc) * ROWS + r_in;
          long long rid = -1;
          if (row < s.T) {
            const int c = find_chunk(s.chunks, s.nchunks, row);
            if (c >= 0) {
              const pkv_chunk ch = s.chunks[c];
              rid = physical_row(s, ch.slot, ch.s0 + (row - ch.t0), row);
            }
          }
          v = rid < 0 ? kNoRow : static_cast<unsigned long long>(rid);
        }
        advance(cl, cloc, unsigned(kResWarps * kBatch) * stride);
      }
      s_res[slot][lane] = v;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&res_full[slot]));
    }
    return;
  }

  // ---- mover ----
  struct Tile {
    unsigned layer, local;
  };
  __shared__ Tile s_tile[STAGES];
  unsigned il = 0, iloc = 0;  // position of the next tile to issue
  if (mine > 0) {
    il = first / per_layer;
    iloc = first - il * per_layer;
  }
  int ready = 0, issued = 0;  // batches known to be resolved; tiles whose loads were started
  bool alive = true;
  auto ensure = [&](int b) {
    while (alive && ready <= b) {
      alive = __all_sync(0xffffffffu, wait_bounded(smem_addr(&res_full[ready % kResBatches]), uint32_t((ready / kResBatches) & 1), int(blockIdx.x)));
      ++ready;
    }
  };
  // Starts the loads of tile j into stage st.
  auto issue = [&](int j, int st) {
    const unsigned layer = il, local = iloc;
    advance(il, iloc, stride);
    const pkv_layer& ly = P.layers[layer];
    unsigned char* stage = smem + size_t(st) * stage_bytes;
    const uint32_t bar = smem_addr(&bars[st]);
    const uint32_t extra = (P.debug_tile == j && blockIdx.x == 0) ? 16u : 0u;
    if (lane == 0) s_tile[st] = Tile{layer, local};
    if (local >= app_tiles) {
      ensure(j / kBatch);
      if (!alive) return;
      const unsigned long long rv = lane < ROWS ? s_res[(j / kBatch) % kResBatches][(j % kBatch) * ROWS + lane] : 0ull;
      const uint4* src = reinterpret_cast<const uint4*>(rv);
      const unsigned valid = __ballot_sync(0xffffffffu, src != nullptr);
      if (lane == 0) mbar_expect_tx(bar, uint32_t(__popc(valid)) * row_bytes + extra);
      // Masked rows (and rows past k, which are never stored) are zero-filled by the whole warp, one row at a time.
      unsigned masked = ~valid & (ROWS == 32 ? 0xffffffffu : ((1u << ROWS) - 1u));
      while (masked) {
        const int r = __ffs(masked) - 1;
        masked &= masked - 1;
        uint4* z = reinterpret_cast<uint4*>(stage + size_t(r) * row_bytes);
        for (uint32_t i = lane; i < row_bytes / 16; i += 32) z[i] = make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
      if (src) bulk_load(smem_addr(stage + size_t(lane) * row_bytes), src, row_bytes, bar);
    } else {
      // Batch rows [a, a + nrows): one load of the contiguous source; where the rows go is looked up when they are stored.
      const int a = int(local) * ROWS, nrows = min(ROWS, s.T - a);
      if (lane == 0) {
        mbar_expect_tx(bar, uint32_t(nrows) * row_bytes + extra);
        bulk_load(smem_addr(stage), reinterpret_cast<const unsigned char*>(ly.rows) + size_t(a) * row_bytes, uint32_t(nrows) * row_bytes, bar);
      }
      __syncwarp();
    }
    ++issued;
  };

  constexpr int ahead = STAGES - 2;
  int st_issue = 0;
  for (int j = 0; j < ahead && j < mine && alive; ++j) {
    issue(j, st_issue);
    st_issue = st_issue + 1 == STAGES ? 0 : st_issue + 1;
  }
  int j_done = 0, st = 0;
  uint32_t parity = 0;
  for (int j = 0; j < mine && alive; ++j) {
    // The stage tile j + ahead goes into was drained by tile j - 2; its stores must have finished reading shared memory
    // (every lane waits on its own bulk groups: append tiles are stored by several lanes).
    if (j + ahead < mine) {
      bulk_wait_read<1>();
      __syncwarp();
      issue(j + ahead, st_issue);
      if (!alive) break;
      st_issue = st_issue + 1 == STAGES ? 0 : st_issue + 1;
    }
    alive = __all_sync(0xffffffffu, wait_bounded(smem_addr(&bars[st]), parity, int(blockIdx.x)));
    if (!alive) break;
    const Tile t = s_tile[st];
    const pkv_layer& ly = P.layers[t.layer];
    unsigned char* stage = smem + size_t(st) * stage_bytes;
    if (t.local >= app_tiles) {
      const unsigned g = t.local - app_tiles;
      const unsigned q = P.tpq_shift >= 0 ? g >> P.tpq_shift : g / tiles_per_q;
      const unsigned e0 = (g - q * tiles_per_q) * ROWS;
      const int nrows = min(ROWS, s.k - int(e0));
      fence_async_smem();  // the zero rows were written through the generic proxy
      __syncwarp();
      if (lane == 0) bulk_store(ly.gathered + (size_t(q) * s.k + e0) * s.width, smem_addr(stage), uint32_t(nrows) * row_bytes);
    } else {
      ensure(j / kBatch);
      if (!alive) break;
      const int a = int(t.local) * ROWS, nrows = min(ROWS, s.T - a);
      // Runs of rows that are contiguous in the pool leave with one bulk store each.
      const unsigned long long rv = lane < nrows ? s_res[(j / kBatch) % kResBatches][(j % kBatch) * ROWS + lane] : kNoRow;
      const long long rid = rv == kNoRow ? -1 : static_cast<long long>(rv);
      const long long prev = __shfl_up_sync(0xffffffffu, rid, 1);
      const bool start = rid >= 0 && (lane == 0 || prev < 0 || rid != prev + 1 || s.row_stride != s.width);
      const unsigned breaks = __ballot_sync(0xffffffffu, start || rid < 0);
      if (start) {
        const unsigned higher = lane == 31 ? 0u : (breaks & ~((2u << lane) - 1u));
        const int next = higher ? __ffs(higher) - 1 : 32;
        bulk_store(ly.row_pool + size_t(rid) * s.row_stride, smem_addr(stage + size_t(lane) * row_bytes), uint32_t(next - lane) * row_bytes);
      }
    }
    bulk_commit();
    __syncwarp();
    if (j % kBatch == kBatch - 1 && lane == 0) mbar_arrive(smem_addr(&res_empty[(j / kBatch) % kResBatches]));
    j_done = j + 1;
    if (++st == STAGES) {
      st = 0;
      parity ^= 1u;
    }
  }
  if (!alive) {
    // Gave up: the loads of the tiles already started get a second, bounded chance to land before the CTA's shared
    // memory is released.
    int st2 = st;
    uint32_t par2 = parity;
    const int polls = min(P.wait_polls, 1 << 18);
    for (int jj = j_done; jj < issued; ++jj) {
      const uint32_t bar = smem_addr(&bars[st2]);
      for (int spin = 0; spin < polls; ++spin) {
        if (mbar_try_wait(bar, par2)) break;
        __nanosleep(256);
      }
      if (++st2 == STAGES) st2 = 0, par2 ^= 1u;
    }
  }
  bulk_wait_all();
  __syncwarp();
}

// ---------------------------------------------------------------------------------------------------------------------
// Reference-shaped single-sequence kernels.
// ---------------------------------------------------------------------------------------------------------------------
struct OneTable {
  const int32_t* table;
  int rows_per_page;
};
__device__ __forceinline__ size_t one_row(const OneTable& t, int r) {
  const int pg = r / t.rows_per_page;
  return size_t(__ldg(&t.table[pg])) * size_t(t.rows_per_page) + size_t(r - pg * t.rows_per_page);
}

// Rows of 16-byte vectors (width % 8 == 0, aligned): one thread per vector.
__global__ void __launch_bounds__(256) store_rows_vec_kernel(const uint4* __restrict__ rows, long long total, int vpr,
                                                             uint16_t* pool, OneTable tb, int row_stride, int row0) {
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
    const int r = int(u / vpr), c = int(u - (long long)r * vpr);
    st_stream(reinterpret_cast<uint4*>(pool + one_row(tb, row0 + r) * size_t(row_stride)) + c, ld_stream(rows + u));
  }
}
// Any width / alignment: one thread per element.
__global__ void __launch_bounds__(256) store_rows_elem_kernel(const uint16_t* __restrict__ rows, long long total, int width,
                                                              uint16_t* pool, OneTable tb, int row_stride, int row0) {
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
    const int r = int(u / width), c = int(u - (long long)r * width);
    pool[one_row(tb, row0 + r) * size_t(row_stride) + c] = rows[u];
  }
}

// fake_quant_fp8 of a row's first quant_cols columns (blocks of `block`, src/kernels/ref_elem.hip:18-41) and store_rows
// in one pass: every 16-byte vector of a row is read once, quantised and dequantised where it lies in the quantised
// columns, and written to its place in the pool. One thread per vector; a block's lanes are neighbours.
__global__ void __launch_bounds__(256) store_rows_fake_fp8_kernel(const uint16_t* __restrict__ rows, long long total, int vpr,
                                                                  int quant_vecs, int group, uint16_t* pool, OneTable tb,
                                                                  int row_stride, int row0) {
  const long long span = ((total + 31) / 32) * 32;  // whole warps stay in the loop: the shuffles need every lane
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < span; u += (long long)gridDim.x * blockDim.x) {
    const bool live = u < total;
    const int r = live ? int(u / vpr) : 0, c = live ? int(u - (long long)r * vpr) : 0;
    const uint4 raw = live ? ld_stream(reinterpret_cast<const uint4*>(rows) + u) : make_uint4(0, 0, 0, 0);
    float v[8];
    pkv::unpack8(raw, v);
    const float amax = pkv::group_max(pkv::absmax8(v), group);
    if (!live) continue;
    uint4* dst = reinterpret_cast<uint4*>(pool + one_row(tb, row0 + r) * size_t(row_stride)) + c;
    if (c < quant_vecs) {
      const float sc = pkv::e8m0_bits_to_f32(pkv::fp8_scale_exp(amax));
      const uint2 codes = pkv::fp8_pack8(v, sc);
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = pkv::f32_to_bf16_bits(pkv::e4m3_bits_to_f32(((i < 2 ? codes.x : codes.y) >> (16 * (i & 1))) & 0xffu) * sc);
        const uint32_t hi = pkv::f32_to_bf16_bits(pkv::e4m3_bits_to_f32(((i < 2 ? codes.x : codes.y) >> (16 * (i & 1) + 8)) & 0xffu) * sc);
        w[i] = lo | (hi << 16);
      }
      st_stream(dst, make_uint4(w[0], w[1], w[2], w[3]));
    } else {
      st_stream(dst, raw);
    }
  }
}

// The KV row chain in front of the append (ewtodd/unholy's kv_chain_row, src/kernels/elem_dev.hip.hpp:50-87) and the
// append itself in one pass: rmsnorm with weight w, rope on the last 2 * npair values, fake_quant_fp8 (block 64) of
// the others, then the row goes to its place in the pool (and / or to rows_out). One warp per row, lane l holds the
// 16-byte vectors l, l + 32, ... of the row (at most kChainVecs each): a quantisation block of 64 values is eight
// neighbouring lanes, a rope pair lies inside one vector. The sum of squares is fp32, lane-partial then a shuffle
// tree; r is the correctly rounded 1 / sqrt (IEEE division and square root, no approximation).
constexpr int kChainVecs = 4;  // rows of up to 1024 values
__global__ void __launch_bounds__(256) kv_chain_store_kernel(const uint16_t* __restrict__ rows, uint16_t* rows_out,
                                                             const uint16_t* __restrict__ w, int n, int dim, float eps,
                                                             const int32_t* __restrict__ pos, const float2* __restrict__ freqs,
                                                             int npair, int quant, uint16_t* pool, OneTable tb, int row_stride, int row0) {
  const int lane = threadIdx.x & 31, vecs = dim >> 3, off = dim - 2 * npair;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n; r += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(rows + size_t(r) * dim);
    float v[kChainVecs][8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kChainVecs; ++i) {
      const int vi = lane + 32 * i;
      pkv::unpack8(vi < vecs ? ld_stream(src + vi) : make_uint4(0, 0, 0, 0), v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    const float rr = 1.0f / sqrtf(ss / float(dim) + eps);
    const int p = __ldg(&pos[r]);
    uint16_t* dst = pool ? pool + one_row(tb, row0 + r) * size_t(row_stride) : nullptr;
#pragma unroll
    for (int i = 0; i < kChainVecs; ++i) {
      const int vi = lane + 32 * i;
      const bool live = vi < vecs;
      float wv[8];
      pkv::unpack8(live ? __ldg(reinterpret_cast<const uint4*>(w) + vi) : make_uint4(0, 0, 0, 0), wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] = pkv::bf16_bits_to_f32(pkv::f32_to_bf16_bits(wv[e] * (v[i][e] * rr)));
      const int c0 = vi * 8;  // first column of this vector
      if (live && c0 >= off) {  // rope: pairs (2t, 2t + 1) of the last 2 * npair columns
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float2 f = __ldg(&freqs[size_t(p) * npair + ((c0 - off + e) >> 1)]);
          const float a = v[i][e], b = v[i][e + 1];
          v[i][e] = pkv::bf16_bits_to_f32(pkv::f32_to_bf16_bits(a * f.x - b * f.y));
          v[i][e + 1] = pkv::bf16_bits_to_f32(pkv::f32_to_bf16_bits(a * f.y + b * f.x));
        }
      }
      // fake_quant_fp8, block 64 = this lane and its seven neighbours (every lane runs the shuffles)
      const float amax = pkv::group_max(pkv::absmax8(v[i]), 8);
      uint32_t out[4];
      if (quant && c0 < off) {
        const float sc = pkv::e8m0_bits_to_f32(pkv::fp8_scale_exp(amax));
        const uint2 codes = pkv::fp8_pack8(v[i], sc);
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const uint32_t lo = pkv::f32_to_bf16_bits(pkv::e4m3_bits_to_f32(((e < 4 ? codes.x : codes.y) >> (8 * (e & 3))) & 0xffu) * sc);
          const uint32_t hi = pkv::f32_to_bf16_bits(pkv::e4m3_bits_to_f32(((e < 4 ? codes.x : codes.y) >> (8 * ((e + 1) & 3))) & 0xffu) * sc);
          out[e >> 1] = lo | (hi << 16);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; e += 2) out[e >> 1] = (__float_as_uint(v[i][e]) >> 16) | (__float_as_uint(v[i][e + 1]) & 0xffff0000u);
      }
      if (live) {
        const uint4 o = make_uint4(out[0], out[1], out[2], out[3]);
        if (dst) st_stream(reinterpret_cast<uint4*>(dst) + vi, o);
        if (rows_out) reinterpret_cast<uint4*>(rows_out + size_t(r) * dim)[vi] = o;
      }
    }
  }
}

// MXFP4 append of 128-wide rows: 16 threads per row.
__global__ void __launch_bounds__(256) store_rows_fp4_kernel(const uint16_t* __restrict__ rows, int n, uint8_t* pool,
                                                             OneTable tb, int row0) {
  const long long span = ((long long)n * 16 + 31) / 32 * 32;
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < span; u += (long long)gridDim.x * blockDim.x) {
    const int r = int(u >> 4), j = int(u & 15);
    const bool live = r < n;
    float v[8];
    if (live) pkv::unpack8(*reinterpret_cast<const uint4*>(rows + size_t(r) * PKV_FP4_ROW_DIM + j * 8), v);
    else
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    const uint32_t se = pkv::fp4_scale_exp(pkv::group_max(pkv::absmax8(v), 4));
    const uint32_t codes = pkv::fp4_pack8(v, pkv::e8m0_bits_to_f32(se));
    const int base = (threadIdx.x & 31) & 16;
    const uint32_t s0 = __shfl_sync(0xffffffffu, se, base), s1 = __shfl_sync(0xffffffffu, se, base + 4),
                   s2 = __shfl_sync(0xffffffffu, se, base + 8), s3 = __shfl_sync(0xffffffffu, se, base + 12);
    if (!live) continue;
    const int lr = row0 + r, pgi = lr / tb.rows_per_page, slot = lr - pgi * tb.rows_per_page;
    uint8_t* pg = pool + size_t(__ldg(&tb.table[pgi])) * size_t(tb.rows_per_page) * 68u;
    *reinterpret_cast<uint32_t*>(pg + size_t(slot) * 64u + j * 4) = codes;
    if (j == 0)
      *reinterpret_cast<uint32_t*>(pg + size_t(tb.rows_per_page) * 64u + size_t(slot) * 4u) =
          s0 | (s1 << 8) | (s2 << 16) | (s3 << 24);
  }
}

// MXFP4 decode: one thread per 8 values (4 code bytes), 16-byte bf16 store.
__global__ void __launch_bounds__(256) load_rows_fp4_kernel(const uint8_t* __restrict__ pool, OneTable tb, int row0, int n,
                                                            uint16_t* __restrict__ out) {
  const long long total = (long long)n * 16;
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
    const int r = int(u >> 4), j = int(u & 15);
    const int lr = row0 + r, pgi = lr / tb.rows_per_page, slot = lr - pgi * tb.rows_per_page;
    const uint8_t* pg = pool + size_t(__ldg(&tb.table[pgi])) * size_t(tb.rows_per_page) * 68u;
    const uint32_t codes = *reinterpret_cast<const uint32_t*>(pg + size_t(slot) * 64u + j * 4);
    const float sc = pkv::e8m0_bits_to_f32(pg[size_t(tb.rows_per_page) * 64u + size_t(slot) * 4u + (j >> 2)]);
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = pkv::e2m1_bits_to_f32((codes >> (4 * i)) & 15u) * sc;
    store8_bf16(out + size_t(r) * PKV_FP4_ROW_DIM + j * 8, o, true);
  }
}

// fp8 append into the two-array layout: one thread per 8 values.
__global__ void __launch_bounds__(256) store_rows_fp8_kernel(const uint16_t* __restrict__ rows, int n, int width, int block,
                                                             uint8_t* codes, uint8_t* scales, OneTable tb, int s0) {
  const int per_row = width >> 3, group = block >> 3, nb = width / block;
  const long long total = (long long)n * per_row;
  const long long span = (total + 31) / 32 * 32;
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < span; u += (long long)gridDim.x * blockDim.x) {
    const bool live = u < total;
    const int r = live ? int(u / per_row) : 0, j = live ? int(u - (long long)r * per_row) : 0;
    float v[8];
    if (live) pkv::unpack8(*reinterpret_cast<const uint4*>(rows + size_t(r) * width + j * 8), v);
    else
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    const uint32_t se = pkv::fp8_scale_exp(pkv::group_max(pkv::absmax8(v), group));
    if (!live) continue;
    const uint2 c8 = pkv::fp8_pack8(v, pkv::e8m0_bits_to_f32(se));
    const size_t rid = one_row(tb, s0 + r);
    *reinterpret_cast<uint2*>(codes + rid * size_t(width) + j * 8) = c8;
    if (j % group == 0) scales[rid * size_t(nb) + j / group] = uint8_t(se);
  }
}

// The gather for one sequence (one block-table row), the shape of one reference attention call.
__global__ void __launch_bounds__(kVecThreads) gather_one_kernel(const uint16_t* __restrict__ pool, OneTable tb,
                                                                int row_stride, int width,
                                                                const int32_t* __restrict__ idx,
                                                                const int32_t* __restrict__ q_visible, int T, int k,
                                                                uint16_t* __restrict__ out) {
  __shared__ const uint4* s_src[kGatherRows];
  const int tiles_per_q = (k + kGatherRows - 1) / kGatherRows;
  const long long total = (long long)T * tiles_per_q;
  for (long long w = blockIdx.x; w < total; w += gridDim.x) {
    const int t = int(w / tiles_per_q), e0 = int(w - (long long)t * tiles_per_q) * kGatherRows;
    if (threadIdx.x < kGatherRows) {
      const int e = e0 + int(threadIdx.x);
      const uint4* p = nullptr;
      if (e < k) {
        const int row = __ldg(&idx[size_t(t) * k + e]);
        if (row >= 0 && row < __ldg(&q_visible[t]))
          p = reinterpret_cast<const uint4*>(pool + one_row(tb, row) * size_t(row_stride));
      }
      s_src[threadIdx.x] = p;
    }
    __syncthreads();
    copy_tile_vec(s_src, reinterpret_cast<uint4*>(out + (size_t(t) * k + e0) * width), min(kGatherRows, k - e0), width >> 3);
    __syncthreads();
  }
}

// Gather with dequantisation for fp8 rows (the gather loop of src/kernels/glm_fast.hip:190-227): entry -> physical
// row -> e4m3 codes [width] and one e8m0 scale per `block` values -> bf16 = code * 2^scale (exact). One unit = 16
// codes: a 16-byte load, sixteen decodes, two 16-byte stores; a thread has four units in flight. Masked entries give
// zero rows.
//
// Decoding without a conversion instruction. A normal e4m3 code b = s eeee mmm times a power of two IS a bf16 number
// with the same three mantissa bits: its low seven bits shifted left by four land exactly on bf16's exponent and
// mantissa fields (eeee in the low exponent bits, mmm in the top mantissa bits), and the scale only adds to the
// exponent. With one code per 16-bit lane of w (a byte permute), w * 16 puts the low seven bits in place and the sign
// at bit 11; adding sign * 0xF0 moves it to bit 15 (0x80 * 16 + 0x80 * 0xF0 = 0x8000); nothing carries between the lanes
// while the result is a normal bf16 number: scale bytes 7 .. 246. Exact: nothing is rounded. Three ways through a unit
// of 16 codes, told apart with carries into bit 7 of each byte of t = code & 0x7f (no sum below exceeds 0xfe):
//   t + 0x78 carries when t >= 8 (a normal code), t + 0x7f when t >= 1 (not a zero), t + 0x01 when t == 0x7f (a NaN);
//   * all codes normal (what quantised rows hold almost everywhere): the integer decode as it stands;
//   * zeros among them, nothing else (padding, rows never written): the same with the zero lanes masked to +-0;
//   * e4m3 subnormals or NaN codes among them (one warp in twenty of a quantised pool meets one somewhere in its 512
//     codes): the masked decode, then those codes alone redone in floating point as the reference does it;
//   * a scale byte outside 7 .. 246: all sixteen codes in floating point.
// (Decoding pairs on the conversion hardware instead, fp16 -> fp32 -> bf16, kept that unit 84 % busy and took the same
// time at 40 registers per thread; what the kernel is short of is issue slots and overlap of its scattered loads.)
__device__ __forceinline__ uint32_t dequant_lanes(uint32_t w, uint32_t exp_add) {
  return w * 16u + exp_add + (w & 0x00800080u) * 0xF0u;
}
__device__ __forceinline__ uint32_t dequant_lanes_zeros(uint32_t w, uint32_t exp_add) {
  const uint32_t t = w & 0x007f007fu;
  const uint32_t keep = (((t + 0x007f007fu) >> 7) & 0x00010001u) * 0xffffu;  // 0xffff in the lanes whose code is not a zero
  return ((t * 16u + exp_add) & keep) | ((w & 0x00800080u) << 8);
}
__device__ __forceinline__ void dequant_unit(const uint4& q, uint32_t scale_bits, uint32_t* w16) {
  const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
  // All sixteen codes normal? Bit 7 of every byte of (t + 0x78) & ~(t + 0x01) says "8 <= t < 0x7f".
  uint32_t normal = 0xffffffffu;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t t = qs[i] & 0x7f7f7f7fu;
    normal &= (t + 0x78787878u) & ~(t + 0x01010101u);
  }
  const bool scale_ok = scale_bits - 7u <= 239u;
  const uint32_t exp_add = ((scale_bits - 7u) << 7) * 0x00010001u;  // the same exponent offset in both 16-bit lanes
  if ((~normal & 0x80808080u) == 0u && scale_ok) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w16[2 * i] = dequant_lanes(__byte_perm(qs[i], 0u, 0x4140u), exp_add);      // codes 0 and 1 of the word
      w16[2 * i + 1] = dequant_lanes(__byte_perm(qs[i], 0u, 0x4342u), exp_add);  // codes 2 and 3
    }
    return;
  }
  // Not all normal. With a scale in range: the masked decode for every code (zeros come out right, normal codes too),
  // then only the codes that are e4m3 subnormals or NaNs are redone one by one in floating point, operation for
  // operation as the reference does it (typically one code of the sixteen). Other scales: all sixteen that way.
  if (scale_ok) {
    uint32_t odd[4], any = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t t = qs[i] & 0x7f7f7f7fu;
      odd[i] = (((t + 0x7f7f7f7fu) & ~(t + 0x78787878u)) | (t + 0x01010101u)) & 0x80808080u;
      any |= odd[i];
      w16[2 * i] = dequant_lanes_zeros(__byte_perm(qs[i], 0u, 0x4140u), exp_add);
      w16[2 * i + 1] = dequant_lanes_zeros(__byte_perm(qs[i], 0u, 0x4342u), exp_add);
    }
    if (any == 0u) return;
    const float sc = pkv::e8m0_bits_to_f32(scale_bits);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((odd[i >> 2] >> (8 * (i & 3) + 7)) & 1u) {
        const uint32_t code = (qs[i >> 2] >> (8 * (i & 3))) & 0xffu;
        const uint32_t bits = pkv::f32_to_bf16_bits(pkv::e4m3_bits_to_f32(code) * sc);
        w16[i >> 1] = (i & 1) ? (w16[i >> 1] & 0x0000ffffu) | (bits << 16) : (w16[i >> 1] & 0xffff0000u) | bits;
      }
    }
    return;
  }
  const float sc = pkv::e8m0_bits_to_f32(scale_bits);
#pragma unroll
  for (int i = 0; i < 8; ++i) w16[i] = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t code = (qs[i >> 2] >> (8 * (i & 3))) & 0xffu;
    w16[i >> 1] |= pkv::f32_to_bf16_bits(pkv::e4m3_bits_to_f32(code) * sc) << (16 * (i & 1));
  }
}
// Where logical row `row` of query row t lives: one sequence's table (the reference-shaped call) ...
struct OneSeqRows {
  OneTable tb;
  __device__ __forceinline__ int begin(int) const { return 0; }
  __device__ __forceinline__ long long rid(int, int, int row) const { return (long long)one_row(tb, row); }
};
// ... or the step's chunk list and block tables (every sequence of a step in one launch; bounds are checked).
struct StepRows {
  pkv_step s;
  // the query row's slot: loaded before (not after) its index entry, so the two chains overlap
  __device__ __forceinline__ int begin(int t) const {
    const int qc = __ldg(&s.q_chunk[t]);
    return unsigned(qc) < unsigned(s.nchunks) ? s.chunks[qc].slot : -1;  // -1: physical_row reports it
  }
  __device__ __forceinline__ long long rid(int slot, int t, int row) const { return physical_row(s, slot, row, t); }
};
// Entries given as selected pools instead of a token list: entry j of query row t is what glm_idx_expand
// (src/kernels/glm_fast.hip:737-748) would have written at idx[t][j] — the tokens of the min((p + 1) / pool, kp) valid
// pools, then the (p + 1) % pool tokens of the query's incomplete pool, then -1 — computed where it is needed.
struct PoolList {
  const int32_t* pools;  // [T][kp]; nullptr: the entries come from idx
  const int32_t* pos;    // [T]
  int kp, pool;
  __device__ __forceinline__ int entry(int t, int j) const {
    const int p = __ldg(&pos[t]);
    const int full = (p + 1) / pool, valid = full < kp ? full : kp, tail = (p + 1) % pool;
    if (j < valid * pool) return __ldg(&pools[size_t(t) * kp + j / pool]) * pool + j % pool;
    if (j < valid * pool + tail) return p + 1 - tail + (j - valid * pool);
    return -1;
  }
};

// 8 warps move data, a ninth resolves the NEXT tile's entries (index -> block table -> physical row) meanwhile, so the
// three dependent loads of a resolution are off the data warps' path: one barrier per tile. Four CTAs per SM: the four
// 16-byte units a data thread keeps in flight need 56 registers; at five CTAs (40 registers) they spill, and launches
// of more than a few tiles per CTA ran 10 % slower for it.
constexpr int kFp8Threads = 256 + 32, kFp8CtasPerSm = 4, kFp8Unroll = 4;
template <class ROWS>
__global__ void __launch_bounds__(kFp8Threads, kFp8CtasPerSm) gather_fp8_kernel(const uint8_t* __restrict__ codes,
                                                                 const uint8_t* __restrict__ scales,
                                                                 const __grid_constant__ ROWS rows, int width, int block,
                                                                 const int32_t* __restrict__ idx,
                                                                 const int32_t* __restrict__ q_visible, int T, int k,
                                                                 uint16_t* __restrict__ out, const PoolList pl) {
  __shared__ long long s_rid[2][kGatherRows];
  // Programmatic dependent launch: the grid may be scheduled while the previous kernel of the stream drains; nothing
  // above reads global memory, everything below waits for that kernel's writes (the index list, the pools).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tiles_per_q = (k + kGatherRows - 1) / kGatherRows, upr = width >> 4, nb = width / block;
  // A unit's row and column by shift and mask where the row length allows (a division costs as much as the decode);
  // the column's scale byte always by a shift: a block is 2, 4 or 8 units.
  const int upr_shift = (upr & (upr - 1)) == 0 ? 31 - __clz(upr) : -1, unit_to_block = 27 - __clz(block);
  const unsigned total_tiles = unsigned(T) * unsigned(tiles_per_q);  // (the host keeps this below 2^31)
  const bool resolver = threadIdx.x >= 256;
  const auto resolve = [&](unsigned t, unsigned tile_in_q, int buf) {
    const int e = int(tile_in_q) * kGatherRows + int(threadIdx.x) - 256;
    long long rid = -1;
    if (e < k) {
      const int slot = rows.begin(int(t)), vis = __ldg(&q_visible[t]);
      const int row = pl.pools ? pl.entry(int(t), e) : __ldg(&idx[size_t(t) * k + e]);
      if (row >= 0 && row < vis) rid = rows.rid(slot, int(t), row);
    }
    s_rid[buf][threadIdx.x - 256] = rid;
  };
  // A CTA's tiles are blockIdx.x, + gridDim.x, ...: (query row, tile in the row) advance by constants, one division per
  // kernel instead of one per tile and thread.
  const unsigned dq = gridDim.x / unsigned(tiles_per_q), dr = gridDim.x - dq * unsigned(tiles_per_q);
  unsigned tq = blockIdx.x / unsigned(tiles_per_q), tile_in_q = blockIdx.x - tq * unsigned(tiles_per_q);
  const auto next_tile = [&](unsigned& t, unsigned& i) {
    t += dq, i += dr;
    if (i >= unsigned(tiles_per_q)) i -= unsigned(tiles_per_q), ++t;
  };
  if (resolver && blockIdx.x < total_tiles) resolve(tq, tile_in_q, 0);
  __syncthreads();
  // A data thread's units of a tile are tid, tid + 256, ...: with a power-of-two row length of at most 256 units their
  // column is the same for every unit and their rows are 256 / upr apart.
  const bool fixed_column = upr_shift >= 0 && upr <= 256;
  const int tid = int(threadIdx.x);
  const int r0 = fixed_column ? tid >> upr_shift : 0, c0 = fixed_column ? tid & (upr - 1) : 0, rstep = fixed_column ? 256 >> upr_shift : 0;
  // A unit's 32 bytes leave as one 256-bit store where the output allows: two 128-bit stores from two instructions
  // reach L2 as two partial writes of the same sector.
  const bool wide_stores = (reinterpret_cast<uintptr_t>(out) & 31u) == 0;
  int buf = 0;
  for (unsigned w = blockIdx.x; w < total_tiles; w += gridDim.x, buf ^= 1) {
    if (resolver) {
      unsigned tn = tq, in = tile_in_q;
      next_tile(tn, in);
      if (w + gridDim.x < total_tiles) resolve(tn, in, buf ^ 1);
    } else {
      const int e0 = int(tile_in_q) * kGatherRows;
      const int nrows = min(kGatherRows, k - e0), total = nrows * upr;
      uint4* o = reinterpret_cast<uint4*>(out + (size_t(tq) * k + e0) * width);
      for (int base = 0; base < total; base += kFp8Unroll * 256) {
        uint4 q[kFp8Unroll];
        uint32_t sb[kFp8Unroll];
        bool live[kFp8Unroll];
        const int rb = fixed_column ? base >> upr_shift : 0;
#pragma unroll
        for (int j = 0; j < kFp8Unroll; ++j) {
          const int u = base + j * 256 + tid;
          live[j] = false;
          if (u < total) {
            const int r = fixed_column ? rb + r0 + j * rstep : u / upr, c = fixed_column ? c0 : u - r * upr;
            const long long rid = s_rid[buf][r];
            if (rid >= 0) {
              live[j] = true;
              q[j] = ld_stream(reinterpret_cast<const uint4*>(codes + size_t(rid) * width) + c);
              sb[j] = __ldg(&scales[size_t(rid) * nb + (c >> unit_to_block)]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < kFp8Unroll; ++j) {
          const int u = base + j * 256 + tid;
          if (u < total) {
            uint32_t w16[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (live[j]) dequant_unit(q[j], sb[j], w16);
            if (wide_stores) {
              st_stream32(o + 2 * u, w16);
            } else {
              st_stream(o + 2 * u, make_uint4(w16[0], w16[1], w16[2], w16[3]));
              st_stream(o + 2 * u + 1, make_uint4(w16[4], w16[5], w16[6], w16[7]));
            }
          }
        }
      }
    }
    next_tile(tq, tile_in_q);
    __syncthreads();  // the next tile's rows are resolved, this tile's are no longer read
  }
}

// hadamard128 in place: 16 lanes per 128-value segment, 8 values each.
__global__ void __launch_bounds__(256) hadamard128_kernel(uint16_t* __restrict__ x, size_t nseg) {
  const size_t groups = (nseg + 1) / 2 * 2;  // whole warps stay in the loop: the shuffles need every lane
  for (size_t g = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 4; g < groups; g += (size_t(gridDim.x) * blockDim.x) >> 4) {
    const int j = threadIdx.x & 15;
    const bool live = g < nseg;
    uint4* p = reinterpret_cast<uint4*>(x + (live ? g : 0) * 128) + j;
    float v[8];
    pkv::unpack8(live ? *p : make_uint4(0, 0, 0, 0), v);
    pkv::hadamard128_lanes(v, j);
    if (live) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = (__float_as_uint(v[2 * i]) >> 16) | (__float_as_uint(v[2 * i + 1]) & 0xffff0000u);
      *p = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

__global__ void __launch_bounds__(256) copy16_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < n; i += 4 * stride) {
    const uint4 a = ld_stream(src + i), b = ld_stream(src + i + stride), c = ld_stream(src + i + 2 * stride),
                d = ld_stream(src + i + 3 * stride);
    st_stream(dst + i, a);
    st_stream(dst + i + stride, b);
    st_stream(dst + i + 2 * stride, c);
    st_stream(dst + i + 3 * stride, d);
  }
  for (; i < n; i += stride) st_stream(dst + i, ld_stream(src + i));
  __threadfence_system();  // as the reference's copy kernels: a flag written after this kernel orders the data for any observer
}
__global__ void __launch_bounds__(256) copy1_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) dst[i] = src[i];
  __threadfence_system();
}

// Page moves: work item = (pool, pair, 16 KB piece of the page).
struct PageCopyParams {
  int npools, n, num_src_pages, num_dst_pages;
  const int32_t* src_ids;
  const int32_t* dst_ids;
  pkv_pool_desc pools[128];
};
constexpr int kPieceVecs = 1536;  // 24 KB = a third of a 73,728-byte row page; six 16-byte vectors per thread
// grid.y = pool; the CTAs of a pool stride over its (pair, piece) items.
__global__ void __launch_bounds__(256) copy_pages_kernel(const __grid_constant__ PageCopyParams P) {
  const pkv_pool_desc d = P.pools[blockIdx.y];
  const unsigned vecs = unsigned(d.page_bytes / 16);
  const unsigned per_page = (vecs + kPieceVecs - 1) / kPieceVecs;
  const unsigned items = unsigned(P.n) * per_page;
  for (unsigned w = blockIdx.x; w < items; w += gridDim.x) {
    const unsigned pair = w / per_page, piece = w - pair * per_page;
    const int sp = __ldg(&P.src_ids[pair]), dp = __ldg(&P.dst_ids[pair]);
    if (sp < 0 || dp < 0 || (P.num_src_pages > 0 && sp >= P.num_src_pages) || (P.num_dst_pages > 0 && dp >= P.num_dst_pages)) {
      if (threadIdx.x == 0) report(1, int(pair));
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(d.src_base) + size_t(sp) * d.page_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(d.dst_base) + size_t(dp) * d.page_bytes);
    const unsigned lo = piece * kPieceVecs, hi = min(vecs, lo + kPieceVecs);
    uint4 v[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      const unsigned u = lo + unsigned(i) * 256u + threadIdx.x;
      if (u < hi) v[i] = ld_stream(src + u);
    }
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      const unsigned u = lo + unsigned(i) * 256u + threadIdx.x;
      if (u < hi) st_stream(dst + u, v[i]);
    }
  }
}

// Page moves inside one device's pools (copy-on-write, compaction: src_base == dst_base for every pool) through the
// bulk-copy engine: an item is one piece (at most kBulkPiece bytes) of one page of one pool; single-warp CTAs stride over
// the items and keep a ring of STAGES pieces rotating (loads of STAGES - 2 pieces in flight while two drain). The
// (source, destination) page ids of 32 items are looked up at a time, one lane per item, a batch ahead. Never used when
// a source pool may belong to another device: bulk copies do not read peer memory in this library.
constexpr unsigned kBulkPiece = 18432;  // a quarter of a 73,728-byte row page
constexpr int kCopyStages = 4;
struct PageCopyBulkParams {
  int npools, n, num_src_pages, num_dst_pages;
  int wait_polls;
  const int32_t* src_ids;
  const int32_t* dst_ids;
  unsigned first_item[129];  // items before pool p; [npools] = all items
  pkv_pool_desc pools[128];
};
__global__ void __launch_bounds__(32) copy_pages_bulk_kernel(const __grid_constant__ PageCopyBulkParams P) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[kCopyStages];
  __shared__ const unsigned char* s_src[2][32];
  __shared__ unsigned char* s_dst[2][32];
  __shared__ unsigned s_bytes[2][32];
  __shared__ unsigned char* s_stage_dst[kCopyStages];
  __shared__ unsigned s_stage_bytes[kCopyStages];
  const int lane = threadIdx.x;
  const unsigned total = P.first_item[P.npools];
  const unsigned first = blockIdx.x, stride = gridDim.x;
  const int mine = first < total ? int((total - first + stride - 1) / stride) : 0;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kCopyStages; ++i) mbar_init(smem_addr(&bars[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  auto resolve_batch = [&](int b) {
    const int j = b * 32 + lane;
    const unsigned char* src = nullptr;
    unsigned char* dst = nullptr;
    unsigned bytes = 0;
    if (j < mine) {
      const unsigned item = first + unsigned(j) * stride;
      int lo = 0, hi = P.npools;  // the pool holding the item: last p with first_item[p] <= item
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (P.first_item[mid] <= item) lo = mid;
        else hi = mid;
      }
      const pkv_pool_desc d = P.pools[lo];
      const unsigned pieces = unsigned((d.page_bytes + kBulkPiece - 1) / kBulkPiece);
      const unsigned rel = item - P.first_item[lo], pair = rel / pieces, piece = rel - pair * pieces;
      const int sp = __ldg(&P.src_ids[pair]), dp = __ldg(&P.dst_ids[pair]);
      if (unsigned(sp) >= unsigned(P.num_src_pages) || unsigned(dp) >= unsigned(P.num_dst_pages)) {
        report(1, int(pair));
      } else {
        const size_t off = size_t(piece) * kBulkPiece;
        bytes = unsigned(min(size_t(kBulkPiece), size_t(d.page_bytes) - off));
        src = static_cast<const unsigned char*>(d.src_base) + size_t(sp) * d.page_bytes + off;
        dst = static_cast<unsigned char*>(d.dst_base) + size_t(dp) * d.page_bytes + off;
      }
    }
    s_src[b & 1][lane] = src;
    s_dst[b & 1][lane] = dst;
    s_bytes[b & 1][lane] = bytes;
    __syncwarp();
  };
  auto issue = [&](int j, int st) {
    if (lane == 0) {
      const int slot = (j >> 5) & 1, i = j & 31;
      const unsigned bytes = s_bytes[slot][i];
      s_stage_dst[st] = s_dst[slot][i];
      s_stage_bytes[st] = bytes;
      const uint32_t bar = smem_addr(&bars[st]);
      mbar_expect_tx(bar, bytes);  // zero bytes (a skipped item): the phase completes with the arrival alone
      if (bytes) bulk_load(smem_addr(smem + size_t(st) * kBulkPiece), s_src[slot][i], bytes, bar);
    }
    __syncwarp();
    if ((j & 31) == 0 && ((j >> 5) + 1) * 32 < mine) resolve_batch((j >> 5) + 1);
  };
  constexpr int ahead = kCopyStages - 2;
  if (mine > 0) resolve_batch(0);
  int st_issue = 0, issued = 0;
  for (; issued < ahead && issued < mine; ++issued) {
    issue(issued, st_issue);
    st_issue = st_issue + 1 == kCopyStages ? 0 : st_issue + 1;
  }
  int st = 0, j = 0;
  uint32_t parity = 0;
  bool alive = true;
  for (; j < mine; ++j) {
    if (issued < mine) {
      if (lane == 0) bulk_wait_read<1>();  // the stage about to be refilled was drained two items ago
      __syncwarp();
      issue(issued++, st_issue);
      st_issue = st_issue + 1 == kCopyStages ? 0 : st_issue + 1;
    }
    const uint32_t bar = smem_addr(&bars[st]);
    alive = false;
    for (int spin = 0; spin < P.wait_polls; ++spin)
      if (mbar_try_wait_for(bar, parity, 1000u)) {
        alive = true;
        break;
      }
    alive = __all_sync(0xffffffffu, alive);
    if (!alive) {
      report(3, int(blockIdx.x));
      break;
    }
    if (lane == 0) {
      if (s_stage_bytes[st]) bulk_store(s_stage_dst[st], smem_addr(smem + size_t(st) * kBulkPiece), s_stage_bytes[st]);
      bulk_commit();
    }
    __syncwarp();
    if (++st == kCopyStages) {
      st = 0;
      parity ^= 1u;
    }
  }
  if (!alive) {  // the loads already started get a second, bounded chance to land before shared memory is released
    const int polls = min(P.wait_polls, 1 << 18);
    for (int jj = j; jj < issued; ++jj) {
      const uint32_t bar = smem_addr(&bars[st]);
      for (int spin = 0; spin < polls; ++spin) {
        if (mbar_try_wait(bar, parity)) break;
        __nanosleep(256);
      }
      if (++st == kCopyStages) st = 0, parity ^= 1u;
    }
  }
  if (lane == 0) bulk_wait_all();
  __syncwarp();
}

int grid_for(long long work_items, int threads, int per_sm) {
  const DeviceInfo& d = device_info();
  const long long cap = (long long)(d.ok ? d.sms : 148) * per_sm;
  const long long want = (work_items + threads - 1) / threads;
  return int(std::max<long long>(1, std::min(want, cap)));
}

int check_quant_shape(int rows, int cols, int block, const char* name) {
  if (rows < 0 || cols < 0) return fail(PKV_ERR_ARG, std::string(name) + ": negative shape");
  if (block != 32 && block != 64 && block != 128) return fail(PKV_ERR_ARG, std::string(name) + ": block must be 32, 64 or 128");
  if (cols % block != 0) return fail(PKV_ERR_ARG, std::string(name) + ": cols must be a multiple of block");
  return PKV_OK;
}

template <int STAGES, int ROWS, int BATCH>
int launch_bulk_b(const StepParams& P0, int ctas_per_sm, cudaStream_t st) {
  StepParams P = P0;
  P.resolve_late = tuning().resolve_late;
  const int row_tiles = (P.s.T + ROWS - 1) / ROWS;
  P.append_tiles = P0.append_tiles ? row_tiles : 0;
  P.key_tiles = P0.key_tiles ? row_tiles : 0;
  const size_t smem = size_t(STAGES) * ROWS * size_t(P.s.width) * 2u;
  if (smem > 224u * 1024u) return fail(PKV_ERR_LIMIT, "pkv_step_run: rows too wide for the bulk pipeline");
  // Dynamic shared memory above 48 KB has to be opted into, per device and per kernel instantiation.
  static thread_local size_t opted[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48u * 1024u && dev >= 0 && dev < 64 && opted[dev] < smem) {
    const cudaError_t e = cudaFuncSetAttribute(step_bulk_kernel<STAGES, ROWS, BATCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
    opted[dev] = smem;
  }
  const DeviceInfo& d = device_info();
  const int sms = d.ok ? d.sms : 148;
  int per_sm = ctas_per_sm > 0 ? ctas_per_sm : int((227u * 1024u) / (smem + 2048u + 8u * ROWS * STAGES));
  per_sm = std::max(1, std::min(per_sm, 32));
  const int tpq = (P.s.k + ROWS - 1) / ROWS;
  P.tpq_shift = -1;
  for (int b = 0; b < 31; ++b)
    if (tpq == (1 << b)) P.tpq_shift = b;
  const long long tiles = (long long)P.L * ((long long)P.s.Q * tpq + P.append_tiles + P.key_tiles);
  if (tiles == 0) return PKV_OK;
  if (tiles >= (1ll << 31) - (1ll << 20)) return fail(PKV_ERR_LIMIT, "pkv_step_run: more than 2^31 tiles in one launch");
  const int grid = int(std::max<long long>(1, std::min<long long>(tiles, (long long)sms * per_sm)));
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(grid));
  cfg.blockDim = dim3(32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tuning().pdl ? 1 : 0;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, step_bulk_kernel<STAGES, ROWS, BATCH>, P);
  if (le != cudaSuccess) return fail_cuda("step_bulk_kernel launch", le);
  return PKV_OK;
}

// Launches with many tiles per CTA (a decode step over long contexts) run best with 8-row tiles resolved one at a
// time; launches with only a few tiles per CTA (a prefill chunk, a small shard) with 4-row tiles, twice the CTAs and
// whole-warp batches (measured on B200: 5.9 vs 5.4 TB/s for the first kind, 4.4 vs 3.0 TB/s for the second).
bool many_tiles_per_cta(const StepParams& P) {
  const DeviceInfo& d = device_info();
  const long long row_tiles = (P.s.T + 7) / 8;
  const long long tiles8 = (long long)P.L * ((long long)P.s.Q * ((P.s.k + 7) / 8) + (P.append_tiles ? row_tiles : 0) + (P.key_tiles ? row_tiles : 0));
  return tiles8 >= 6ll * 8 * (d.ok ? d.sms : 148);
}

template <int STAGES, int ROWS>
int launch_bulk(const StepParams& P, int ctas_per_sm, cudaStream_t st) {
  constexpr int kFull = 32 / ROWS;
  const int want = tuning().batch >= 0 ? tuning().batch : (many_tiles_per_cta(P) ? 1 : 0);
  if (want == 1) return launch_bulk_b<STAGES, ROWS, 1>(P, ctas_per_sm, st);
  if constexpr (kFull >= 2) {
    if (want == 2) return launch_bulk_b<STAGES, ROWS, 2>(P, ctas_per_sm, st);
  }
  return launch_bulk_b<STAGES, ROWS, kFull>(P, ctas_per_sm, st);
}

int dispatch_bulk(const StepParams& P, int shape, int ctas_per_sm, cudaStream_t st) {
  if (shape == 0) shape = many_tiles_per_cta(P) ? 308 : 304;
  switch (shape) {  // STAGES * 100 + ROWS
    case 304: return launch_bulk<3, 4>(P, ctas_per_sm, st);
    case 308: return launch_bulk<3, 8>(P, ctas_per_sm, st);
    case 408: return launch_bulk<4, 8>(P, ctas_per_sm, st);
    case 316: return launch_bulk<3, 16>(P, ctas_per_sm, st);
    default: return fail(PKV_ERR_ARG, "PKV_BULK_SHAPE names no compiled shape of the single-warp pipeline (304, 308, 408, 316)");
  }
}

template <int STAGES, int ROWS>
int launch_pipe(const StepParams& P0, int ctas_per_sm, cudaStream_t st) {
  StepParams P = P0;
  P.wait_polls = std::max(1, tuning().wait_polls);
  P.debug_tile = tuning().debug_tile;
  P.append_tiles = P0.append_tiles ? (P.s.T + ROWS - 1) / ROWS : 0;
  const bool keys = P0.key_tiles != 0;
  // Key workers per CTA: two when a CTA's share of the key rows is small (a chunk of one layer), kKeyWarps when it is
  // large (many layers per launch): each worker runs its address chains one after the other.
  const long long key_units = keys ? (long long)P.L * ((P.s.T + 1) / 2) : 0;
  const int key_warps = !keys ? 0 : (key_units > 8ll * 148 * 7 ? kKeyWarps : 2);
  const int threads = 32 * (kFirstKeyWarp + key_warps);
  const size_t smem = size_t(STAGES) * ROWS * size_t(P.s.width) * 2u;
  if (smem > 224u * 1024u) return fail(PKV_ERR_LIMIT, "pkv_step_run: rows too wide for the bulk pipeline");
  static thread_local size_t opted[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48u * 1024u && dev >= 0 && dev < 64 && opted[dev] < smem) {
    const cudaError_t e = cudaFuncSetAttribute(step_pipe_kernel<STAGES, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
    opted[dev] = smem;
  }
  const DeviceInfo& d = device_info();
  const int sms = d.ok ? d.sms : 148;
  int per_sm = ctas_per_sm > 0 ? ctas_per_sm : int((227u * 1024u) / (smem + 2048u));
  int resident = 0;  // registers may allow fewer CTAs than shared memory does
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, step_pipe_kernel<STAGES, ROWS>, threads, smem) == cudaSuccess && resident > 0)
    per_sm = std::min(per_sm, resident);
  per_sm = std::max(1, std::min({per_sm, 2048 / threads, 32}));
  const int tpq = (P.s.k + ROWS - 1) / ROWS;
  P.tpq_shift = -1;
  for (int b = 0; b < 31; ++b)
    if (tpq == (1 << b)) P.tpq_shift = b;
  const long long tiles = (long long)P.L * ((long long)P.s.Q * tpq + P.append_tiles);
  const long long key_ctas = keys ? (key_units + key_warps - 1) / key_warps : 0;
  if (tiles == 0 && key_ctas == 0) return PKV_OK;
  if (tiles >= (1ll << 31) - (1ll << 20)) return fail(PKV_ERR_LIMIT, "pkv_step_run: more than 2^31 tiles in one launch");
  const int grid = int(std::max<long long>(1, std::min<long long>(std::max(tiles, key_ctas), (long long)sms * per_sm)));
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(grid));
  cfg.blockDim = dim3(unsigned(threads));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tuning().pdl ? 1 : 0;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, step_pipe_kernel<STAGES, ROWS>, P);
  if (le != cudaSuccess) return fail_cuda("step_pipe_kernel launch", le);
  return PKV_OK;
}

// Which of the two bulk pipelines takes a launch. A long run of gather tiles per CTA (a decode step over long contexts)
// goes to the single-warp kernel: its CTAs are paced by their own address chains, finish within a few microseconds of
// each other and the launch ends when the data does, while the free-running movers of the warp-specialised kernel end
// up to 25 us apart on the same launch (measured on B200: 50.7 against 55.5 us per launch). Launches with few tiles per
// CTA, long appends and key quantisation go to the warp-specialised kernel (prefill call 11.0 -> 9.0 us, 4096-row
// appends of 43 layers in one launch 1.6 -> 3.3 TB/s).
bool use_pipe(const StepParams& P) {
  const int knob = tuning().pipe;
  if (knob >= 0) return knob != 0;
  const bool gather_heavy = (long long)P.s.Q * P.s.k >= 8ll * P.s.T;
  return !(many_tiles_per_cta(P) && gather_heavy);
}

int dispatch_pipe(const StepParams& P, int shape, int ctas_per_sm, cudaStream_t st) {
  if (shape == 0) shape = 308;
  switch (shape) {  // STAGES * 100 + ROWS
    case 304: return launch_pipe<3, 4>(P, ctas_per_sm, st);
    case 308: return launch_pipe<3, 8>(P, ctas_per_sm, st);
    case 408: return launch_pipe<4, 8>(P, ctas_per_sm, st);
    case 316: return launch_pipe<3, 16>(P, ctas_per_sm, st);
    default: return fail(PKV_ERR_ARG, "PKV_BULK_SHAPE names no compiled shape of the warp-specialised pipeline (304, 308, 408, 316)");
  }
}

// Both fp8 gathers launch the same way: one wave of CTAs, programmatic dependent launch as the step kernels.
template <class ROWSRC>
int launch_gather_fp8(const ROWSRC& rows, const uint8_t* codes, const uint8_t* scales, int width, int block, const int32_t* idx,
                      const int32_t* q_visible, int T, int k, uint16_t* out, const PoolList& pl, cudaStream_t stream) {
  const long long tiles = (long long)T * ((k + kGatherRows - 1) / kGatherRows);
  if (tiles >= (1ll << 31) - (1 << 20)) return fail(PKV_ERR_LIMIT, "fp8 gather: more than 2^31 tiles of 32 entries in one call");
  const DeviceInfo& d = device_info();
  const int sms = d.ok ? d.sms : 148;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(std::max<long long>(1, std::min<long long>(tiles, (long long)sms * kFp8CtasPerSm))));
  cfg.blockDim = dim3(kFp8Threads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tuning().pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gather_fp8_kernel<ROWSRC>, codes, scales, rows, width, block, idx, q_visible, T, k, out, pl);
  if (e != cudaSuccess) return fail_cuda("gather_fp8_kernel launch", e);
  return PKV_OK;
}

}  // namespace

extern "C" {

const char* pkv_last_error(void) { return g_err.c_str(); }
int pkv_abi_version(void) { return 2; }

int pkv_tune(int knob, int value) {
  Tuning& t = tuning();
  switch (knob) {
    case 0: t.bulk_shape = value; return PKV_OK;
    case 1: t.bulk_ctas_per_sm = value; return PKV_OK;
    case 2: t.pdl = value; return PKV_OK;
    case 3: t.vec_ctas_per_sm = value > 0 ? value : 5; return PKV_OK;
    case 4: t.fuse = value; return PKV_OK;
    case 5: t.batch = value; return PKV_OK;
    case 6: t.resolve_late = value; return PKV_OK;
    case 7: pkv_g_topk_path = value; return PKV_OK;
    case 8: t.pipe = value; return PKV_OK;
    case 9: t.wait_polls = value > 0 ? value : 1 << 21; return PKV_OK;
    case 10: t.debug_tile = value; return PKV_OK;
    case 11: t.copy_bulk = value; return PKV_OK;
    default: return fail(PKV_ERR_ARG, "pkv_tune: unknown knob");
  }
}

int pkv_device_status(int* status_out) {
  if (!status_out) return fail(PKV_ERR_ARG, "pkv_device_status: null output");
  int v = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda("cudaDeviceSynchronize", e);
  e = cudaMemcpyFromSymbol(&v, g_status, sizeof(int));
  if (e != cudaSuccess) return fail_cuda("cudaMemcpyFromSymbol", e);
  const int zero = 0;
  e = cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  if (e != cudaSuccess) return fail_cuda("cudaMemcpyToSymbol", e);
  *status_out = v;
  return PKV_OK;
}

int pkv_stream_check(pkv_stream_t stream) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&v, g_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail_cuda("pkv_stream_check", e);
  if (v == 0) return PKV_OK;
  const int zero = 0;
  e = cudaMemcpyToSymbolAsync(g_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail_cuda("pkv_stream_check", e);
  static const char* const kinds[] = {"?", "page id out of range", "chunk row, chunk index or slot out of range", "bounded wait gave up"};
  const int kind = v & 0xff;
  return fail(PKV_ERR_DEVICE, std::string("device-side check failed: ") + kinds[kind >= 1 && kind <= 3 ? kind : 0] + " (entry " +
                                  std::to_string(v >> 8) + ")");
}

int pkv_store_rows(const uint16_t* rows, int n, int width, uint16_t* pool, const int32_t* table, int rows_per_page,
                   int row_stride, int row0, pkv_stream_t stream) {
  if (n <= 0) return PKV_OK;
  if (!rows || !pool || !table) return fail(PKV_ERR_ARG, "pkv_store_rows: null pointer");
  if (width <= 0 || rows_per_page <= 0 || row_stride < width || row0 < 0) return fail(PKV_ERR_ARG, "pkv_store_rows: bad shape");
  const OneTable tb{table, rows_per_page};
  const bool vec = width % 8 == 0 && row_stride % 8 == 0 && aligned16(rows) && aligned16(pool);
  if (vec) {
    const long long total = (long long)n * (width / 8);
    store_rows_vec_kernel<<<grid_for(total, 256, 16), 256, 0, stream>>>(reinterpret_cast<const uint4*>(rows), total, width / 8,
                                                                        pool, tb, row_stride, row0);
  } else {
    const long long total = (long long)n * width;
    store_rows_elem_kernel<<<grid_for(total, 256, 16), 256, 0, stream>>>(rows, total, width, pool, tb, row_stride, row0);
  }
  PKV_LAUNCH_CHECK("store_rows");
  return PKV_OK;
}

int pkv_store_rows_fake_fp8(const uint16_t* rows, int n, int width, int quant_cols, int block, uint16_t* pool,
                            const int32_t* table, int rows_per_page, int row_stride, int row0, pkv_stream_t stream) {
  if (n <= 0) return PKV_OK;
  if (!rows || !pool || !table) return fail(PKV_ERR_ARG, "pkv_store_rows_fake_fp8: null pointer");
  if (const int rc = check_quant_shape(n, quant_cols, block, "pkv_store_rows_fake_fp8")) return rc;
  if (width <= 0 || width % block != 0 || quant_cols > width || rows_per_page <= 0 || row_stride < width || row_stride % 8 != 0 ||
      row0 < 0)
    return fail(PKV_ERR_ARG, "pkv_store_rows_fake_fp8: width must be a multiple of block, quant_cols <= width, row_stride % 8 == 0");
  if (!aligned16(rows) || !aligned16(pool)) return fail(PKV_ERR_ARG, "pkv_store_rows_fake_fp8: rows and pool must be 16-byte aligned");
  const long long total = (long long)n * (width / 8);
  store_rows_fake_fp8_kernel<<<grid_for(total, 256, 16), 256, 0, stream>>>(rows, total, width / 8, quant_cols / 8, block / 8, pool,
                                                                           OneTable{table, rows_per_page}, row_stride, row0);
  PKV_LAUNCH_CHECK("store_rows_fake_fp8");
  return PKV_OK;
}

int pkv_store_rows_kv_chain(const uint16_t* rows, uint16_t* rows_out, const uint16_t* w, int n, int dim, float eps, const int32_t* pos,
                            const float* freqs, int npair, int quant, uint16_t* pool, const int32_t* table, int rows_per_page,
                            int row_stride, int row0, pkv_stream_t stream) {
  if (n <= 0) return PKV_OK;
  if (!rows || !w || !pos || (npair > 0 && !freqs)) return fail(PKV_ERR_ARG, "pkv_store_rows_kv_chain: null pointer");
  if (!pool && !rows_out) return fail(PKV_ERR_ARG, "pkv_store_rows_kv_chain: neither a pool nor rows_out to write to");
  if (pool && (!table || rows_per_page <= 0 || row_stride < dim || row_stride % 8 != 0 || row0 < 0))
    return fail(PKV_ERR_ARG, "pkv_store_rows_kv_chain: bad pool geometry");
  if (dim <= 0 || dim % 8 != 0 || dim > 256 * kChainVecs || npair < 0 || 2 * npair > dim || (2 * npair) % 8 != 0 || (dim - 2 * npair) % 64 != 0)
    return fail(PKV_ERR_ARG, "pkv_store_rows_kv_chain: dim <= 1024, a multiple of 8; the rope part a multiple of 8 values, the rest of 64");
  if (!aligned16(rows) || !aligned16(w) || !aligned16(pool) || !aligned16(rows_out) || (reinterpret_cast<uintptr_t>(freqs) & 7u))
    return fail(PKV_ERR_ARG, "pkv_store_rows_kv_chain: rows, w, pool and rows_out must be 16-byte aligned, freqs 8-byte");
  kv_chain_store_kernel<<<grid_for((long long)n * 32, 256, 8), 256, 0, stream>>>(rows, rows_out, w, n, dim, eps, pos, reinterpret_cast<const float2*>(freqs),
                                                                                  npair, quant, pool, OneTable{table, rows_per_page}, row_stride, row0);
  PKV_LAUNCH_CHECK("kv_chain_store_kernel");
  return PKV_OK;
}

int pkv_store_rows_fp4(const uint16_t* rows, int n, uint8_t* pool, const int32_t* table, int rows_per_page, int row0,
                       pkv_stream_t stream) {
  if (n <= 0) return PKV_OK;
  if (!rows || !pool || !table) return fail(PKV_ERR_ARG, "pkv_store_rows_fp4: null pointer");
  if (rows_per_page <= 0 || row0 < 0) return fail(PKV_ERR_ARG, "pkv_store_rows_fp4: bad shape");
  if (!aligned16(rows) || (reinterpret_cast<uintptr_t>(pool) & 3u)) return fail(PKV_ERR_ARG, "pkv_store_rows_fp4: rows must be 16-byte and pool 4-byte aligned");
  store_rows_fp4_kernel<<<grid_for((long long)n * 16, 256, 16), 256, 0, stream>>>(rows, n, pool, OneTable{table, rows_per_page}, row0);
  PKV_LAUNCH_CHECK("store_rows_fp4");
  return PKV_OK;
}

int pkv_load_rows_fp4(const uint8_t* pool, const int32_t* table, int rows_per_page, int row0, int n, uint16_t* out,
                      pkv_stream_t stream) {
  if (n <= 0) return PKV_OK;
  if (!pool || !table || !out) return fail(PKV_ERR_ARG, "pkv_load_rows_fp4: null pointer");
  if (rows_per_page <= 0 || row0 < 0) return fail(PKV_ERR_ARG, "pkv_load_rows_fp4: bad shape");
  if (!aligned16(out) || (reinterpret_cast<uintptr_t>(pool) & 3u)) return fail(PKV_ERR_ARG, "pkv_load_rows_fp4: out must be 16-byte and pool 4-byte aligned");
  load_rows_fp4_kernel<<<grid_for((long long)n * 16, 256, 16), 256, 0, stream>>>(pool, OneTable{table, rows_per_page}, row0, n, out);
  PKV_LAUNCH_CHECK("load_rows_fp4");
  return PKV_OK;
}

static int quant_launch(int mode, const uint16_t* x, int ldx, uint8_t* q, uint8_t* s, int rows, int cols, int block,
                        pkv_stream_t stream, const char* name) {
  if (const int rc = check_quant_shape(rows, cols, block, name)) return rc;
  if (rows == 0 || cols == 0) return PKV_OK;
  if (!x || ldx < cols) return fail(PKV_ERR_ARG, std::string(name) + ": bad input");
  const bool vec = aligned16(x) && ldx % 8 == 0;
  const long long total = (long long)rows * (cols / 8);
  const int grid = grid_for(total, 256, 16);
  if (mode == kFp8Codes) quant_rows_kernel<kFp8Codes><<<grid, 256, 0, stream>>>(x, ldx, q, s, rows, cols, block, vec);
  else if (mode == kFp8Fake) quant_rows_kernel<kFp8Fake><<<grid, 256, 0, stream>>>(x, ldx, nullptr, nullptr, rows, cols, block, vec);
  else quant_rows_kernel<kFp4Fake><<<grid, 256, 0, stream>>>(x, ldx, nullptr, nullptr, rows, cols, block, vec);
  PKV_LAUNCH_CHECK("quant_rows_kernel");
  return PKV_OK;
}

int pkv_hadamard128(uint16_t* x, size_t nseg, pkv_stream_t stream) {
  if (nseg == 0) return PKV_OK;
  if (!x || !aligned16(x)) return fail(PKV_ERR_ARG, "pkv_hadamard128: x must be a 16-byte aligned device pointer");
  hadamard128_kernel<<<grid_for((long long)std::min<size_t>(nseg, size_t(1) << 40) * 16, 256, 16), 256, 0, stream>>>(x, nseg);
  PKV_LAUNCH_CHECK("hadamard128_kernel");
  return PKV_OK;
}

int pkv_act_quant_fp8(const uint16_t* x, int ldx, uint8_t* q, uint8_t* s, int rows, int cols, int block,
                      pkv_stream_t stream) {
  if (rows > 0 && cols > 0 && (!q || !s)) return fail(PKV_ERR_ARG, "pkv_act_quant_fp8: null output");
  return quant_launch(kFp8Codes, x, ldx, q, s, rows, cols, block, stream, "pkv_act_quant_fp8");
}
int pkv_fake_quant_fp8(uint16_t* x, int ldx, int rows, int cols, int block, pkv_stream_t stream) {
  return quant_launch(kFp8Fake, x, ldx, nullptr, nullptr, rows, cols, block, stream, "pkv_fake_quant_fp8");
}
int pkv_fake_quant_fp4(uint16_t* x, int ldx, int rows, int cols, int block, pkv_stream_t stream) {
  return quant_launch(kFp4Fake, x, ldx, nullptr, nullptr, rows, cols, block, stream, "pkv_fake_quant_fp4");
}

int pkv_store_rows_fp8(const uint16_t* rows, int n, int width, int block, uint8_t* codes, uint8_t* scales,
                       const int32_t* table, int rows_per_page, int s0, pkv_stream_t stream) {
  if (n <= 0) return PKV_OK;
  if (const int rc = check_quant_shape(n, width, block, "pkv_store_rows_fp8")) return rc;
  if (!rows || !codes || !scales || !table) return fail(PKV_ERR_ARG, "pkv_store_rows_fp8: null pointer");
  if (rows_per_page <= 0 || s0 < 0) return fail(PKV_ERR_ARG, "pkv_store_rows_fp8: bad shape");
  if (!aligned16(rows) || (reinterpret_cast<uintptr_t>(codes) & 7u)) return fail(PKV_ERR_ARG, "pkv_store_rows_fp8: rows must be 16-byte and codes 8-byte aligned");
  store_rows_fp8_kernel<<<grid_for((long long)n * (width / 8), 256, 16), 256, 0, stream>>>(rows, n, width, block, codes, scales,
                                                                                         OneTable{table, rows_per_page}, s0);
  PKV_LAUNCH_CHECK("store_rows_fp8");
  return PKV_OK;
}

int pkv_copy(void* dst, const void* src, size_t bytes, pkv_stream_t stream) {
  if (bytes == 0) return PKV_OK;
  if (!dst || !src) return fail(PKV_ERR_ARG, "pkv_copy: null pointer");
  const bool v16 = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | bytes) & 15u) == 0;
  if (v16) {
    const size_t n = bytes / 16;
    copy16_kernel<<<grid_for((long long)((n + 3) / 4), 256, 8), 256, 0, stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), n);
  } else {
    copy1_kernel<<<grid_for((long long)bytes, 256, 8), 256, 0, stream>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), bytes);
  }
  PKV_LAUNCH_CHECK("copy_kernel");
  return PKV_OK;
}

int pkv_step_run(const pkv_step* step, const pkv_layer* layers, int L, int flags, pkv_stream_t stream) {
  if (!step || !layers) return fail(PKV_ERR_ARG, "pkv_step_run: null argument");
  if (L <= 0) return PKV_OK;
  if (L > PKV_MAX_LAYERS) return fail(PKV_ERR_LIMIT, "pkv_step_run: more than PKV_MAX_LAYERS layers in one launch");
  const pkv_step& s = *step;
  if (s.width <= 0 || s.width % 8 != 0 || s.row_stride < s.width || s.row_stride % 8 != 0)
    return fail(PKV_ERR_ARG, "pkv_step_run: width and row_stride must be positive multiples of 8 with row_stride >= width");
  if (s.rows_per_page <= 0 || s.max_pages_per_seq <= 0 || s.nchunks < 0 || s.T < 0 || s.Q < 0 || s.k < 0)
    return fail(PKV_ERR_ARG, "pkv_step_run: bad geometry");
  if (s.num_pages <= 0 || s.max_slots <= 0)
    return fail(PKV_ERR_ARG, "pkv_step_run: num_pages and max_slots must be positive (the kernels check page ids and slots against them)");
  const bool append = (flags & (PKV_DO_ROWS | PKV_DO_KEYS_FP4 | PKV_DO_KEYS_FP8)) != 0 && s.T > 0 && s.nchunks > 0;
  const bool gather = (flags & PKV_DO_GATHER) != 0 && s.Q > 0 && s.k > 0;
  if (!append && !gather) return PKV_OK;
  if (!s.tables || !s.chunks) return fail(PKV_ERR_ARG, "pkv_step_run: tables and chunks are required");
  if (gather && (!s.q_chunk || !s.q_visible)) return fail(PKV_ERR_ARG, "pkv_step_run: q_chunk and q_visible are required for a gather");
  if ((flags & PKV_DO_KEYS_FP8) && s.fp8_block != 32 && s.fp8_block != 64 && s.fp8_block != 128)
    return fail(PKV_ERR_ARG, "pkv_step_run: fp8_block must be 32, 64 or 128");
  for (int l = 0; l < L; ++l) {
    const pkv_layer& y = layers[l];
    if (!aligned16(y.rows) || !aligned16(y.row_pool) || !aligned16(y.keys) || !aligned16(y.gathered) ||
        (reinterpret_cast<uintptr_t>(y.key_pool_fp4) & 3u) || (reinterpret_cast<uintptr_t>(y.key_fp8_codes) & 7u))
      return fail(PKV_ERR_ARG, "pkv_step_run: layer pointers must be 16-byte aligned (fp4 pool 4, fp8 codes 8)");
    if (gather && (!y.idx || !y.gathered || !y.row_pool)) return fail(PKV_ERR_ARG, "pkv_step_run: a layer lacks idx, gathered or row_pool");
  }
  const int grid_mult = tuning().vec_ctas_per_sm, bulk_shape = tuning().bulk_shape, bulk_ctas = tuning().bulk_ctas_per_sm;

  StepParams P;
  std::memset(&P, 0, sizeof(P));
  P.s = s;
  P.L = L;
  P.flags = flags;
  std::memcpy(P.layers, layers, sizeof(pkv_layer) * size_t(L));
  const bool bulk = gather && (flags & PKV_VARIANT_BULK);
  // With the bulk pipeline the step's appends are tiles of the same launch (rows of at least 256 bytes, so that a
  // tile of 128-wide keys fits the stage a tile of rows uses).
  const bool rows_on = append && (flags & PKV_DO_ROWS), keys_on = append && (flags & (PKV_DO_KEYS_FP4 | PKV_DO_KEYS_FP8));
  if ((flags & PKV_VARIANT_BULK) && append && tuning().fuse && s.width >= PKV_FP4_ROW_DIM) {
    StepParams B = P;
    B.append_tiles = rows_on ? 1 : 0;   // flags here; launch_bulk counts the tiles for its ROWS
    B.key_tiles = keys_on ? 1 : 0;
    if (!gather) B.s.Q = 0;
    for (int l = 0; l < L; ++l) {       // a layer without the arrays of a part cannot take part in it
      if (rows_on && (!B.layers[l].rows || !B.layers[l].row_pool)) return fail(PKV_ERR_ARG, "pkv_step_run: a layer lacks rows or row_pool");
      if (keys_on && !B.layers[l].keys) return fail(PKV_ERR_ARG, "pkv_step_run: a layer lacks keys");
    }
    return use_pipe(B) ? dispatch_pipe(B, bulk_shape, bulk_ctas, stream) : dispatch_bulk(B, bulk_shape, bulk_ctas, stream);
  }
  P.append_tiles = append ? (s.T + kAppendRows - 1) / kAppendRows : 0;
  P.tiles_per_q = (s.k + kGatherRows - 1) / kGatherRows;
  P.gather_tiles = gather && !bulk ? s.Q * P.tiles_per_q : 0;
  const long long vec_work = (long long)(P.append_tiles + P.gather_tiles) * L;
  if (vec_work > 0) {
    const DeviceInfo& d = device_info();
    const int sms = d.ok ? d.sms : 148;
    // One wave: as many CTAs as are resident at once (asked of the runtime, capped by the tuning knob).
    int resident = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, step_vec_kernel, kVecThreads, 0) != cudaSuccess || resident < 1) resident = 1;
    resident = std::min(resident, std::max(1, grid_mult));
    const int grid = int(std::max<long long>(1, std::min<long long>(vec_work, (long long)sms * resident)));
    step_vec_kernel<<<grid, kVecThreads, 0, stream>>>(P);
    PKV_LAUNCH_CHECK("step_vec_kernel");
  }
  if (bulk) {
    P.append_tiles = 0;
    P.key_tiles = 0;
    return use_pipe(P) ? dispatch_pipe(P, bulk_shape, bulk_ctas, stream) : dispatch_bulk(P, bulk_shape, bulk_ctas, stream);
  }
  return PKV_OK;
}

int pkv_gather_rows(const uint16_t* pool, const int32_t* table, int rows_per_page, int row_stride, int width,
                    const int32_t* idx, const int32_t* q_visible, int T, int k, uint16_t* out, pkv_stream_t stream) {
  if (T <= 0 || k <= 0) return PKV_OK;
  if (!pool || !table || !idx || !q_visible || !out) return fail(PKV_ERR_ARG, "pkv_gather_rows: null pointer");
  if (width <= 0 || width % 8 != 0 || row_stride < width || row_stride % 8 != 0 || rows_per_page <= 0)
    return fail(PKV_ERR_ARG, "pkv_gather_rows: width and row_stride must be positive multiples of 8 with row_stride >= width");
  if (!aligned16(pool) || !aligned16(out)) return fail(PKV_ERR_ARG, "pkv_gather_rows: pool and out must be 16-byte aligned");
  const long long tiles = (long long)T * ((k + kGatherRows - 1) / kGatherRows);
  const DeviceInfo& d = device_info();
  const int sms = d.ok ? d.sms : 148;
  const int grid = int(std::max<long long>(1, std::min<long long>(tiles, (long long)sms * 5)));
  gather_one_kernel<<<grid, kVecThreads, 0, stream>>>(pool, OneTable{table, rows_per_page}, row_stride, width, idx,
                                                      q_visible, T, k, out);
  PKV_LAUNCH_CHECK("gather_one_kernel");
  return PKV_OK;
}

int pkv_gather_rows_fp8(const uint8_t* codes, const uint8_t* scales, const int32_t* table, int rows_per_page, int width,
                        int block, const int32_t* idx, const int32_t* q_visible, int T, int k, uint16_t* out,
                        pkv_stream_t stream) {
  if (T <= 0 || k <= 0) return PKV_OK;
  if (!codes || !scales || !table || !idx || !q_visible || !out) return fail(PKV_ERR_ARG, "pkv_gather_rows_fp8: null pointer");
  if (const int rc = check_quant_shape(T, width, block, "pkv_gather_rows_fp8")) return rc;
  if (width <= 0 || width % 16 != 0 || block % 16 != 0 || rows_per_page <= 0)
    return fail(PKV_ERR_ARG, "pkv_gather_rows_fp8: width must be a positive multiple of 16");
  if (!aligned16(codes) || !aligned16(out)) return fail(PKV_ERR_ARG, "pkv_gather_rows_fp8: codes and out must be 16-byte aligned");
  return launch_gather_fp8(OneSeqRows{OneTable{table, rows_per_page}}, codes, scales, width, block, idx, q_visible, T, k, out,
                           PoolList{nullptr, nullptr, 0, 0}, static_cast<cudaStream_t>(stream));
}

// Shared by the two step-wide fp8 gathers: entries from idx [Q][k], or from pools [Q][kp] + pos (k = kp * pool + pool - 1).
static int step_gather_fp8(const pkv_step* step, const uint8_t* codes, const uint8_t* scales, int width, int block,
                           const int32_t* idx, const PoolList& pl, int k, uint16_t* out, cudaStream_t stream, const char* name) {
  if (!step) return fail(PKV_ERR_ARG, std::string(name) + ": null step");
  const pkv_step& s = *step;
  if (s.Q <= 0 || k <= 0) return PKV_OK;
  if (!codes || !scales || !(idx || pl.pools) || !out || !s.tables || !s.chunks || !s.q_chunk || !s.q_visible)
    return fail(PKV_ERR_ARG, std::string(name) + ": null pointer");
  if (const int rc = check_quant_shape(s.Q, width, block, name)) return rc;
  if (width <= 0 || width % 16 != 0 || block % 16 != 0 || s.rows_per_page <= 0 || s.max_pages_per_seq <= 0 || s.nchunks <= 0)
    return fail(PKV_ERR_ARG, std::string(name) + ": width must be a positive multiple of 16, the step needs pages and chunks");
  if (s.num_pages <= 0 || s.max_slots <= 0) return fail(PKV_ERR_ARG, std::string(name) + ": num_pages and max_slots must be positive");
  if (!aligned16(codes) || !aligned16(out)) return fail(PKV_ERR_ARG, std::string(name) + ": codes and out must be 16-byte aligned");
  return launch_gather_fp8(StepRows{s}, codes, scales, width, block, idx, s.q_visible, s.Q, k, out, pl, stream);
}

int pkv_step_gather_fp8(const pkv_step* step, const uint8_t* codes, const uint8_t* scales, int width, int block,
                        const int32_t* idx, uint16_t* out, pkv_stream_t stream) {
  return step_gather_fp8(step, codes, scales, width, block, idx, PoolList{nullptr, nullptr, 0, 0}, step ? step->k : 0, out, stream,
                         "pkv_step_gather_fp8");
}

int pkv_step_gather_fp8_pools(const pkv_step* step, const uint8_t* codes, const uint8_t* scales, int width, int block,
                              const int32_t* pools, const int32_t* pos, int kp, int pool, uint16_t* out, pkv_stream_t stream) {
  if (kp <= 0 || pool <= 0 || !pools || !pos) return fail(PKV_ERR_ARG, "pkv_step_gather_fp8_pools: pools, pos, kp > 0 and pool > 0 are required");
  return step_gather_fp8(step, codes, scales, width, block, nullptr, PoolList{pools, pos, kp, pool}, kp * pool + pool - 1, out, stream,
                         "pkv_step_gather_fp8_pools");
}

int pkv_copy_pages(const pkv_pool_desc* pools, int npools, const int32_t* src_ids, const int32_t* dst_ids, int n,
                   int num_src_pages, int num_dst_pages, pkv_stream_t stream) {
  if (n <= 0 || npools <= 0) return PKV_OK;
  if (!pools || !src_ids || !dst_ids) return fail(PKV_ERR_ARG, "pkv_copy_pages: null pointer");
  if (npools > 128) return fail(PKV_ERR_LIMIT, "pkv_copy_pages: more than 128 pools in one call");
  bool same_pool = tuning().copy_bulk != 0;
  for (int p = 0; p < npools && same_pool; ++p) same_pool = pools[p].src_base == pools[p].dst_base;
  if (same_pool) {
    // Moves inside pools of this device: the bulk-copy ring.
    PageCopyBulkParams B;
    std::memset(&B, 0, sizeof(B));
    B.npools = npools;
    B.n = n;
    B.num_src_pages = num_src_pages > 0 ? num_src_pages : 0x7fffffff;
    B.num_dst_pages = num_dst_pages > 0 ? num_dst_pages : 0x7fffffff;
    B.wait_polls = std::max(1, tuning().wait_polls);
    B.src_ids = src_ids;
    B.dst_ids = dst_ids;
    unsigned long long items = 0;
    for (int p = 0; p < npools; ++p) {
      if (!pools[p].src_base || pools[p].page_bytes == 0 || pools[p].page_bytes % 16 != 0 || !aligned16(pools[p].src_base))
        return fail(PKV_ERR_ARG, "pkv_copy_pages: pool bases must be 16-byte aligned and page_bytes a multiple of 16");
      if (pools[p].page_bytes > (1ull << 30)) return fail(PKV_ERR_LIMIT, "pkv_copy_pages: page_bytes above 1 GiB");
      B.pools[p] = pools[p];
      B.first_item[p] = unsigned(items);
      items += (unsigned long long)n * ((pools[p].page_bytes + kBulkPiece - 1) / kBulkPiece);
      if (items > 0x7fffffffull) return fail(PKV_ERR_LIMIT, "pkv_copy_pages: too many pages in one call");
    }
    B.first_item[npools] = unsigned(items);
    const size_t smem = size_t(kCopyStages) * kBulkPiece;
    static thread_local bool opted[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !opted[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(copy_pages_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
      opted[dev] = true;
    }
    const DeviceInfo& d = device_info();
    const int sms = d.ok ? d.sms : 148;
    const int per_sm = int((227u * 1024u) / (smem + 2048u));
    const unsigned grid = unsigned(std::max<unsigned long long>(1, std::min<unsigned long long>(items, (unsigned long long)sms * per_sm)));
    copy_pages_bulk_kernel<<<grid, 32, smem, stream>>>(B);
    PKV_LAUNCH_CHECK("copy_pages_bulk_kernel");
    return PKV_OK;
  }
  PageCopyParams P;
  std::memset(&P, 0, sizeof(P));
  P.npools = npools;
  P.n = n;
  P.num_src_pages = num_src_pages;
  P.num_dst_pages = num_dst_pages;
  P.src_ids = src_ids;
  P.dst_ids = dst_ids;
  long long max_items = 0;
  for (int p = 0; p < npools; ++p) {
    if (!pools[p].src_base || !pools[p].dst_base || pools[p].page_bytes == 0 || pools[p].page_bytes % 16 != 0 ||
        !aligned16(pools[p].src_base) || !aligned16(pools[p].dst_base))
      return fail(PKV_ERR_ARG, "pkv_copy_pages: pool bases must be 16-byte aligned and page_bytes a multiple of 16");
    if (pools[p].page_bytes > (1ull << 30)) return fail(PKV_ERR_LIMIT, "pkv_copy_pages: page_bytes above 1 GiB");
    P.pools[p] = pools[p];
    max_items = std::max<long long>(max_items, (long long)n * (long long)((pools[p].page_bytes / 16 + kPieceVecs - 1) / kPieceVecs));
  }
  if (max_items > 0x7fffffffLL) return fail(PKV_ERR_LIMIT, "pkv_copy_pages: too many pages in one call");
  const DeviceInfo& d = device_info();
  const int sms = d.ok ? d.sms : 148;
  const long long per_pool = std::max<long long>(1, ((long long)sms * 8 + npools - 1) / npools);
  const dim3 grid(unsigned(std::min<long long>(max_items, per_pool)), unsigned(npools));
  copy_pages_kernel<<<grid, 256, 0, stream>>>(P);
  PKV_LAUNCH_CHECK("copy_pages_kernel");
  return PKV_OK;
}

int pkv_device_alloc(void** ptr_out, size_t bytes) {
  if (!ptr_out) return fail(PKV_ERR_ARG, "pkv_device_alloc: null output");
  const cudaError_t e = cudaMalloc(ptr_out, bytes);
  return e == cudaSuccess ? PKV_OK : fail_cuda("cudaMalloc", e);
}
int pkv_device_free(void* ptr) {
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? PKV_OK : fail_cuda("cudaFree", e);
}
int pkv_ipc_export(void* base, unsigned char handle_out[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (!base || !handle_out) return fail(PKV_ERR_ARG, "pkv_ipc_export: null argument");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, base);
  if (e != cudaSuccess) return fail_cuda("cudaIpcGetMemHandle", e);
  std::memcpy(handle_out, &h, 64);
  return PKV_OK;
}
int pkv_ipc_open(const unsigned char handle[64], void** ptr_out) {
  if (!handle || !ptr_out) return fail(PKV_ERR_ARG, "pkv_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  const cudaError_t e = cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? PKV_OK : fail_cuda("cudaIpcOpenMemHandle", e);
}
int pkv_ipc_close(void* ptr) {
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? PKV_OK : fail_cuda("cudaIpcCloseMemHandle", e);
}

}  // extern "C"
