// Index-list producer: top-k per row of bf16 scores, the step immediately before the sparse gather.
//
// Contract of ewtodd/unholy's topk_bf16 (src/kernels/indexer.hpp:74, src/kernels/indexer.hip:408-560; fp32 twin
// topk_rows: src/kernels/ref_attn.hip:143-240): per row the want = min(k, #valid) largest scores, a score being valid
// when it is greater than -inf in the order-preserving 16-bit key (so -inf and negative-NaN patterns are never
// selected); ties at the threshold go to the lowest indices; the output is ordered by (score descending, index
// ascending) and padded with -1. That contract fixes every output element, so any algorithm that meets it is
// bit-exact with the reference.
//
// B200 design: a row of 128k bf16 scores is 256 KB and a decode step has only 64 rows, so one CTA per row would leave
// most SMs idle. Rows are cut into slices of kSlice keys and a launch covers (slice, row): 16 x 64 = 1024 CTAs for the
// benchmark shape. Radix select on the 16-bit key takes two 8-bit histogram passes; every CTA writes ITS OWN
// histograms to scratch (no global atomics, nothing to zero), and the next pass re-derives the threshold from the sum
// over slices, which also gives each slice the exact output offsets of its keys above the threshold and of its share
// of the threshold ties in index order. Four short launches: high-byte histogram, low-byte histogram, collect, sort
// (one CTA per row, bitonic on (key, ~index) packed in 64 bits). Scratch is caller-provided (pkv_topk_scratch_words).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/unholy_pkv.h"

namespace pkv_topk {

constexpr int kThreads = 512;
constexpr int kSlice = 8192;          // keys per CTA
constexpr int kMaxK = 4096;
constexpr int kMaxSlices = 256;       // rows of up to 2M keys
constexpr uint32_t kNegInfKey = 0x007Fu;  // key16 of the bf16 pattern 0xFF80

__device__ __forceinline__ uint32_t key16(uint32_t b) { return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u); }

// Scratch layout (uint32 words): per-slice histograms hist[row][slice][2][256]; per-row results info[row][8]
// (kWant.. below; the two arrival counters are the only words that must be zero when a call starts: the launcher
// clears info); per-slice output offsets offs[row][slice][2]; candidates as uint64 [row][k] (8-byte aligned).
enum Info { kWant = 0, kHiBin = 1, kNeed1 = 2, kLoBin = 3, kNeedTies = 4, kAboveTotal = 5, kArrived0 = 6, kArrived1 = 7 };
struct Layout {
  int slices;
  size_t hist_words, info_offset, offs_offset, cand_offset_words, total_words;
};
__host__ __device__ inline Layout layout(int T, int n, int k) {
  Layout l;
  l.slices = (n + kSlice - 1) / kSlice;
  if (l.slices < 1) l.slices = 1;
  l.hist_words = size_t(T) * l.slices * 512;
  l.info_offset = l.hist_words;
  l.offs_offset = l.info_offset + size_t(T) * 8;
  l.cand_offset_words = (l.offs_offset + size_t(T) * l.slices * 2 + 1) & ~size_t(1);
  l.total_words = l.cand_offset_words + size_t(T) * k * 2;
  return l;
}

constexpr int kPerThread = kSlice / kThreads;  // 16 consecutive keys per thread: two 16-byte loads

// This thread's kPerThread consecutive keys of the slice, as order-preserving 16-bit keys; 0 (never valid) past the end.
__device__ __forceinline__ void load_keys(const uint16_t* __restrict__ r, int base, int hi, uint32_t* key) {
  const uint16_t* p = r + base;
  if (base + kPerThread <= hi && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
    for (int v = 0; v < kPerThread / 8; ++v) {
      const uint4 w = __ldcg(reinterpret_cast<const uint4*>(p) + v);
      const uint32_t x[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        key[v * 8 + 2 * i] = key16(x[i] & 0xffffu);
        key[v * 8 + 2 * i + 1] = key16(x[i] >> 16);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) key[i] = base + i < hi ? key16(p[i]) : 0u;
  }
}

// Threshold bin of a 256-bin histogram h (plain counts in shared memory): the highest bin b >= 1 whose suffix sum
// S[b] = sum of bins >= b reaches `need`, else bin 0 — what the reference's walk from the top finds
// (src/kernels/indexer.hip:447-462). need < 0 means "min(k, number of valid keys)" (the first pass). Outputs through
// shared memory: s_out[0] = bin, s_out[1] = how many are still needed inside that bin, s_out[2] = S[0] (all counted
// keys). Called by every thread of the CTA; threads 0..255 hold one bin each; suffix sums by warp shuffles.
__device__ void pick_bin(const uint32_t* h, int need_in, int k, uint32_t* s_wsum, uint32_t* s_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t mine = 0, v = 0;
  if (tid < 256) {
    mine = h[tid];
    v = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_down_sync(0xffffffffu, v, o);
      if (lane + o < 32) v += t;
    }
    if (lane == 0) s_wsum[warp] = v;
  }
  __syncthreads();
  if (tid < 256)
    for (int w = warp + 1; w < 8; ++w) v += s_wsum[w];
  if (tid == 0) {
    s_out[2] = v;
    const uint32_t need = need_in < 0 ? min(uint32_t(k), v) : uint32_t(need_in);
    s_out[0] = 0;
    s_out[1] = need - (v - mine);  // bin 0: everything above it counts
    s_out[3] = need;
  }
  __syncthreads();
  const uint32_t need = s_out[3];
  if (tid >= 1 && tid < 256 && v >= need && v - mine < need) {
    s_out[0] = uint32_t(tid);
    s_out[1] = need - (v - mine);
  }
  __syncthreads();
}

// Sum over slices of one of the two histograms of a row into shared memory.
__device__ void sum_hist(const uint32_t* __restrict__ row_hist, int slices, int which, uint32_t* out) {
  for (int b = threadIdx.x; b < 256; b += blockDim.x) {
    uint32_t s = 0;
    for (int sl = 0; sl < slices; ++sl) s += __ldcg(&row_hist[(size_t(sl) * 2 + which) * 256 + b]);
    out[b] = s;
  }
  __syncthreads();
}

// Pass 1 (which = 0): histogram of the high key byte over the slice's valid keys. Pass 2 (which = 1): histogram of
// the low byte over the keys whose high byte is the threshold's. In both, the CTA that finishes LAST for its row (an
// arrival counter; writers fence before they count, the last one fences before it reads) folds the row's per-slice
// histograms once for everybody: after pass 1 it leaves want / high threshold byte / remaining need in info[row];
// after pass 2 the low byte, the number of threshold ties to take, and for every slice where its keys above the
// threshold and its ties start in the output. No other CTA repeats that work.
__global__ void __launch_bounds__(kThreads) hist_kernel(const uint16_t* __restrict__ scores, int n, long long ld, int k,
                                                        uint32_t* __restrict__ scratch, Layout L, int which) {
  asm volatile("griddepcontrol.wait;" ::: "memory");            // launched with programmatic stream serialisation:
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // only the launch latency overlaps the previous kernel
  __shared__ uint32_t hist[256], total[256], s_wsum[kThreads / 32], s_out[4], s_last;
  __shared__ uint32_t s_slice_above[kMaxSlices], s_slice_ties[kMaxSlices];
  const int row = blockIdx.y, sl = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, slices = L.slices;
  uint32_t* row_hist = scratch + size_t(row) * slices * 512;
  uint32_t* info = scratch + L.info_offset + size_t(row) * 8;
  const uint16_t* r = scores + size_t(row) * ld;
  const int lo = sl * kSlice, hi = min(n, lo + kSlice);
  uint32_t key[kPerThread];
  load_keys(r, lo + tid * kPerThread, hi, key);
  const uint32_t hi_bin = which == 1 ? __ldcg(&info[kHiBin]) : 0u;
  for (int b = tid; b < 256; b += kThreads) hist[b] = 0;
  __syncthreads();
  // Plain shared-memory atomics: measured faster here than electing one lane per bin (match.any or ballot rounds cost
  // more than the same-address queueing they avoid).
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    if (key[i] <= kNegInfKey) continue;
    if (which == 0) atomicAdd(&hist[key[i] >> 8], 1u);
    else if ((key[i] >> 8) == hi_bin) atomicAdd(&hist[key[i] & 0xffu], 1u);
  }
  __syncthreads();
  for (int b = tid; b < 256; b += kThreads) row_hist[(size_t(sl) * 2 + which) * 256 + b] = hist[b];
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&info[which == 0 ? kArrived0 : kArrived1], 1u) == uint32_t(slices - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  sum_hist(row_hist, slices, which, total);
  if (which == 0) {
    pick_bin(total, -1, k, s_wsum, s_out);
    if (tid == 0) {
      info[kWant] = s_out[3];
      info[kHiBin] = s_out[0];
      info[kNeed1] = s_out[1];
    }
    return;
  }
  const uint32_t need1 = __ldcg(&info[kNeed1]);
  pick_bin(total, int(need1), k, s_wsum, s_out);
  const uint32_t lo_bin = s_out[0], need_ties = s_out[1];
  // One warp per slice: that slice's keys above the threshold and its ties.
  for (int s2 = warp; s2 < slices; s2 += kThreads / 32) {
    const uint32_t* h0 = row_hist + (size_t(s2) * 2) * 256;
    const uint32_t* h1 = h0 + 256;
    uint32_t a = 0;
    for (uint32_t b = lane; b < 256; b += 32) a += (b > hi_bin ? __ldcg(&h0[b]) : 0u) + (b > lo_bin ? __ldcg(&h1[b]) : 0u);
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) {
      s_slice_above[s2] = a;
      s_slice_ties[s2] = __ldcg(&h1[lo_bin]);
    }
  }
  __syncthreads();
  if (tid == 0) {
    uint32_t* offs = scratch + L.offs_offset + size_t(row) * slices * 2;
    uint32_t above = 0, ties = 0;
    for (int s2 = 0; s2 < slices; ++s2) {
      offs[2 * s2] = above;
      offs[2 * s2 + 1] = ties;
      above += s_slice_above[s2];
      ties += s_slice_ties[s2];
    }
    info[kLoBin] = lo_bin;
    info[kNeedTies] = need_ties;
    info[kAboveTotal] = above;
  }
}

// Collect: every slice writes its keys above the threshold and its share of the threshold ties (lowest indices first
// across the whole row) into the row's candidate array at the offsets pass 2 left in scratch. Each thread owns 16
// consecutive keys, so index order is thread order and one block-wide scan places everything.
__global__ void __launch_bounds__(kThreads) collect_kernel(const uint16_t* __restrict__ scores, int n, long long ld, int k,
                                                           uint32_t* __restrict__ scratch, Layout L) {
  asm volatile("griddepcontrol.wait;" ::: "memory");            // launched with programmatic stream serialisation:
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // only the launch latency overlaps the previous kernel
  __shared__ uint32_t s_wsum[kThreads / 32];
  const int row = blockIdx.y, sl = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t* info = scratch + L.info_offset + size_t(row) * 8;
  const uint32_t* offs = scratch + L.offs_offset + (size_t(row) * L.slices + sl) * 2;
  unsigned long long* cand = reinterpret_cast<unsigned long long*>(scratch + L.cand_offset_words) + size_t(row) * k;
  const uint16_t* r = scores + size_t(row) * ld;
  const int lo = sl * kSlice, hi = min(n, lo + kSlice), base = lo + tid * kPerThread;
  uint32_t key[kPerThread];
  load_keys(r, base, hi, key);
  const uint32_t want = __ldcg(&info[kWant]);
  if (want == 0) return;
  const uint32_t thr = (__ldcg(&info[kHiBin]) << 8) | __ldcg(&info[kLoBin]), need_ties = __ldcg(&info[kNeedTies]);
  const uint32_t above_total = __ldcg(&info[kAboveTotal]), above_before = __ldcg(&offs[0]), ties_before = __ldcg(&offs[1]);
  // This thread's counts, packed (above << 16 | ties; a slice holds 8192 keys), and their block-wide exclusive scan.
  uint32_t cnt = 0;
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) cnt += key[i] > kNegInfKey ? (key[i] > thr ? 0x10000u : (key[i] == thr ? 1u : 0u)) : 0u;
  uint32_t incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_wsum[warp] = incl;
  __syncthreads();
  uint32_t before = incl - cnt;
  for (int w = 0; w < warp; ++w) before += s_wsum[w];
  uint32_t a_pos = above_before + (before >> 16), t_rank = ties_before + (before & 0xffffu);
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    if (key[i] <= kNegInfKey) continue;
    const unsigned long long packed = (static_cast<unsigned long long>(key[i]) << 32) | (0xffffffffu - uint32_t(base + i));
    if (key[i] > thr) {
      cand[a_pos++] = packed;
    } else if (key[i] == thr) {
      if (t_rank < need_ties) cand[above_total + t_rank] = packed;
      ++t_rank;
    }
  }
}

// Sort: one CTA per row; (key, ~index) descending = (score descending, index ascending); -1 padding. Bitonic network,
// one compare-exchange per thread per stage (thread p owns the p-th pair of the stage).
constexpr int kSortThreads = 1024;
__global__ void __launch_bounds__(kSortThreads) sort_kernel(const uint32_t* __restrict__ scratch, int k, Layout L,
                                                            int32_t* __restrict__ idx) {
  asm volatile("griddepcontrol.wait;" ::: "memory");            // launched with programmatic stream serialisation:
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // only the launch latency overlaps the previous kernel
  extern __shared__ unsigned long long s_keys[];
  const int row = blockIdx.x, tid = threadIdx.x;
  const size_t cand_offset = L.cand_offset_words;
  const uint32_t want = __ldcg(&scratch[L.info_offset + size_t(row) * 8 + kWant]);
  int size = 2;
  while (size < k) size <<= 1;
  const unsigned long long* cand = reinterpret_cast<const unsigned long long*>(scratch + cand_offset) + size_t(row) * k;
  for (int i = tid; i < size; i += kSortThreads) s_keys[i] = uint32_t(i) < want ? __ldcg(&cand[i]) : 0ull;
  __syncthreads();
  const int pairs = size >> 1;
  for (int len = 2; len <= size; len <<= 1)
    for (int stride = len >> 1; stride > 0; stride >>= 1) {
      for (int p = tid; p < pairs; p += kSortThreads) {
        const int i = ((p & ~(stride - 1)) << 1) | (p & (stride - 1)), j = i | stride;
        const bool desc = (i & len) == 0;
        const unsigned long long a = s_keys[i], b = s_keys[j];
        if ((a < b) == desc) {
          s_keys[i] = b;
          s_keys[j] = a;
        }
      }
      __syncthreads();
    }
  int32_t* out = idx + size_t(row) * k;
  for (int i = tid; i < k; i += kSortThreads)
    out[i] = uint32_t(i) < want ? int32_t(0xffffffffu - uint32_t(s_keys[i] & 0xffffffffull)) : -1;
}

// The same sort for 64 <= size <= 2048 with size / 2 threads, two elements per thread (2t, 2t + 1): strides 1..32 are
// exchanges inside a thread or between lanes of a warp (shuffles, no barrier); only strides >= 64 go through shared
// memory. 15 of the 66 stages of a 2048-element sort need a barrier instead of all of them.
__device__ __forceinline__ unsigned long long shfl_xor64(unsigned long long v, int lane_mask) {
  const uint32_t lo = __shfl_xor_sync(0xffffffffu, uint32_t(v), lane_mask);
  const uint32_t hi = __shfl_xor_sync(0xffffffffu, uint32_t(v >> 32), lane_mask);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}
__global__ void __launch_bounds__(1024) sort_pairs_kernel(const uint32_t* __restrict__ scratch, int k, Layout L,
                                                          int32_t* __restrict__ idx, int size) {
  asm volatile("griddepcontrol.wait;" ::: "memory");            // launched with programmatic stream serialisation:
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // only the launch latency overlaps the previous kernel
  extern __shared__ unsigned long long s_keys[];
  const int row = blockIdx.x, tid = threadIdx.x;
  const size_t cand_offset = L.cand_offset_words;
  const uint32_t want = __ldcg(&scratch[L.info_offset + size_t(row) * 8 + kWant]);
  const unsigned long long* cand = reinterpret_cast<const unsigned long long*>(scratch + cand_offset) + size_t(row) * k;
  const int i0 = 2 * tid, i1 = i0 + 1;
  unsigned long long a = uint32_t(i0) < want ? __ldcg(&cand[i0]) : 0ull, b = uint32_t(i1) < want ? __ldcg(&cand[i1]) : 0ull;
  // Position i keeps the larger of the pair when it is the lower position of a descending run (or the upper of an
  // ascending one).
  auto keep = [](unsigned long long mine, unsigned long long other, bool take_max) {
    return take_max == (mine > other) ? mine : other;
  };
  for (int len = 2; len <= size; len <<= 1) {
    for (int stride = len >> 1; stride > 0; stride >>= 1) {
      const bool desc = (i0 & len) == 0;  // i0 and i1 lie in the same run of length len >= 2
      if (stride == 1) {
        const unsigned long long hi = a > b ? a : b, lo = a > b ? b : a;
        a = desc ? hi : lo;
        b = desc ? lo : hi;
      } else if (stride <= 32) {
        const bool lower = (i0 & stride) == 0;  // i1 shares the bit (stride >= 2)
        const unsigned long long oa = shfl_xor64(a, stride >> 1), ob = shfl_xor64(b, stride >> 1);
        a = keep(a, oa, lower == desc);
        b = keep(b, ob, lower == desc);
      } else {
        s_keys[i0] = a;
        s_keys[i1] = b;
        __syncthreads();
        const bool lower = (i0 & stride) == 0;
        const unsigned long long oa = s_keys[i0 ^ stride], ob = s_keys[i1 ^ stride];
        a = keep(a, oa, lower == desc);
        b = keep(b, ob, lower == desc);
        __syncthreads();
      }
    }
  }
  int32_t* out = idx + size_t(row) * k;
  if (i0 < k) out[i0] = uint32_t(i0) < want ? int32_t(0xffffffffu - uint32_t(a & 0xffffffffull)) : -1;
  if (i1 < k) out[i1] = uint32_t(i1) < want ? int32_t(0xffffffffu - uint32_t(b & 0xffffffffull)) : -1;
}

// glm_idx_expand (src/kernels/glm_fast.hip:737-748): selected pools -> compact token list, one thread per entry.
__global__ void __launch_bounds__(256) idx_expand_kernel(const int32_t* __restrict__ pools, const int32_t* __restrict__ pos,
                                                         int32_t* __restrict__ idx, int n, int k, int pool) {
  const int w = k * pool + pool - 1;
  const long long total = (long long)n * w;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / w), j = int(i - (long long)t * w), p = __ldg(&pos[t]);
    const int full = (p + 1) / pool, valid = full < k ? full : k, tail = (p + 1) % pool;
    int v = -1;
    if (j < valid * pool) v = __ldg(&pools[size_t(t) * k + j / pool]) * pool + j % pool;
    else if (j < valid * pool + tail) v = p + 1 - tail + (j - valid * pool);
    idx[i] = v;
  }
}

}  // namespace pkv_topk

#include "pkv_internal.hpp"

// Scratch for pkv_topk_bf16_static: 4 MiB that every GPU which loads the library holds until the process exits.
// In host code this name is only a handle for the runtime (not a device address): the device address is looked up once
// per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
constexpr size_t kStaticScratchWords = size_t(1) << 20;
static __device__ __align__(256) uint32_t g_topk_static_scratch[kStaticScratchWords];

namespace {
constexpr int kMaxDevices = 64;
uint32_t* g_static_ptr[kMaxDevices] = {};
std::mutex g_static_mu;

// The device address of the static scratch on the CURRENT device; looked up on the first call per device.
int static_scratch(uint32_t** out, std::string& err) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    err = std::string("built-in top-k scratch: cudaGetDevice: ") + cudaGetErrorString(e);
    return PKV_ERR_CUDA;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    err = "built-in top-k scratch: device ordinal " + std::to_string(dev) + " is outside the " + std::to_string(kMaxDevices) + " this library tracks";
    return PKV_ERR_LIMIT;
  }
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_topk_static_scratch);
    if (e != cudaSuccess || !p) {
      err = std::string("built-in top-k scratch: cudaGetSymbolAddress: ") + cudaGetErrorString(e);
      return PKV_ERR_CUDA;
    }
    g_static_ptr[dev] = static_cast<uint32_t*>(p);
  }
  *out = g_static_ptr[dev];
  return PKV_OK;
}

// Launches the four kernels on `stream` with caller-provided scratch. Shared by pkv_topk_bf16 and the entry point that
// brings its own static scratch.
int pkv_topk_launch(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, uint32_t* scratch,
                    cudaStream_t stream, std::string& err) {
  using namespace pkv_topk;
  const Layout l = layout(T, n, k);
  const dim3 grid(unsigned(l.slices), unsigned(T));
  int size = 2;
  while (size < k) size <<= 1;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  auto config = [&](dim3 g, unsigned threads, size_t smem) {
    cudaLaunchConfig_t c;
    std::memset(&c, 0, sizeof(c));
    c.gridDim = g;
    c.blockDim = dim3(threads);
    c.dynamicSmemBytes = smem;
    c.stream = stream;
    c.attrs = attr;
    c.numAttrs = 1;
    return c;
  };
  // The two arrival counters of every row (and the rest of the per-row results) start at zero: a memset node on the
  // stream, not an allocation.
  cudaMemsetAsync(scratch + l.info_offset, 0, size_t(T) * 8 * sizeof(uint32_t), stream);
  cudaLaunchConfig_t c = config(grid, kThreads, 0);
  cudaLaunchKernelEx(&c, hist_kernel, scores, n, ld, k, scratch, l, 0);
  cudaLaunchKernelEx(&c, hist_kernel, scores, n, ld, k, scratch, l, 1);
  cudaLaunchKernelEx(&c, collect_kernel, scores, n, ld, k, scratch, l);
  const uint32_t* cscratch = scratch;
  if (size >= 64 && size <= 2048) {
    c = config(dim3(unsigned(T)), unsigned(size / 2), size_t(size) * 8);
    cudaLaunchKernelEx(&c, sort_pairs_kernel, cscratch, k, l, idx, size);
  } else {
    c = config(dim3(unsigned(T)), kSortThreads, size_t(size) * 8);
    cudaLaunchKernelEx(&c, sort_kernel, cscratch, k, l, idx);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    err = std::string("top-k launch: ") + cudaGetErrorString(e);
    return PKV_ERR_CUDA;
  }
  return PKV_OK;
}

// The scratch the four-launch path uses: the caller's when it is there, aligned and large enough, else the library's
// built-in array (the one pkv_topk_bf16_static uses) when the shape fits it.
int pkv_topk_pick_scratch(uint32_t* scratch, size_t scratch_words, size_t need, uint32_t** out, std::string& err) {
  if (scratch && scratch_words >= need && (reinterpret_cast<uintptr_t>(scratch) & 7u) == 0) {
    *out = scratch;
    return PKV_OK;
  }
  if (need <= kStaticScratchWords) return static_scratch(out, err);
  err = "pkv_topk_bf16: this shape runs as four launches that need " + std::to_string(need) +
        " uint32 words of 8-byte aligned scratch (pkv_topk_scratch_words); the caller gave " + std::to_string(scratch ? scratch_words : 0) +
        " and the built-in scratch holds " + std::to_string(kStaticScratchWords);
  return PKV_ERR_LIMIT;
}

// One cluster launch when the shape and the device allow it (no scratch), else the four launches through scratch.
int pkv_topk_dispatch(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, uint32_t* scratch,
                      size_t scratch_words, cudaStream_t stream, std::string& err) {
  if (pkv_g_topk_path != 1 && pkv_topk_cluster_eligible(T, n, k)) {
    bool usable = false;
    const pkv_topk_cluster_group g{0, ld, 0, T, n, k, 0};
    if (const int rc = pkv_topk_cluster_launch(scores, &g, 1, idx, stream, &usable, err)) return rc;
    if (usable) return PKV_OK;
  }
  uint32_t* use = nullptr;
  if (const int rc = pkv_topk_pick_scratch(scratch, scratch_words, pkv_topk::layout(T, n > 0 ? n : 1, k).total_words, &use, err)) return rc;
  return pkv_topk_launch(scores, T, n, ld, k, idx, use, stream, err);
}

int pkv_topk_check(const uint16_t* scores, int T, int n, long long ld, int k, const int32_t* idx, std::string& err) {
  if (T < 0 || n < 0 || k <= 0 || ld < n) {
    err = "pkv_topk_bf16: bad shape";
    return PKV_ERR_ARG;
  }
  if (k > pkv_topk::kMaxK || n > pkv_topk::kSlice * pkv_topk::kMaxSlices) {
    err = "pkv_topk_bf16: k above 4096 or more than 2,097,152 keys per row";
    return PKV_ERR_LIMIT;
  }
  if (T > 0 && (!scores || !idx)) {
    err = "pkv_topk_bf16: null pointer";
    return PKV_ERR_ARG;
  }
  return PKV_OK;
}

}  // namespace

extern "C" {

size_t pkv_topk_scratch_words(int T, int n, int k) {
  if (T <= 0 || k <= 0) return 0;
  return pkv_topk::layout(T, n > 0 ? n : 1, k).total_words;
}

int pkv_topk_bf16(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, uint32_t* scratch,
                  size_t scratch_words, pkv_stream_t stream) {
  if (const int rc = pkv_topk_check(scores, T, n, ld, k, idx, pkv_g_err)) return rc;
  if (T == 0) return PKV_OK;
  return pkv_topk_dispatch(scores, T, n, ld, k, idx, scratch, scratch_words, reinterpret_cast<cudaStream_t>(stream), pkv_g_err);
}

size_t pkv_topk_batch_scratch_words(const pkv_topk_group* groups, int ngroups) {
  size_t need = 0;
  for (int g = 0; groups && g < ngroups; ++g)
    need = std::max(need, pkv_topk_scratch_words(groups[g].rows, groups[g].n, groups[g].k));
  return need;
}

int pkv_topk_bf16_batch(const uint16_t* scores, const pkv_topk_group* groups, int ngroups, int32_t* idx, uint32_t* scratch,
                        size_t scratch_words, pkv_stream_t stream) {
  if (ngroups < 0 || (ngroups > 0 && !groups)) {
    pkv_g_err = "pkv_topk_bf16_batch: bad group list";
    return PKV_ERR_ARG;
  }
  for (int g = 0; g < ngroups; ++g)
    if (groups[g].rows > 0)
      if (const int rc = pkv_topk_check(scores + groups[g].off, groups[g].rows, groups[g].n, groups[g].n, groups[g].k,
                                        idx + groups[g].idx_off, pkv_g_err))
        return rc;
  // All groups in one launch of thread-block clusters (32 groups per launch) when every group's shape allows it.
  if (pkv_g_topk_path != 1 && ngroups > 0) {
    std::vector<pkv_topk_cluster_group> cg;
    long long rows = 0;
    bool ok = true;
    for (int g = 0; g < ngroups && ok; ++g) {
      const pkv_topk_group& q = groups[g];
      if (q.rows <= 0) continue;
      ok = pkv_topk_cluster_eligible(q.rows, q.n, q.k);
      cg.push_back({(long long)q.off, q.n, q.idx_off, q.rows, q.n, q.k, 0});
      rows += q.rows;
    }
    if (ok && rows > 0 && rows <= 65535) {
      bool usable = false;
      if (const int rc = pkv_topk_cluster_launch(scores, cg.data(), int(cg.size()), idx, reinterpret_cast<cudaStream_t>(stream),
                                                 &usable, pkv_g_err))
        return rc;
      if (usable) return PKV_OK;
    }
  }
  // Otherwise the groups run one after the other on the stream, so they can share the scratch.
  for (int g = 0; g < ngroups; ++g) {
    const pkv_topk_group& q = groups[g];
    if (q.rows <= 0) continue;
    if (const int rc = pkv_topk_dispatch(scores + q.off, q.rows, q.n, q.n, q.k, idx + q.idx_off, scratch, scratch_words,
                                         reinterpret_cast<cudaStream_t>(stream), pkv_g_err))
      return rc;
  }
  return PKV_OK;
}

size_t pkv_topk_static_scratch_words(void) { return kStaticScratchWords; }

int pkv_topk_bf16_static(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, pkv_stream_t stream) {
  if (const int rc = pkv_topk_check(scores, T, n, ld, k, idx, pkv_g_err)) return rc;
  if (T == 0) return PKV_OK;
  const size_t need = pkv_topk::layout(T, n > 0 ? n : 1, k).total_words;
  if (need > kStaticScratchWords) {
    pkv_g_err = "pkv_topk_bf16_static: this shape needs " + std::to_string(need) + " scratch words, the built-in scratch holds " +
                std::to_string(kStaticScratchWords) + " (use pkv_topk_bf16 with your own scratch)";
    return PKV_ERR_LIMIT;
  }
  uint32_t* scratch = nullptr;
  if (const int rc = static_scratch(&scratch, pkv_g_err)) return rc;
  return pkv_topk_launch(scores, T, n, ld, k, idx, scratch, reinterpret_cast<cudaStream_t>(stream), pkv_g_err);
}

int pkv_idx_expand(const int32_t* pools, const int32_t* pos, int32_t* idx, int n, int k, int pool, pkv_stream_t stream) {
  if (n < 0 || k < 0 || pool <= 0) {
    pkv_g_err = "pkv_idx_expand: bad shape";
    return PKV_ERR_ARG;
  }
  const long long total = (long long)n * ((long long)k * pool + pool - 1);
  if (total == 0) return PKV_OK;
  if (!pools || !pos || !idx) {
    pkv_g_err = "pkv_idx_expand: null pointer";
    return PKV_ERR_ARG;
  }
  const long long blocks = (total + 255) / 256;
  pkv_topk::idx_expand_kernel<<<unsigned(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pools, pos, idx, n, k, pool);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    pkv_g_err = std::string("idx_expand launch: ") + cudaGetErrorString(e);
    return PKV_ERR_CUDA;
  }
  return PKV_OK;
}

}  // extern "C"
