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

#include <cstdint>
#include <mutex>
#include <string>

#include "../../include/unholy_pkv.h"

namespace pkv_topk {

constexpr int kThreads = 512;
constexpr int kSlice = 8192;          // keys per CTA
constexpr int kMaxK = 4096;
constexpr int kMaxSlices = 256;       // rows of up to 2M keys
constexpr uint32_t kNegInfKey = 0x007Fu;  // key16 of the bf16 pattern 0xFF80

__device__ __forceinline__ uint32_t key16(uint32_t b) { return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u); }

// Scratch layout (uint32 words): hist[row][slice][2][256], then candidates as uint64 [row][k] (8-byte aligned).
struct Layout {
  int slices;
  size_t hist_words, cand_offset_words, total_words;
};
__host__ __device__ inline Layout layout(int T, int n, int k) {
  Layout l;
  l.slices = (n + kSlice - 1) / kSlice;
  if (l.slices < 1) l.slices = 1;
  l.hist_words = size_t(T) * l.slices * 512;
  l.cand_offset_words = (l.hist_words + 1) & ~size_t(1);
  l.total_words = l.cand_offset_words + size_t(T) * k * 2;
  return l;
}

// Inclusive suffix sums of hist[0..255] in place (S[b] = sum of bins >= b), then the bin the reference's walk from the
// top finds: the highest b >= 1 with S[b] >= need, else 0. Returns through shared variables. blockDim.x >= 256.
__device__ void pick_bin(uint32_t* hist, uint32_t need, uint32_t* s_bin, uint32_t* s_need) {
  const int tid = threadIdx.x;
  for (int d = 1; d < 256; d <<= 1) {
    uint32_t add = 0;
    if (tid < 256 && tid + d < 256) add = hist[tid + d];
    __syncthreads();
    if (tid < 256) hist[tid] += add;
    __syncthreads();
  }
  if (tid == 0) {
    *s_bin = 0;
    *s_need = need - hist[1];
  }
  __syncthreads();
  if (tid >= 1 && tid < 256) {
    const uint32_t above = tid < 255 ? hist[tid + 1] : 0u;
    if (hist[tid] >= need && above < need) {
      *s_bin = uint32_t(tid);
      *s_need = need - above;
    }
  }
  __syncthreads();
}

// Sum over slices of one of the two histograms of a row into shared memory.
__device__ void sum_hist(const uint32_t* row_hist, int slices, int which, uint32_t* out) {
  for (int b = threadIdx.x; b < 256; b += blockDim.x) {
    uint32_t s = 0;
    for (int sl = 0; sl < slices; ++sl) s += row_hist[(size_t(sl) * 2 + which) * 256 + b];
    out[b] = s;
  }
  __syncthreads();
}

// Pass 1 (which = 0): histogram of the high key byte over the slice's valid keys. Pass 2 (which = 1): the threshold's
// high byte is derived from the summed pass-1 histograms, then the low byte is histogrammed over the keys that share it.
__global__ void __launch_bounds__(kThreads) hist_kernel(const uint16_t* __restrict__ scores, int n, long long ld, int k,
                                                        uint32_t* __restrict__ scratch, int slices, int which) {
  __shared__ uint32_t hist[256], total[256];
  __shared__ uint32_t s_bin, s_need;
  const int row = blockIdx.y, sl = blockIdx.x, tid = threadIdx.x;
  uint32_t* row_hist = scratch + size_t(row) * slices * 512;
  uint32_t hi_bin = 0;
  if (which == 1) {
    sum_hist(row_hist, slices, 0, total);
    uint32_t nvalid = 0;
    // total[] still holds plain counts here: the number of valid keys is their sum (computed by every thread).
    for (int b = 0; b < 256; ++b) nvalid += total[b];
    const uint32_t want = min(uint32_t(k), nvalid);
    __syncthreads();
    pick_bin(total, want, &s_bin, &s_need);
    hi_bin = s_bin;
  }
  for (int b = tid; b < 256; b += kThreads) hist[b] = 0;
  __syncthreads();
  const uint16_t* r = scores + size_t(row) * ld;
  const int lo = sl * kSlice, hi = min(n, lo + kSlice);
  for (int i = lo + tid; i < hi; i += kThreads) {
    const uint32_t key = key16(r[i]);
    if (key <= kNegInfKey) continue;
    if (which == 0) atomicAdd(&hist[key >> 8], 1u);
    else if ((key >> 8) == hi_bin) atomicAdd(&hist[key & 0xffu], 1u);
  }
  __syncthreads();
  for (int b = tid; b < 256; b += kThreads) row_hist[(size_t(sl) * 2 + which) * 256 + b] = hist[b];
}

// Collect: every slice writes its keys above the threshold and its share of the threshold ties (lowest indices first
// across the whole row) into the row's candidate array at offsets known from the per-slice histograms.
__global__ void __launch_bounds__(kThreads) collect_kernel(const uint16_t* __restrict__ scores, int n, long long ld, int k,
                                                           uint32_t* __restrict__ scratch, int slices, size_t cand_offset) {
  __shared__ uint32_t total[256];
  __shared__ uint32_t s_bin, s_need, s_above, s_warp[kThreads / 32], s_run;
  __shared__ uint32_t s_slice_above[kMaxSlices], s_slice_ties[kMaxSlices];
  const int row = blockIdx.y, sl = blockIdx.x, tid = threadIdx.x;
  const uint32_t* row_hist = scratch + size_t(row) * slices * 512;
  unsigned long long* cand = reinterpret_cast<unsigned long long*>(scratch + cand_offset) + size_t(row) * k;
  sum_hist(row_hist, slices, 0, total);
  uint32_t nvalid = 0;
  for (int b = 0; b < 256; ++b) nvalid += total[b];
  const uint32_t want = min(uint32_t(k), nvalid);
  __syncthreads();
  if (want == 0) return;
  pick_bin(total, want, &s_bin, &s_need);
  const uint32_t hi_bin = s_bin, need1 = s_need;
  __syncthreads();
  sum_hist(row_hist, slices, 1, total);
  pick_bin(total, need1, &s_bin, &s_need);
  const uint32_t lo_bin = s_bin, need_ties = s_need;
  const uint32_t thr = (hi_bin << 8) | lo_bin;
  // Offsets: keys above the threshold come first (any order: the sort follows), then the ties in index order. One warp
  // per slice sums that slice's bins above the threshold.
  for (int s2 = tid >> 5; s2 < slices; s2 += kThreads / 32) {
    const uint32_t* h0 = row_hist + (size_t(s2) * 2) * 256;
    const uint32_t* h1 = h0 + 256;
    uint32_t a = 0;
    for (uint32_t b = tid & 31; b < 256; b += 32) a += (b > hi_bin ? h0[b] : 0u) + (b > lo_bin ? h1[b] : 0u);
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if ((tid & 31) == 0) {
      s_slice_above[s2] = a;
      s_slice_ties[s2] = h1[lo_bin];
    }
  }
  __syncthreads();
  uint32_t above_before = 0, ties_before = 0, above_total = 0;
  for (int s2 = 0; s2 < slices; ++s2) {
    above_total += s_slice_above[s2];
    if (s2 < sl) {
      above_before += s_slice_above[s2];
      ties_before += s_slice_ties[s2];
    }
  }
  if (tid == 0) {
    s_above = 0;
    s_run = 0;
  }
  __syncthreads();
  const uint16_t* r = scores + size_t(row) * ld;
  const int lo = sl * kSlice, hi = min(n, lo + kSlice);
  for (int base = lo; base < hi; base += kThreads) {
    const int i = base + tid;
    const uint32_t key = i < hi ? key16(r[i]) : 0u;
    const bool valid = i < hi && key > kNegInfKey;
    if (valid && key > thr) {
      const uint32_t slot = above_before + atomicAdd(&s_above, 1u);
      cand[slot] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - uint32_t(i));
    }
    // ordered positions of the ties of this chunk
    const bool tie = valid && key == thr;
    const unsigned ballot = __ballot_sync(0xffffffffu, tie);
    const int lane = tid & 31, warp = tid >> 5;
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    uint32_t before = s_run;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    before += __popc(ballot & ((1u << lane) - 1u));
    if (tie) {
      const uint32_t rank = ties_before + before;
      if (rank < need_ties) cand[above_total + rank] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - uint32_t(i));
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t t = 0;
      for (int w = 0; w < kThreads / 32; ++w) t += s_warp[w];
      s_run += t;
    }
    __syncthreads();
  }
}

// Sort: one CTA per row; (key, ~index) descending = (score descending, index ascending); -1 padding.
__global__ void __launch_bounds__(kThreads) sort_kernel(const uint32_t* __restrict__ scratch, int k, int slices,
                                                        size_t cand_offset, int32_t* __restrict__ idx) {
  extern __shared__ unsigned long long s_keys[];
  __shared__ uint32_t s_want;
  const int row = blockIdx.x, tid = threadIdx.x;
  const uint32_t* row_hist = scratch + size_t(row) * slices * 512;
  if (tid == 0) s_want = 0;
  __syncthreads();
  uint32_t local = 0;
  for (int j = tid; j < slices * 256; j += kThreads) local += row_hist[(size_t(j >> 8) * 2) * 256 + (j & 255)];
  atomicAdd(&s_want, local);
  __syncthreads();
  const uint32_t want = min(uint32_t(k), s_want);
  int size = 1;
  while (size < k) size <<= 1;
  const unsigned long long* cand = reinterpret_cast<const unsigned long long*>(scratch + cand_offset) + size_t(row) * k;
  for (int i = tid; i < size; i += kThreads) s_keys[i] = uint32_t(i) < want ? cand[i] : 0ull;
  __syncthreads();
  for (int len = 2; len <= size; len <<= 1)
    for (int stride = len >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < size; i += kThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const bool desc = (i & len) == 0;
          const unsigned long long a = s_keys[i], b = s_keys[j];
          if ((a < b) == desc) {
            s_keys[i] = b;
            s_keys[j] = a;
          }
        }
      }
      __syncthreads();
    }
  int32_t* out = idx + size_t(row) * k;
  for (int i = tid; i < k; i += kThreads)
    out[i] = uint32_t(i) < want ? int32_t(0xffffffffu - uint32_t(s_keys[i] & 0xffffffffull)) : -1;
}

}  // namespace pkv_topk

extern thread_local std::string pkv_g_err;  // defined in pkv_kernels.cu: what pkv_last_error() returns

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
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    err = std::string("pkv_topk_bf16_static: cudaGetDevice: ") + cudaGetErrorString(e);
    return PKV_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_topk_static_scratch);
    if (e != cudaSuccess || !p) {
      err = std::string("pkv_topk_bf16_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e);
      return PKV_ERR_CUDA;
    }
    g_static_ptr[dev] = static_cast<uint32_t*>(p);
  }
  *out = g_static_ptr[dev];
  return PKV_OK;
}
}  // namespace

extern "C" {

size_t pkv_topk_scratch_words(int T, int n, int k) {
  if (T <= 0 || k <= 0) return 0;
  return pkv_topk::layout(T, n > 0 ? n : 1, k).total_words;
}

// Launches the four kernels on `stream` with caller-provided scratch. Shared by pkv_topk_bf16 and the entry point that
// brings its own static scratch.
int pkv_topk_launch(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, uint32_t* scratch,
                    cudaStream_t stream, std::string& err) {
  using namespace pkv_topk;
  const Layout l = layout(T, n, k);
  const dim3 grid(unsigned(l.slices), unsigned(T));
  hist_kernel<<<grid, kThreads, 0, stream>>>(scores, n, ld, k, scratch, l.slices, 0);
  hist_kernel<<<grid, kThreads, 0, stream>>>(scores, n, ld, k, scratch, l.slices, 1);
  collect_kernel<<<grid, kThreads, 0, stream>>>(scores, n, ld, k, scratch, l.slices, l.cand_offset_words);
  int size = 1;
  while (size < k) size <<= 1;
  sort_kernel<<<unsigned(T), kThreads, size_t(size) * 8, stream>>>(scratch, k, l.slices, l.cand_offset_words, idx);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    err = std::string("top-k launch: ") + cudaGetErrorString(e);
    return PKV_ERR_CUDA;
  }
  return PKV_OK;
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

int pkv_topk_bf16(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, uint32_t* scratch,
                  size_t scratch_words, pkv_stream_t stream) {
  if (const int rc = pkv_topk_check(scores, T, n, ld, k, idx, pkv_g_err)) return rc;
  if (T == 0) return PKV_OK;
  const size_t need = pkv_topk::layout(T, n > 0 ? n : 1, k).total_words;
  if (!scratch || scratch_words < need || (reinterpret_cast<uintptr_t>(scratch) & 7u)) {
    pkv_g_err = "pkv_topk_bf16: scratch must be 8-byte aligned and hold pkv_topk_scratch_words(T, n, k) words";
    return PKV_ERR_ARG;
  }
  return pkv_topk_launch(scores, T, n, ld, k, idx, scratch, reinterpret_cast<cudaStream_t>(stream), pkv_g_err);
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

}  // extern "C"
