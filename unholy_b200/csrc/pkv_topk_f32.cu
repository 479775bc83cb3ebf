// Index-list producer on fp32 scores: top-k per row, the fp32 twin of pkv_topk_bf16.
//
// Contract of ewtodd/unholy's topk_rows (src/kernels/ref.hpp:107, src/kernels/ref_attn.hip:143-254) and glm_topk
// (src/kernels/glm_fast.hpp:86-93, src/kernels/glm_fast.hip:557-681,852-874; one- or two-stage, same result): per row
// the want = min(k, #valid) largest scores, a score being valid when its order-preserving 32-bit key is greater than
// the key of -inf (-inf and negative NaN patterns are never selected; -0.0 sorts below +0.0); ties at the threshold
// go to the lowest indices; the output is ordered by (score descending, index ascending) and padded with -1; k <= 1024.
// That contract fixes every output element, so any algorithm that meets it is bit-exact with the reference.
//
// B200 design: one CTA of 512 threads per row, no scratch in global memory. Rows of up to kListKeys scores take
// topk_f32_list_kernel (group maxima, floor, list: see there); what follows describes the kernel for longer rows, whose
// building blocks the list kernel shares. The row is read from HBM ONCE: its keys
// are kept in shared memory (rows of up to kCacheKeys keys; longer rows are re-read through L2) while the first
// histogram is built. Radix select in three passes of 12 + 10 + 10 bits instead of four of 8: the first digit holds
// sign, exponent and three mantissa bits, so scores of similar magnitude still spread over dozens of bins and the
// shared-memory atomics do not pile up on one address; passes two and three only count the few keys inside the chosen
// bin. The selected keys are placed without atomics: every warp counts the keys above the threshold and the ties in
// its contiguous range of indices, the counts give each warp its bases, ballots give the rank inside a group of 32,
// so the threshold ties come out in index order (no serial scan of the row by one warp). The final sort of up to 1024
// (key, ~index) pairs keeps two elements per thread in registers and its network is unrolled at compile time: strides
// up to 32 are register or shuffle exchanges, only strides >= 64 go through shared memory.
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/unholy_pkv.h"

#include "pkv_internal.hpp"

namespace pkv_topkf {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxK = 1024;               // the reference's limit (ref_attn.hip:391, glm_fast.hip:854)
constexpr int kCacheKeys = 49152;         // 192 KB of keys in shared memory (rows above kListKeys)
constexpr int kListKeys = 40960;          // rows up to this length: keys (160 KB) and group maxima (20 KB) in shared memory
constexpr int kBins = 4096;               // first pass: 12 bits
constexpr uint32_t kNegInfKey = 0x007fffffu;  // sort_key(-inf) = ~0xff800000

__device__ __forceinline__ uint32_t sort_key(uint32_t u) { return (u & 0x80000000u) ? ~u : (u | 0x80000000u); }

struct Shared {
  uint32_t hist[kBins];
  unsigned long long sel[kMaxK];
  unsigned long long wsum64[kWarps];
  uint32_t wsum[kWarps];
  uint32_t wties[kWarps];
  uint32_t bin, need;
};

// Sum over all bins (BINS / kThreads consecutive bins per thread); every thread returns the total.
template <int BINS>
__device__ uint32_t block_total(Shared& s) {
  constexpr int PER = BINS / kThreads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t v = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) v += s.hist[tid * PER + j];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) s.wsum[warp] = v;
  __syncthreads();
  uint32_t t = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t += s.wsum[w];
  __syncthreads();
  return t;
}

// The highest bin b with (count in bins > b) < need <= (count in bins >= b): s.bin = b, s.need = need - count above.
// need is in 1..total, so exactly one thread writes.
template <int BINS>
__device__ void pick_bin(Shared& s, uint32_t need) {
  constexpr int PER = BINS / kThreads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t h[PER], local = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    h[j] = s.hist[tid * PER + j];
    local += h[j];
  }
  uint32_t sfx = local;  // inclusive suffix sum over threads
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_down_sync(0xffffffffu, sfx, o);
    if (lane + o < 32) sfx += t;
  }
  if (lane == 0) s.wsum[warp] = sfx;
  __syncthreads();
  for (int w = warp + 1; w < kWarps; ++w) sfx += s.wsum[w];
  uint32_t above = sfx - local;
#pragma unroll
  for (int j = PER - 1; j >= 0; --j) {
    if (above < need && above + h[j] >= need) {
      s.bin = uint32_t(tid * PER + j);
      s.need = need - above;
    }
    above += h[j];
  }
  __syncthreads();
}

template <int BINS>
__device__ __forceinline__ void clear_hist(Shared& s) {
  for (int b = threadIdx.x; b < BINS; b += kThreads) s.hist[b] = 0;
  __syncthreads();
}

__device__ __forceinline__ unsigned long long keep(unsigned long long mine, unsigned long long other, bool take_max) {
  return take_max == (mine > other) ? mine : other;
}
__device__ __forceinline__ unsigned long long shfl_xor64(unsigned long long v, int m) {
  const uint32_t lo = __shfl_xor_sync(0xffffffffu, uint32_t(v), m);
  const uint32_t hi = __shfl_xor_sync(0xffffffffu, uint32_t(v >> 32), m);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}

// Bitonic sort, descending, of 2^LOG (key, ~index) words held two per thread (words 2t, 2t + 1) by the first 2^LOG / 2
// threads; the network is unrolled at compile time: stride 1 inside the thread, 2..32 by shuffles, larger ones through
// s.sel with a named barrier over the sorting threads. Then the indices, -1 padded.
template <int LOG>
__device__ __forceinline__ void sort_and_write(Shared& s, int tid, int k, uint32_t want, int32_t* __restrict__ out) {
  constexpr int kSortThreads = (1 << LOG) / 2;
  if (tid >= kSortThreads) return;
  const int i0 = 2 * tid, i1 = i0 + 1;
  unsigned long long a = uint32_t(i0) < want ? s.sel[i0] : 0ull, b = uint32_t(i1) < want ? s.sel[i1] : 0ull;
  if (LOG > 6) asm volatile("bar.sync 1, %0;" ::"n"(kSortThreads) : "memory");  // s.sel is the exchange buffer below
#pragma unroll
  for (int L = 1; L <= LOG; ++L) {
    const bool desc = (i0 & (1 << L)) == 0;
#pragma unroll
    for (int S = L - 1; S >= 0; --S) {
      const int stride = 1 << S;
      if (stride == 1) {
        const unsigned long long hi = a > b ? a : b, lo = a > b ? b : a;
        a = desc ? hi : lo;
        b = desc ? lo : hi;
      } else if (stride <= 32) {
        const bool take_max = ((i0 & stride) == 0) == desc;
        a = keep(a, shfl_xor64(a, stride >> 1), take_max);
        b = keep(b, shfl_xor64(b, stride >> 1), take_max);
      } else {
        s.sel[i0] = a;
        s.sel[i1] = b;
        asm volatile("bar.sync 1, %0;" ::"n"(kSortThreads) : "memory");
        const bool take_max = ((i0 & stride) == 0) == desc;
        const unsigned long long oa = s.sel[i0 ^ stride], ob = s.sel[i1 ^ stride];
        a = keep(a, oa, take_max);
        b = keep(b, ob, take_max);
        asm volatile("bar.sync 1, %0;" ::"n"(kSortThreads) : "memory");
      }
    }
  }
  if (i0 < k) out[i0] = uint32_t(i0) < want ? int32_t(0xffffffffu - uint32_t(a & 0xffffffffull)) : -1;
  if (i1 < k) out[i1] = uint32_t(i1) < want ? int32_t(0xffffffffu - uint32_t(b & 0xffffffffull)) : -1;
}

// Exclusive prefix sums over the CTA's threads, in thread order. Two barriers each.
__device__ __forceinline__ uint32_t block_exclusive_scan(Shared& s, uint32_t v, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) s.wsum[warp] = inc;
  __syncthreads();
  const uint32_t w = lane < kWarps ? s.wsum[lane] : 0u;
  uint32_t before = lane < warp ? w : 0u, all = w;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, o);
    all += __shfl_xor_sync(0xffffffffu, all, o);
  }
  __syncthreads();
  total = all;
  return before + inc - v;
}
__device__ __forceinline__ unsigned long long block_exclusive_scan(Shared& s, unsigned long long v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) s.wsum64[warp] = inc;
  __syncthreads();
  unsigned long long before = lane < warp ? s.wsum64[lane] : 0ull;  // lane < warp < kWarps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
  __syncthreads();
  return before + inc - v;
}

__device__ __forceinline__ uint32_t key_of(const uint4& q, int j) { return j == 0 ? q.x : j == 1 ? q.y : j == 2 ? q.z : q.w; }

// Rows of up to kListKeys scores. The same selection as topk_f32_kernel below, but most of the row drops out after one
// cheap pass: with the largest key of every group of four, the histogram of those group maxima (n / 4 atomics) gives a
// floor below which no key can be selected (with at least k groups whose maximum is >= x, at least k keys are >= x);
// the groups that hold a key >= floor are compacted into a list in index order (about a third of the groups for
// k = 1024 of 32,768) and the three radix passes, the placement and its scan walk that list only.
__global__ void __launch_bounds__(kThreads) topk_f32_list_kernel(const float* __restrict__ scores, int n, long long ld,
                                                                 int k, int32_t* __restrict__ idx) {
  extern __shared__ __align__(16) uint32_t s_key[];  // keys [n + 8], then 16-bit group maxima [(n + 8) / 4 + 16]
  __shared__ Shared s;
  const int tid = threadIdx.x;
  const uint32_t* row = reinterpret_cast<const uint32_t*>(scores) + size_t(blockIdx.x) * size_t(ld);
  int32_t* out = idx + size_t(blockIdx.x) * size_t(k);
  // Position p of the cache holds element p - mis, so 16-byte groups of the row are 16-byte groups of the cache.
  const int mis = int((reinterpret_cast<uintptr_t>(row) >> 2) & 3u);
  const int padded = (mis + n + 3) & ~3, groups = padded >> 2, sgroups = (groups + 7) >> 3;
  const uint4* s_groups = reinterpret_cast<const uint4*>(s_key);
  uint16_t* s_gmax = reinterpret_cast<uint16_t*>(s_key + ((n + 8) & ~3));
  const uint4* s_sg = reinterpret_cast<const uint4*>(s_gmax);

  // ---- 1: load, cache, group maxima and their histogram (top 12 bits) ----
  clear_hist<kBins>(s);
  if (tid < mis) s_key[tid] = 0;  // key 0 is never valid, never selected
  if (tid < padded - (mis + n)) s_key[mis + n + tid] = 0;
  if (tid < sgroups * 8 - groups) s_gmax[groups + tid] = 0;
  const int head = min(n, (4 - mis) & 3), nvec = (n - head) >> 2, gbase = (mis + head) >> 2;
  const auto note_group = [&](int g, const uint4& q) {
    const uint32_t gm = max(max(q.x, q.y), max(q.z, q.w));
    s_gmax[g] = uint16_t(gm >> 16);
    if (gm > kNegInfKey) atomicAdd(&s.hist[gm >> 20], 1u);
  };
  if (tid < head) s_key[mis + tid] = sort_key(__ldg(row + tid));
  {
    const uint4* gv = reinterpret_cast<const uint4*>(row + head);
    uint4* sv = reinterpret_cast<uint4*>(s_key + mis + head);
#pragma unroll 4
    for (int v = tid; v < nvec; v += kThreads) {
      uint4 q = __ldg(gv + v);
      q.x = sort_key(q.x), q.y = sort_key(q.y), q.z = sort_key(q.z), q.w = sort_key(q.w);
      sv[v] = q;
      note_group(gbase + v, q);
    }
  }
  for (int i = head + 4 * nvec + tid; i < n; i += kThreads) s_key[mis + i] = sort_key(__ldg(row + i));
  __syncthreads();
  if (tid < 2) {  // the first and the last group when the 16-byte loads did not cover them
    const int g = tid == 0 ? 0 : groups - 1;
    const bool todo = tid == 0 ? (groups > 0 && !(gbase == 0 && nvec > 0)) : (groups > 1 && gbase + nvec != groups);
    if (todo) note_group(g, s_groups[g]);
  }
  __syncthreads();
  // ---- 2: the floor, then the list of groups with a key >= floor (it takes the place of the group maxima: every
  // thread reads the maxima of its three supergroups before anyone writes) ----
  const uint32_t valid_groups = block_total<kBins>(s);
  uint32_t floor_key = kNegInfKey + 1u;
  if (valid_groups >= uint32_t(k)) {
    pick_bin<kBins>(s, uint32_t(k));
    floor_key = s.bin << 20;
  }
  uint16_t* s_list = s_gmax;
  uint32_t listed = 0;
  {
    const uint32_t floor16 = floor_key >> 16;  // the floor's low 16 bits are zero
    uint32_t mask[3] = {0, 0, 0};
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      const int sg = 3 * tid + u;
      if (sg < sgroups) {
        const uint4 m = s_sg[sg];
        const uint32_t w[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) mask[u] |= (((w[j >> 1] >> (16 * (j & 1))) & 0xffffu) >= floor16 ? 1u : 0u) << j;
      }
    }
    uint32_t pos = block_exclusive_scan(s, uint32_t(__popc(mask[0]) + __popc(mask[1]) + __popc(mask[2])), listed);
#pragma unroll
    for (int u = 0; u < 3; ++u)
      for (uint32_t m = mask[u]; m != 0; m &= m - 1) s_list[pos++] = uint16_t((3 * tid + u) * 8 + (__ffs(int(m)) - 1));
  }
  __syncthreads();
  // ---- 3: radix select (12 + 10 + 10 bits) over the listed groups' keys >= floor ----
  clear_hist<kBins>(s);
  for (uint32_t eb = 0; eb < listed; eb += kThreads) {
    const uint32_t e = eb + tid;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (e < listed) q = s_groups[s_list[e]];
    // a shared-memory atomic costs about the same with one active lane as with 32: every lane marks its keys that are
    // in the race and the warp pops one marked key per lane and step
    uint32_t m = (q.x >= floor_key ? 1u : 0u) | (q.y >= floor_key ? 2u : 0u) | (q.z >= floor_key ? 4u : 0u) |
                 (q.w >= floor_key ? 8u : 0u);
    while (__any_sync(0xffffffffu, m != 0)) {
      if (m != 0) {
        atomicAdd(&s.hist[key_of(q, __ffs(int(m)) - 1) >> 20], 1u);
        m &= m - 1;
      }
    }
  }
  __syncthreads();
  const uint32_t in_race = block_total<kBins>(s);
  const uint32_t want = min(uint32_t(k), in_race);
  if (want == 0) {
    for (int i = tid; i < k; i += kThreads) out[i] = -1;
    return;
  }
  pick_bin<kBins>(s, want);
  uint32_t prefix = s.bin << 20, need = s.need;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int shift = pass == 0 ? 10 : 0;
    const uint32_t mask_hi = pass == 0 ? 0xfff00000u : 0xfffffc00u;
    __syncthreads();
    clear_hist<1024>(s);
    for (uint32_t e = tid; e < listed; e += kThreads) {
      const uint4 q = s_groups[s_list[e]];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t key = key_of(q, j);
        if ((key & mask_hi) == prefix) atomicAdd(&s.hist[(key >> shift) & 0x3ffu], 1u);
      }
    }
    __syncthreads();
    pick_bin<1024>(s, need);
    prefix |= s.bin << shift;
    need = s.need;
  }
  // ---- 4: placement. prefix = the threshold key, need = threshold ties to take. The list is in index order and every
  // thread takes a contiguous run of it: one exclusive scan over the threads' counts (keys above the threshold in the
  // low word, ties in the high word) gives every thread the places of its keys; ties go to the lowest indices. ----
  {
    const uint32_t per = (listed + kThreads - 1) / kThreads;
    const uint32_t e0 = min(listed, uint32_t(tid) * per), e1 = min(listed, e0 + per);
    unsigned long long c = 0;
    for (uint32_t e = e0; e < e1; ++e) {
      const uint4 q = s_groups[s_list[e]];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t key = key_of(q, j);
        c += (key > prefix ? 1ull : 0ull) + (key == prefix ? (1ull << 32) : 0ull);
      }
    }
    const unsigned long long exc = block_exclusive_scan(s, c);
    uint32_t a = uint32_t(exc), t = uint32_t(exc >> 32);
    const uint32_t base = want - need;  // keys above the threshold in the whole row
    if (c != 0)
      for (uint32_t e = e0; e < e1; ++e) {
        const int g = s_list[e];
        const uint4 q = s_groups[g];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t key = key_of(q, j);
          const unsigned long long word = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - uint32_t(g * 4 + j - mis));
          if (key > prefix) {
            s.sel[a++] = word;
          } else if (key == prefix) {
            if (t < need) s.sel[base + t] = word;
            ++t;
          }
        }
      }
  }
  __syncthreads();
  int log_size = 6;
  while ((1 << log_size) < k) ++log_size;
  switch (log_size) {
    case 6: sort_and_write<6>(s, tid, k, want, out); break;
    case 7: sort_and_write<7>(s, tid, k, want, out); break;
    case 8: sort_and_write<8>(s, tid, k, want, out); break;
    case 9: sort_and_write<9>(s, tid, k, want, out); break;
    default: sort_and_write<10>(s, tid, k, want, out); break;
  }
}

__global__ void __launch_bounds__(kThreads) topk_f32_kernel(const float* __restrict__ scores, int n, long long ld, int k,
                                                            int32_t* __restrict__ idx, int cached) {
  extern __shared__ __align__(16) uint32_t s_key[];  // [n + 3] when cached
  __shared__ Shared s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t* row = reinterpret_cast<const uint32_t*>(scores) + size_t(blockIdx.x) * size_t(ld);
  int32_t* out = idx + size_t(blockIdx.x) * size_t(k);
  uint32_t* sk = s_key + ((reinterpret_cast<uintptr_t>(row) >> 2) & 3u);  // sk + i is 16-byte aligned where row + i is
  const auto key_at = [&](int i) { return cached ? sk[i] : sort_key(__ldg(row + i)); };

  // Pass 1: the only read of the row from HBM, 16 bytes per load from the first aligned element on; 12-bit digit.
  // Keys that are not valid are not counted. sk is shifted so that the 16-byte groups are aligned in the cache too.
  clear_hist<kBins>(s);
  const int head = min(n, int((4u - uint32_t((reinterpret_cast<uintptr_t>(row) >> 2) & 3u)) & 3u));
  const int nvec = (n - head) >> 2;
  const auto count = [&](uint32_t key) {
    if (key > kNegInfKey) atomicAdd(&s.hist[key >> 20], 1u);
  };
  if (tid < head) {
    const uint32_t key = sort_key(__ldg(row + tid));
    if (cached) sk[tid] = key;
    count(key);
  }
  const uint4* rv = reinterpret_cast<const uint4*>(row + head);
#pragma unroll 4
  for (int v = tid; v < nvec; v += kThreads) {
    uint4 q = __ldg(rv + v);
    q.x = sort_key(q.x), q.y = sort_key(q.y), q.z = sort_key(q.z), q.w = sort_key(q.w);
    if (cached) *reinterpret_cast<uint4*>(sk + head + 4 * v) = q;
    count(q.x), count(q.y), count(q.z), count(q.w);
  }
  for (int i = head + 4 * nvec + tid; i < n; i += kThreads) {
    const uint32_t key = sort_key(__ldg(row + i));
    if (cached) sk[i] = key;
    count(key);
  }
  __syncthreads();
  const uint32_t nvalid = block_total<kBins>(s);
  const uint32_t want = min(uint32_t(k), nvalid);
  if (want == 0) {
    for (int i = tid; i < k; i += kThreads) out[i] = -1;
    return;
  }
  pick_bin<kBins>(s, want);
  uint32_t prefix = s.bin << 20, need = s.need;
  // Passes 2 and 3: 10 bits each, over the keys that share the prefix.
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int shift = pass == 0 ? 10 : 0;
    const uint32_t mask_hi = pass == 0 ? 0xfff00000u : 0xfffffc00u;
    __syncthreads();
    clear_hist<1024>(s);
#pragma unroll 4
    for (int i = tid; i < n; i += kThreads) {
      const uint32_t key = key_at(i);
      if ((key & mask_hi) == prefix) atomicAdd(&s.hist[(key >> shift) & 0x3ffu], 1u);
    }
    __syncthreads();
    pick_bin<1024>(s, need);
    prefix |= s.bin << shift;
    need = s.need;
  }
  // prefix = the threshold key (valid: it is the key of a counted score); need = threshold ties to take.
  // Each warp owns a contiguous range of indices. First sweep: how many keys above the threshold and how many ties
  // the range holds. Second sweep: every such key goes to its slot — the warps' counts give the bases, ballots the
  // rank inside a group of 32 — so no atomic is needed and the ties come out in index order.
  const int per_warp = ((n + kWarps - 1) / kWarps + 31) & ~31;
  const int w0 = warp * per_warp, w1 = min(n, w0 + per_warp);
  uint32_t above = 0, ties = 0;
#pragma unroll 4
  for (int i = w0 + lane; i < w1; i += 32) {
    const uint32_t key = key_at(i);
    above += key > prefix;
    ties += key == prefix;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    above += __shfl_xor_sync(0xffffffffu, above, o);
    ties += __shfl_xor_sync(0xffffffffu, ties, o);
  }
  if (lane == 0) {
    s.wsum[warp] = above;
    s.wties[warp] = ties;
  }
  __syncthreads();
  uint32_t above_before = 0, ties_before = 0;
  for (int w = 0; w < warp; ++w) {
    above_before += s.wsum[w];
    ties_before += s.wties[w];
  }
  const uint32_t base = want - need;  // = keys above the threshold in the whole row
  const bool take_ties = ties > 0 && ties_before < need;
  if (above > 0 || take_ties) {
    const uint32_t lt = (1u << lane) - 1u;
    uint32_t a_rank = above_before, t_rank = ties_before;
    for (int i0 = w0; i0 < w1; i0 += 32) {
      const int i = i0 + lane;
      const uint32_t key = i < w1 ? key_at(i) : 0u;  // 0 is below every threshold
      const uint32_t ba = __ballot_sync(0xffffffffu, key > prefix);
      const uint32_t bt = __ballot_sync(0xffffffffu, key == prefix);
      const unsigned long long packed = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - uint32_t(i));
      if (key > prefix) s.sel[a_rank + __popc(ba & lt)] = packed;
      const uint32_t r = t_rank + __popc(bt & lt);
      if (key == prefix && r < need) s.sel[base + r] = packed;
      a_rank += __popc(ba);
      t_rank += __popc(bt);
    }
  }
  __syncthreads();
  // Sort 2^log_size >= max(k, 64) (<= 1024) words, two per thread, descending; padding 0 sorts last.
  int log_size = 6;
  while ((1 << log_size) < k) ++log_size;
  switch (log_size) {
    case 6: sort_and_write<6>(s, tid, k, want, out); break;
    case 7: sort_and_write<7>(s, tid, k, want, out); break;
    case 8: sort_and_write<8>(s, tid, k, want, out); break;
    case 9: sort_and_write<9>(s, tid, k, want, out); break;
    default: sort_and_write<10>(s, tid, k, want, out); break;
  }
}

// Dynamic shared memory of the list kernel: keys [n + 8] and 16-bit group maxima [(n + 8) / 4 + 16].
static size_t list_smem_bytes(int n) { return size_t((n + 8) & ~3) * 4 + size_t((n + 8) / 4 + 16) * 2; }

}  // namespace pkv_topkf

extern "C" {

int pkv_topk_f32(const float* scores, int T, int n, long long ld, int k, int32_t* idx, pkv_stream_t stream) {
  using namespace pkv_topkf;
  if (T <= 0 || n <= 0) return PKV_OK;  // nothing to do, as the reference (ref_attn.hip:390 launches T blocks)
  if (k > kMaxK) {
    pkv_g_err = "pkv_topk_f32: k > 1024";
    return PKV_ERR_ARG;
  }
  if (!scores || !idx || k <= 0 || ld < n || n > (1 << 30)) {
    pkv_g_err = "pkv_topk_f32: null pointer, k <= 0, ld < n or n > 2^30";
    return PKV_ERR_ARG;
  }
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  static thread_local int opted_dev = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && dev != opted_dev) {  // once per device and thread: both kernels may use the whole shared memory
    e = cudaFuncSetAttribute(topk_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int((kCacheKeys + 3) * 4));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(topk_f32_list_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(list_smem_bytes(kListKeys)));
    if (e == cudaSuccess) opted_dev = dev;
  }
  if (e != cudaSuccess) {
    pkv_g_err = std::string("pkv_topk_f32: ") + cudaGetErrorString(e);
    return PKV_ERR_CUDA;
  }
  if (n <= kListKeys) {
    topk_f32_list_kernel<<<T, kThreads, list_smem_bytes(n), st>>>(scores, n, ld, k, idx);
  } else {
    const int cached = n <= kCacheKeys;
    topk_f32_kernel<<<T, kThreads, cached ? size_t(n + 3) * 4 : 0, st>>>(scores, n, ld, k, idx, cached);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    pkv_g_err = std::string("pkv_topk_f32: ") + cudaGetErrorString(e);
    return PKV_ERR_CUDA;
  }
  return PKV_OK;
}

}  // extern "C"
