// Top-k of bf16 scores in ONE launch: a thread-block cluster of 1, 2, 4 or 8 CTAs per row, no scratch in global memory.
//
// Same contract as pkv_topk.cu (ewtodd/unholy's topk_bf16, src/kernels/indexer.hpp:74, src/kernels/indexer.hip:408-560):
// per row the min(k, #valid) largest scores, valid = 16-bit order-preserving key above the key of -inf, threshold
// ties to the lowest indices, output ordered by (score descending, index ascending), -1 padded.
//
// The four-launch path in pkv_topk.cu reads a row three times (the second and third time from L2) and passes
// histograms, offsets and candidates through global scratch. Here the CTAs of a cluster split the row, every CTA reads
// its slice from HBM once and keeps the keys in shared memory (up to 160 KB: one CTA of 1024 threads per SM), and the
// CTAs exchange their histograms through distributed shared memory. The cluster size is chosen by the host so that
// the launch is about one CTA per SM (64 rows of 131,072 keys: 2 CTAs per row on 128 SMs):
//   1. load the slice (16-byte loads), keys to shared memory together with the largest key of every group of 8
//      (DPX three-way 16-bit maxima), histogram of those group maxima by their top 12 bits. With at least k groups
//      whose maximum is >= x, at least k keys are >= x: the bin of the k-th largest group maximum gives this CTA a
//      floor below which no key can be selected. Cluster barrier A; the row's floor `base` is the largest of the CTAs'.
//   2. the groups with a key >= base are compacted, in index order, into a list (about a quarter of the groups for
//      k = 2048 of 131,072): every later pass walks the list with all lanes busy;
//   3. exact counts, one bin per key value, of the keys in the window [base, base + 4096) — equal scores are the only
//      same-address atomics —, keys above the window counted apart; cluster barrier B; the sum over the CTAs gives the
//      threshold key and the number of threshold ties to take. (If the keys above the window alone reach k, a coarse
//      histogram names the 16 keys around the threshold and a second round of the same pass looks at those: two rounds
//      at most, two more barriers.) Every CTA publishes how many selected keys it holds; cluster barrier C;
//   4. every CTA writes its selected keys, in index order, into the candidate list in CTA 0's shared memory (remote
//      stores). A candidate is (key << 16 | 0xffff - ordinal) plus its index: the ordinal is the candidate's place
//      in index order, so sorting the 32-bit words descending IS the (score descending, index ascending) order;
//      cluster barrier D; CTA 0 sorts the words (bitonic network unrolled at compile time, four words per thread in
//      registers: strides up to 64 are register or shuffle exchanges) and writes the indices.
// Every thread of every CTA passes the same cluster barriers whatever its own data (the branch that adds a round is
// taken from cluster-wide sums, identical in every CTA; no early exit before the last barrier), and no CTA touches
// another's shared memory after the last barrier.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>

#include "../../include/unholy_pkv.h"
#include "pkv_internal.hpp"

namespace cg = cooperative_groups;

namespace pkv_topkc {

constexpr int kMaxCluster = 8;
constexpr int kMaxGroups = 32;
constexpr int kMaxThreads = 1024;         // CTAs of 256, 512 or 1024 threads (chosen by the host)
constexpr int kMaxWarps = kMaxThreads / 32;
constexpr int kMaxK = 2048;
constexpr int k256Slice = 16384, k512Slice = 32768;  // the longest slices the smaller CTAs take (64 keys per thread)
constexpr int kMaxSlice = 81920;          // keys per CTA kept in shared memory (160 KB, and 20 KB of group maxima)
constexpr int kBins = 4096;               // top 12 bits: four bins per thread
constexpr uint32_t kNegInfKey = 0x007Fu;  // key of the bf16 pattern 0xFF80; valid keys are above it (their top 12 bits >= 8)

// Two bf16 patterns in one word -> their order-preserving keys: ~b when the sign is set, b | 0x8000 otherwise.
__device__ __forceinline__ uint32_t key_pair(uint32_t w) { return w ^ ((((w >> 15) & 0x00010001u) * 0xffffu) | 0x80008000u); }
__device__ __forceinline__ uint32_t key_one(uint32_t b) { return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u); }

struct __align__(16) Shared {
  uint32_t hist0[kBins];   // group maxima by their top 12 bits; then the keys above the window, 16 to a bin; after
                           // barrier C, in CTA 0, the candidates' sort words
  uint32_t fine[kBins];    // exact counts of the keys base + v of the window; after barrier C, in CTA 0, the
                           // candidates' indices (cand_idx below)
  unsigned long long wsum64[kMaxWarps];
  uint32_t wsum[kMaxWarps], wsum2[kMaxWarps];
  uint32_t floor_pub;      // this CTA's floor: read by the others after barrier A
  uint32_t over;           // this CTA's keys above the window
  uint32_t pub_above, pub_ties;  // this CTA's selected keys above the threshold, and its ties: read after barrier C
  uint32_t bin, need;
};

// The rows of one launch: up to kMaxGroups blocks of `rows` rows of n scores (row r of a block at scores + off + r * ld,
// its k indices at idx + idx_off + r * k); row0 = the block's first row in the launch.
struct Batch {
  int ngroups, slice_max;
  pkv_topk_cluster_group g[kMaxGroups];
};

template <class F>
__device__ __forceinline__ void for_each_key(const uint4& q, F&& f) {
  f(q.x & 0xffffu, 0), f(q.x >> 16, 1), f(q.y & 0xffffu, 2), f(q.y >> 16, 3);
  f(q.z & 0xffffu, 4), f(q.z >> 16, 5), f(q.w & 0xffffu, 6), f(q.w >> 16, 7);
}

// The largest of the eight 16-bit keys of a group.
__device__ __forceinline__ uint32_t group_max(const uint4& q) {
  const uint32_t m = __vmaxu2(__vimax3_u16x2(q.x, q.y, q.z), q.w);
  return max(m >> 16, m & 0xffffu);
}

// Key j (0..7) of a group.
__device__ __forceinline__ uint32_t key_at(const uint4& q, int j) {
  const uint32_t w = (j & 4) ? ((j & 2) ? q.w : q.z) : ((j & 2) ? q.y : q.x);
  return (j & 1) ? (w >> 16) : (w & 0xffffu);
}

// Bit j set when key j of the group is >= floor_key.
__device__ __forceinline__ uint32_t mask_at_least(const uint4& q, uint32_t floor_key) {
  uint32_t m = 0;
  for_each_key(q, [&](uint32_t key, int j) { m |= (key >= floor_key ? 1u : 0u) << j; });
  return m;
}

// Keys above the threshold in the low half, keys equal to it in the high half.
__device__ __forceinline__ uint32_t count_selected(const uint4& q, uint32_t thr) {
  uint32_t c = 0;
  for_each_key(q, [&](uint32_t key, int) { c += (key > thr ? 1u : 0u) + (key == thr ? 0x10000u : 0u); });
  return c;
}

__device__ __forceinline__ uint32_t keep(uint32_t mine, uint32_t other, bool take_max) {
  return take_max ? max(mine, other) : min(mine, other);
}

// Bitonic sort, descending, of SIZE words: thread t < SIZE / 4 holds words 4t..4t+3. The network is unrolled at compile
// time, so a stage is a handful of instructions: strides 1 and 2 inside the thread, 4..64 by shuffles, larger ones
// through `buf` with a named barrier over the SIZE / 4 sorting threads.
template <int LOG>
__device__ __forceinline__ void sort_desc(uint32_t& e0, uint32_t& e1, uint32_t& e2, uint32_t& e3, uint32_t* buf, int tid) {
  constexpr int kSortThreads = (1 << LOG) / 4;
#pragma unroll
  for (int L = 1; L <= LOG; ++L) {
    const int len = 1 << L;
    const bool desc = L == 1 ? true : ((4 * tid) & len) == 0;  // for len >= 4 the thread's four words share the direction
#pragma unroll
    for (int S = L - 1; S >= 0; --S) {
      const int stride = 1 << S;
      if (stride == 1) {
        const bool d23 = L == 1 ? false : desc;
        const uint32_t a = keep(e0, e1, desc), b = keep(e1, e0, !desc), c = keep(e2, e3, d23), d = keep(e3, e2, !d23);
        e0 = a, e1 = b, e2 = c, e3 = d;
      } else if (stride == 2) {
        const uint32_t a = keep(e0, e2, desc), b = keep(e1, e3, desc), c = keep(e2, e0, !desc), d = keep(e3, e1, !desc);
        e0 = a, e1 = b, e2 = c, e3 = d;
      } else if (stride <= 64) {
        const int m = stride >> 2;
        const bool take_max = ((tid & m) == 0) == desc;
        e0 = keep(e0, __shfl_xor_sync(0xffffffffu, e0, m), take_max);
        e1 = keep(e1, __shfl_xor_sync(0xffffffffu, e1, m), take_max);
        e2 = keep(e2, __shfl_xor_sync(0xffffffffu, e2, m), take_max);
        e3 = keep(e3, __shfl_xor_sync(0xffffffffu, e3, m), take_max);
      } else {
        const int m = stride >> 2;
        reinterpret_cast<uint4*>(buf)[tid] = make_uint4(e0, e1, e2, e3);
        asm volatile("bar.sync 1, %0;" ::"n"(kSortThreads) : "memory");
        const uint4 o = reinterpret_cast<const uint4*>(buf)[tid ^ m];
        const bool take_max = ((tid & m) == 0) == desc;
        e0 = keep(e0, o.x, take_max), e1 = keep(e1, o.y, take_max);
        e2 = keep(e2, o.z, take_max), e3 = keep(e3, o.w, take_max);
        asm volatile("bar.sync 1, %0;" ::"n"(kSortThreads) : "memory");
      }
    }
  }
}

template <int LOG>
__device__ __forceinline__ void sort_and_write(Shared& s, int tid, int k, uint32_t want, int32_t* __restrict__ out) {
  if (tid >= (1 << LOG) / 4) return;
  const uint4 q = reinterpret_cast<const uint4*>(s.hist0)[tid];
  uint32_t e0 = q.x, e1 = q.y, e2 = q.z, e3 = q.w;
  sort_desc<LOG>(e0, e1, e2, e3, s.hist0, tid);
  const uint32_t e[4] = {e0, e1, e2, e3};
  int32_t v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = uint32_t(4 * tid + j) < want ? reinterpret_cast<const int32_t*>(s.fine)[0xffffu - (e[j] & 0xffffu)] : -1;
  if (4 * tid + 3 < k && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
    reinterpret_cast<int4*>(out)[tid] = make_int4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (4 * tid + j < k) out[4 * tid + j] = v[j];
  }
}

// Exclusive prefix sum over the CTA's threads (in thread order) and the total. Two barriers; uses s.wsum.
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
  const uint32_t w = lane < int(blockDim.x >> 5) ? s.wsum[lane] : 0u;
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

// The same for 64-bit values (two counters side by side), without the total.
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
  unsigned long long before = lane < warp ? s.wsum64[lane] : 0ull;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
  __syncthreads();
  return before + inc - v;
}

// One suffix scan over a 4096-bin histogram (each thread owns 4096 / THREADS consecutive bins): of this CTA alone (nc == 0,
// plain shared-memory reads) or summed over CTAs 0 .. nc - 1 of the cluster (distributed shared memory). Returns the
// total; when need_fn(total) > 0, s.bin is the highest bin with (count above it) < need <= (count from it up) and
// s.need = need - (count above it). Two barriers; the caller reads s.bin / s.need after the call.
template <int THREADS, class NeedFn>
__device__ __forceinline__ uint32_t reduce_and_pick(cg::cluster_group& cluster, Shared& s, uint32_t* hist, int nc,
                                                    NeedFn&& need_fn) {
  constexpr int PER = kBins / THREADS, WARPS = THREADS / 32;  // this thread's bins: PER consecutive ones
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t r[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) r[j] = 0;
  for (int c = 0; c < (nc == 0 ? 1 : nc); ++c) {
    const uint32_t* h = nc == 0 ? hist : cluster.map_shared_rank(hist, c);
#pragma unroll
    for (int j = 0; j < PER; j += 4) {
      const uint4 v = *reinterpret_cast<const uint4*>(&h[PER * tid + j]);
      r[j] += v.x, r[j + 1] += v.y, r[j + 2] += v.z, r[j + 3] += v.w;
    }
  }
  uint32_t local = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) local += r[j];
  uint32_t sfx = local;  // inclusive suffix sum over threads (higher bins first)
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_down_sync(0xffffffffu, sfx, o);
    if (lane + o < 32) sfx += t;
  }
  if (lane == 0) s.wsum[warp] = sfx;
  __syncthreads();
  const uint32_t w = lane < WARPS ? s.wsum[lane] : 0u;
  uint32_t higher = lane > warp ? w : 0u, total = w;  // the totals of the warps above this one, and of all warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    higher += __shfl_xor_sync(0xffffffffu, higher, o);
    total += __shfl_xor_sync(0xffffffffu, total, o);
  }
  sfx += higher;
  const uint32_t need = need_fn(total);
  if (need > 0) {
    uint32_t above = sfx - local;
#pragma unroll
    for (int j = PER - 1; j >= 0; --j) {
      if (above < need && above + r[j] >= need) {
        s.bin = uint32_t(PER * tid + j);
        s.need = need - above;
      }
      above += r[j];
    }
  }
  __syncthreads();
  return total;
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS, kMaxThreads / THREADS) topk_cluster_kernel(const uint16_t* __restrict__ scores,
                                                                                      int32_t* __restrict__ idx,
                                                                                      const __grid_constant__ Batch B) {
  constexpr int kThreads = THREADS, PER = kBins / THREADS;  // PER consecutive histogram bins per thread
  extern __shared__ __align__(16) uint16_t s_keys[];  // keys [slice_max + 16], then group maxima [(slice_max + 16) / 8 + 8]
  __shared__ Shared s;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = int(cluster.block_rank()), csize = int(cluster.num_blocks());
  // blockIdx.y is a row of the launch; the groups' rows follow one another (row0 ascending)
  int gi = 0;
  while (gi + 1 < B.ngroups && B.g[gi + 1].row0 <= int(blockIdx.y)) ++gi;
  const int n = B.g[gi].n, k = B.g[gi].k, row = int(blockIdx.y) - B.g[gi].row0;
  const uint16_t* rp = scores + B.g[gi].off + (long long)row * B.g[gi].ld;
  const int slice = ((n + csize - 1) / csize + 7) & ~7;
  const int lo = min(n, rank * slice), cnt = min(n, lo + slice) - lo;
  // Position p of the cache holds element lo + p - mis, so 16-byte groups of the row are 16-byte groups of the cache.
  const int mis = int((reinterpret_cast<uintptr_t>(rp) >> 1) & 7u);
  const int padded = (mis + cnt + 7) & ~7;
  const int groups = padded >> 3;            // groups of 8 keys
  const int sgroups = (groups + 7) >> 3;     // groups of 8 group maxima = 64 keys
  const uint4* s_groups = reinterpret_cast<const uint4*>(s_keys);
  uint16_t* s_gmax = s_keys + B.slice_max + 16;
  const uint4* s_sg = reinterpret_cast<const uint4*>(s_gmax);

  // ---- 1: load, cache, the largest key of every group of 8, histogram of those maxima (top 12 bits) ----
  for (int b = tid; b < kBins; b += kThreads) s.hist0[b] = 0, s.fine[b] = 0;
  if (tid == 0) s.over = 0;
  if (tid < mis) s_keys[tid] = 0;                                   // key 0 is never valid, never selected
  if (tid < padded - (mis + cnt)) s_keys[mis + cnt + tid] = 0;
  if (tid < sgroups * 8 - groups) s_gmax[groups + tid] = 0;
  __syncthreads();
  const int head = min(cnt, (8 - mis) & 7), nvec = (cnt - head) >> 3, gbase = (mis + head) >> 3;
  {
    const uint16_t* src = rp + lo;
    if (tid < head) s_keys[mis + tid] = uint16_t(key_one(__ldg(src + tid)));
    const uint4* gv = reinterpret_cast<const uint4*>(src + head);
    uint4* sv = reinterpret_cast<uint4*>(s_keys + mis + head);
#pragma unroll 8
    for (int v = tid; v < nvec; v += kThreads) {
      uint4 q = __ldg(gv + v);
      q.x = key_pair(q.x), q.y = key_pair(q.y), q.z = key_pair(q.z), q.w = key_pair(q.w);
      sv[v] = q;
      const uint32_t gm = group_max(q);
      s_gmax[gbase + v] = uint16_t(gm);
      if (gm > kNegInfKey) atomicAdd(&s.hist0[gm >> 4], 1u);
    }
    for (int i = head + 8 * nvec + tid; i < cnt; i += kThreads) s_keys[mis + i] = uint16_t(key_one(__ldg(src + i)));
  }
  __syncthreads();
  if (tid < 2) {  // the first and the last group when the 16-byte loads did not cover them
    const int g = tid == 0 ? 0 : groups - 1;
    const bool todo = tid == 0 ? (groups > 0 && !(gbase == 0 && nvec > 0)) : (groups > 1 && gbase + nvec != groups);
    if (todo) {
      const uint32_t gm = group_max(s_groups[g]);
      s_gmax[g] = uint16_t(gm);
      if (gm > kNegInfKey) atomicAdd(&s.hist0[gm >> 4], 1u);
    }
  }
  __syncthreads();

  // This CTA's floor: with at least k valid groups here, at least k of this CTA's keys are >= the lower edge of the
  // bin that holds its k-th largest group maximum, so the row's k-th largest key is too; with fewer valid groups this
  // CTA says nothing (floor = the smallest valid key). The row's floor is the largest of the CTAs' floors: no key
  // below it can be selected.
  {
    const uint32_t valid_groups =
        reduce_and_pick<THREADS>(cluster, s, s.hist0, 0, [&](uint32_t v) { return v >= uint32_t(k) ? uint32_t(k) : 0u; });
    if (tid == 0) s.floor_pub = valid_groups >= uint32_t(k) ? (s.bin << 4) : (kNegInfKey + 1u);
    // hist0 now becomes the coarse histogram (16 keys per bin) of the keys above the exact window, see below
#pragma unroll
    for (int j = 0; j < PER; j += 4) *reinterpret_cast<uint4*>(&s.hist0[PER * tid + j]) = make_uint4(0, 0, 0, 0);
  }
  cluster.sync();  // barrier A: the floors
  uint32_t base = 0;
  for (int c = 0; c < csize; ++c) base = max(base, *cluster.map_shared_rank(&s.floor_pub, c));

  // ---- 2: the groups that hold a key >= base, as a list in index order (it takes the place of the group maxima:
  // every thread reads the maxima of its two supergroups before anyone writes). Later passes go over the list only,
  // so all lanes work. ----
  uint16_t* s_list = s_gmax;
  uint32_t listed = 0;
  {
    uint32_t mask[2] = {0, 0};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int sg = 2 * tid + u;
      if (sg < sgroups) for_each_key(s_sg[sg], [&](uint32_t gm, int j) { mask[u] |= (gm >= base ? 1u : 0u) << j; });
    }
    uint32_t pos = block_exclusive_scan(s, uint32_t(__popc(mask[0]) + __popc(mask[1])), listed);
#pragma unroll
    for (int u = 0; u < 2; ++u)
      for (uint32_t m = mask[u]; m != 0; m &= m - 1) s_list[pos++] = uint16_t((2 * tid + u) * 8 + (__ffs(int(m)) - 1));
  }
  __syncthreads();

  // ---- 3: exact counts of the keys in the window [base, base + window): one bin per key value, so equal scores are
  // the only same-address atomics. Keys above the window are counted in `over` and, 16 to a bin, in the coarse
  // histogram. The threshold lies in the window unless `over` alone reaches want; then the coarse histogram names
  // the 16 keys around the threshold and a second round looks at those (two rounds at most). ----
  uint32_t want = 0, thr = 0xffffffffu, need_ties = 0;
  int vstar = -1;  // the threshold's bin in the window; -1: every key of the window is selected
  uint32_t window = kBins;
  for (int round = 0; round < 2; ++round) {
    // A shared-memory atomic costs about the same with one active lane as with 32, so every lane first marks its
    // keys that are in the race and the warp then pops one marked key per lane and step: two or three atomic
    // instructions per 32 groups instead of eight.
    uint32_t my_over = 0;
    for (uint32_t eb = 0; eb < listed; eb += kThreads) {
      const uint32_t e = eb + tid;
      uint4 q = make_uint4(0, 0, 0, 0);
      if (e < listed) q = s_groups[s_list[e]];
      uint32_t m = mask_at_least(q, base);
      while (__any_sync(0xffffffffu, m != 0)) {
        if (m != 0) {
          const uint32_t key = key_at(q, __ffs(int(m)) - 1);
          m &= m - 1;
          const uint32_t v = key - base;
          if (v < window) {
            atomicAdd(&s.fine[v], 1u);
          } else {
            ++my_over;
            if (round == 0) atomicAdd(&s.hist0[key >> 4], 1u);
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) my_over += __shfl_xor_sync(0xffffffffu, my_over, o);
    if (lane == 0 && my_over != 0) atomicAdd(&s.over, my_over);
    cluster.sync();  // barrier B: fine, over (and the coarse histogram) of every CTA are complete
    uint32_t over_all = 0;
    for (int c = 0; c < csize; ++c) over_all += *cluster.map_shared_rank(&s.over, c);
    const uint32_t in_window = reduce_and_pick<THREADS>(cluster, s, s.fine, csize, [&](uint32_t v) {
      const uint32_t w = round == 0 ? min(uint32_t(k), v + over_all) : want;
      return w > over_all ? w - over_all : 0u;
    });
    if (round == 0) want = min(uint32_t(k), in_window + over_all);  // the same in every CTA of the cluster
    if (want == 0) break;
    if (want > over_all) {
      if (round == 0 && in_window + over_all <= uint32_t(k)) {
        thr = base - 1u;  // fewer keys in the race than k: all of them are selected, none is a tie
      } else {
        vstar = int(s.bin);
        thr = base + s.bin;
        need_ties = s.need;
      }
      break;
    }
    // The threshold is above the window (first window only: the second window holds it by construction).
    reduce_and_pick<THREADS>(cluster, s, s.hist0, csize, [&](uint32_t) { return want; });
    const uint32_t coarse_bin = s.bin;
    cluster.sync();  // everyone has read this CTA's fine, over and coarse histogram
    base = coarse_bin << 4;
    window = 16;
#pragma unroll
    for (int j = 0; j < PER; j += 4) *reinterpret_cast<uint4*>(&s.fine[PER * tid + j]) = make_uint4(0, 0, 0, 0);
    if (tid == 0) s.over = 0;
    __syncthreads();
  }
  {
    // This CTA's selected keys above the threshold and its ties, published for the others.
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (PER * tid + j > vstar && uint32_t(PER * tid + j) < window) mine += s.fine[PER * tid + j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) s.wsum2[warp] = mine;
    __syncthreads();
    if (warp == 0) {
      uint32_t t = lane < THREADS / 32 ? s.wsum2[lane] : 0u;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) {
        s.pub_above = want > 0 ? t + s.over : 0u;
        s.pub_ties = (want > 0 && vstar >= 0) ? s.fine[vstar] : 0u;
      }
    }
  }
  cluster.sync();  // barrier C: every CTA's counts
  uint32_t base_above = 0, ties_before = 0;
  for (int c = 0; c < rank; ++c) {
    base_above += *cluster.map_shared_rank(&s.pub_above, c);
    ties_before += *cluster.map_shared_rank(&s.pub_ties, c);
  }
  const uint32_t total_above = want - need_ties;

  // ---- 4: place this CTA's selected keys, in index order, into CTA 0's candidate list ----
  int log_size = 7;
  while ((1 << log_size) < k) ++log_size;
  if (rank == 0)
    for (int i = int(want) + tid; i < (1 << log_size); i += kThreads) s.hist0[i] = 0;  // padding sorts last
  if (want > 0) {
    uint32_t* cand_key = cluster.map_shared_rank(s.hist0, 0);
    int32_t* cand_idx = reinterpret_cast<int32_t*>(cluster.map_shared_rank(s.fine, 0));
    // The listed groups are in index order and every thread takes a contiguous run of them: one exclusive scan over
    // the threads' counts (keys above the threshold in the low word, ties in the high word) gives every thread the
    // places of its keys.
    const uint32_t per = (listed + kThreads - 1) / kThreads;
    const uint32_t e0 = min(listed, uint32_t(tid) * per), e1 = min(listed, e0 + per);
    unsigned long long c = 0;
    for (uint32_t e = e0; e < e1; ++e) {
      const uint32_t cs = count_selected(s_groups[s_list[e]], thr);
      c += (cs & 0xffffu) | (static_cast<unsigned long long>(cs >> 16) << 32);
    }
    const unsigned long long exc = block_exclusive_scan(s, c);
    uint32_t a = base_above + uint32_t(exc), t = ties_before + uint32_t(exc >> 32);
    // The same popping for the stores: a lane's selected keys leave in slot order, so index order is kept.
    if (__any_sync(0xffffffffu, c != 0))
      for (uint32_t i = 0; i < per; ++i) {
        const uint32_t e = e0 + i;
        uint4 q = make_uint4(0, 0, 0, 0);
        int g = 0;
        if (e < e1) {
          g = s_list[e];
          q = s_groups[g];
        }
        uint32_t m = mask_at_least(q, thr);
        const int i0 = lo + g * 8 - mis;
        while (__any_sync(0xffffffffu, m != 0)) {
          if (m != 0) {
            const int j = __ffs(int(m)) - 1;
            m &= m - 1;
            const uint32_t key = key_at(q, j);
            if (key > thr) {
              cand_key[a] = (key << 16) | (0xffffu - a);
              cand_idx[a] = i0 + j;
              ++a;
            } else {
              if (t < need_ties) {
                const uint32_t o = total_above + t;
                cand_key[o] = (key << 16) | (0xffffu - o);
                cand_idx[o] = i0 + j;
              }
              ++t;
            }
          }
        }
      }
  }
  cluster.sync();  // barrier D: the candidate list in CTA 0 is complete; no remote access after this point
  if (rank != 0) return;

  // ---- sort in CTA 0: 2^log_size words (128..2048), four per thread, descending ----
  int32_t* out = idx + B.g[gi].idx_off + (long long)row * k;
  switch (log_size) {
    case 7: sort_and_write<7>(s, tid, k, want, out); break;
    case 8: sort_and_write<8>(s, tid, k, want, out); break;
    case 9: sort_and_write<9>(s, tid, k, want, out); break;
    case 10: sort_and_write<10>(s, tid, k, want, out); break;
    default: sort_and_write<11>(s, tid, k, want, out); break;
  }
}


}  // namespace pkv_topkc

// Library-internal entry points (declared in pkv_internal.hpp).

// Whether the one-launch path takes this shape.
bool pkv_topk_cluster_eligible(int T, int n, int k) {
  using namespace pkv_topkc;
  return T > 0 && T <= 65535 && n > 0 && k > 0 && k <= kMaxK && n <= kMaxCluster * kMaxSlice;
}

// Keys [slice + 16] and group maxima [(slice + 16) / 8 + 8], 16 bits each.
static size_t smem_bytes(int slice) { return size_t(slice + 16) * 2 + size_t((slice + 16) / 8 + 8) * 2; }

// CTAs per row: the fewest whose slices fit in shared memory, then doubled while the launch stays within about one
// CTA per SM and a slice keeps at least 4096 keys.
static int cluster_size_for(int rows, int n_max, int sms) {
  using namespace pkv_topkc;
  int c = 1;
  while (c < kMaxCluster && (n_max + c - 1) / c > kMaxSlice) c *= 2;
  while (c < kMaxCluster && (long long)rows * c * 2 <= sms + sms / 8 && n_max / (c * 2) >= 4096) c *= 2;
  return c;
}

// Launches the cluster kernel for up to 32 blocks of rows per launch (more blocks: more launches); returns PKV_OK, or
// PKV_ERR_CUDA with `err` set. `usable` (per device, found on the first call) is false when the device cannot
// co-schedule the largest cluster: the caller then takes the four-launch path. Every block must be eligible.
int pkv_topk_cluster_launch(const uint16_t* scores, const pkv_topk_cluster_group* groups, int ngroups, int32_t* idx,
                            cudaStream_t stream, bool* usable, std::string& err) {
  using namespace pkv_topkc;
  constexpr int kMaxDevices = 64;
  static thread_local signed char state[kMaxDevices];  // 0 unknown, 1 usable, -1 not
  static thread_local int sm_count[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *usable = false;
    return PKV_OK;
  }
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kMaxCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t c;
  std::memset(&c, 0, sizeof(c));
  c.blockDim = dim3(kMaxThreads);
  c.stream = stream;
  c.attrs = attr;
  if (state[dev] == 0) {
    const size_t max_smem = smem_bytes(kMaxSlice);
    e = cudaFuncSetAttribute(topk_cluster_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(max_smem));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(topk_cluster_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes(k512Slice)));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(topk_cluster_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes(k256Slice)));
    int clusters = 0, sms = 0;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) {
      c.gridDim = dim3(kMaxCluster, 1);
      c.dynamicSmemBytes = max_smem;
      c.numAttrs = 1;
      e = cudaOccupancyMaxActiveClusters(&clusters, topk_cluster_kernel<1024>, &c);
    }
    if (e != cudaSuccess) cudaGetLastError();  // not sticky: clear it
    state[dev] = (e == cudaSuccess && clusters > 0 && sms > 0) ? 1 : -1;
    sm_count[dev] = sms;
  }
  *usable = state[dev] == 1;
  if (!*usable) return PKV_OK;
  for (int g0 = 0; g0 < ngroups; g0 += kMaxGroups) {
    Batch B;
    B.ngroups = 0;
    int rows = 0, n_max = 1;
    for (int g = g0; g < ngroups && g < g0 + kMaxGroups; ++g) {
      if (groups[g].rows <= 0) continue;
      B.g[B.ngroups] = groups[g];
      B.g[B.ngroups].row0 = rows;
      rows += groups[g].rows;
      n_max = std::max(n_max, groups[g].n);
      ++B.ngroups;
    }
    if (rows == 0) continue;
    const int csize = cluster_size_for(rows, n_max, sm_count[dev]);
    B.slice_max = ((n_max + csize - 1) / csize + 7) & ~7;
    attr[0].val.clusterDim.x = unsigned(csize);
    c.gridDim = dim3(unsigned(csize), unsigned(rows));
    c.dynamicSmemBytes = smem_bytes(B.slice_max);
    c.numAttrs = 2;
    // One CTA of 1024 threads per SM when the launch fits the SMs anyway (a decode batch at long context); with more
    // rows than that, smaller CTAs so that two or four rows share an SM and fill each other's barrier and latency gaps.
    int k_max = 1;
    for (int g = 0; g < B.ngroups; ++g) k_max = std::max(k_max, B.g[g].k);
    const bool one_wave = (long long)rows * csize <= sm_count[dev] + sm_count[dev] / 8;
    if (!one_wave && B.slice_max <= k256Slice && k_max <= 1024) {
      c.blockDim = dim3(256);
      e = cudaLaunchKernelEx(&c, topk_cluster_kernel<256>, scores, idx, B);
    } else if (!one_wave && B.slice_max <= k512Slice) {
      c.blockDim = dim3(512);
      e = cudaLaunchKernelEx(&c, topk_cluster_kernel<512>, scores, idx, B);
    } else {
      c.blockDim = dim3(1024);
      e = cudaLaunchKernelEx(&c, topk_cluster_kernel<1024>, scores, idx, B);
    }
    if (e != cudaSuccess) {
      err = std::string("top-k cluster launch: ") + cudaGetErrorString(e);
      return PKV_ERR_CUDA;
    }
  }
  return PKV_OK;
}
