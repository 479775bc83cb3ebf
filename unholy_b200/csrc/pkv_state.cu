// Slot-state snapshots: the other half of a prefix-cache hit. Block tables only cover the paged pools; the per-slot
// state that is not paged (attention windows, compressor and indexer rings) is saved into a snapshot when a prefix is
// registered and restored into the slot of a request that matches it.
//
// ewtodd/unholy's ResidentModel::state_copies (src/engine/resident.hip:545-557) walks the ops and the model's segment
// list (SnapSeg, src/engine/resident.hpp:180-183: buffer, bytes per slot, offset in the snapshot) and issues one
// copy_kernel per (op, segment): hundreds of launches per saved prefix. Here all (op, segment) pairs of a call are
// copied by one launch (per 256 segments x 32 ops): grid (24 KB pieces of all segments, 1, op), six 16-byte vectors in
// flight per thread, streaming loads and stores. The snapshot memory is whatever the caller maps for the device:
// pinned host memory as in the reference (resident.hip:538-541; the copy then runs at PCIe speed), or HBM — a B200 has
// room to keep snapshots on the card, where the same kernel runs at HBM speed.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>

#include "../../include/unholy_pkv.h"

#include "pkv_internal.hpp"

namespace pkv_state {

constexpr int kSegsPerLaunch = 256, kOpsPerLaunch = 32;  // 7.5 KB of kernel parameters
constexpr unsigned kPieceVecs = 1536;  // 24 KB

struct Params {
  uint8_t* snap;
  size_t snap_bytes;
  int save;
  int nsegs;
  pkv_state_op ops[kOpsPerLaunch];
  pkv_state_seg segs[kSegsPerLaunch];
  unsigned first_piece[kSegsPerLaunch + 1];  // segment i owns the launch's pieces first_piece[i] .. first_piece[i + 1] - 1
};

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(uint4* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// grid (pieces of all segments of the launch, 1, op): a CTA finds its segment by bisection over first_piece, then moves
// one piece of 24 KB (a segment that is not a multiple of 16 bytes, or not 16-byte aligned, goes byte by byte).
__global__ void __launch_bounds__(256) state_copies_kernel(const __grid_constant__ Params P) {
  int lo_s = 0, hi_s = P.nsegs;  // first_piece[lo_s] <= blockIdx.x < first_piece[hi_s]
  while (hi_s - lo_s > 1) {
    const int mid = (lo_s + hi_s) >> 1;
    if (P.first_piece[mid] <= blockIdx.x) lo_s = mid;
    else hi_s = mid;
  }
  const pkv_state_seg sg = P.segs[lo_s];
  const pkv_state_op op = P.ops[blockIdx.z];
  const size_t piece = blockIdx.x - P.first_piece[lo_s];
  uint8_t* slot = static_cast<uint8_t*>(sg.dev) + size_t(op.slot) * sg.bytes;
  uint8_t* snap = P.snap + size_t(op.snapshot) * P.snap_bytes + sg.off;
  const uint8_t* src = P.save ? slot : snap;
  uint8_t* dst = P.save ? snap : slot;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | sg.bytes) & 15u) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const size_t vecs = sg.bytes / 16, lo = piece * kPieceVecs, hi = min(vecs, lo + kPieceVecs);
    uint4 v[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      const size_t u = lo + size_t(i) * 256u + threadIdx.x;
      if (u < hi) v[i] = ld_stream(s4 + u);
    }
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      const size_t u = lo + size_t(i) * 256u + threadIdx.x;
      if (u < hi) st_stream(d4 + u, v[i]);
    }
  } else {
    const size_t lo = piece * kPieceVecs * 16, hi = min(sg.bytes, lo + size_t(kPieceVecs) * 16);
    for (size_t i = lo + threadIdx.x; i < hi; i += 256u) dst[i] = src[i];
  }
  __threadfence_system();  // snapshots in host memory: visible to the host when the stream reaches this point
}

}  // namespace pkv_state

extern "C" {

int pkv_state_copies(const pkv_state_seg* segs, int nsegs, const pkv_state_op* ops, int nops, void* snap_base,
                     size_t snap_bytes, int num_snapshots, int max_slots, int save, pkv_stream_t stream) {
  using namespace pkv_state;
  if (nops <= 0 || nsegs <= 0) return PKV_OK;
  if (!segs || !ops || !snap_base) {
    pkv_g_err = "pkv_state_copies: null pointer";
    return PKV_ERR_ARG;
  }
  size_t end = 0;
  for (int i = 0; i < nsegs; ++i) {
    if (!segs[i].dev) {
      pkv_g_err = "pkv_state_copies: null segment";
      return PKV_ERR_ARG;
    }
    end = std::max(end, segs[i].off + segs[i].bytes);
  }
  if (end > snap_bytes) {
    pkv_g_err = "pkv_state_copies: a segment ends past the snapshot size";
    return PKV_ERR_ARG;
  }
  for (int i = 0; i < nops; ++i)
    if (ops[i].snapshot < 0 || ops[i].snapshot >= num_snapshots || ops[i].slot < 0 || ops[i].slot >= max_slots) {
      pkv_g_err = "step: bad state op";  // the reference's message (resident.hip:549)
      return PKV_ERR_ARG;
    }
  Params P;
  P.snap = static_cast<uint8_t*>(snap_base);
  P.snap_bytes = snap_bytes;
  P.save = save ? 1 : 0;
  constexpr size_t kPieceBytes = size_t(kPieceVecs) * 16;
  for (int o0 = 0; o0 < nops; o0 += kOpsPerLaunch) {
    const int no = std::min(kOpsPerLaunch, nops - o0);
    std::memcpy(P.ops, ops + o0, size_t(no) * sizeof(pkv_state_op));
    for (int s0 = 0; s0 < nsegs; s0 += kSegsPerLaunch) {
      const int ns = std::min(kSegsPerLaunch, nsegs - s0);
      std::memcpy(P.segs, segs + s0, size_t(ns) * sizeof(pkv_state_seg));
      P.nsegs = ns;
      size_t pieces = 0;
      for (int i = 0; i < ns; ++i) {
        P.first_piece[i] = unsigned(pieces);
        pieces += (segs[s0 + i].bytes + kPieceBytes - 1) / kPieceBytes;
      }
      P.first_piece[ns] = unsigned(pieces);
      if (pieces == 0) continue;
      if (pieces > 0x7fffffffu) {
        pkv_g_err = "pkv_state_copies: segments too large for one launch";
        return PKV_ERR_LIMIT;
      }
      state_copies_kernel<<<dim3(unsigned(pieces), 1, unsigned(no)), 256, 0, static_cast<cudaStream_t>(stream)>>>(P);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) {
        pkv_g_err = std::string("pkv_state_copies: ") + cudaGetErrorString(e);
        return PKV_ERR_CUDA;
      }
    }
  }
  return PKV_OK;
}

}  // extern "C"
