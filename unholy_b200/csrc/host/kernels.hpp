// C++ face of the paged KV-cache kernels with the reference's names, argument order and error behaviour, so that the
// reference's call sites (src/model/forward_ref.hip:719-745,843-857; src/model/glm5_fast.hip:229-250) compile against
// it unchanged apart from hipStream_t -> cudaStream_t. Every function forwards to the C ABI (include/unholy_pkv.h) and
// turns a non-zero status into std::runtime_error, the reference's convention (src/rt/hip.hpp:11-19). Launches are
// asynchronous on `st`; nullptr is the default stream. Header-only; link with libunholy_pkv.so.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../../include/unholy_pkv.h"

namespace unholy::kernels {

using bf16 = uint16_t;

inline void pkv_throw(int rc, const char* what) {
  if (rc != PKV_OK) throw std::runtime_error(std::string(what) + ": " + pkv_last_error());
}

// src/kernels/ref.hpp:92-99.
struct PagedRows {
  bf16* pool = nullptr;
  const int32_t* table = nullptr;
  int rows_per_page = 0;
  int row_stride = 0;
};
// src/kernels/ref.hpp:100.
inline void store_rows(const bf16* rows, int n, int width, PagedRows dst, int row0, cudaStream_t st) {
  pkv_throw(pkv_store_rows(rows, n, width, dst.pool, dst.table, dst.rows_per_page, dst.row_stride, row0,
                           reinterpret_cast<pkv_stream_t>(st)), "store_rows");
}

// src/kernels/indexer.hpp:20-34.
constexpr int kFp4RowsPerPage = 64;
constexpr int kFp4RowBytes = 64;
constexpr int kFp4PageBytes = kFp4RowsPerPage * (kFp4RowBytes + 4);
struct PagedFp4 {
  uint8_t* pool = nullptr;
  const int32_t* table = nullptr;
};
inline void store_rows_fp4(const bf16* rows, int n, PagedFp4 dst, int row0, cudaStream_t st) {
  pkv_throw(pkv_store_rows_fp4(rows, n, dst.pool, dst.table, kFp4RowsPerPage, row0, reinterpret_cast<pkv_stream_t>(st)),
            "store_rows_fp4");
}
inline void load_rows_fp4(PagedFp4 src, int row0, int n, bf16* out, cudaStream_t st) {
  pkv_throw(pkv_load_rows_fp4(src.pool, src.table, kFp4RowsPerPage, row0, n, out, reinterpret_cast<pkv_stream_t>(st)),
            "load_rows_fp4");
}

// src/kernels/ref.hpp:22-25.
inline void act_quant_fp8(const bf16* x, int ldx, uint8_t* q, uint8_t* s, int rows, int cols, int block, cudaStream_t st) {
  pkv_throw(pkv_act_quant_fp8(x, ldx, q, s, rows, cols, block, reinterpret_cast<pkv_stream_t>(st)), "act_quant_fp8");
}
inline void fake_quant_fp8(bf16* x, int ldx, int rows, int cols, int block, cudaStream_t st) {
  pkv_throw(pkv_fake_quant_fp8(x, ldx, rows, cols, block, reinterpret_cast<pkv_stream_t>(st)), "fake_quant_fp8");
}
inline void fake_quant_fp4(bf16* x, int ldx, int rows, int cols, int block, cudaStream_t st) {
  pkv_throw(pkv_fake_quant_fp4(x, ldx, rows, cols, block, reinterpret_cast<pkv_stream_t>(st)), "fake_quant_fp4");
}

// src/kernels/glm_fast.hpp:21-32 (the pooled-key array of the reference's struct belongs to a kernel outside this path).
constexpr int kGlmPageRows = 256;
struct GlmPaged {
  uint8_t* lat = nullptr;    // e4m3 [pages][256][512]
  uint8_t* lat_s = nullptr;  // e8m0 [pages][256][8]
  bf16* pk = nullptr;        // kept for layout compatibility; not touched here
  const int32_t* table = nullptr;
};
inline void glm_store_latent(const bf16* lat, GlmPaged pg, int s0, int n, cudaStream_t st) {
  pkv_throw(pkv_store_rows_fp8(lat, n, 512, 64, pg.lat, pg.lat_s, pg.table, kGlmPageRows, s0,
                               reinterpret_cast<pkv_stream_t>(st)), "glm_store_latent");
}

// The gather of the reference's GLM attention over fp8 latent rows (src/kernels/glm_fast.hip:190-227) as a call of its
// own: idx [T][k] positions of the slot behind `pg`, dequantised to bf16 [T][k][512].
inline void glm_gather_latent(GlmPaged pg, const int32_t* idx, const int32_t* visible, int T, int k, bf16* out, cudaStream_t st) {
  pkv_throw(pkv_gather_rows_fp8(pg.lat, pg.lat_s, pg.table, kGlmPageRows, 512, 64, idx, visible, T, k, out,
                                reinterpret_cast<pkv_stream_t>(st)), "glm_gather_latent");
}

// src/kernels/ref.hpp:90.
inline void copy_kernel(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  pkv_throw(pkv_copy(dst, src, bytes, reinterpret_cast<pkv_stream_t>(st)), "copy_kernel");
}

// The gather the reference carries inside its attention kernels (src/kernels/attn_wmma.hip:75-113), as a call of its
// own: idx [T][k] entries of the sequence behind `src`, masked entries (< 0 or >= visible[t]) give zero rows.
inline void gather_rows(PagedRows src, int width, const int32_t* idx, const int32_t* visible, int T, int k, bf16* out,
                        cudaStream_t st) {
  pkv_throw(pkv_gather_rows(src.pool, src.table, src.rows_per_page, src.row_stride, width, idx, visible, T, k, out,
                            reinterpret_cast<pkv_stream_t>(st)), "gather_rows");
}

// src/kernels/indexer.hpp:74-94: the reference's declarations, argument for argument.
inline void topk_bf16(const uint16_t* scores, int T, int n, int k, int32_t* idx, cudaStream_t st) {
  pkv_throw(pkv_topk_bf16(scores, T, n, n, k, idx, nullptr, 0, reinterpret_cast<pkv_stream_t>(st)), "topk_bf16");
}
struct TopkRows {
  size_t off;
  int rows, n, k, idx_off;
};
static_assert(sizeof(TopkRows) == sizeof(pkv_topk_group), "TopkRows is passed to the C ABI as pkv_topk_group");
struct TopkBatch {
  static constexpr int kMax = 32;
  int ngroups = 0;
  TopkRows g[kMax];
};
constexpr int kTopkSplitMinKeys = 8192, kTopkSplitMaxRows = 64;
// The reference sizes the scratch of its several-workgroups-per-row path with this. Here the CTAs of a row exchange
// through distributed shared memory, so that path needs no scratch: 0. (Shapes outside it, k > 2048 or rows longer
// than 655,360 keys, use the caller's scratch when it holds topk_scratch_words(rows, n, k) words and the library's
// built-in array otherwise.)
inline size_t topk_split_scratch_words(int /*rows*/) { return 0; }
inline size_t topk_scratch_words(int rows, int n, int k) { return pkv_topk_scratch_words(rows, n, k); }
inline void topk_bf16_batch(const uint16_t* scores, const TopkBatch& b, int32_t* idx, cudaStream_t st, uint32_t* scratch = nullptr,
                            size_t scratch_words = 0) {
  pkv_throw(pkv_topk_bf16_batch(scores, reinterpret_cast<const pkv_topk_group*>(b.g), b.ngroups, idx, scratch, scratch_words,
                                reinterpret_cast<pkv_stream_t>(st)), "topk_bf16_batch");
}
// src/kernels/ref.hpp:107 (k > 1024 throws, as ref_attn.hip:391 does) and src/kernels/glm_fast.hpp:86-93: the same
// selection; glm_topk keeps its cand argument (unused: one CTA per row selects in shared memory) and its size query.
inline void topk_rows(const float* scores, int T, int n, int k, int32_t* idx, cudaStream_t st) {
  pkv_throw(pkv_topk_f32(scores, T, n, n, k, idx, reinterpret_cast<pkv_stream_t>(st)), "topk_rows");
}
constexpr int kGlmTopkSeg = 4096;
inline size_t glm_topk_cand_bytes(int rows, int cols, int k) {
  return size_t(rows) * size_t((cols + kGlmTopkSeg - 1) / kGlmTopkSeg) * size_t(k) * 8;
}
inline void glm_topk(const float* scores, int ld, int n, int cols, int k, int32_t* idx, void* /*cand*/, cudaStream_t st) {
  pkv_throw(pkv_topk_f32(scores, n, cols, ld, k, idx, reinterpret_cast<pkv_stream_t>(st)), "glm_topk");
}
inline void glm_idx_expand(const int32_t* pools, const int32_t* pos, int32_t* idx, int n, int k, int pool, cudaStream_t st) {
  pkv_throw(pkv_idx_expand(pools, pos, idx, n, k, pool, reinterpret_cast<pkv_stream_t>(st)), "glm_idx_expand");
}
// fake_quant_fp8(rows, width, n, quant_cols, block) followed by store_rows(rows, n, width, dst, row0) (ref.hpp:24,100;
// the pair of src/model/forward_ref.hip:739-741) in one pass; rows is not modified.
inline void store_rows_fake_fp8(const bf16* rows, int n, int width, int quant_cols, int block, PagedRows dst, int row0,
                                cudaStream_t st) {
  pkv_throw(pkv_store_rows_fake_fp8(rows, n, width, quant_cols, block, dst.pool, dst.table, dst.rows_per_page, dst.row_stride,
                                    row0, reinterpret_cast<pkv_stream_t>(st)), "store_rows_fake_fp8");
}
// src/kernels/elem_fast.hpp:29: kv_chain in place, and the same chain fused with the append that follows it in
// compress_chunk (kv_chain, then store_rows of the same rows: one pass, the rows are read once).
inline void kv_chain(bf16* kv, const bf16* w, int rows, int dim, float eps, const int32_t* pos, const float2* freqs, int npair,
                     cudaStream_t st) {
  pkv_throw(pkv_store_rows_kv_chain(kv, kv, w, rows, dim, eps, pos, reinterpret_cast<const float*>(freqs), npair, 1, nullptr, nullptr,
                                    0, 0, 0, reinterpret_cast<pkv_stream_t>(st)), "kv_chain");
}
inline void store_rows_kv_chain(const bf16* kv, bf16* kv_out, const bf16* w, int rows, int dim, float eps, const int32_t* pos,
                                const float2* freqs, int npair, PagedRows dst, int row0, cudaStream_t st) {
  pkv_throw(pkv_store_rows_kv_chain(kv, kv_out, w, rows, dim, eps, pos, reinterpret_cast<const float*>(freqs), npair, 1, dst.pool,
                                    dst.table, dst.rows_per_page, dst.row_stride, row0, reinterpret_cast<pkv_stream_t>(st)),
            "store_rows_kv_chain");
}
// src/kernels/ref.hpp:63.
inline void hadamard128(bf16* x, size_t nseg, cudaStream_t st) {
  pkv_throw(pkv_hadamard128(x, nseg, reinterpret_cast<pkv_stream_t>(st)), "hadamard128");
}
// ResidentModel::state_copies (src/engine/resident.hip:545-557): SnapSeg and StateOp keep their field names.
using SnapSeg = pkv_state_seg;
using StateOp = pkv_state_op;
inline void state_copies(const SnapSeg* segs, int nsegs, const StateOp* ops, int nops, void* snap_base, size_t snap_bytes,
                         int num_snapshots, int max_slots, bool save, cudaStream_t st) {
  pkv_throw(pkv_state_copies(segs, nsegs, ops, nops, snap_base, snap_bytes, num_snapshots, max_slots, save ? 1 : 0,
                             reinterpret_cast<pkv_stream_t>(st)), "state_copies");
}
inline int glm_sel_count(int p, int k, int pool) {
  const int full = (p + 1) / pool;
  return (full < k ? full : k) * pool + (p + 1) % pool;
}

}  // namespace unholy::kernels
