// CPU oracle for the paged KV-cache path. TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared
// with and the timed CPU baseline of the benchmark. Nothing in the product library links, loads or calls this file.
//
// Every function restates, in plain scalar C++, the arithmetic of one piece of the reference (ewtodd/unholy); the
// comment above each names the reference file:line it follows. Pinning: tests/test_oracle_pins.py checks these
// functions against the reference's own scalar helpers compiled in place (oracle/_ref/libref_numeric.so, built from
// src/kernels/dev.hip.hpp by oracle/build_oracle.py) and against the golden vectors under tests/golden/ produced
// from the reference's pure-torch quantisers (tools/ref/oracle/kernel.py). Page duplication, compaction and
// migration have no counterpart in the reference: for those three the rule is stated here and parity is unpinned.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

inline uint32_t f2u(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float u2f(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// src/kernels/dev.hip.hpp:40 — a bf16 is the top half of an fp32.
inline float bf16_to_f32(uint16_t v) { return u2f(uint32_t(v) << 16); }

// src/kernels/dev.hip.hpp:43-48 — round to nearest even; a NaN keeps its top bits and gets the quiet bit.
inline uint16_t f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40u);
  const uint32_t lsb = (u >> 16) & 1u;
  return uint16_t((u + 0x7fffu + lsb) >> 16);
}

// src/kernels/dev.hip.hpp:59-63 — OCP e4m3fn decode: subnormals are m * 2^-9, normals rebias 7 -> 127.
inline float e4m3_to_f32(uint8_t c) {
  const uint32_t ex = (c >> 3) & 15u, man = c & 7u;
  const float mag = ex == 0 ? float(man) * (1.0f / 512.0f) : u2f(((ex + 120u) << 23) | (man << 20));
  return (c & 0x80u) ? -mag : mag;
}

// src/kernels/dev.hip.hpp:82-94 — RNE encode for |x| <= 448. Below 2^-6 the code is rint(|x| * 512) (which may
// round up into the smallest normal, code 8); otherwise RNE at the 3 kept mantissa bits and rebias.
inline uint8_t f32_to_e4m3(float x) {
  uint32_t u = f2u(x);
  const uint8_t sign = uint8_t((u >> 24) & 0x80u);
  u &= 0x7fffffffu;
  const int ex = int(u >> 23) - 127;
  if (ex < -6) return uint8_t(sign | uint8_t(std::nearbyintf(u2f(u) * 512.0f)));
  u += 0x7ffffu + ((u >> 20) & 1u);
  const uint32_t e2 = (u >> 23) - 127u + 7u, m2 = (u >> 20) & 7u;
  return uint8_t(sign | uint8_t((e2 << 3) | m2));
}

// src/kernels/dev.hip.hpp:96 — an e8m0 byte is an fp32 exponent field.
inline float e8m0_to_f32(uint8_t e) { return u2f(uint32_t(e) << 23); }

// src/kernels/dev.hip.hpp:99-104 — e2m1 grid 0, .5, 1, 1.5, 2, 3, 4, 6 with bit 3 the sign.
inline float e2m1_to_f32(uint32_t nib) {
  static const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const float mag = grid[nib & 7u];
  return (nib & 8u) ? -mag : mag;
}

// src/kernels/dev.hip.hpp:107-119 — nearest grid point, ties to the even code; sign applied with `x < 0`, so a
// small negative becomes -0.0 while an input of -0.0 stays +0.0.
inline float round_e2m1(float x) {
  const float a = std::fabs(x);
  float r = 6.0f;
  if (a <= 0.25f) r = 0.0f;
  else if (a < 0.75f) r = 0.5f;
  else if (a <= 1.25f) r = 1.0f;
  else if (a < 1.75f) r = 1.5f;
  else if (a <= 2.5f) r = 2.0f;
  else if (a < 3.5f) r = 3.0f;
  else if (a <= 5.0f) r = 4.0f;
  return x < 0 ? -r : r;
}

// src/kernels/dev.hip.hpp:123-127 — exponent of the next power of two >= v, as a biased byte.
inline uint8_t pow2_ceil_e8m0(float v) {
  const uint32_t b = f2u(v);
  const int ex = int((b >> 23) & 0xffu) - 127 + ((b & 0x7fffffu) ? 1 : 0);
  return uint8_t(ex + 127);
}

// src/kernels/indexer.hip:20-24 — nibble of a value already on the grid; the sign comes from signbit, so -0.0 -> 8.
inline uint32_t e2m1_code(float r) {
  const float a = std::fabs(r);
  const uint32_t m = a < 2.0f ? uint32_t(a * 2.0f) : (a == 6.0f ? 7u : uint32_t(a) + 2u);
  return m | (std::signbit(r) ? 8u : 0u);
}

// src/kernels/indexer.hip:36-41 and src/kernels/ref_elem.hip:43-59 — one 32-value block: absmax floored at
// 6 * 2^-126, power-of-two scale of amax / 6, x / scale clamped to [-6, 6], rounded onto the grid.
inline uint8_t fp4_block_scale(const uint16_t* x, int count) {
  float amax = 0.0f;
  for (int i = 0; i < count; ++i) amax = std::fmax(amax, std::fabs(bf16_to_f32(x[i])));
  amax = std::fmax(amax, 6.0f * 1.1754943508222875e-38f);
  return pow2_ceil_e8m0(amax * (1.0f / 6.0f));
}
inline float fp4_round(uint16_t x, float sc) {
  return round_e2m1(std::fmin(std::fmax(bf16_to_f32(x) / sc, -6.0f), 6.0f));
}

// src/kernels/ref_elem.hip:18-41 and src/kernels/glm_fast.hip:37-51 — one block: absmax floored at 1e-4,
// power-of-two scale of amax / 448, x / scale clamped to [-448, 448], encoded e4m3.
inline uint8_t fp8_block_scale(const uint16_t* x, int count) {
  float amax = 0.0f;
  for (int i = 0; i < count; ++i) amax = std::fmax(amax, std::fabs(bf16_to_f32(x[i])));
  amax = std::fmax(amax, 1e-4f);
  return pow2_ceil_e8m0(amax * (1.0f / 448.0f));
}
inline uint8_t fp8_code(uint16_t x, float sc) {
  return f32_to_e4m3(std::fmin(std::fmax(bf16_to_f32(x) / sc, -448.0f), 448.0f));
}

// src/kernels/ref_attn.hip:15-18 (also attn_wmma.hip:29-32, glm_fast.hip:29-31) — physical row of logical row r.
inline size_t phys_row(const int32_t* table, int rows_per_page, int r) {
  return size_t(table[r / rows_per_page]) * size_t(rows_per_page) + size_t(r % rows_per_page);
}

template <class F>
void parallel_for(int n, int threads, F&& body) {
  if (threads <= 1 || n <= 1) {
    for (int i = 0; i < n; ++i) body(i);
    return;
  }
  threads = std::min(threads, n);
  std::vector<std::thread> pool;
  pool.reserve(size_t(threads));
  for (int w = 0; w < threads; ++w)
    pool.emplace_back([&, w] {
      for (int i = w; i < n; i += threads) body(i);
    });
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

// ---- scalar helpers, exported so the pin tests can sweep them against the reference's own ----
float orc_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }
uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_e4m3_to_f32(uint8_t c) { return e4m3_to_f32(c); }
uint8_t orc_f32_to_e4m3(float x) { return f32_to_e4m3(x); }
float orc_e8m0_to_f32(uint8_t e) { return e8m0_to_f32(e); }
float orc_e2m1_to_f32(uint32_t n) { return e2m1_to_f32(n); }
float orc_round_e2m1(float x) { return round_e2m1(x); }
uint8_t orc_pow2_ceil_e8m0(float v) { return pow2_ceil_e8m0(v); }
uint32_t orc_e2m1_code(float r) { return e2m1_code(r); }

// src/kernels/ref_attn.hip:88-93,377-381 (store_rows) — rows [n][width] become logical rows [row0, row0 + n) of the
// sequence whose block-table row is `table`; a pure bit copy.
void orc_store_rows(const uint16_t* rows, int n, int width, uint16_t* pool, const int32_t* table, int rows_per_page,
                    int row_stride, int row0) {
  for (int r = 0; r < n; ++r)
    std::memcpy(pool + phys_row(table, rows_per_page, row0 + r) * size_t(row_stride), rows + size_t(r) * width,
                size_t(width) * 2);
}

// src/kernels/indexer.hip:26-33,43-53,802-806 (store_rows_fp4) with the page layout of src/kernels/indexer.hpp:20-28:
// page p starts at pool + p * rows_per_page * (dim/2 + dim/32); first the code rows (dim/2 bytes each, even column in
// the low nibble), then the scale rows (dim/32 e8m0 bytes each).
void orc_store_rows_fp4(const uint16_t* rows, int n, int dim, uint8_t* pool, const int32_t* table, int rows_per_page,
                        int row0) {
  const int code_bytes = dim / 2, nblk = dim / 32;
  const size_t page_bytes = size_t(rows_per_page) * size_t(code_bytes + nblk);
  for (int r = 0; r < n; ++r) {
    const int lr = row0 + r;
    uint8_t* page = pool + size_t(table[lr / rows_per_page]) * page_bytes;
    const int slot = lr % rows_per_page;
    uint8_t* codes = page + size_t(slot) * code_bytes;
    uint8_t* scales = page + size_t(rows_per_page) * code_bytes + size_t(slot) * nblk;
    const uint16_t* x = rows + size_t(r) * dim;
    for (int b = 0; b < nblk; ++b) {
      const uint8_t se = fp4_block_scale(x + b * 32, 32);
      const float sc = e8m0_to_f32(se);
      for (int j = 0; j < 16; ++j) {
        const uint32_t lo = e2m1_code(fp4_round(x[b * 32 + 2 * j], sc));
        const uint32_t hi = e2m1_code(fp4_round(x[b * 32 + 2 * j + 1], sc));
        codes[b * 16 + j] = uint8_t(lo | (hi << 4));
      }
      scales[b] = se;
    }
  }
}

// src/kernels/indexer.hip:55-62 (load_rows_fp4) — grid value times the block's power of two, rounded to bf16 (exact).
void orc_load_rows_fp4(const uint8_t* pool, const int32_t* table, int rows_per_page, int dim, int row0, int n,
                       uint16_t* out) {
  const int code_bytes = dim / 2, nblk = dim / 32;
  const size_t page_bytes = size_t(rows_per_page) * size_t(code_bytes + nblk);
  for (int r = 0; r < n; ++r) {
    const int lr = row0 + r;
    const uint8_t* page = pool + size_t(table[lr / rows_per_page]) * page_bytes;
    const int slot = lr % rows_per_page;
    const uint8_t* codes = page + size_t(slot) * code_bytes;
    const uint8_t* scales = page + size_t(rows_per_page) * code_bytes + size_t(slot) * nblk;
    for (int c = 0; c < dim; ++c) {
      const uint8_t byte = codes[c / 2];
      const float v = e2m1_to_f32((c & 1) ? uint32_t(byte >> 4) : uint32_t(byte & 15u)) * e8m0_to_f32(scales[c / 32]);
      out[size_t(r) * dim + c] = f32_to_bf16(v);
    }
  }
}

// src/kernels/ref_elem.hip:43-59,292-296 (fake_quant_fp4) — quantise and write the bf16 value back in place.
void orc_fake_quant_fp4(uint16_t* x, int ldx, int rows, int cols, int block) {
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < cols / block; ++b) {
      uint16_t* xb = x + size_t(r) * ldx + size_t(b) * block;
      const float sc = e8m0_to_f32(fp4_block_scale(xb, block));
      for (int i = 0; i < block; ++i) xb[i] = f32_to_bf16(fp4_round(xb[i], sc) * sc);
    }
}

// src/kernels/ref_elem.hip:18-41,282-286 (act_quant_fp8) — codes [rows][cols] and one e8m0 scale per block.
void orc_act_quant_fp8(const uint16_t* x, int ldx, uint8_t* q, uint8_t* s, int rows, int cols, int block) {
  const int nb = cols / block;
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < nb; ++b) {
      const uint16_t* xb = x + size_t(r) * ldx + size_t(b) * block;
      const uint8_t se = fp8_block_scale(xb, block);
      const float sc = e8m0_to_f32(se);
      for (int i = 0; i < block; ++i) q[size_t(r) * cols + size_t(b) * block + i] = fp8_code(xb[i], sc);
      s[size_t(r) * nb + b] = se;
    }
}

// src/kernels/ref_elem.hip:18-41,287-291 (fake_quant_fp8) — the same codes decoded, rescaled and rounded to bf16.
void orc_fake_quant_fp8(uint16_t* x, int ldx, int rows, int cols, int block) {
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < cols / block; ++b) {
      uint16_t* xb = x + size_t(r) * ldx + size_t(b) * block;
      const float sc = e8m0_to_f32(fp8_block_scale(xb, block));
      for (int i = 0; i < block; ++i) xb[i] = f32_to_bf16(e4m3_to_f32(fp8_code(xb[i], sc)) * sc);
    }
}

// src/kernels/elem_dev.hip.hpp:50-87 (kv_chain_row; launcher src/kernels/elem_fast.hip:87-92,124-128): the chain a KV
// row goes through before it is appended, in place: rmsnorm with weight w (fp32: sum of squares, r = 1 / sqrt(mean +
// eps), x = bf16(w * (x * r))), rope on the last 2 * npair dims with freqs[pos][pair] = (cos, sin) on the bf16-rounded
// values, then fake_quant_fp8 (block 64) of the other dims. The reference's sum runs over 256 threads and a block
// reduction and its r is the GPU's rsqrtf: the order of the additions and the last bit of r are not fixed by the
// source, so this restatement (sequential fp32 sum, correctly rounded 1 / sqrt) pins the chain only to a tolerance:
// one bf16 step on the normalised values (a rotated value inherits the steps of its two inputs); the quantisation
// itself is exact on equal inputs (quant = 0 stops in front of it).
void orc_kv_chain(uint16_t* x, const uint16_t* w, int rows, int dim, float eps, const int32_t* pos, const float* freqs,
                  int npair, int quant) {
  const int off = dim - 2 * npair;
  for (int r = 0; r < rows; ++r) {
    uint16_t* xr = x + size_t(r) * dim;
    float ss = 0.0f;
    for (int i = 0; i < dim; ++i) {
      const float v = bf16_to_f32(xr[i]);
      ss += v * v;
    }
    const float rr = 1.0f / std::sqrt(ss / float(dim) + eps);
    for (int i = 0; i < dim; ++i) {
      const float t = bf16_to_f32(xr[i]) * rr;
      xr[i] = f32_to_bf16(bf16_to_f32(w[i]) * t);
    }
    for (int t = 0; t < npair; ++t) {
      uint16_t* e = xr + off + 2 * t;
      const float a = bf16_to_f32(e[0]), b = bf16_to_f32(e[1]);
      const float c = freqs[(size_t(pos[r]) * npair + t) * 2], sn = freqs[(size_t(pos[r]) * npair + t) * 2 + 1];
      e[0] = f32_to_bf16(a * c - b * sn);
      e[1] = f32_to_bf16(a * sn + b * c);
    }
    if (quant) orc_fake_quant_fp8(xr, dim, 1, off, 64);
  }
}

// src/kernels/glm_fast.hip:29-31,37-51,752-756 (glm_store_latent), layout src/kernels/glm_fast.hpp:23-28: codes
// [pages * rows_per_page][width] and scales [pages * rows_per_page][width / block] are two separate arrays, both
// indexed by the physical row id of position s0 + r.
void orc_store_rows_fp8(const uint16_t* rows, int n, int width, int block, uint8_t* codes, uint8_t* scales,
                        const int32_t* table, int rows_per_page, int s0) {
  const int nb = width / block;
  for (int r = 0; r < n; ++r) {
    const size_t rid = phys_row(table, rows_per_page, s0 + r);
    orc_act_quant_fp8(rows + size_t(r) * width, width, codes + rid * size_t(width), scales + rid * size_t(nb), 1, width,
                      block);
  }
}

// The sparse gather as a standalone operation. Entry semantics follow src/kernels/attn_wmma.hip:75-92 (row_of),
// src/kernels/ref_attn.hip:285-301 and src/kernels/glm_fast.hip:190-195: entry e of query t names logical row
// idx[t][e] of the query's slot; a negative entry or one >= visible[t] is masked. A masked entry reads as a row of
// zeros (src/kernels/attn_wmma.hip:107,277-291: the split path points masked entries at one shared zero row).
// Output out[t][e][0..width) is contiguous. Queries are independent; `threads` splits them over host threads.
void orc_gather_rows(const uint16_t* pool, const int32_t* tables, int max_pages_per_seq, int rows_per_page,
                     int row_stride, int width, const int32_t* idx, const int32_t* q_slot, const int32_t* q_visible,
                     int T, int k, uint16_t* out, int threads) {
  parallel_for(T, threads, [&](int t) {
    const int32_t* table = tables + size_t(q_slot[t]) * max_pages_per_seq;
    for (int e = 0; e < k; ++e) {
      const int row = idx[size_t(t) * k + e];
      uint16_t* dst = out + (size_t(t) * k + e) * size_t(width);
      if (row >= 0 && row < q_visible[t])
        std::memcpy(dst, pool + phys_row(table, rows_per_page, row) * size_t(row_stride), size_t(width) * 2);
      else
        std::memset(dst, 0, size_t(width) * 2);
    }
  });
}

// A batched append in the shape of the reference's step (src/engine/step.hpp:20-26 Chunk{slot, s0, n, t0};
// src/model/forward_ref.hip:843-857 calls store_rows once per chunk): batch rows [t0, t0 + n) of `rows` become
// logical rows [s0, s0 + n) of the chunk's slot. chunks is [nchunks][4] int32 (slot, s0, n, t0).
void orc_store_rows_chunks(const uint16_t* rows, int width, uint16_t* pool, const int32_t* tables,
                           int max_pages_per_seq, int rows_per_page, int row_stride, const int32_t* chunks, int nchunks,
                           int threads) {
  parallel_for(nchunks, threads, [&](int c) {
    const int32_t* ch = chunks + size_t(c) * 4;
    orc_store_rows(rows + size_t(ch[3]) * width, ch[2], width, pool, tables + size_t(ch[0]) * max_pages_per_seq,
                   rows_per_page, row_stride, ch[1]);
  });
}
void orc_store_rows_fp4_chunks(const uint16_t* rows, int dim, uint8_t* pool, const int32_t* tables,
                               int max_pages_per_seq, int rows_per_page, const int32_t* chunks, int nchunks,
                               int threads) {
  parallel_for(nchunks, threads, [&](int c) {
    const int32_t* ch = chunks + size_t(c) * 4;
    orc_store_rows_fp4(rows + size_t(ch[3]) * dim, ch[2], dim, pool, tables + size_t(ch[0]) * max_pages_per_seq,
                       rows_per_page, ch[1]);
  });
}
void orc_store_rows_fp8_chunks(const uint16_t* rows, int width, int block, uint8_t* codes, uint8_t* scales,
                               const int32_t* tables, int max_pages_per_seq, int rows_per_page, const int32_t* chunks,
                               int nchunks, int threads) {
  parallel_for(nchunks, threads, [&](int c) {
    const int32_t* ch = chunks + size_t(c) * 4;
    orc_store_rows_fp8(rows + size_t(ch[3]) * width, ch[2], width, block, codes, scales,
                       tables + size_t(ch[0]) * max_pages_per_seq, rows_per_page, ch[1]);
  });
}

// Whole-page copies inside one pool (no reference counterpart; the copy primitive is src/kernels/ref_elem.hip:269-278).
// Rule: page dst[i] becomes a byte-for-byte copy of page src[i]; the src and dst id sets are disjoint, so order is
// irrelevant. Serves copy-on-write duplication and hole-filling compaction.
void orc_copy_pages(uint8_t* pool, size_t page_bytes, const int32_t* src, const int32_t* dst, int n, int threads) {
  parallel_for(n, threads, [&](int i) {
    std::memcpy(pool + size_t(dst[i]) * page_bytes, pool + size_t(src[i]) * page_bytes, page_bytes);
  });
}
// The same between two pools (migration between shards: source pool on one device, destination on another).
void orc_move_pages(const uint8_t* src_pool, uint8_t* dst_pool, size_t page_bytes, const int32_t* src,
                    const int32_t* dst, int n, int threads) {
  parallel_for(n, threads, [&](int i) {
    std::memcpy(dst_pool + size_t(dst[i]) * page_bytes, src_pool + size_t(src[i]) * page_bytes, page_bytes);
  });
}

// src/kernels/ref_elem.hip:269-278,358-366 (copy_kernel) — a byte copy.
void orc_copy(void* dst, const void* src, size_t bytes) { std::memcpy(dst, src, bytes); }

// src/kernels/indexer.hip:408-560 (topk_bf16; the fp32 twin is src/kernels/ref_attn.hip:143-240): per row the
// want = min(k, #valid) largest scores, valid meaning key16(score) > key16(-inf) (indexer.hip:409,424-437); ties at the
// threshold to the lowest indices; output ordered (score descending, index ascending), -1 padded. The contract fixes
// every output element, so it is restated as a full sort of the valid keys.
void orc_topk_bf16(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, int threads) {
  parallel_for(T, threads, [&](int t) {
    const uint16_t* row = scores + size_t(t) * size_t(ld);
    std::vector<uint64_t> keys;
    keys.reserve(size_t(n));
    for (int i = 0; i < n; ++i) {
      const uint32_t b = row[i];
      const uint32_t key = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);  // indexer.hip:409
      if (key > 0x007Fu) keys.push_back((uint64_t(key) << 32) | (0xffffffffu - uint32_t(i)));
    }
    const size_t want = std::min(size_t(k), keys.size());
    std::partial_sort(keys.begin(), keys.begin() + ptrdiff_t(want), keys.end(), std::greater<uint64_t>());
    for (int j = 0; j < k; ++j)
      idx[size_t(t) * k + j] = size_t(j) < want ? int32_t(0xffffffffu - uint32_t(keys[size_t(j)] & 0xffffffffu)) : -1;
  });
}

// src/kernels/ref_attn.hip:137-254 (sort_key, topk_rows_kernel) = src/kernels/glm_fast.hip:551-681 (topk_seg_kernel; the
// two-stage form of glm_topk, :852-874, selects the same set): valid = key above the key of -inf; the min(k, #valid)
// largest by (key descending, index ascending), -1 padded.
void orc_topk_f32(const float* scores, int T, int n, long long ld, int k, int32_t* idx, int threads) {
  parallel_for(T, threads, [&](int t) {
    const float* row = scores + size_t(t) * size_t(ld);
    std::vector<uint64_t> keys;
    keys.reserve(size_t(n));
    for (int i = 0; i < n; ++i) {
      uint32_t u;
      std::memcpy(&u, row + i, 4);
      const uint32_t key = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ref_attn.hip:138-141
      if (key > 0x007fffffu) keys.push_back((uint64_t(key) << 32) | (0xffffffffu - uint32_t(i)));
    }
    const size_t want = std::min(size_t(k), keys.size());
    std::partial_sort(keys.begin(), keys.begin() + ptrdiff_t(want), keys.end(), std::greater<uint64_t>());
    for (int j = 0; j < k; ++j)
      idx[size_t(t) * k + j] = size_t(j) < want ? int32_t(0xffffffffu - uint32_t(keys[size_t(j)] & 0xffffffffu)) : -1;
  });
}

// src/kernels/glm_fast.hip:737-748 (idx_expand_compact_kernel) — selected pools -> compact token list.
void orc_idx_expand(const int32_t* pools, const int32_t* pos, int32_t* idx, int n, int k, int pool) {
  const int w = k * pool + pool - 1;
  for (int t = 0; t < n; ++t) {
    const int p = pos[t], full = (p + 1) / pool, valid = full < k ? full : k, tail = (p + 1) % pool;
    for (int j = 0; j < w; ++j) {
      int v = -1;
      if (j < valid * pool) v = pools[size_t(t) * k + j / pool] * pool + j % pool;
      else if (j < valid * pool + tail) v = p + 1 - tail + (j - valid * pool);
      idx[size_t(t) * w + j] = v;
    }
  }
}

// src/kernels/glm_fast.hip:190-227 (the gather loop of mla_attn_kernel): entry -> row id (glm_fast.hip:29-31), codes
// dequantised on the fly as bf16(e4m3 * 2^scale) (:203-218), masked entries zero (:219-222).
void orc_gather_rows_fp8(const uint8_t* codes, const uint8_t* scales, const int32_t* table, int rows_per_page, int width,
                         int block, const int32_t* idx, const int32_t* q_visible, int T, int k, uint16_t* out) {
  const int nb = width / block;
  for (int t = 0; t < T; ++t)
    for (int e = 0; e < k; ++e) {
      const int row = idx[size_t(t) * k + e];
      uint16_t* dst = out + (size_t(t) * k + e) * size_t(width);
      if (row < 0 || row >= q_visible[t]) {
        std::memset(dst, 0, size_t(width) * 2);
        continue;
      }
      const size_t rid = phys_row(table, rows_per_page, row);
      for (int c = 0; c < width; ++c)
        dst[c] = f32_to_bf16(e4m3_to_f32(codes[rid * size_t(width) + c]) * e8m0_to_f32(scales[rid * size_t(nb) + c / block]));
    }
}

// src/engine/resident.hip:545-557 (state_copies): for every op and segment one copy between the slot's slice
// (dev + slot * bytes) and the snapshot (snap + snapshot * snap_bytes + off). Host memory on both sides here.
void orc_state_copies(uint8_t* const* seg_dev, const size_t* seg_bytes, const size_t* seg_off, int nsegs, const int32_t* op_slot,
                      const int32_t* op_snapshot, int nops, uint8_t* snap, size_t snap_bytes, int save) {
  for (int o = 0; o < nops; ++o)
    for (int i = 0; i < nsegs; ++i) {
      uint8_t* slot = seg_dev[i] + size_t(op_slot[o]) * seg_bytes[i];
      uint8_t* sn = snap + size_t(op_snapshot[o]) * snap_bytes + seg_off[i];
      if (save) std::memcpy(sn, slot, seg_bytes[i]);
      else std::memcpy(slot, sn, seg_bytes[i]);
    }
}

// src/kernels/ref_elem.hip:111-135 (hadamard128_kernel): per 128-value segment seven butterfly stages in fp32,
// (b[i], b[i + h]) <- (a + c, a - c) for i = (t / h) * 2h + t % h, t = 0..63, then * 128^-0.5 and bf16 rounding, in place.
void orc_hadamard128(uint16_t* x, size_t nseg) {
  for (size_t g = 0; g < nseg; ++g) {
    uint16_t* p = x + g * 128;
    float b[128];
    for (int i = 0; i < 128; ++i) b[i] = bf16_to_f32(p[i]);
    for (int h = 1; h < 128; h <<= 1)
      for (int t = 0; t < 64; ++t) {
        const int i = (t / h) * 2 * h + (t % h);
        const float a = b[i], c = b[i + h];
        b[i] = a + c;
        b[i + h] = a - c;
      }
    const float sc = 0.08838834764831845f;
    for (int i = 0; i < 128; ++i) p[i] = f32_to_bf16(b[i] * sc);
  }
}

int orc_hardware_threads() { return int(std::thread::hardware_concurrency()); }

}  // extern "C"
