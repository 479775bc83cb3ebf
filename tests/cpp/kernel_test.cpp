// GPU test of the C++ wrappers (unholy_b200/csrc/host/kernels.hpp) in the style of the reference's standalone kernel
// tests (tools/kernel_test/indexer.hip:40-95): seeded rows, a shuffled block table, store -> load round trip equal to
// fake_quant_fp4, store_rows + gather_rows equal to the rows, errors thrown as std::runtime_error. Prints and returns
// non-zero on failure. Built and run by tests/test_gpu_cpp_wrappers.py.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <random>
#include <vector>

#include "../../unholy_b200/csrc/host/kernels.hpp"

namespace k = unholy::kernels;

#define CK(x)                                                                  \
  do {                                                                         \
    cudaError_t e_ = (x);                                                      \
    if (e_ != cudaSuccess) {                                                   \
      std::printf("cuda error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
      return 2;                                                                \
    }                                                                          \
  } while (0)

static uint16_t to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}

template <class T>
struct Dev {
  T* p = nullptr;
  size_t n = 0;
  explicit Dev(size_t count) : n(count) { cudaMalloc(&p, count * sizeof(T)); }
  ~Dev() { cudaFree(p); }
  void up(const std::vector<T>& h) { cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice); }
  std::vector<T> down() const {
    std::vector<T> h(n);
    cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost);
    return h;
  }
};

int main() {
  int fails = 0;
  std::mt19937_64 rng(1);
  std::normal_distribution<float> nd(0.0f, 1.0f);
  // ---- fp4 keys: store -> load == fake_quant_fp4 over a shuffled table ----
  {
    const int nkeys = 5000, D = 128, pages = (nkeys + k::kFp4RowsPerPage - 1) / k::kFp4RowsPerPage;
    std::vector<uint16_t> hk(size_t(nkeys) * D);
    for (int r = 0; r < nkeys; ++r) {
      const float m = std::ldexp(1.0f, int(rng() % 7) - 3);
      for (int c = 0; c < D; ++c) hk[size_t(r) * D + c] = to_bf16(nd(rng) * m);
    }
    std::vector<int32_t> table(static_cast<size_t>(pages));
    std::iota(table.begin(), table.end(), 0);
    std::shuffle(table.begin(), table.end(), rng);
    Dev<uint16_t> dk(hk.size()), back(hk.size());
    Dev<int32_t> dt(table.size());
    Dev<uint8_t> pool(size_t(pages) * k::kFp4PageBytes);
    dk.up(hk);
    dt.up(table);
    const k::PagedFp4 keys{pool.p, dt.p};
    k::store_rows_fp4(dk.p, nkeys, keys, 0, nullptr);
    k::load_rows_fp4(keys, 0, nkeys, back.p, nullptr);
    k::fake_quant_fp4(dk.p, D, nkeys, D, 32, nullptr);
    CK(cudaDeviceSynchronize());
    const auto a = back.down(), b = dk.down();
    size_t diff = 0;
    for (size_t i = 0; i < a.size(); ++i) diff += a[i] != b[i];
    std::printf("fp4 store/load vs fake_quant_fp4: %zu / %zu differ\n", diff, a.size());
    fails += diff != 0;
  }
  // ---- bf16 rows: store_rows then gather_rows returns the rows; masked entries are zero ----
  {
    const int n = 1000, W = 576, rpp = 64, pages = 16;
    std::vector<uint16_t> rows(size_t(n) * W);
    for (auto& v : rows) v = to_bf16(nd(rng));
    std::vector<int32_t> table(pages);
    std::iota(table.begin(), table.end(), 0);
    std::shuffle(table.begin(), table.end(), rng);
    const int T = 2, kk = 600;
    std::vector<int32_t> idx(size_t(T) * kk), vis = {n, 500};
    for (int t = 0; t < T; ++t)
      for (int e = 0; e < kk; ++e) idx[size_t(t) * kk + e] = e % 7 == 6 ? -1 : int(rng() % n);
    Dev<uint16_t> drows(rows.size()), pool(size_t(pages) * rpp * W), out(size_t(T) * kk * W);
    Dev<int32_t> dt(table.size()), didx(idx.size()), dvis(vis.size());
    drows.up(rows);
    dt.up(table);
    didx.up(idx);
    dvis.up(vis);
    const k::PagedRows pr{pool.p, dt.p, rpp, W};
    k::store_rows(drows.p, n, W, pr, 0, nullptr);
    k::gather_rows(pr, W, didx.p, dvis.p, T, kk, out.p, nullptr);
    CK(cudaDeviceSynchronize());
    const auto got = out.down();
    size_t diff = 0;
    for (int t = 0; t < T; ++t)
      for (int e = 0; e < kk; ++e) {
        const int r = idx[size_t(t) * kk + e];
        const bool masked = r < 0 || r >= vis[size_t(t)];
        for (int c = 0; c < W; ++c) {
          const uint16_t want = masked ? 0 : rows[size_t(r) * W + c];
          diff += got[(size_t(t) * kk + e) * W + c] != want;
        }
      }
    std::printf("store_rows + gather_rows: %zu values differ\n", diff);
    fails += diff != 0;
  }
  // ---- topk_rows == glm_topk == a host sort by (score desc, index asc); k > 1024 throws as in the reference ----
  {
    const int T = 9, n = 6000, kk = 300;
    std::vector<float> sc(size_t(T) * n);
    for (auto& v : sc) v = float(int(rng() % 4001) - 2000) * 0.25f;   // many equal scores
    for (int i = 4000; i < n; ++i) sc[size_t(2) * n + i] = -INFINITY;
    Dev<float> d_sc(sc.size());
    d_sc.up(sc);
    Dev<int32_t> d_a(size_t(T) * kk), d_b(size_t(T) * kk);
    k::topk_rows(d_sc.p, T, n, kk, d_a.p, nullptr);
    k::glm_topk(d_sc.p, n, T, n, kk, d_b.p, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    const auto a = d_a.down(), b = d_b.down();
    size_t diff = 0;
    std::vector<int32_t> order(static_cast<size_t>(n));
    for (int t = 0; t < T; ++t) {
      std::iota(order.begin(), order.end(), 0);
      const float* row = sc.data() + size_t(t) * n;
      std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return row[x] > row[y]; });
      for (int e = 0; e < kk; ++e) {
        const int32_t want = row[order[size_t(e)]] == -INFINITY ? -1 : order[size_t(e)];
        diff += a[size_t(t) * kk + e] != want;
        diff += b[size_t(t) * kk + e] != want;
      }
    }
    std::printf("topk_rows / glm_topk: %zu entries differ\n", diff);
    fails += diff != 0;
    bool threw = false;
    try {
      k::topk_rows(d_sc.p, T, n, 1025, d_a.p, nullptr);
    } catch (const std::runtime_error& e) {
      threw = std::strstr(e.what(), "k > 1024") != nullptr;
    }
    std::printf("topk_rows k > 1024 throws: %s\n", threw ? "yes" : "NO");
    fails += !threw;
  }
  // ---- topk_bf16 / topk_bf16_batch with the reference's signatures (src/kernels/indexer.hpp:74-94), called the way
  //      src/model/forward_ref.hip:890-935 calls them: score blocks of several chunks in one buffer, the rest of the
  //      buffer (possibly very little) offered as scratch; and without any scratch at all ----
  {
    const int n0 = 9000, n1 = 700, kk = 512, rows0 = 3, rows1 = 5;
    std::vector<uint16_t> sc(size_t(rows0) * n0 + size_t(rows1) * n1 + 64);
    for (auto& v : sc) v = to_bf16(float(int(rng() % 2001) - 1000) * 0.125f);   // many ties
    Dev<uint16_t> d_sc(sc.size());
    d_sc.up(sc);
    Dev<int32_t> d_idx(size_t(rows0 + rows1) * kk), d_one(size_t(rows0) * kk);
    k::TopkBatch tb;
    tb.g[tb.ngroups++] = {0, rows0, n0, kk, 0};
    tb.g[tb.ngroups++] = {size_t(rows0) * n0, rows1, n1, kk, rows0 * kk};
    const size_t used = size_t(rows0) * n0 + size_t(rows1) * n1;
    k::topk_bf16_batch(d_sc.p, tb, d_idx.p, nullptr, reinterpret_cast<uint32_t*>(d_sc.p + used), (sc.size() - used) / 2);  // 32 words
    k::topk_bf16(d_sc.p, rows0, n0, kk, d_one.p, nullptr);
    CK(cudaDeviceSynchronize());
    const auto got = d_idx.down(), one = d_one.down();
    auto f = [](uint16_t b) {
      uint32_t u = uint32_t(b) << 16;
      float x;
      std::memcpy(&x, &u, 4);
      return x;
    };
    size_t diff = 0;
    for (int gi = 0; gi < 2; ++gi) {
      const int rows = gi ? rows1 : rows0, n = gi ? n1 : n0;
      const uint16_t* base = sc.data() + (gi ? size_t(rows0) * n0 : 0);
      std::vector<int32_t> order(static_cast<size_t>(n));
      for (int t = 0; t < rows; ++t) {
        std::iota(order.begin(), order.end(), 0);
        const uint16_t* row = base + size_t(t) * n;
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return f(row[x]) > f(row[y]); });
        for (int e = 0; e < kk; ++e) {
          const int32_t want = e < n ? order[size_t(e)] : -1;
          diff += got[(gi ? size_t(rows0) * kk : 0) + size_t(t) * kk + e] != want;
          if (!gi) diff += one[size_t(t) * kk + e] != want;
        }
      }
    }
    std::printf("topk_bf16 / topk_bf16_batch (reference signatures, 32 words of scratch): %zu entries differ\n", diff);
    fails += diff != 0;
    // the four-launch path without caller scratch falls back to the library's own; a shape too large for it throws
    pkv_tune(7, 1);
    k::topk_bf16(d_sc.p, rows0, n0, kk, d_one.p, nullptr);
    CK(cudaDeviceSynchronize());
    const auto again = d_one.down();
    size_t d2 = 0;
    for (size_t i = 0; i < again.size(); ++i) d2 += again[i] != one[i];
    std::printf("topk_bf16 through the built-in scratch: %zu entries differ\n", d2);
    fails += d2 != 0;
    bool threw = false;
    try {
      k::topk_bf16(d_sc.p, 4096, 2, 4096, d_one.p, nullptr);   // needs far more scratch than the built-in array holds
    } catch (const std::runtime_error& e) {
      threw = std::strstr(e.what(), "scratch") != nullptr;
    }
    pkv_tune(7, 0);
    std::printf("top-k beyond the built-in scratch throws: %s\n", threw ? "yes" : "NO");
    fails += !threw;
  }
  // ---- errors are exceptions ----
  {
    bool threw = false;
    try {
      k::act_quant_fp8(reinterpret_cast<const uint16_t*>(16), 128, reinterpret_cast<uint8_t*>(16),
                       reinterpret_cast<uint8_t*>(16), 1, 128, 48, nullptr);
    } catch (const std::runtime_error& e) {
      threw = std::strstr(e.what(), "block must be") != nullptr;
    }
    std::printf("bad block size throws: %s\n", threw ? "yes" : "NO");
    fails += !threw;
  }
  std::printf(fails ? "FAILED\n" : "all ok\n");
  return fails ? 1 : 0;
}
