// Host-side code of the library under AddressSanitizer and UndefinedBehaviorSanitizer (test infrastructure).
// Built by tests/test_host_sanitizers.py from hp-spmm-sddmm_b200/csrc/host_side.cpp; exercises the generators,
// the .smtx and row-order readers, the partitioner and the needed-rows planner, including their edge cases.
// Exit code 0 and no sanitizer report = pass.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "hpspmm.h"

#define CHECK(cond)                                                         \
  do {                                                                      \
    if (!(cond)) {                                                          \
      std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      return 1;                                                             \
    }                                                                       \
  } while (0)

static int export_graph(hpspmm_graph* g, std::vector<int32_t>& rp, std::vector<int32_t>& ci, std::vector<float>& v) {
  int64_t M = 0, N = 0, nnz = 0;
  if (hpspmm_gen_shape(g, &M, &N, &nnz) != HPSPMM_OK) return 1;
  rp.assign((size_t)M + 1, 0);
  ci.assign((size_t)(nnz > 0 ? nnz : 1), 0);
  v.assign((size_t)(nnz > 0 ? nnz : 1), 0.f);
  if (hpspmm_gen_export(g, rp.data(), ci.data(), v.data()) != HPSPMM_OK) return 1;
  ci.resize((size_t)nnz);
  v.resize((size_t)nnz);
  return hpspmm_gen_free(g) != HPSPMM_OK;
}

int main(int argc, char** argv) {
  const char* tmp = argc > 1 ? argv[1] : "/tmp";
  std::vector<int32_t> rp, ci;
  std::vector<float> v;
  hpspmm_graph* g = nullptr;

  // generators
  CHECK(hpspmm_gen_uniform_degree(300, 200, 0, 12, 3, HPSPMM_VALS_UPM1, &g) == HPSPMM_OK);
  CHECK(export_graph(g, rp, ci, v) == 0);
  CHECK(rp.size() == 301 && rp[0] == 0 && (size_t)rp[300] == ci.size());
  CHECK(hpspmm_gen_rmat(10, 8, 0.57, 0.19, 0.19, 7, HPSPMM_VALS_U01, &g) == HPSPMM_OK);
  CHECK(export_graph(g, rp, ci, v) == 0);
  const int64_t M = (int64_t)rp.size() - 1, nnz = (int64_t)ci.size();
  CHECK(M == 1024 && nnz > 0);
  for (int64_t r = 0; r < M; ++r)
    for (int32_t j = rp[r] + 1; j < rp[r + 1]; ++j) CHECK(ci[j - 1] < ci[j]);   // sorted, no duplicates
  CHECK(hpspmm_gen_erdos_renyi(500, 500, 6.0, 11, HPSPMM_VALS_ONES, &g) == HPSPMM_OK);
  std::vector<int32_t> rp2, ci2;
  std::vector<float> v2;
  CHECK(export_graph(g, rp2, ci2, v2) == 0);
  CHECK(hpspmm_gen_uniform_degree(-1, 10, 0, 1, 1, 0, &g) != HPSPMM_OK);

  // host fill
  std::vector<float> x(1000);
  CHECK(hpspmm_host_fill_uniform_f32(x.data(), 1000, 2, 3, -1.f, 1.f) == HPSPMM_OK);
  for (float f : x) CHECK(f >= -1.f && f < 1.f);
  CHECK(hpspmm_host_fill_uniform_f32(x.data(), 0, 2, 3, -1.f, 1.f) == HPSPMM_OK);

  // partitioner: every world size, degenerate shards
  for (int G = 1; G <= 9; ++G) {
    std::vector<int64_t> b((size_t)G + 1);
    CHECK(hpspmm_shard_bounds(M, rp.data(), G, b.data()) == HPSPMM_OK);
    CHECK(b[0] == 0 && b[G] == M);
    int64_t total = 0;
    for (int s = 0; s < G; ++s) {
      CHECK(b[s] <= b[s + 1]);
      std::vector<int32_t> local((size_t)(b[s + 1] - b[s]) + 1);
      int64_t lo = 0, n = 0;
      CHECK(hpspmm_shard_row_ptr(rp.data(), b[s], b[s + 1], local.data(), &lo, &n) == HPSPMM_OK);
      CHECK(local[0] == 0 && local.back() == n);
      total += n;
      // needed rows of this shard
      std::vector<int32_t> cc((size_t)(n > 0 ? n : 1)), need((size_t)(n > 0 ? (n < M ? n : M) : 1));
      std::vector<int64_t> off((size_t)G + 1);
      int64_t n_needed = -1;
      CHECK(hpspmm_shard_needed_rows(n, ci.data() + lo, M, G, b.data(), cc.data(), need.data(), off.data(), &n_needed) ==
            HPSPMM_OK);
      CHECK(off[0] == 0 && off[G] == n_needed);
      for (int64_t j = 0; j < n; ++j) CHECK(need[cc[j]] == ci[lo + j]);
    }
    CHECK(total == nnz);
  }
  {
    const int32_t empty_rp[5] = {0, 0, 0, 0, 0};
    int64_t b[4];
    CHECK(hpspmm_shard_bounds(4, empty_rp, 3, b) == HPSPMM_OK && b[0] == 0 && b[3] == 4);
    int64_t off[3], n_needed = 7;
    const int64_t bb[3] = {0, 2, 4};
    CHECK(hpspmm_shard_needed_rows(0, nullptr, 4, 2, bb, nullptr, nullptr, off, &n_needed) == HPSPMM_OK && n_needed == 0);
    const int32_t bad_col[2] = {1, 4};
    int32_t cc[2], need[2];
    CHECK(hpspmm_shard_needed_rows(2, bad_col, 4, 2, bb, cc, need, off, &n_needed) == HPSPMM_ERR_BAD_CSR);
    CHECK(hpspmm_shard_bounds(4, nullptr, 3, b) != HPSPMM_OK);
  }

  // .smtx and row-order readers: a good file, truncated files, a non-permutation
  char path[512];
  std::snprintf(path, sizeof(path), "%s/g.smtx", tmp);
  FILE* f = std::fopen(path, "w");
  CHECK(f != nullptr);
  std::fprintf(f, "%lld,%lld,%lld\n", (long long)M, (long long)M, (long long)nnz);
  for (int64_t r = 0; r <= M; ++r) std::fprintf(f, "%d ", rp[r]);
  std::fprintf(f, "\n");
  for (int64_t j = 0; j < nnz; ++j) std::fprintf(f, "%d ", ci[j]);
  std::fprintf(f, "\n");
  std::fclose(f);
  CHECK(hpspmm_read_smtx(path, &g) == HPSPMM_OK);
  std::vector<int32_t> rp3, ci3;
  std::vector<float> v3;
  CHECK(export_graph(g, rp3, ci3, v3) == 0);
  CHECK(rp3 == rp && ci3 == ci);
  std::snprintf(path, sizeof(path), "%s/short.smtx", tmp);
  f = std::fopen(path, "w");
  std::fprintf(f, "4,4,5\n0 1 2 3 5\n0 1 2\n");     // fewer column ids than announced
  std::fclose(f);
  CHECK(hpspmm_read_smtx(path, &g) != HPSPMM_OK);
  std::snprintf(path, sizeof(path), "%s/none.smtx", tmp);
  CHECK(hpspmm_read_smtx(path, &g) != HPSPMM_OK);   // no such file
  std::snprintf(path, sizeof(path), "%s/order.txt", tmp);
  f = std::fopen(path, "w");
  std::fprintf(f, "3 1 0 2\n");
  std::fclose(f);
  int32_t order[4];
  CHECK(hpspmm_read_row_order(path, 4, order) == HPSPMM_OK && order[0] == 3 && order[3] == 2);
  f = std::fopen(path, "w");
  std::fprintf(f, "3 1 1 2\n");
  std::fclose(f);
  CHECK(hpspmm_read_row_order(path, 4, order) != HPSPMM_OK);
  f = std::fopen(path, "w");
  std::fprintf(f, "3 1\n");
  std::fclose(f);
  CHECK(hpspmm_read_row_order(path, 4, order) != HPSPMM_OK);

  // metric helpers
  CHECK(hpspmm_gflops(1000, 32, 1.0) > 0.0);
  CHECK(hpspmm_row_length_cv(M, rp.data()) > 0.0);
  CHECK(hpspmm_spmm_algorithmic_bytes(10, 10, 32, 100) == 4.0 * 11 + 800.0 + 4.0 * 32 * 20);
  std::printf("host sanitizer run: ok\n");
  return 0;
}
