// Host-side parts of the C ABI: the seeded synthetic CSR generator that takes the place
// of the reference's dataset loaders (spmm/mm/spmm_common.cpp:125-296), a one-pass .smtx
// reader, the multi-GPU row partitioner, and the metric formulas.  No CUDA here.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <new>
#include <vector>

#include "hpspmm_internal.h"

struct hpspmm_graph {
  int64_t M = 0, N = 0, nnz = 0;
  std::vector<int32_t> row_ptr;
  std::vector<int32_t> col_idx;
  std::vector<float> vals;
};

namespace {

// PRNG stream ids, one per generated array
enum : uint64_t {
  kStreamDegree = 1,
  kStreamColumn = 2,
  kStreamValue = 3,
  kStreamRmat = 4,
};

inline double u01d(uint64_t bits) { return (double)(bits >> 11) * (1.0 / 9007199254740992.0); }

void fill_values(hpspmm_graph* g, uint64_t seed, int32_t kind) {
  g->vals.resize((size_t)g->nnz);
  float* v = g->vals.data();
  const int64_t n = g->nnz;
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < n; ++j) {
    if (kind == HPSPMM_VALS_ONES) {
      v[j] = 1.0f;  // the reference's loaders set every value to 1.0 (spmm_common.cpp:154)
    } else {
      const float u = hpspmm_u01(hpspmm_rand64(seed, kStreamValue, (uint64_t)j));
      v[j] = (kind == HPSPMM_VALS_U01) ? u : fmaf(2.0f, u, -1.0f);
    }
  }
}

// deg distinct columns in [0, N), ascending, drawn from the (row, t) counter stream
void draw_row_columns(uint64_t seed, int64_t row, int64_t N, int32_t deg, std::vector<int32_t>& out) {
  out.clear();
  uint64_t t = 0;
  while ((int32_t)out.size() < deg) {
    const int32_t need = deg - (int32_t)out.size();
    for (int32_t i = 0; i < need; ++i, ++t) {
      const uint64_t r = hpspmm_rand64(seed, kStreamColumn, ((uint64_t)row << 28) + t);
      out.push_back((int32_t)(r % (uint64_t)N));
    }
    std::sort(out.begin(), out.end());
    out.erase(std::unique(out.begin(), out.end()), out.end());
  }
}

int32_t poisson_draw(double lambda, double u) {
  // inverse CDF; lambda is moderate (tens), so the walk is short
  double p = std::exp(-lambda), cdf = p;
  int32_t k = 0;
  while (u > cdf && k < 100000) {
    ++k;
    p *= lambda / (double)k;
    cdf += p;
  }
  return k;
}

int build_from_degrees(int64_t M, int64_t N, const std::vector<int32_t>& deg, uint64_t seed,
                       int32_t vals_kind, hpspmm_graph** out) {
  hpspmm_graph* g = new (std::nothrow) hpspmm_graph();
  if (!g) return HPSPMM_ERR_OOM;
  try {
    g->M = M;
    g->N = N;
    g->row_ptr.assign((size_t)M + 1, 0);
    int64_t total = 0;
    for (int64_t r = 0; r < M; ++r) {
      total += deg[(size_t)r];
      if (total > 2147483647ll) {
        delete g;
        return HPSPMM_ERR_UNSUPPORTED;
      }
      g->row_ptr[(size_t)r + 1] = (int32_t)total;
    }
    g->nnz = total;
    g->col_idx.resize((size_t)total);
#pragma omp parallel
    {
      std::vector<int32_t> tmp;
#pragma omp for schedule(dynamic, 1024)
      for (int64_t r = 0; r < M; ++r) {
        draw_row_columns(seed, r, N, deg[(size_t)r], tmp);
        std::copy(tmp.begin(), tmp.end(), g->col_idx.begin() + g->row_ptr[(size_t)r]);
      }
    }
    fill_values(g, seed, vals_kind);
  } catch (const std::bad_alloc&) {
    delete g;
    return HPSPMM_ERR_OOM;
  }
  *out = g;
  return HPSPMM_OK;
}

}  // namespace

extern "C" {

int hpspmm_host_fill_uniform_f32(float* host_ptr, int64_t count, uint64_t seed, uint64_t stream_id,
                                 float lo, float hi) {
  if (count < 0 || (count > 0 && !host_ptr)) return HPSPMM_ERR_INVALID;
  const float span = hi - lo;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i)
    host_ptr[i] = fmaf(span, hpspmm_u01(hpspmm_rand64(seed, stream_id, (uint64_t)i)), lo);
  return HPSPMM_OK;
}

int hpspmm_gen_uniform_degree(int64_t M, int64_t N, int32_t deg_lo, int32_t deg_hi, uint64_t seed,
                              int32_t vals_kind, hpspmm_graph** out) {
  if (!out || M < 0 || N <= 0 || deg_lo < 0 || deg_hi < deg_lo || deg_hi > N) return HPSPMM_ERR_INVALID;
  *out = nullptr;
  std::vector<int32_t> deg;
  try {
    deg.resize((size_t)M);
  } catch (const std::bad_alloc&) {
    return HPSPMM_ERR_OOM;
  }
  const uint64_t span = (uint64_t)(deg_hi - deg_lo + 1);
  for (int64_t r = 0; r < M; ++r)
    deg[(size_t)r] = deg_lo + (int32_t)(hpspmm_rand64(seed, kStreamDegree, (uint64_t)r) % span);
  return build_from_degrees(M, N, deg, seed, vals_kind, out);
}

int hpspmm_gen_erdos_renyi(int64_t M, int64_t N, double mean_degree, uint64_t seed,
                           int32_t vals_kind, hpspmm_graph** out) {
  if (!out || M < 0 || N <= 0 || !(mean_degree >= 0.0) || mean_degree > 600.0) return HPSPMM_ERR_INVALID;
  *out = nullptr;
  std::vector<int32_t> deg;
  try {
    deg.resize((size_t)M);
  } catch (const std::bad_alloc&) {
    return HPSPMM_ERR_OOM;
  }
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < M; ++r) {
    int32_t d = poisson_draw(mean_degree, u01d(hpspmm_rand64(seed, kStreamDegree, (uint64_t)r)));
    if ((int64_t)d > N) d = (int32_t)N;
    deg[(size_t)r] = d;
  }
  return build_from_degrees(M, N, deg, seed, vals_kind, out);
}

int hpspmm_gen_rmat(int32_t scale, int32_t edge_factor, double a, double b, double c, uint64_t seed,
                    int32_t vals_kind, hpspmm_graph** out) {
  if (!out || scale < 1 || scale > 27 || edge_factor < 1 || a <= 0 || b < 0 || c < 0 || a + b + c >= 1.0)
    return HPSPMM_ERR_INVALID;
  *out = nullptr;
  const int64_t n = (int64_t)1 << scale;
  const int64_t draws = (int64_t)edge_factor * n / 2;
  if (2 * draws > 2147483647ll) return HPSPMM_ERR_UNSUPPORTED;
  hpspmm_graph* g = new (std::nothrow) hpspmm_graph();
  if (!g) return HPSPMM_ERR_OOM;
  try {
    std::vector<int32_t> eu((size_t)draws), ev((size_t)draws);
    const double ab = a + b, abc = a + b + c;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < draws; ++e) {
      int32_t u = 0, v = 0;
      for (int32_t l = 0; l < scale; ++l) {
        const double x = u01d(hpspmm_rand64(seed, kStreamRmat, (uint64_t)e * 32u + (uint64_t)l));
        const int32_t ubit = x >= ab;
        const int32_t vbit = (x >= a && x < ab) || x >= abc;
        u = (u << 1) | ubit;
        v = (v << 1) | vbit;
      }
      eu[(size_t)e] = u;
      ev[(size_t)e] = v;
    }
    // bucket both directions by source vertex
    std::vector<int64_t> off((size_t)n + 1, 0);
    for (int64_t e = 0; e < draws; ++e) {
      off[(size_t)eu[(size_t)e] + 1]++;
      off[(size_t)ev[(size_t)e] + 1]++;
    }
    for (int64_t r = 0; r < n; ++r) off[(size_t)r + 1] += off[(size_t)r];
    std::vector<int32_t> adj((size_t)(2 * draws));
    {
      std::vector<int64_t> cur(off.begin(), off.end() - 1);
      for (int64_t e = 0; e < draws; ++e) {
        const int32_t u = eu[(size_t)e], v = ev[(size_t)e];
        adj[(size_t)cur[(size_t)u]++] = v;
        adj[(size_t)cur[(size_t)v]++] = u;
      }
    }
    std::vector<int32_t>().swap(eu);
    std::vector<int32_t>().swap(ev);
    // sort and de-duplicate each row in place
    std::vector<int32_t> deg((size_t)n);
#pragma omp parallel for schedule(dynamic, 512)
    for (int64_t r = 0; r < n; ++r) {
      int32_t* lo = adj.data() + off[(size_t)r];
      int32_t* hi = adj.data() + off[(size_t)r + 1];
      std::sort(lo, hi);
      deg[(size_t)r] = (int32_t)(std::unique(lo, hi) - lo);
    }
    g->M = g->N = n;
    g->row_ptr.assign((size_t)n + 1, 0);
    int64_t total = 0;
    for (int64_t r = 0; r < n; ++r) {
      total += deg[(size_t)r];
      g->row_ptr[(size_t)r + 1] = (int32_t)total;
    }
    g->nnz = total;
    g->col_idx.resize((size_t)total);
#pragma omp parallel for schedule(dynamic, 512)
    for (int64_t r = 0; r < n; ++r)
      std::copy(adj.data() + off[(size_t)r], adj.data() + off[(size_t)r] + deg[(size_t)r],
                g->col_idx.data() + g->row_ptr[(size_t)r]);
    fill_values(g, seed, vals_kind);
  } catch (const std::bad_alloc&) {
    delete g;
    return HPSPMM_ERR_OOM;
  }
  *out = g;
  return HPSPMM_OK;
}

int hpspmm_gen_shape(const hpspmm_graph* g, int64_t* M, int64_t* N, int64_t* nnz) {
  if (!g) return HPSPMM_ERR_INVALID;
  if (M) *M = g->M;
  if (N) *N = g->N;
  if (nnz) *nnz = g->nnz;
  return HPSPMM_OK;
}

int hpspmm_gen_export(const hpspmm_graph* g, int32_t* row_ptr, int32_t* col_idx, float* vals) {
  if (!g) return HPSPMM_ERR_INVALID;
  if (row_ptr) memcpy(row_ptr, g->row_ptr.data(), g->row_ptr.size() * sizeof(int32_t));
  if (col_idx && g->nnz) memcpy(col_idx, g->col_idx.data(), (size_t)g->nnz * sizeof(int32_t));
  if (vals && g->nnz) memcpy(vals, g->vals.data(), (size_t)g->nnz * sizeof(float));
  return HPSPMM_OK;
}

int hpspmm_gen_free(hpspmm_graph* g) {
  delete g;
  return HPSPMM_OK;
}

int hpspmm_read_smtx(const char* path, hpspmm_graph** out) {
  if (!path || !out) return HPSPMM_ERR_INVALID;
  *out = nullptr;
  FILE* f = fopen(path, "rb");
  if (!f) return HPSPMM_ERR_INVALID;
  fseek(f, 0, SEEK_END);
  const long size = ftell(f);
  fseek(f, 0, SEEK_SET);
  std::vector<char> buf;
  try {
    buf.resize((size_t)size + 1);
  } catch (const std::bad_alloc&) {
    fclose(f);
    return HPSPMM_ERR_OOM;
  }
  const size_t got = fread(buf.data(), 1, (size_t)size, f);
  fclose(f);
  buf[got] = 0;
  char* p = buf.data();
  char* end = nullptr;
  long dims[3];
  for (int i = 0; i < 3; ++i) {
    dims[i] = strtol(p, &end, 10);
    if (end == p) return HPSPMM_ERR_INVALID;
    p = end;
    while (*p == ',' || *p == ' ') ++p;
  }
  if (dims[0] < 0 || dims[1] < 0 || dims[2] < 0) return HPSPMM_ERR_INVALID;
  hpspmm_graph* g = new (std::nothrow) hpspmm_graph();
  if (!g) return HPSPMM_ERR_OOM;
  try {
    g->M = dims[0];
    g->N = dims[1];
    g->nnz = dims[2];
    g->row_ptr.resize((size_t)g->M + 1);
    g->col_idx.resize((size_t)g->nnz);
    for (int64_t i = 0; i <= g->M; ++i) {
      const long v = strtol(p, &end, 10);
      if (end == p) {
        delete g;
        return HPSPMM_ERR_BAD_CSR;
      }
      g->row_ptr[(size_t)i] = (int32_t)v;
      p = end;
    }
    for (int64_t j = 0; j < g->nnz; ++j) {
      const long v = strtol(p, &end, 10);
      if (end == p) {
        delete g;
        return HPSPMM_ERR_BAD_CSR;
      }
      g->col_idx[(size_t)j] = (int32_t)v;
      p = end;
    }
    if (g->row_ptr[0] != 0 || g->row_ptr[(size_t)g->M] != g->nnz) {
      delete g;
      return HPSPMM_ERR_BAD_CSR;
    }
    g->vals.assign((size_t)g->nnz, 1.0f);
  } catch (const std::bad_alloc&) {
    delete g;
    return HPSPMM_ERR_OOM;
  }
  *out = g;
  return HPSPMM_OK;
}

// Row order file of the reference (".cugraph_reorder", spmm/mm/spmm_common.cpp:262-267): one
// line of M whitespace-separated row ids, the order in which rows are to be emitted.  Unlike
// the reference this checks that the line is a permutation of 0..M-1.
int hpspmm_read_row_order(const char* path, int64_t M, int32_t* order_out) {
  if (!path || M < 0 || (M > 0 && !order_out)) return HPSPMM_ERR_INVALID;
  FILE* f = fopen(path, "rb");
  if (!f) return HPSPMM_ERR_INVALID;
  fseek(f, 0, SEEK_END);
  const long size = ftell(f);
  fseek(f, 0, SEEK_SET);
  std::vector<char> buf;
  std::vector<char> seen;
  try {
    buf.resize((size_t)size + 1);
    seen.assign((size_t)M, 0);
  } catch (const std::bad_alloc&) {
    fclose(f);
    return HPSPMM_ERR_OOM;
  }
  const size_t got = fread(buf.data(), 1, (size_t)size, f);
  fclose(f);
  buf[got] = 0;
  char* p = buf.data();
  char* end = nullptr;
  for (int64_t i = 0; i < M; ++i) {
    const long v = strtol(p, &end, 10);
    if (end == p || v < 0 || v >= M || seen[(size_t)v]) return HPSPMM_ERR_BAD_CSR;
    seen[(size_t)v] = 1;
    order_out[i] = (int32_t)v;
    p = end;
  }
  return HPSPMM_OK;
}

int hpspmm_shard_bounds(int64_t M, const int32_t* row_ptr_host, int32_t G, int64_t* bounds) {
  if (M < 0 || !row_ptr_host || G < 1 || !bounds) return HPSPMM_ERR_INVALID;
  const int64_t nnz = row_ptr_host[M];
  bounds[0] = 0;
  for (int32_t g = 1; g < G; ++g) {
    const int64_t target = (int64_t)(((__int128)nnz * g) / G);
    const int32_t* it = std::lower_bound(row_ptr_host, row_ptr_host + M, target,
                                         [](int32_t v, int64_t t) { return (int64_t)v < t; });
    bounds[g] = (int64_t)(it - row_ptr_host);
  }
  bounds[G] = M;
  return HPSPMM_OK;
}

int hpspmm_shard_bounds_weighted(int64_t M, const int32_t* row_ptr_host, int32_t G, double row_weight,
                                 int64_t* bounds) {
  if (M < 0 || !row_ptr_host || G < 1 || !bounds || !(row_weight >= 0.0)) return HPSPMM_ERR_INVALID;
  // cost of rows [0, r): their entries plus row_weight per row; monotone in r, so every cut is a binary search
  const double total = (double)row_ptr_host[M] + row_weight * (double)M;
  bounds[0] = 0;
  for (int32_t g = 1; g < G; ++g) {
    const double target = total * (double)g / (double)G;
    int64_t lo = 0, hi = M;
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if ((double)row_ptr_host[mid] + row_weight * (double)mid < target)
        lo = mid + 1;
      else
        hi = mid;
    }
    bounds[g] = lo < bounds[g - 1] ? bounds[g - 1] : lo;
  }
  bounds[G] = M;
  return HPSPMM_OK;
}

int hpspmm_shard_row_ptr(const int32_t* row_ptr_host, int64_t row_lo, int64_t row_hi,
                         int32_t* local_row_ptr, int64_t* nnz_lo_out, int64_t* nnz_local_out) {
  if (!row_ptr_host || !local_row_ptr || row_lo < 0 || row_hi < row_lo) return HPSPMM_ERR_INVALID;
  const int32_t base = row_ptr_host[row_lo];
  for (int64_t i = 0; i <= row_hi - row_lo; ++i) local_row_ptr[i] = row_ptr_host[row_lo + i] - base;
  if (nnz_lo_out) *nnz_lo_out = base;
  if (nnz_local_out) *nnz_local_out = (int64_t)row_ptr_host[row_hi] - base;
  return HPSPMM_OK;
}

int hpspmm_shard_needed_rows(int64_t nnz_local, const int32_t* col_idx_host, int64_t N, int32_t world,
                             const int64_t* b_bounds, int32_t* col_compact_out, int32_t* need_rows_out,
                             int64_t* need_off_out, int64_t* n_needed_out) {
  if (nnz_local < 0 || N < 1 || N > 2147483646ll || world < 1 || !b_bounds || !need_off_out || !n_needed_out)
    return HPSPMM_ERR_INVALID;
  if (nnz_local > 0 && (!col_idx_host || !col_compact_out || !need_rows_out)) return HPSPMM_ERR_INVALID;
  if (b_bounds[0] != 0 || b_bounds[world] != N) return HPSPMM_ERR_INVALID;
  for (int32_t s = 0; s < world; ++s)
    if (b_bounds[s] > b_bounds[s + 1]) return HPSPMM_ERR_INVALID;
  // mark, number (an exclusive scan over the marks), renumber
  std::vector<int32_t> id((size_t)N + 1, 0);
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t j = 0; j < nnz_local; ++j) {
    const int32_t c = col_idx_host[j];
    if (c < 0 || c >= N)
      bad |= 1;
    else
      id[(size_t)c] = 1;   // benign race: every writer stores the same value
  }
  if (bad) return HPSPMM_ERR_BAD_CSR;
  int32_t run = 0;
  for (int64_t c = 0; c < N; ++c) {
    const int32_t m = id[(size_t)c];
    id[(size_t)c] = run;
    if (m) need_rows_out[run++] = (int32_t)c;
  }
  id[(size_t)N] = run;
  for (int32_t s = 0; s <= world; ++s) need_off_out[s] = id[(size_t)b_bounds[s]];
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < nnz_local; ++j) col_compact_out[j] = id[(size_t)col_idx_host[j]];
  *n_needed_out = run;
  return HPSPMM_OK;
}

double hpspmm_gflops(int64_t nnz, int64_t K, double ms) {
  return (double)nnz * (double)K * 2.0 / ms / 1.0e6;
}

double hpspmm_row_length_cv(int64_t M, const int32_t* row_ptr_host) {
  if (M <= 0 || !row_ptr_host) return 0.0;
  double sum = 0.0;
  for (int64_t r = 0; r < M; ++r) sum += (double)(row_ptr_host[r + 1] - row_ptr_host[r]);
  const double mean = sum / (double)M;
  double acc = 0.0;
  for (int64_t r = 0; r < M; ++r) {
    const double d = (double)(row_ptr_host[r + 1] - row_ptr_host[r]) - mean;
    acc += d * d;
  }
  return std::sqrt(acc / (double)M) / mean;
}

double hpspmm_spmm_algorithmic_bytes(int64_t M, int64_t N_ref, int64_t K, int64_t nnz) {
  return 4.0 * (double)(M + 1) + 8.0 * (double)nnz + 4.0 * (double)K * (double)N_ref +
         4.0 * (double)K * (double)M;
}

double hpspmm_sddmm_algorithmic_bytes(int64_t M_ref, int64_t N_ref, int64_t K, int64_t M, int64_t nnz) {
  return 4.0 * (double)(M + 1) + 8.0 * (double)nnz + 4.0 * (double)K * (double)(M_ref + N_ref);
}

}  // extern "C"
