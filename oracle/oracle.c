/*
 * CPU oracle for the FP32 CSR SpMM / SDDMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's GPU
 * kernels so that the CUDA path can be checked against it.  It is never part
 * of the product: only tests, the smoke check and the CPU-baseline leg of the
 * benchmark may load it.  The product path has no CPU fallback.
 *
 * Pinning: the reference ships no golden vectors, no known-answer tests and
 * no CPU SpMM.  This restatement is pinned (a) against scipy.sparse on the
 * host and (b) against outputs of the reference's own GESpMM / LBSpMM kernels
 * run on a B200 (fixtures under tests/golden/, see tests/golden/README.md).
 * SDDMM and CSR transpose have no counterpart in the reference: for those
 * two functions parity with the reference is UNPINNED; they are pinned only
 * against scipy.
 *
 * Every function takes 64-bit element offsets into the dense operands; the
 * reference uses 32-bit ints throughout (include/starml/basic/matrix.h:71,
 * spmm/mm/spmm_kernel.cu:269,332,454).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/*
 * C = A * B, FP32, one sequential CSR-order accumulation per output element.
 * Follows the row loop of topoCacheSPMMKernel / topoCacheCoarsenSPMMKernel
 * (spmm/mm/spmm_kernel.cu:324-346 and :259-283): for every row, for every
 * stored entry in storage order, acc += val * B[col*K + c]; then the row of
 * C is overwritten (empty rows become zeros).  nvcc contracts the multiply
 * and add of that loop into one FMA, hence fmaf here.
 */
ORACLE_API void oracle_spmm_csr_f32(int64_t M, int64_t K, const int32_t* row_ptr,
                                    const int32_t* col_idx, const float* vals,
                                    const float* B, float* C) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < M; ++r) {
    float* crow = C + r * K;
    for (int64_t c = 0; c < K; ++c) crow[c] = 0.0f;
    for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
      const float v = vals[j];
      const float* brow = B + (int64_t)col_idx[j] * K;
      for (int64_t c = 0; c < K; ++c) crow[c] = fmaf(v, brow[c], crow[c]);
    }
  }
}

/*
 * Same product accumulated in FP64 (the error yardstick), plus, when
 * abs_sum != NULL, the sum of |val * B| per output element, which bounds the
 * rounding error of any FP32 summation order.
 */
ORACLE_API void oracle_spmm_csr_f64(int64_t M, int64_t K, const int32_t* row_ptr,
                                    const int32_t* col_idx, const float* vals,
                                    const float* B, double* C, double* abs_sum) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < M; ++r) {
    double* crow = C + r * K;
    double* arow = abs_sum ? abs_sum + r * K : NULL;
    for (int64_t c = 0; c < K; ++c) crow[c] = 0.0;
    if (arow)
      for (int64_t c = 0; c < K; ++c) arow[c] = 0.0;
    for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
      const double v = vals[j];
      const float* brow = B + (int64_t)col_idx[j] * K;
      for (int64_t c = 0; c < K; ++c) {
        const double t = v * (double)brow[c];
        crow[c] += t;
        if (arow) arow[c] += fabs(t);
      }
    }
  }
}

/*
 * The COO form the reference's LBSpMM consumes: C += A * B, entry by entry in
 * storage order, padded entries (row 0, col 0, value 0) included
 * (spmm/mm/spmm_kernel.cu:451-476; padding spmm/mm/spmm_common.cpp:220-226).
 * The GPU kernel adds per-warp partial sums with atomics, so its summation
 * order is not defined; this sequential form is one admissible order.
 * C must be zeroed by the caller, as the reference's driver does
 * (test/test_all.cpp:101).
 */
ORACLE_API void oracle_spmm_coo_f32(int64_t K, int64_t nnz_padded, const int32_t* row_idx,
                                    const int32_t* col_idx, const float* vals,
                                    const float* B, float* C) {
  for (int64_t j = 0; j < nnz_padded; ++j) {
    const float v = vals[j];
    const float* brow = B + (int64_t)col_idx[j] * K;
    float* crow = C + (int64_t)row_idx[j] * K;
    for (int64_t c = 0; c < K; ++c) crow[c] = fmaf(v, brow[c], crow[c]);
  }
}

/*
 * SDDMM over the CSR pattern: out[j] = sum_c X[row(j)*K + c] * Y[col[j]*K + c].
 * A's values are not multiplied in.  The reference has no SDDMM code (only the
 * unused ResInfo::sddmm_* fields, include/spmm/mm/spmm_common.h:130-135); the
 * definition is the pattern-masked X * Y^T.
 */
ORACLE_API void oracle_sddmm_csr_f32(int64_t M, int64_t K, const int32_t* row_ptr,
                                     const int32_t* col_idx, const float* X,
                                     const float* Y, float* out) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < M; ++r) {
    const float* xrow = X + r * K;
    for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
      const float* yrow = Y + (int64_t)col_idx[j] * K;
      float acc = 0.0f;
      for (int64_t c = 0; c < K; ++c) acc = fmaf(xrow[c], yrow[c], acc);
      out[j] = acc;
    }
  }
}

ORACLE_API void oracle_sddmm_csr_f64(int64_t M, int64_t K, const int32_t* row_ptr,
                                     const int32_t* col_idx, const float* X,
                                     const float* Y, double* out, double* abs_sum) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < M; ++r) {
    const float* xrow = X + r * K;
    for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
      const float* yrow = Y + (int64_t)col_idx[j] * K;
      double acc = 0.0, aacc = 0.0;
      for (int64_t c = 0; c < K; ++c) {
        const double t = (double)xrow[c] * (double)yrow[c];
        acc += t;
        aacc += fabs(t);
      }
      out[j] = acc;
      if (abs_sum) abs_sum[j] = aacc;
    }
  }
}

/*
 * CSR transpose by counting sort on the column index, stable in storage
 * order, so every row of the transpose lists its entries by ascending source
 * row.  No counterpart in the reference.  perm[t] (optional) is the source
 * position of transposed entry t.
 */
ORACLE_API void oracle_csr_transpose(int64_t M, int64_t N, const int32_t* row_ptr,
                                     const int32_t* col_idx, const float* vals,
                                     int32_t* row_ptr_t, int32_t* col_idx_t, float* vals_t,
                                     int32_t* perm) {
  const int64_t nnz = row_ptr[M];
  memset(row_ptr_t, 0, (size_t)(N + 1) * sizeof(int32_t));
  for (int64_t j = 0; j < nnz; ++j) row_ptr_t[col_idx[j] + 1]++;
  for (int64_t c = 0; c < N; ++c) row_ptr_t[c + 1] += row_ptr_t[c];
  int32_t* cursor = (int32_t*)malloc((size_t)(N > 0 ? N : 1) * sizeof(int32_t));
  memcpy(cursor, row_ptr_t, (size_t)N * sizeof(int32_t));
  for (int64_t r = 0; r < M; ++r) {
    for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
      const int32_t t = cursor[col_idx[j]]++;
      col_idx_t[t] = (int32_t)r;
      if (vals_t) vals_t[t] = vals[j];
      if (perm) perm[t] = (int32_t)j;
    }
  }
  free(cursor);
}

/*
 * CSR -> COO row expansion with padding to a multiple of `padding`
 * (spmm/mm/spmm_common.cpp:210-216 expansion, :220-226 padding with zeros,
 * :179-184 round-up).  Outputs hold nnz_padded entries; returns nnz_padded.
 */
ORACLE_API int64_t oracle_csr_to_coo_padded(int64_t M, const int32_t* row_ptr,
                                            const int32_t* col_idx, const float* vals,
                                            int64_t padding, int32_t* row_out,
                                            int32_t* col_out, float* val_out) {
  const int64_t nnz = row_ptr[M];
  int64_t padded = nnz;
  if (padding > 0 && nnz % padding != 0) padded = nnz + padding - nnz % padding;
  for (int64_t j = 0; j < padded; ++j) {
    row_out[j] = 0;
    col_out[j] = 0;
    val_out[j] = 0.0f;
  }
  for (int64_t r = 0; r < M; ++r)
    for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) row_out[j] = (int32_t)r;
  memcpy(col_out, col_idx, (size_t)nnz * sizeof(int32_t));
  memcpy(val_out, vals, (size_t)nnz * sizeof(float));
  return padded;
}

/*
 * Reordered COO emission: rows are written in the order a permutation names,
 * each keeping its original row id (spmm/mm/spmm_common.cpp:269-277), then
 * padded like the plain form.  Returns nnz_padded.
 */
ORACLE_API int64_t oracle_csr_to_coo_reordered(int64_t M, const int32_t* row_ptr,
                                               const int32_t* col_idx, const float* vals,
                                               const int32_t* row_order, int64_t padding,
                                               int32_t* row_out, int32_t* col_out,
                                               float* val_out) {
  const int64_t nnz = row_ptr[M];
  int64_t padded = nnz;
  if (padding > 0 && nnz % padding != 0) padded = nnz + padding - nnz % padding;
  int64_t t = 0;
  for (int64_t i = 0; i < M; ++i) {
    const int32_t r = row_order[i];
    for (int64_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j, ++t) {
      row_out[t] = r;
      col_out[t] = col_idx[j];
      val_out[t] = vals[j];
    }
  }
  for (; t < padded; ++t) {
    row_out[t] = 0;
    col_out[t] = 0;
    val_out[t] = 0.0f;
  }
  return padded;
}

/*
 * Coefficient of variation of the row lengths, population standard deviation
 * over mean (spmm/mm/spmm_common.cpp:57-67 calCV, :349-374 get_standard_CV).
 */
ORACLE_API double oracle_row_length_cv(int64_t M, const int32_t* row_ptr) {
  if (M <= 0) return 0.0;
  double sum = 0.0;
  for (int64_t r = 0; r < M; ++r) sum += (double)(row_ptr[r + 1] - row_ptr[r]);
  const double mean = sum / (double)M;
  double acc = 0.0;
  for (int64_t r = 0; r < M; ++r) {
    const double d = (double)(row_ptr[r + 1] - row_ptr[r]) - mean;
    acc += d * d;
  }
  return sqrt(acc / (double)M) / mean;
}

/* Throughput figure of the reference's CSV: 2*nnz*K / ms / 1e6
 * (spmm/mm/spmm_common.cpp:24-31). */
ORACLE_API double oracle_gflops(int64_t nnz, int64_t K, double ms) {
  return (double)nnz * (double)K * 2.0 / ms / 1000.0 / 1000.0;
}

/*
 * nnz-balanced contiguous row blocks for G shards: bounds[g] is the first row
 * r with row_ptr[r] >= g*nnz/G (bounds[0] = 0, bounds[G] = M).  No counterpart
 * in the reference, which is single-GPU.
 */
ORACLE_API void oracle_shard_bounds(int64_t M, const int32_t* row_ptr, int32_t G,
                                    int64_t* bounds) {
  const int64_t nnz = row_ptr[M];
  bounds[0] = 0;
  for (int32_t g = 1; g < G; ++g) {
    const int64_t target = (int64_t)(((__int128)nnz * g) / G);
    int64_t r = 0;
    while (r < M && row_ptr[r] < target) ++r;
    bounds[g] = r;
  }
  bounds[G] = M;
}

/* Max absolute-error check of the reference's checker, threshold 0.1, with the
 * optional division by the 200 accumulating launches
 * (spmm/utils/compare.cpp:9-21; include/spmm/utils/timer_cuda.h:4). */
ORACLE_API double oracle_max_abs_err(int64_t n, const float* got, const float* want,
                                     int div_by_launches) {
  double err_max = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    const float g = div_by_launches ? got[i] / (float)200 : got[i];
    const double e = fabs((double)g - (double)want[i]);
    if (e > err_max) err_max = e;
  }
  return err_max;
}
