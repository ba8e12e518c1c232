// Sparse containers, transfers, seeded generators and the CSV result row for the SpMM path.
// Mirrors the call surface of the reference's include/spmm/mm/spmm_common.h:58-164 on top of the
// C ABI; the `.smtx` loaders keep their names, the dataset files are replaced for benchmarking
// by seeded synthetic generators (uniform degree, Erdos-Renyi, R-MAT).
#pragma once
#include <cmath>
#include <fstream>
#include <sstream>
#include <iostream>
#include <string>
#include <vector>

#include "spmm/utils/timer_cuda.h"
#include "starml/basic/matrix.h"
#include "starml/operators/factories.h"

using namespace starml;

class CSR_Matrix {
 public:
  int64_t num_rows_ = 0, num_cols_ = 0, num_nonzeros_ = 0;
  Matrix row_offsets_, column_indices_, values_;
  Matrix row_offsets() const { return row_offsets_; }
  Matrix column_indices() const { return column_indices_; }
  Matrix values() const { return values_; }
  int64_t num_rows() const { return num_rows_; }
  int64_t num_cols() const { return num_cols_; }
  int64_t num_nonzeros() const { return num_nonzeros_; }
};

// num_nonzeros_ is the UNPADDED count; values().size() is the padded one (the reference is
// inconsistent between its two loaders, spmm/mm/spmm_common.cpp:233 vs :294; kernels use
// values().size(), spmm/mm/spmm_kernel.cu:742, and so do the wrappers here).
class COO_Matrix {
 public:
  int64_t num_rows_ = 0, num_cols_ = 0, num_nonzeros_ = 0;
  Matrix row_indices_, column_indices_, values_;
  Matrix row_indices() const { return row_indices_; }
  Matrix column_indices() const { return column_indices_; }
  Matrix values() const { return values_; }
  int64_t num_rows() const { return num_rows_; }
  int64_t num_cols() const { return num_cols_; }
  int64_t num_nonzeros() const { return num_nonzeros_; }
};

// One CSV row per run; the SpMM fields of the reference's ResInfo (spmm_common.h:111-141) plus
// the SDDMM fields it declares but never fills.
struct ResInfo {
  std::string filename_;
  float spmm_ge_time_ = 0.f, spmm_ge_throughput_ = 0.f;   // row-split kernel (GESpMM shape)
  float spmm_hp_time_ = 0.f, spmm_hp_throughput_ = 0.f;   // nnz-balanced kernel
  float spmm_coo_time_ = 0.f, spmm_coo_throughput_ = 0.f; // LBSpMM-compatible COO entry
  float sddmm_hp_time_ = 0.f, sddmm_hp_throughput_ = 0.f;
  float spmm_cpu_time_ = 0.f, spmm_cpu_throughput_ = 0.f; // filled by callers that time a CPU loop
  int64_t num_rows_ = 0, num_cols_ = 0, num_nnz_ = 0, dense_dim_ = 0;
  double stdv = 0.0;
};

namespace hpspmm {

inline CSR_Matrix csr_from_graph(hpspmm_graph* g) {
  int64_t M = 0, N = 0, nnz = 0;
  hpspmm_gen_shape(g, &M, &N, &nnz);
  CSR_Matrix m;
  m.num_rows_ = M;
  m.num_cols_ = N;
  m.num_nonzeros_ = nnz;
  m.row_offsets_ = Matrix({M + 1}, Device(kCPU), DataType(kInt32));
  m.column_indices_ = Matrix({nnz}, Device(kCPU), DataType(kInt32));
  m.values_ = Matrix({nnz}, Device(kCPU), DataType(kFloat));
  hpspmm_gen_export(g, m.row_offsets_.mutable_data<int32_t>(),
                    nnz ? m.column_indices_.mutable_data<int32_t>() : nullptr,
                    nnz ? m.values_.mutable_data<float>() : nullptr);
  hpspmm_gen_free(g);
  return m;
}

}  // namespace hpspmm

// ---- inputs ---------------------------------------------------------------------------------
// .smtx text format (reference: spmm/mm/spmm_common.cpp:125-174), parsed once.
inline CSR_Matrix get_csr_mat_from_smtx(const std::string& filename, long long& num, long long& dim,
                                        long long& real_nonezero_num) {
  hpspmm_graph* g = nullptr;
  const int st = hpspmm_read_smtx(filename.c_str(), &g);
  if (st != HPSPMM_OK) throw hpspmm::Error(st, "cannot read " + filename);
  CSR_Matrix m = hpspmm::csr_from_graph(g);
  num = m.num_rows_;
  dim = m.num_cols_;
  real_nonezero_num = m.num_nonzeros_;
  return m;
}

// small benchmark configuration: per-row degree uniform in [deg_lo, deg_hi], values U(-1,1)
inline CSR_Matrix gen_csr_uniform_degree(int64_t M, int64_t N, int deg_lo, int deg_hi, uint64_t seed) {
  hpspmm_graph* g = nullptr;
  const int st = hpspmm_gen_uniform_degree(M, N, deg_lo, deg_hi, seed, HPSPMM_VALS_UPM1, &g);
  if (st != HPSPMM_OK) throw hpspmm::Error(st, "hpspmm_gen_uniform_degree");
  return hpspmm::csr_from_graph(g);
}
// uniform sparse configuration: Poisson(mean_degree) degrees, values U(0,1)
inline CSR_Matrix gen_csr_erdos_renyi(int64_t M, int64_t N, double mean_degree, uint64_t seed) {
  hpspmm_graph* g = nullptr;
  const int st = hpspmm_gen_erdos_renyi(M, N, mean_degree, seed, HPSPMM_VALS_U01, &g);
  if (st != HPSPMM_OK) throw hpspmm::Error(st, "hpspmm_gen_erdos_renyi");
  return hpspmm::csr_from_graph(g);
}
// power-law configurations: symmetric R-MAT (0.57, 0.19, 0.19, 0.05), values U(0,1)
inline CSR_Matrix gen_csr_rmat(int scale, int edge_factor, uint64_t seed) {
  hpspmm_graph* g = nullptr;
  const int st = hpspmm_gen_rmat(scale, edge_factor, 0.57, 0.19, 0.19, seed, HPSPMM_VALS_U01, &g);
  if (st != HPSPMM_OK) throw hpspmm::Error(st, "hpspmm_gen_rmat");
  return hpspmm::csr_from_graph(g);
}

// ---- transfers (reference: spmm/mm/spmm_common.cpp:377-416) ------------------------------------
inline CSR_Matrix csr_to_cuda(const CSR_Matrix& h) {
  CSR_Matrix d = h;
  d.row_offsets_ = h.row_offsets_.to(kCUDA);
  d.column_indices_ = h.column_indices_.to(kCUDA);
  d.values_ = h.values_.to(kCUDA);
  return d;
}
inline CSR_Matrix csr_to_host(const CSR_Matrix& d) {
  CSR_Matrix h = d;
  h.row_offsets_ = d.row_offsets_.to(kCPU);
  h.column_indices_ = d.column_indices_.to(kCPU);
  h.values_ = d.values_.to(kCPU);
  return h;
}
inline COO_Matrix coo_to_cuda(const COO_Matrix& h) {
  COO_Matrix d = h;
  d.row_indices_ = h.row_indices_.to(kCUDA);
  d.column_indices_ = h.column_indices_.to(kCUDA);
  d.values_ = h.values_.to(kCUDA);
  return d;
}
inline COO_Matrix coo_to_host(const COO_Matrix& d) {
  COO_Matrix h = d;
  h.row_indices_ = d.row_indices_.to(kCPU);
  h.column_indices_ = d.column_indices_.to(kCPU);
  h.values_ = d.values_.to(kCPU);
  return h;
}

// Device CSR -> device COO padded to a multiple of `padding` (the reference does this with
// host loops while loading, spmm/mm/spmm_common.cpp:210-226).
inline COO_Matrix csr_to_coo_cuda(const CSR_Matrix& d_csr, int padding) {
  const int64_t padded = hpspmm_padded_nnz(d_csr.num_nonzeros_, padding);
  COO_Matrix c;
  c.num_rows_ = d_csr.num_rows_;
  c.num_cols_ = d_csr.num_cols_;
  c.num_nonzeros_ = d_csr.num_nonzeros_;
  c.row_indices_ = Matrix({padded}, Device(kCUDA), DataType(kInt32));
  c.column_indices_ = Matrix({padded}, Device(kCUDA), DataType(kInt32));
  c.values_ = Matrix({padded}, Device(kCUDA), DataType(kFloat));
  if (padded > 0) {
    hpspmm_ctx* ctx = hpspmm::context(0);
    hpspmm::check(hpspmm_csr_to_coo_padded(ctx, d_csr.num_rows_, d_csr.num_nonzeros_,
                                           d_csr.row_offsets_.data<int32_t>(),
                                           d_csr.column_indices_.data<int32_t>(),
                                           d_csr.values_.data<float>(), padding,
                                           c.row_indices_.mutable_data<int32_t>(),
                                           c.column_indices_.mutable_data<int32_t>(),
                                           c.values_.mutable_data<float>(), nullptr), "csr_to_coo_padded");
    hpspmm::check(hpspmm_stream_sync(ctx, nullptr), "sync");
  }
  return c;
}

// Row-length coefficient of variation of a host CSR (reference: get_standard_CV re-parses the
// file, spmm/mm/spmm_common.cpp:349-374; the formula is calCV, :57-67).
inline double get_standard_CV(const CSR_Matrix& h_csr) {
  return hpspmm_row_length_cv(h_csr.num_rows_, h_csr.row_offsets_.data<int32_t>());
}

// Appends one CSV row: file,M,N,nnz,K,rowlenCV, then label,ms,GFLOPS triples
// (reference: spmm/mm/spmm_common.cpp:22-44; GFLOPS = 2*nnz*K/ms/1e6 with the unpadded nnz).
// True when `filename` already holds a row for this graph and dense width (columns 1 and 5 of the layout
// below).  The reference's harness appends blindly (spmm/mm/spmm_common.cpp:33), so a sweep restarted after a
// failure measures everything again; a driver can ask first and skip what is there.
inline bool result_row_present(const std::string& filename, const std::string& graph, long long dense_dim) {
  std::ifstream f(filename);
  std::string line;
  while (std::getline(f, line)) {
    std::vector<std::string> col;
    std::stringstream ss(line);
    std::string item;
    while (std::getline(ss, item, ',')) col.push_back(item);
    if (col.size() > 4 && col[0] == graph && std::atoll(col[4].c_str()) == dense_dim) return true;
  }
  return false;
}

inline void write_info_to_file(const std::string& filename, ResInfo& info) {
  auto tp = [&](float ms) { return ms > 0.f ? (float)hpspmm_gflops(info.num_nnz_, info.dense_dim_, ms) : 0.f; };
  info.spmm_ge_throughput_ = tp(info.spmm_ge_time_);
  info.spmm_hp_throughput_ = tp(info.spmm_hp_time_);
  info.spmm_coo_throughput_ = tp(info.spmm_coo_time_);
  info.sddmm_hp_throughput_ = tp(info.sddmm_hp_time_);
  info.spmm_cpu_throughput_ = tp(info.spmm_cpu_time_);
  std::ofstream f(filename, std::ios::app);
  f << info.filename_ << "," << info.num_rows_ << "," << info.num_cols_ << "," << info.num_nnz_ << ","
    << info.dense_dim_ << "," << info.stdv
    << ",GE-SpMM: ," << info.spmm_ge_time_ << "," << info.spmm_ge_throughput_
    << ",HP-SpMM ," << info.spmm_hp_time_ << "," << info.spmm_hp_throughput_
    << ",HP-SpMM(COO): ," << info.spmm_coo_time_ << "," << info.spmm_coo_throughput_
    << ",HP-SDDMM: ," << info.sddmm_hp_time_ << "," << info.sddmm_hp_throughput_
    << ",CPU CSR loop: ," << info.spmm_cpu_time_ << "," << info.spmm_cpu_throughput_ << std::endl;
}
