// Bench driver: successor of the reference's test/test_all.cpp (lines 27-109).
//
//   test_all <graph> <K> [timed_launches] [--force]
//
// <graph> is a .smtx file (the reference's dataset format) or one of the seeded synthetic
// specs  cfg1 | rmat:<scale>[:<edge_factor>[:<seed>]] | er:<rows>:<mean_degree>[:<seed>] .
// Runs the row-split (GE-SpMM shaped) kernel, the nnz-balanced kernel, the COO entry and the
// SDDMM, checks each against a CPU CSR loop when the graph is small, and appends one CSV row to
// ./full_graph_res.csv in the reference's layout (spmm/mm/spmm_common.cpp:34-42).  A (graph, K) pair
// that already has a row there is skipped, so a sweep that was interrupted resumes where it stopped;
// --force measures it again.
#include <cstdio>
#include <cstdlib>
#include <sstream>

#include "spmm/mm/spmm_kernel.h"
#include "spmm/utils/compare.h"
#include "spmm/utils/timer_cpu.h"

static std::vector<std::string> split(const std::string& s, char sep) {
  std::vector<std::string> out;
  std::stringstream ss(s);
  std::string item;
  while (std::getline(ss, item, sep)) out.push_back(item);
  return out;
}

// CSR-order FP32 row loop, the arithmetic of spmm/mm/spmm_kernel.cu:324-346 on the host
static void cpu_csr_spmm(const CSR_Matrix& A, const Matrix& B, Matrix& C) {
  const int64_t M = A.num_rows(), K = B.dim(1);
  const int32_t* rp = A.row_offsets_.data<int32_t>();
  const int32_t* ci = A.column_indices_.data<int32_t>();
  const float* v = A.values_.data<float>();
  const float* b = B.data<float>();
  float* c = C.mutable_data<float>();
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < M; ++r) {
    float* crow = c + r * K;
    for (int64_t x = 0; x < K; ++x) crow[x] = 0.f;
    for (int64_t j = rp[r]; j < rp[r + 1]; ++j) {
      const float* brow = b + (int64_t)ci[j] * K;
      for (int64_t x = 0; x < K; ++x) crow[x] = fmaf(v[j], brow[x], crow[x]);
    }
  }
}

int main(int argc, char** argv) {
  if (argc < 3) {
    std::fprintf(stderr, "usage: %s <graph.smtx | cfg1 | rmat:S[:EF[:seed]] | er:M:deg[:seed]> <K> [launches] [--force]\n", argv[0]);
    return 2;
  }
  try {
    const std::string spec = argv[1];
    const long long k = std::atoll(argv[2]);
    bool force = false;
    int launches = EXE_NUM_CUDA;
    for (int a = 3; a < argc; ++a) {
      if (std::string(argv[a]) == "--force")
        force = true;
      else
        launches = std::atoi(argv[a]);
    }
    if (!force && result_row_present("./full_graph_res.csv", spec, k)) {
      std::cout << spec << " at k = " << k << " is already in ./full_graph_res.csv: skipped (--force measures it again)"
                << std::endl;
      return 0;
    }
    ResInfo info;
    info.filename_ = spec;
    long long num = 0, dim = 0, real_nnz = 0;
    CSR_Matrix h_csr;
    std::vector<std::string> p = split(spec, ':');
    if (spec == "cfg1") {
      h_csr = gen_csr_uniform_degree(4096, 4096, 1, 32, 1);
    } else if (p[0] == "rmat" && p.size() >= 2) {
      h_csr = gen_csr_rmat(std::atoi(p[1].c_str()), p.size() > 2 ? std::atoi(p[2].c_str()) : 16,
                           p.size() > 3 ? std::strtoull(p[3].c_str(), nullptr, 10) : 2);
    } else if (p[0] == "er" && p.size() >= 3) {
      const long long m = std::atoll(p[1].c_str());
      h_csr = gen_csr_erdos_renyi(m, m, std::atof(p[2].c_str()),
                                  p.size() > 3 ? std::strtoull(p[3].c_str(), nullptr, 10) : 3);
    } else {
      h_csr = get_csr_mat_from_smtx(spec, num, dim, real_nnz);
    }
    num = h_csr.num_rows();
    dim = h_csr.num_cols();
    real_nnz = h_csr.num_nonzeros();
    info.stdv = get_standard_CV(h_csr);
    info.num_rows_ = num;
    info.num_cols_ = dim;
    info.dense_dim_ = k;
    info.num_nnz_ = real_nnz;
    std::cout << "row_num: " << num << "\ncol_num: " << dim << "\nk: " << k << "\nnonzero_num: " << real_nnz
              << "\nrow length CV: " << info.stdv << std::endl;

    Matrix dense_mat_cpu = rand({dim, k}, Device(kCPU), DataType(kFloat), -1.0, 1.0, /*seed=*/2, /*stream=*/100 + k);
    Matrix d_dense = dense_mat_cpu.to(kCUDA);
    CSR_Matrix d_csr = csr_to_cuda(h_csr);
    COO_Matrix d_coo = csr_to_coo_cuda(d_csr, 32);
    Matrix d_res_ge = full({num, k}, Device(kCUDA), DataType(kFloat), 0.0);
    Matrix d_res_hp = full({num, k}, Device(kCUDA), DataType(kFloat), 0.0);
    Matrix d_res_coo = full({num, k}, Device(kCUDA), DataType(kFloat), 0.0);

    float t = 0.f;
    // the reference's two CSR / COO entry points by their own names (test/test_all.cpp:91-92, :101-102) ...
    GESpMM(d_csr, d_dense, d_res_ge, t, launches);
    info.spmm_ge_time_ = t;
    // ... the row-split arithmetic of the reference's GESpMM kernels, for the bit-exact check below ...
    Matrix d_res_rs = full({num, k}, Device(kCUDA), DataType(kFloat), 0.0);
    GESpMM_rowsplit(d_csr, d_dense, d_res_rs, t, launches < 3 ? launches : 3, 1);
    // ... and the balanced kernel under its own name
    HPSpMM(d_csr, d_dense, d_res_hp, t, launches);
    info.spmm_hp_time_ = t;
    std::cout << "HP-SpMM time: " << t << " ms" << std::endl;
    fill_matrix(d_res_coo, 0.0f);
    LBSpMM(d_coo, d_dense, d_res_coo, t, launches);
    info.spmm_coo_time_ = t;

    Matrix d_x = rand({num, k}, Device(kCUDA), DataType(kFloat), -1.0, 1.0, 2, 300 + k);
    Matrix d_out = Matrix({real_nnz}, Device(kCUDA), DataType(kFloat));
    HPSDDMM(d_csr, d_x, d_dense, d_out, t, launches);
    info.sddmm_hp_time_ = t;
    std::cout << "HP-SDDMM time: " << t << " ms" << std::endl;

    int rc = 0;
    if ((double)real_nnz * (double)k <= 4.5e9) {
      Matrix c_ref({num, k}, Device(kCPU), DataType(kFloat));
      cpu_csr_spmm(h_csr, dense_mat_cpu, c_ref);  // warm-up
      CpuTimer ct;
      ct.Start();
      for (int i = 0; i < EXE_NUM_CPU; ++i) cpu_csr_spmm(h_csr, dense_mat_cpu, c_ref);
      ct.Stop();
      info.spmm_cpu_time_ = ct.Elapsed() / EXE_NUM_CPU;
      if (ExpectEqualDenseWithError(d_res_rs, c_ref) != 0.0) rc = 1;          // row split: bit exact
      if (ExpectEqualDenseWithError(d_res_ge, c_ref, "", 1e-2) >= 1e-2) rc = 1;
      if (ExpectEqualDenseWithError(d_res_hp, c_ref, "", 1e-2) >= 1e-2) rc = 1;
      if (ExpectEqualDenseWithError(d_res_coo, c_ref, "", 1e-2) >= 1e-2) rc = 1;
    }
    write_info_to_file("./full_graph_res.csv", info);
    return rc;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "test_all: %s\n", e.what());
    return 3;
  }
}
