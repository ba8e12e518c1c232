// Layer handle for the caller either side of the product: one aggregation layer of a GNN.
//   forward            C  = A  · H          (CSR SpMM, cached plan)
//   backward, features dH = Aᵀ · dC         (SpMM on the device-built transpose, cached plan)
//   backward, weights  dA = pattern(A) ⊙ (dC · Hᵀ)   (SDDMM, same plan as forward)
// The reference has no such layer: its driver calls one product at a time
// (test/test_all.cpp:63-107) and ships neither a transpose nor an SDDMM.  What the
// handle owns is what a training loop would otherwise rebuild every step: the two
// chunk tables, Aᵀ, and the permutation that carries new edge weights into Aᵀ.
#include <new>

#include "hpspmm_internal.h"

struct hpspmm_layer {
  int device;
  int64_t M, N, nnz, max_K;
  // borrowed from the caller
  const int32_t* row_ptr;
  const int32_t* col_idx;
  const float* vals;
  // owned: Aᵀ as CSR (N rows), source position of every transposed entry, plans
  int32_t* row_ptr_t;
  int32_t* col_idx_t;
  float* vals_t;
  int32_t* perm;
  // chunk tables per width class (K <= 32, <= 64, wider): the best chunk size depends on K.
  // The class of max_K is built by create, the others on first use.
  hpspmm_plan* plan[3];
  hpspmm_plan* plan_t[3];
  size_t bytes;
};

namespace {

constexpr int kThreads = 256;

__global__ void gather_by_perm_kernel(int64_t n, const int* __restrict__ perm, const float* __restrict__ src,
                                      float* __restrict__ dst) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += stride)
    dst[t] = __ldg(src + perm[t]);
}

void release(hpspmm_ctx* ctx, hpspmm_layer* g) {
  if (!g) return;
  for (int i = 0; i < 3; ++i) {
    if (g->plan[i]) hpspmm_plan_destroy(ctx, g->plan[i]);
    if (g->plan_t[i]) hpspmm_plan_destroy(ctx, g->plan_t[i]);
  }
  cudaFree(g->row_ptr_t);
  cudaFree(g->col_idx_t);
  cudaFree(g->vals_t);
  cudaFree(g->perm);
  delete g;
}

int width_class(int64_t K) { return K <= 32 ? 0 : (K <= 64 ? 1 : 2); }

// plans of A and of its transpose for the width class of K, built on first use
int plans_for(hpspmm_ctx* ctx, hpspmm_layer* g, int64_t K, hpspmm_stream stream, int* cls_out) {
  const int cls = width_class(K);
  *cls_out = cls;
  if (g->plan[cls] && g->plan_t[cls]) return HPSPMM_OK;
  const int64_t width = cls == 0 ? 32 : (cls == 1 ? 64 : g->max_K);
  int st = HPSPMM_OK;
  if (!g->plan[cls])
    st = hpspmm_plan_create(ctx, g->M, g->N, g->nnz, g->row_ptr, g->col_idx, width, nullptr, stream, &g->plan[cls]);
  if (st == HPSPMM_OK && !g->plan_t[cls])
    st = hpspmm_plan_create(ctx, g->N, g->M, g->nnz, g->row_ptr_t, g->col_idx_t, width, nullptr, stream,
                            &g->plan_t[cls]);
  if (st == HPSPMM_OK) g->bytes += g->plan[cls]->bytes + g->plan_t[cls]->bytes;
  return st;
}

}  // namespace

extern "C" {

int hpspmm_layer_create(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz, const int32_t* row_ptr,
                        const int32_t* col_idx, const float* vals, int64_t max_K, hpspmm_stream stream,
                        hpspmm_layer** out) {
  HPSPMM_TRACE("hpspmm_layer_create");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && out != nullptr, "null context or output");
  *out = nullptr;
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0 && max_K >= 1, "bad size");
  HPSPMM_REQUIRE(ctx, row_ptr != nullptr && (nnz == 0 || (col_idx != nullptr && vals != nullptr)),
                 "null pointer");
  if (M > 2147483646ll || N > 2147483646ll || nnz > 2147483647ll - 4096) return HPSPMM_ERR_UNSUPPORTED;
  hpspmm_device_guard guard(ctx->device);
  hpspmm_layer* g = new (std::nothrow) hpspmm_layer();
  if (!g) return HPSPMM_ERR_OOM;
  memset(g, 0, sizeof(*g));
  g->device = ctx->device;
  g->M = M;
  g->N = N;
  g->nnz = nnz;
  g->max_K = max_K;
  g->row_ptr = row_ptr;
  g->col_idx = col_idx;
  g->vals = vals;
  const size_t b_rp = (size_t)(N + 1) * 4, b_e = (size_t)(nnz > 0 ? nnz : 1) * 4;
  cudaError_t e = hpspmm_device_malloc((void**)&g->row_ptr_t, b_rp);
  if (e == cudaSuccess) e = hpspmm_device_malloc((void**)&g->col_idx_t, b_e);
  if (e == cudaSuccess) e = hpspmm_device_malloc((void**)&g->vals_t, b_e);
  if (e == cudaSuccess) e = hpspmm_device_malloc((void**)&g->perm, b_e);
  if (e != cudaSuccess) {
    release(ctx, g);
    return hpspmm_set_err(ctx, HPSPMM_ERR_OOM, "layer cudaMalloc", e);
  }
  g->bytes = b_rp + 3 * b_e;
  int st = hpspmm_csr_transpose(ctx, M, N, nnz, row_ptr, col_idx, vals, g->row_ptr_t, g->col_idx_t,
                                vals ? g->vals_t : nullptr, g->perm, stream);
  int cls = 0;
  if (st == HPSPMM_OK) st = plans_for(ctx, g, max_K, stream, &cls);
  if (st != HPSPMM_OK) {
    release(ctx, g);
    return st;
  }
  *out = g;
  return HPSPMM_OK;
}

int hpspmm_layer_destroy(hpspmm_ctx* ctx, hpspmm_layer* g) {
  if (!g) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  hpspmm_device_guard guard(g->device);
  release(ctx, g);
  return HPSPMM_OK;
}

int hpspmm_layer_info(const hpspmm_layer* g, int64_t* M, int64_t* N, int64_t* nnz, int64_t* max_K,
                      int64_t* owned_bytes) {
  if (!g) return HPSPMM_ERR_INVALID;
  if (M) *M = g->M;
  if (N) *N = g->N;
  if (nnz) *nnz = g->nnz;
  if (max_K) *max_K = g->max_K;
  if (owned_bytes) *owned_bytes = (int64_t)g->bytes;
  return HPSPMM_OK;
}

int hpspmm_layer_transposed(const hpspmm_layer* g, const int32_t** row_ptr_t, const int32_t** col_idx_t,
                            const float** vals_t, const int32_t** perm) {
  if (!g) return HPSPMM_ERR_INVALID;
  if (row_ptr_t) *row_ptr_t = g->row_ptr_t;
  if (col_idx_t) *col_idx_t = g->col_idx_t;
  if (vals_t) *vals_t = g->vals_t;
  if (perm) *perm = g->perm;
  return HPSPMM_OK;
}

int hpspmm_layer_forward(hpspmm_ctx* ctx, hpspmm_layer* g, int64_t K, const float* H, float* C,
                         hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_layer_forward");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && g != nullptr, "null context or layer");
  HPSPMM_REQUIRE(ctx, K >= 1 && K <= g->max_K, "K outside [1, max_K] of the layer");
  int cls;
  const int st = plans_for(ctx, g, K, stream, &cls);
  if (st != HPSPMM_OK) return st;
  return hpspmm_spmm_csr_f32(ctx, g->plan[cls], g->M, g->N, K, g->nnz, g->row_ptr, g->col_idx, g->vals, H, C,
                             nullptr, stream);
}

int hpspmm_layer_backward_features(hpspmm_ctx* ctx, hpspmm_layer* g, int64_t K, const float* dC,
                                   float* dH, hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_layer_backward_features");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && g != nullptr, "null context or layer");
  HPSPMM_REQUIRE(ctx, K >= 1 && K <= g->max_K, "K outside [1, max_K] of the layer");
  int cls;
  const int st = plans_for(ctx, g, K, stream, &cls);
  if (st != HPSPMM_OK) return st;
  return hpspmm_spmm_csr_f32(ctx, g->plan_t[cls], g->N, g->M, K, g->nnz, g->row_ptr_t, g->col_idx_t, g->vals_t, dC,
                             dH, nullptr, stream);
}

int hpspmm_layer_backward_weights(hpspmm_ctx* ctx, hpspmm_layer* g, int64_t K, const float* dC,
                                  const float* H, float* dA, hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_layer_backward_weights");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && g != nullptr, "null context or layer");
  HPSPMM_REQUIRE(ctx, K >= 1 && K <= g->max_K, "K outside [1, max_K] of the layer");
  int cls;
  const int st = plans_for(ctx, g, K, stream, &cls);
  if (st != HPSPMM_OK) return st;
  return hpspmm_sddmm_csr_f32(ctx, g->plan[cls], g->M, g->N, K, g->nnz, g->row_ptr, g->col_idx, dC, H, dA, nullptr,
                              stream);
}

int hpspmm_layer_update_values(hpspmm_ctx* ctx, hpspmm_layer* g, const float* vals, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr && g != nullptr, "null context or layer");
  HPSPMM_REQUIRE(ctx, g->nnz == 0 || vals != nullptr, "null values");
  g->vals = vals;
  if (g->nnz == 0) return HPSPMM_OK;
  hpspmm_device_guard guard(g->device);
  int64_t blocks = (g->nnz + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)ctx->sm_count * 32;
  if (blocks > cap) blocks = cap;
  gather_by_perm_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(g->nnz, g->perm, vals,
                                                                                g->vals_t);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

}  // extern "C"
