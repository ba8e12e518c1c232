// FP32 SDDMM over a CSR pattern for sm_100a: out[j] = dot(X[row(j), :], Y[col[j], :]).
//
// The reference names SDDMM but ships no code for it (only the unused ResInfo::sddmm_*
// fields, include/spmm/mm/spmm_common.h:130-135).  The kernel reuses the nnz-balanced
// chunk table of the SpMM: a sub-warp of W = K/4 lanes owns one chunk, keeps its
// fragment of the current row of X in registers, gathers fragments of rows of Y as
// float4, and reduces U = 8 partial dot products across the sub-warp at once with a
// transposing butterfly (7 shuffles for 8 results instead of 8 * log2(W)).
#include "device_utils.cuh"
#include "hpspmm_internal.h"

namespace {

using namespace hpspmm;

constexpr int kBlockThreads = 256;

__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  acc = fmaf(a.w, b.w, acc);
  return acc;
}

// Row holding entry j, searching upward from `row` (entry j lies beyond the end of `row`).
__device__ __forceinline__ void next_row(const int* __restrict__ row_ptr, int M, int j, int& row,
                                         int& row_end) {
  ++row;
  int e = __ldg(row_ptr + row + 1);
  int probes = 0;
  while (e <= j) {
    if (++probes == 8) {
      int lo = row + 1, hi = M + 1;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(row_ptr + mid) <= j)
          lo = mid + 1;
        else
          hi = mid;
      }
      row = lo - 1;
      e = __ldg(row_ptr + row + 1);
      break;
    }
    ++row;
    e = __ldg(row_ptr + row + 1);
  }
  row_end = e;
}

// Sums p[0..7] over each group of 8 adjacent lanes; on return p[0] of lane l holds the
// group total of the value whose index is the 3-bit reversal of (l & 7).
__device__ __forceinline__ void reduce8_transposed(float (&p)[8], unsigned mask, int lane) {
  {
    const bool up = lane & 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float send = up ? p[i] : p[i + 4];
      const float keep = up ? p[i + 4] : p[i];
      p[i] = keep + __shfl_xor_sync(mask, send, 1);
    }
  }
  {
    const bool up = lane & 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = up ? p[i] : p[i + 2];
      const float keep = up ? p[i + 2] : p[i];
      p[i] = keep + __shfl_xor_sync(mask, send, 2);
    }
  }
  {
    const bool up = lane & 4;
    const float send = up ? p[0] : p[1];
    const float keep = up ? p[1] : p[0];
    p[0] = keep + __shfl_xor_sync(mask, send, 4);
  }
}

__device__ __forceinline__ int bitrev3(int x) { return ((x & 1) << 2) | (x & 2) | ((x >> 2) & 1); }

template <int W, int R, bool HINT>
__global__ void __launch_bounds__(kBlockThreads)
sddmm_balanced_kernel(int M, int n_chunks, const int* __restrict__ row_ptr,
                      const int* __restrict__ col_idx, const float* __restrict__ X,
                      const float* __restrict__ Y, float* __restrict__ out,
                      const int* __restrict__ chunk_start, const int* __restrict__ chunk_row) {
  constexpr int K = 4 * W * R;
  constexpr int U = 8;
  const int lane = threadIdx.x & (W - 1);
  const int worker = (int)(((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) / W);
  if (worker >= n_chunks) return;
  const unsigned mask = subwarp_mask<W>();
  const uint64_t policy = policy_evict_last();

  const int n0 = __ldg(chunk_start + worker);
  const int n1 = __ldg(chunk_start + worker + 1);
  int row = __ldg(chunk_row + worker);
  int row_end = __ldg(row_ptr + row + 1);

  float4 x[R];
  auto load_x = [&]() {
    const float* xr = X + (int64_t)row * K + lane * 4;
#pragma unroll
    for (int r = 0; r < R; ++r) x[r] = __ldg(reinterpret_cast<const float4*>(xr + r * W * 4));
  };
  load_x();
  const float* Yl = Y + lane * 4;

  for (int base = n0; base < n1; base += W) {
    const int jj = base + lane;
    int mycol = 0;
    if (jj < n1) mycol = ld_stream(col_idx + jj);
#pragma unroll 1
    for (int u0 = 0; u0 < W; u0 += U) {
      const int j0 = base + u0;
      if (j0 >= n1) break;
      const int cnt = min(U, n1 - j0);
      float4 y[U][R];
#pragma unroll
      for (int i = 0; i < U; ++i) {
        const int c = __shfl_sync(mask, mycol, u0 + i, W);  // lanes past n1 hold column 0
        const float* p = Yl + (int64_t)c * K;
#pragma unroll
        for (int r = 0; r < R; ++r) y[i][r] = ld_gather<HINT>(p + r * W * 4, policy);
      }
      float part[U];
#pragma unroll
      for (int i = 0; i < U; ++i) {
        if (i < cnt && j0 + i >= row_end) {
          next_row(row_ptr, M, j0 + i, row, row_end);
          load_x();
        }
        float s = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) s = dot4(x[r], y[i][r], s);
        part[i] = s;
      }
      reduce8_transposed(part, mask, lane);
      float total = part[0];
      if (W >= 16) total += __shfl_xor_sync(mask, total, 8);
      if (W >= 32) total += __shfl_xor_sync(mask, total, 16);
      const int slot = bitrev3(lane & 7);
      if (lane < 8 && slot < cnt) out[j0 + slot] = total;
    }
  }
}

// Any K: one warp per chunk, one entry at a time, lanes stride over the columns.
template <int VEC>
__global__ void __launch_bounds__(kBlockThreads)
sddmm_generic_kernel(int M, int K, int n_chunks, const int* __restrict__ row_ptr,
                     const int* __restrict__ col_idx, const float* __restrict__ X,
                     const float* __restrict__ Y, float* __restrict__ out,
                     const int* __restrict__ chunk_start, const int* __restrict__ chunk_row) {
  const int lane = threadIdx.x & 31;
  const int worker = (int)(((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) >> 5);
  if (worker >= n_chunks) return;
  const int n0 = __ldg(chunk_start + worker);
  const int n1 = __ldg(chunk_start + worker + 1);
  int row = __ldg(chunk_row + worker);
  int row_end = __ldg(row_ptr + row + 1);
  for (int j = n0; j < n1; ++j) {
    if (j >= row_end) next_row(row_ptr, M, j, row, row_end);
    const float* xr = X + (int64_t)row * K;
    const float* yr = Y + (int64_t)__ldg(col_idx + j) * K;
    float s = 0.f;
    if (VEC == 4) {
      for (int c = lane * 4; c < K; c += 128) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(xr + c));
        const float4 b = __ldg(reinterpret_cast<const float4*>(yr + c));
        s = dot4(a, b, s);
      }
    } else {
      for (int c = lane; c < K; c += 32) s = fmaf(__ldg(xr + c), __ldg(yr + c), s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[j] = s;
  }
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <int W, int R>
void launch_sddmm(bool hint, int M, int n_chunks, const int32_t* row_ptr, const int32_t* col_idx,
                  const float* X, const float* Y, float* out, const int32_t* chunk_start,
                  const int32_t* chunk_row, cudaStream_t s) {
  const int wpb = kBlockThreads / W;
  const unsigned grid = (unsigned)((n_chunks + wpb - 1) / wpb);
  if (hint)
    sddmm_balanced_kernel<W, R, true><<<grid, kBlockThreads, 0, s>>>(
        M, n_chunks, row_ptr, col_idx, X, Y, out, chunk_start, chunk_row);
  else
    sddmm_balanced_kernel<W, R, false><<<grid, kBlockThreads, 0, s>>>(
        M, n_chunks, row_ptr, col_idx, X, Y, out, chunk_start, chunk_row);
}

}  // namespace

extern "C" int hpspmm_sddmm_csr_f32(hpspmm_ctx* ctx, const hpspmm_plan* plan, int64_t M, int64_t N,
                                    int64_t K, int64_t nnz, const int32_t* row_ptr,
                                    const int32_t* col_idx, const float* X, const float* Y,
                                    float* out_vals, const hpspmm_opts* opts,
                                    hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0, "negative size");
  HPSPMM_REQUIRE(ctx, K >= 1, "K must be >= 1");
  if (M > 2147483646ll || N > 2147483647ll || nnz > 2147483647ll || K > (1 << 20)) {
    snprintf(ctx->err, sizeof(ctx->err), "sizes beyond 32-bit CSR indices");
    return HPSPMM_ERR_UNSUPPORTED;
  }
  if (nnz == 0 || M == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, row_ptr && col_idx && X && Y && out_vals, "null operand");
  if ((K & 3) == 0 && (((uintptr_t)X & 15u) || ((uintptr_t)Y & 15u))) {
    snprintf(ctx->err, sizeof(ctx->err), "dense operands must be 16-byte aligned");
    return HPSPMM_ERR_INVALID;
  }
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  const int hint_mode = opts ? opts->b_l2_hint : 0;
  const bool hint = hint_mode == 2 || (hint_mode == 0 && K >= 64);
  const int32_t* chunk_start;
  const int32_t* chunk_row;
  int64_t n_chunks;
  if (plan) {
    HPSPMM_REQUIRE(ctx, plan->M == M && plan->nnz == nnz, "plan built for another matrix");
    HPSPMM_REQUIRE(ctx, plan->device == ctx->device, "plan built on another device");
    chunk_start = plan->chunk_start;
    chunk_row = plan->chunk_row;
    n_chunks = plan->n_chunks;
  } else {
    int32_t S = (opts && opts->chunk_nnz > 0) ? opts->chunk_nnz : hpspmm_default_chunk_nnz(K);
    S = (S + 31) / 32 * 32;
    n_chunks = (nnz + S - 1) / S;
    const size_t b_int = align_up((size_t)(n_chunks + 1) * 4, 256);
    int st = hpspmm_ensure_scratch(ctx, 2 * b_int);
    if (st != HPSPMM_OK) return st;
    int32_t* cs = (int32_t*)ctx->scratch;
    int32_t* cr = (int32_t*)((char*)ctx->scratch + b_int);
    st = hpspmm_launch_chunk_table(ctx, M, nnz, row_ptr, S, n_chunks, cs, cr, nullptr, s);
    if (st != HPSPMM_OK) return st;
    chunk_start = cs;
    chunk_row = cr;
  }
  const int m = (int)M, nc = (int)n_chunks;
  if (K == 32) {
    launch_sddmm<8, 1>(hint, m, nc, row_ptr, col_idx, X, Y, out_vals, chunk_start, chunk_row, s);
  } else if (K == 64) {
    launch_sddmm<16, 1>(hint, m, nc, row_ptr, col_idx, X, Y, out_vals, chunk_start, chunk_row, s);
  } else if (K == 128) {
    launch_sddmm<32, 1>(hint, m, nc, row_ptr, col_idx, X, Y, out_vals, chunk_start, chunk_row, s);
  } else {
    const unsigned grid = (unsigned)((n_chunks + kBlockThreads / 32 - 1) / (kBlockThreads / 32));
    if ((K & 3) == 0)
      sddmm_generic_kernel<4><<<grid, kBlockThreads, 0, s>>>(m, (int)K, nc, row_ptr, col_idx, X, Y,
                                                             out_vals, chunk_start, chunk_row);
    else
      sddmm_generic_kernel<1><<<grid, kBlockThreads, 0, s>>>(m, (int)K, nc, row_ptr, col_idx, X, Y,
                                                             out_vals, chunk_start, chunk_row);
  }
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}
