// FP32 SDDMM over a CSR pattern for sm_100a: out[j] = dot(X[row(j), :], Y[col[j], :]).
//
// The reference names SDDMM but ships no code for it (only the unused ResInfo::sddmm_*
// fields, include/spmm/mm/spmm_common.h:130-135).  The kernels reuse the nnz-balanced chunk
// table of the SpMM (one warp per chunk); A's values are not multiplied in.
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

// ---- warp kernel: one warp per chunk, G = 32/W interleaved lane groups, K = 4 * W --------
// Same shape as the SpMM warp kernel: (col) tiles of 32 entries staged in shared memory with
// asynchronous copies; in every step group g takes entry G*s+g and gathers its float4 of that
// row of Y, U = 4 steps at a time.  The fragment of the current row of X stays in registers;
// row changes are warp-uniform.  The four partial dot products of a batch are reduced across
// the W lanes of each group with a transposing butterfly (4 shuffles for 4 results at W = 8).

// Sums p[0..3] over each group of 4 adjacent lanes; afterwards p[0] of lane l holds the total
// of the value whose index is the 2-bit reversal of (l & 3).
__device__ __forceinline__ void reduce4_transposed(float (&p)[4], int lane) {
  {
    const bool up = lane & 1;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = up ? p[i] : p[i + 2];
      const float keep = up ? p[i + 2] : p[i];
      p[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
    }
  }
  {
    const bool up = lane & 2;
    const float send = up ? p[0] : p[1];
    const float keep = up ? p[1] : p[0];
    p[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
}

// SLAB = 0: X and Y are 4 * W columns wide.  SLAB = 1 / 2: the kernel covers a slab of 4 * W columns of wider
// X and Y (row stride ld); 1 writes the partial dot products, 2 adds them to what earlier slabs wrote.
// When a row ends the kernel steps to the next row that holds entries through the list nz_id / nz_end (chunk_ri:
// position in that list of the row holding a chunk's first entry), so it never looks at an empty row.
// resident 64-thread blocks per SM the kernel is compiled for: 20 (48 registers) measured 0.193 / 0.318 /
// 0.542 ms at K = 32 / 64 / 128 on the R-MAT scale-20 graph against 0.204 / 0.318 / 0.555 ms at 18 (56 registers)
#ifndef HPSPMM_SDDMM_MINB
#define HPSPMM_SDDMM_MINB 20
#endif
template <int W, bool HINT, int BT, int SLAB>
__global__ void __launch_bounds__(BT, HPSPMM_SDDMM_MINB)
sddmm_warp_kernel(int M, int n_chunks, const int* __restrict__ row_ptr,
                  const int* __restrict__ col_idx, const float* __restrict__ X,
                  const float* __restrict__ Y, float* __restrict__ out,
                  const int* __restrict__ chunk_start, const int* __restrict__ chunk_row,
                  const int* __restrict__ chunk_order, int ld, const int* __restrict__ nz_id,
                  const int* __restrict__ nz_end, const int* __restrict__ chunk_ri) {
  const int64_t K = SLAB ? (int64_t)ld : (int64_t)(4 * W);
  constexpr int G = 32 / W;
  constexpr int T = 32;
  constexpr int U = 4;
  constexpr int BATCH = U * G;
  constexpr int STAGES = 2;
  static_assert(T % BATCH == 0, "batch must tile the staged tile");
  __shared__ int tiles[BT / 32][STAGES][T];

  const int lane = threadIdx.x & 31;
  const int g = lane / W;
  const int l = lane % W;
  const int slot = (int)(((int64_t)blockIdx.x * BT + threadIdx.x) >> 5);
  if (slot >= n_chunks) return;
  const int chunk = chunk_order != nullptr ? __ldg(chunk_order + slot) : slot;
  const uint64_t policy = HINT ? policy_evict_last() : 0ull;
  int(*my)[T] = tiles[threadIdx.x >> 5];

  const int n0 = __ldg(chunk_start + chunk);
  const int n1 = __ldg(chunk_start + chunk + 1);
  int ri = __ldg(chunk_ri + chunk);
  int row = __ldg(nz_id + ri);
  int row_end = __ldg(nz_end + ri);

  auto stage_tile = [&](int stage, int base) {
    const int j = base + lane;
    if (j < n1)
      cp_async_4(&my[stage][lane], col_idx + j);
    else
      my[stage][lane] = 0;   // past the chunk: column 0 (a valid row of Y), result discarded
    cp_async_commit();
  };
  stage_tile(0, n0);
  stage_tile(1, n0 + T);

  float4 x = __ldg(reinterpret_cast<const float4*>(X + (int64_t)row * K + l * 4));
  const float* Yl = Y + l * 4;
  // entry `next_entry` starts a later row: find it and fetch its fragment of X
  auto next_x = [&](int next_entry) {
    (void)next_entry;   // the list of rows that hold entries names the row directly
    ++ri;
    row = __ldg(nz_id + ri);
    row_end = __ldg(nz_end + ri);
    x = __ldg(reinterpret_cast<const float4*>(X + (int64_t)row * K + l * 4));
  };

  // reduce the U partial dot products of a batch over the W lanes of each group and store the U * G results
  auto finish_batch = [&](float (&part)[U], int j0) {
    reduce4_transposed(part, lane);
    float total = part[0];
    total += __shfl_xor_sync(0xffffffffu, total, 4);
    if (W >= 16) total += __shfl_xor_sync(0xffffffffu, total, 8);
    if (W >= 32) total += __shfl_xor_sync(0xffffffffu, total, 16);
    const int which = ((l & 1) << 1) | ((l >> 1) & 1);   // which of the U entries lane l holds
    const int j = j0 + which * G + g;
    if (l < 4 && j < n1) out[j] = SLAB == 2 ? out[j] + total : total;
  };

  int stage = 0;
  for (int base = n0; base < n1; base += T) {
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const int* tile = &my[stage][g];
    if (base + T <= n1 && row_end >= base + T) {
      // Fast tile: all 32 entries belong to the current row.  Fully unrolled, every shared-memory offset a
      // compile-time constant, no tests between gathers (two thirds of the tiles of a power-law graph).
#pragma unroll
      for (int u0 = 0; u0 < T; u0 += BATCH) {
        float4 y[U];
#pragma unroll
        for (int i = 0; i < U; ++i) y[i] = ld_gather<HINT>(Yl + (int64_t)tile[u0 + i * G] * K, policy);
        float part[U];
#pragma unroll
        for (int i = 0; i < U; ++i) part[i] = dot4(x, y[i], 0.f);
        finish_batch(part, base + u0);
      }
    } else {
#pragma unroll 1
      for (int u0 = 0; u0 < T; u0 += BATCH) {
        const int j0 = base + u0;
        if (j0 >= n1) break;
        float4 y[U];
#pragma unroll
        for (int i = 0; i < U; ++i) y[i] = ld_gather<HINT>(Yl + (int64_t)tile[u0 + i * G] * K, policy);
        float part[U];
        if (row_end >= j0 + BATCH) {
#pragma unroll
          for (int i = 0; i < U; ++i) part[i] = dot4(x, y[i], 0.f);
        } else {
#pragma unroll
          for (int i = 0; i < U; ++i) {
            const int lo = j0 + i * G;
            const int hi = min(lo + G, n1);
            const int mine = lo + g;
            int cur = lo;
            part[i] = 0.f;
            while (row_end < hi) {   // warp-uniform: the current row ends inside this step
              if (mine >= cur && mine < row_end) part[i] = dot4(x, y[i], 0.f);
              cur = row_end;
              next_x(cur);
            }
            if (mine >= cur) part[i] = dot4(x, y[i], 0.f);
          }
        }
        finish_batch(part, j0);
      }
    }
    __syncwarp();
    stage_tile(stage, base + STAGES * T);
    stage ^= 1;
  }
  cp_async_wait<0>();
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

struct sddmm_row_list {
  const int32_t* nz_id;
  const int32_t* nz_end;
  const int32_t* chunk_ri;
};

template <int W, int SLAB>
void launch_sddmm(bool hint, int M, int n_chunks, const int32_t* row_ptr, const int32_t* col_idx,
                  const float* X, const float* Y, float* out, const int32_t* chunk_start,
                  const int32_t* chunk_row, const int32_t* chunk_order, cudaStream_t s, sddmm_row_list rows,
                  int ld = 4 * W) {
  constexpr int BT = 64;
  const int cpb = BT / 32;
  const unsigned grid = (unsigned)((n_chunks + cpb - 1) / cpb);
#define HPSPMM_SDDMM_LAUNCH(H)                                                                            \
  sddmm_warp_kernel<W, H, BT, SLAB><<<grid, BT, 0, s>>>(M, n_chunks, row_ptr, col_idx, X, Y, out,          \
                                                        chunk_start, chunk_row, chunk_order, ld,          \
                                                        rows.nz_id, rows.nz_end, rows.chunk_ri)
  if (hint) HPSPMM_SDDMM_LAUNCH(true); else HPSPMM_SDDMM_LAUNCH(false);
#undef HPSPMM_SDDMM_LAUNCH
}

}  // namespace

extern "C" int hpspmm_sddmm_csr_f32(hpspmm_ctx* ctx, const hpspmm_plan* plan, int64_t M, int64_t N,
                                    int64_t K, int64_t nnz, const int32_t* row_ptr,
                                    const int32_t* col_idx, const float* X, const float* Y,
                                    float* out_vals, const hpspmm_opts* opts,
                                    hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_sddmm_csr_f32");
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0, "negative size");
  HPSPMM_REQUIRE(ctx, K >= 1, "K must be >= 1");
  if (M > 2147483646ll || N > 2147483647ll || nnz > 2147483647ll - 4096 || K > (1 << 20)) {
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
  const int32_t* chunk_order = nullptr;
  sddmm_row_list rows = {nullptr, nullptr, nullptr};
  int64_t n_chunks;
  if (plan) {
    HPSPMM_REQUIRE(ctx, plan->M == M && plan->nnz == nnz, "plan built for another matrix");
    HPSPMM_REQUIRE(ctx, plan->device == ctx->device, "plan built on another device");
    chunk_start = plan->chunk_start;
    chunk_row = plan->chunk_row;
    chunk_order = plan->chunk_order;
    n_chunks = plan->n_chunks;
    rows = sddmm_row_list{plan->nz_id, plan->nz_end, plan->chunk_ri};
  } else {
    int32_t S = (opts && opts->chunk_nnz > 0) ? opts->chunk_nnz : hpspmm_default_chunk_nnz(K, nnz);
    S = (S + 31) / 32 * 32;
    n_chunks = (nnz + S - 1) / S;
    const size_t b_int = align_up((size_t)(n_chunks + 1) * 4, 256);
    const size_t b_nz = align_up((size_t)(M + 2) * 4, 256);
    const size_t b_sort = hpspmm_order_scratch_bytes(n_chunks), b_list = hpspmm_row_list_scratch_bytes(M);
    int st = hpspmm_ensure_scratch(ctx, 4 * b_int + 2 * b_nz + (b_sort > b_list ? b_sort : b_list));
    if (st != HPSPMM_OK) return st;
    char* sb = (char*)ctx->scratch;
    int32_t* cs = (int32_t*)sb;
    int32_t* cr = (int32_t*)(sb + b_int);
    int32_t* co = (int32_t*)(sb + 2 * b_int);
    int32_t* cri = (int32_t*)(sb + 3 * b_int);
    int32_t* nzi = (int32_t*)(sb + 4 * b_int);
    int32_t* nze = (int32_t*)(sb + 4 * b_int + b_nz);
    void* tmp = sb + 4 * b_int + 2 * b_nz;
    st = hpspmm_launch_chunk_table(ctx, M, nnz, row_ptr, S, n_chunks, cs, cr, nullptr, s, nullptr);
    if (st != HPSPMM_OK) return st;
    st = hpspmm_order_chunks_by_cost(ctx, M, N, n_chunks, row_ptr, nullptr, cs, cr, co, tmp, s);
    if (st != HPSPMM_OK) return st;
    st = hpspmm_build_row_list(ctx, M, n_chunks, row_ptr, cr, nzi, nze, cri, tmp, s);
    if (st != HPSPMM_OK) return st;
    rows = sddmm_row_list{nzi, nze, cri};
    chunk_start = cs;
    chunk_row = cr;
    chunk_order = co;
  }
  const int m = (int)M, nc = (int)n_chunks;
  if (K == 32) {
    launch_sddmm<8, 0>(hint, m, nc, row_ptr, col_idx, X, Y, out_vals, chunk_start, chunk_row, chunk_order, s, rows);
  } else if (K == 64) {
    launch_sddmm<16, 0>(hint, m, nc, row_ptr, col_idx, X, Y, out_vals, chunk_start, chunk_row, chunk_order, s, rows);
  } else if (K == 128) {
    launch_sddmm<32, 0>(hint, m, nc, row_ptr, col_idx, X, Y, out_vals, chunk_start, chunk_row, chunk_order, s, rows);
  } else if (K % 32 == 0 && K <= 512) {
    // other multiples of 32: column slabs of 128, 64 and 32; the first writes, the others add their share
    int64_t off = 0;
    while (off < K) {
      const int64_t w = K - off >= 128 ? 128 : (K - off >= 64 ? 64 : 32);
#define HPSPMM_SDDMM(WW)                                                                                  \
  if (off == 0)                                                                                           \
    launch_sddmm<WW, 1>(hint, m, nc, row_ptr, col_idx, X + off, Y + off, out_vals, chunk_start, chunk_row, \
                        chunk_order, s, rows, (int)K);                                                    \
  else                                                                                                    \
    launch_sddmm<WW, 2>(hint, m, nc, row_ptr, col_idx, X + off, Y + off, out_vals, chunk_start, chunk_row, \
                        chunk_order, s, rows, (int)K)
      if (w == 128) { HPSPMM_SDDMM(32); }
      else if (w == 64) { HPSPMM_SDDMM(16); }
      else { HPSPMM_SDDMM(8); }
#undef HPSPMM_SDDMM
      off += w;
      if (off < K) ctx->launches++;
    }
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
