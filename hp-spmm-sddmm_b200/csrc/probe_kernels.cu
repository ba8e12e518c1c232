// Load-path probes: how fast can this GPU deliver rows of a dense matrix to registers?
//
// The product kernels gather nnz rows of B (K * 4 bytes each) per launch; whatever the cache
// hit rates, every gathered byte crosses the L2 -> SM port and the L1 data path.  These probes
// measure those ceilings with the gather shape of the product kernels (G = 32 / W lane groups,
// one float4 per lane, U = 4 gathers in flight per lane, 64-thread blocks) and nothing else:
// no sparse stream, no row ends, no stores.  Row indices come from a multiplicative hash of the
// gather counter, so no index array is read.  The reference has no counterpart; its README
// reports kernel GFLOPS only.
#include "device_utils.cuh"
#include "hpspmm_internal.h"

namespace {

using namespace hpspmm;

// pattern 0: consecutive rows (a stream); 1: uniformly random rows; 2: random, but a share
// `hot_share_q16 / 65536` of the gathers falls on the first hot_rows rows (hub columns)
template <int W, int U>
__global__ void __launch_bounds__(64, 20)
probe_gather_kernel(const float* __restrict__ table, unsigned table_rows, int64_t n_gathers, int per_warp,
                    int pattern, unsigned hot_rows, unsigned hot_share_q16, float* __restrict__ sink) {
  constexpr int G = 32 / W;
  const int lane = threadIdx.x & 31;
  const int g = lane / W, l = lane % W;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t first = warp * per_warp;
  if (first >= n_gathers) return;
  const int64_t last = min(n_gathers, first + (int64_t)per_warp);
  const float* base = table + l * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t j = first; j < last; j += U * G) {
    float4 b[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const unsigned idx = (unsigned)(j + i * G + g);
      unsigned row;
      if (pattern == 0) {
        row = idx % table_rows;
      } else {
        const unsigned h = idx * 2654435761u;
        const unsigned h2 = (h ^ (h >> 15)) * 2246822519u;
        row = __umulhi(h2, table_rows);
        if (pattern == 2 && (h >> 16) < hot_share_q16) row = __umulhi(h2, hot_rows);
      }
      b[i] = ld_gather_plain(base + (int64_t)row * (W * 4));
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      acc.x += b[i].x;
      acc.y += b[i].y;
      acc.z += b[i].z;
      acc.w += b[i].w;
    }
  }
  // never true for a zero-filled table; keeps the loads alive
  if (acc.x + acc.y + acc.z + acc.w == 12345.f) sink[warp] = acc.x;
}

template <int W>
void launch_probe(const float* table, unsigned rows, int64_t n, int per_warp, int pattern, unsigned hot_rows,
                  unsigned hot_q16, float* sink, cudaStream_t s) {
  const int64_t warps = (n + per_warp - 1) / per_warp;
  const unsigned blocks = (unsigned)((warps + 1) / 2);
  probe_gather_kernel<W, 4><<<blocks, 64, 0, s>>>(table, rows, n, per_warp, pattern, hot_rows, hot_q16, sink);
}

}  // namespace

extern "C" int hpspmm_probe_gather_gbs(hpspmm_ctx* ctx, int32_t row_bytes, int64_t table_rows, int64_t n_gathers,
                                       int32_t pattern, int64_t hot_rows, double hot_share, int32_t repeats,
                                       double* gbs_out, double* ms_out) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr && gbs_out != nullptr, "null context or output");
  HPSPMM_REQUIRE(ctx, row_bytes == 128 || row_bytes == 256 || row_bytes == 512, "row_bytes must be 128, 256 or 512");
  HPSPMM_REQUIRE(ctx, table_rows >= 1 && table_rows <= 0x7fffffffll && n_gathers >= 1 && n_gathers <= 0x7fffffffll,
                 "table_rows and n_gathers must be in [1, 2^31)");
  HPSPMM_REQUIRE(ctx, pattern >= 0 && pattern <= 2 && repeats >= 1 && repeats <= 1000, "bad pattern or repeats");
  HPSPMM_REQUIRE(ctx, pattern != 2 || (hot_rows >= 1 && hot_rows <= table_rows && hot_share >= 0.0 && hot_share <= 1.0),
                 "bad hot set");
  hpspmm_device_guard guard(ctx->device);
  const int per_warp = 256;
  const int64_t warps = (n_gathers + per_warp - 1) / per_warp;
  float* table = nullptr;
  float* sink = nullptr;
  cudaEvent_t a = nullptr, b = nullptr;
  const size_t table_bytes = (size_t)table_rows * (size_t)row_bytes;
  cudaError_t e = hpspmm_device_malloc((void**)&table, table_bytes);
  if (e == cudaSuccess) e = hpspmm_device_malloc((void**)&sink, (size_t)warps * 4);
  if (e == cudaSuccess) e = cudaMemset(table, 0, table_bytes);
  if (e == cudaSuccess) e = cudaEventCreate(&a);
  if (e == cudaSuccess) e = cudaEventCreate(&b);
  float ms = 0.f;
  if (e == cudaSuccess) {
    const unsigned q16 = (unsigned)(hot_share * 65536.0);
    cudaStream_t s = 0;
    for (int it = 0; it < 3 + repeats && e == cudaSuccess; ++it) {
      if (it == 3) e = cudaEventRecord(a, s);
      if (row_bytes == 128)
        launch_probe<8>(table, (unsigned)table_rows, n_gathers, per_warp, pattern, (unsigned)hot_rows, q16, sink, s);
      else if (row_bytes == 256)
        launch_probe<16>(table, (unsigned)table_rows, n_gathers, per_warp, pattern, (unsigned)hot_rows, q16, sink, s);
      else
        launch_probe<32>(table, (unsigned)table_rows, n_gathers, per_warp, pattern, (unsigned)hot_rows, q16, sink, s);
      ctx->launches++;
    }
    if (e == cudaSuccess) e = cudaEventRecord(b, s);
    if (e == cudaSuccess) e = cudaEventSynchronize(b);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
  }
  if (a) cudaEventDestroy(a);
  if (b) cudaEventDestroy(b);
  if (table) cudaFree(table);
  if (sink) cudaFree(sink);
  if (e != cudaSuccess)
    return hpspmm_set_err(ctx, e == cudaErrorMemoryAllocation ? HPSPMM_ERR_OOM : HPSPMM_ERR_CUDA, "gather probe", e);
  ms /= (float)repeats;
  *gbs_out = (double)n_gathers * (double)row_bytes / ((double)ms * 1e-3) / 1e9;
  if (ms_out) *ms_out = ms;
  return HPSPMM_OK;
}
