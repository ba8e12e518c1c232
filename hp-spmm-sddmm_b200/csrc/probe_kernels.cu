// Load-path probes: how fast can this GPU deliver rows of a dense matrix to registers?
//
// The product kernels gather nnz rows of B (K * 4 bytes each) per launch; whatever the cache
// hit rates, every gathered byte crosses the L2 -> SM port and the L1 data path.  These probes
// measure those ceilings with the gather shape of the product kernels (G = 32 / W lane groups,
// one float4 per lane, U = 4 gathers in flight per lane, 64-thread blocks) and nothing else:
// no sparse stream, no row ends, no stores.  Row indices come from a multiplicative hash of the
// gather counter, so no index array is read.  The reference has no counterpart; its README
// reports kernel GFLOPS only.
#include <cuda.h>   // CUtensorMap and the encode prototype only; the entry point is looked up at run time

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

// ---- the same rows through the tensor memory accelerator ----------------------------------------
// Blackwell's TMA can fetch four rows of a 2-D tensor, named by four row indices, into shared memory
// with one instruction (cp.async.bulk.tensor ... tile::gather4; the tensor map's box is one row wide,
// each operation completes 4 * row_bytes on the mbarrier).  The probe is a producer / consumer ring:
// PW producer warps issue gather4 operations into STAGES buffers of 16 KB, eight consumer warps read
// every delivered byte from shared memory into registers and release the buffer.  It answers whether
// this path delivers rows to an SM faster than per-lane 16-byte loads do.
//
// Every wait is bounded: a wait that outlasts kTmaWaitCycles records a code in *err and the kernel
// winds down (each role stops at its next wait), so a fault in the protocol shows up as a status, not
// as a hang.
constexpr int kTmaStageBytes = 16384;
constexpr int kTmaConsumerWarps = 8;
constexpr long long kTmaWaitCycles = 1000000000ll;   // about half a second

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* err, int code) {
  const long long t0 = clock64();
  for (unsigned n = 1;; ++n) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((n & 63u) == 0 && (clock64() - t0 > kTmaWaitCycles || *(volatile int*)err != 0)) {
      atomicCAS(err, 0, code);
      return false;
    }
  }
}

__device__ __forceinline__ unsigned probe_hash_row(unsigned idx, unsigned table_rows) {
  const unsigned h = idx * 2654435761u;
  const unsigned h2 = (h ^ (h >> 15)) * 2246822519u;
  return __umulhi(h2, table_rows);
}

// sums[thread] receives the sum of everything the thread read (producer threads write 0), so that a
// table with known contents checks that the right rows arrived.
template <int ROW_FLOATS, int STAGES, int PW>
__global__ void __launch_bounds__((kTmaConsumerWarps + PW) * 32)
probe_tma_gather_kernel(const __grid_constant__ CUtensorMap tmap, unsigned table_rows, int iters,
                        float* __restrict__ sums, int* err) {
  constexpr int ROW_BYTES = ROW_FLOATS * 4;
  constexpr int ROWS = kTmaStageBytes / ROW_BYTES;   // rows per stage
  constexpr int OPS = ROWS / 4;                      // gather4 operations per stage
  static_assert(STAGES % PW == 0, "each producer warp owns every PW-th stage");
  extern __shared__ __align__(1024) unsigned char ring[];
  __shared__ __align__(8) uint64_t full[STAGES];
  __shared__ __align__(8) uint64_t empty[STAGES];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&full[s])), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&empty[s])), "r"(kTmaConsumerWarps)
                   : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const unsigned cta_first = (unsigned)blockIdx.x * (unsigned)iters * (unsigned)ROWS;
  float total = 0.f;
  if (warp >= kTmaConsumerWarps) {
    bool ok = true;
    for (int it = warp - kTmaConsumerWarps; it < iters && ok; it += PW) {
      const int s = it % STAGES;
      const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
      if (it >= STAGES) {   // the buffer's previous contents must have been read
        if (lane == 0) ok = mbar_wait_bounded(smem_addr(&empty[s]), ph ^ 1u, err, 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&full[s])),
                     "r"(kTmaStageBytes)
                     : "memory");
      __syncwarp();
      for (int q = lane; q < OPS; q += 32) {
        const unsigned g0 = cta_first + (unsigned)it * ROWS + (unsigned)q * 4u;
        const int r0 = (int)probe_hash_row(g0, table_rows), r1 = (int)probe_hash_row(g0 + 1, table_rows);
        const int r2 = (int)probe_hash_row(g0 + 2, table_rows), r3 = (int)probe_hash_row(g0 + 3, table_rows);
        const uint32_t dst = smem_addr(ring + (size_t)s * kTmaStageBytes + (size_t)q * 4 * ROW_BYTES);
        // column coordinate 0: a multiple of 16 bytes, as every tiled TMA copy requires
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
            "l"(&tmap), "r"(0), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(smem_addr(&full[s]))
            : "memory");
      }
    }
  } else {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int it = 0; it < iters; ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
      const bool ok = mbar_wait_bounded(smem_addr(&full[s]), ph, err, 2);
      if (!__all_sync(0xffffffffu, ok)) break;
      const float4* src = reinterpret_cast<const float4*>(ring + (size_t)s * kTmaStageBytes);
#pragma unroll
      for (int k = 0; k < kTmaStageBytes / 16 / (kTmaConsumerWarps * 32); ++k) {
        const float4 v = src[(k * kTmaConsumerWarps + warp) * 32 + lane];
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&empty[s])) : "memory");
    }
    total = (acc.x + acc.y) + (acc.z + acc.w);
  }
  sums[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = total;
}

__global__ void probe_fill_rows_kernel(float* __restrict__ table, int64_t rows, int row_floats) {
  const int64_t n = rows * row_floats;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    table[i] = (float)((i / row_floats) % 251);
}

typedef CUresult (*tensor_map_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int ROW_FLOATS>
cudaError_t launch_tma_probe(const CUtensorMap& tmap, unsigned rows, int grid, int iters, float* sums, int* err,
                             cudaStream_t s) {
  constexpr int STAGES = 4, PW = 4;
  auto kern = probe_tma_gather_kernel<ROW_FLOATS, STAGES, PW>;
  const int smem = STAGES * kTmaStageBytes;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  kern<<<grid, (kTmaConsumerWarps + PW) * 32, smem, s>>>(tmap, rows, iters, sums, err);
  return cudaGetLastError();
}

}  // namespace

extern "C" int hpspmm_probe_tma_gather_gbs(hpspmm_ctx* ctx, int32_t row_bytes, int64_t table_rows, int64_t n_gathers,
                                           int32_t ctas_per_sm, int32_t repeats, double* gbs_out, double* ms_out,
                                           double* checksum_out, int64_t* gathers_done_out) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr && gbs_out != nullptr, "null context or output");
  HPSPMM_REQUIRE(ctx, row_bytes == 128 || row_bytes == 256 || row_bytes == 512, "row_bytes must be 128, 256 or 512");
  HPSPMM_REQUIRE(ctx, table_rows >= 1 && table_rows <= 0x7fffffffll && n_gathers >= 1 && n_gathers <= 0x7fffffffll,
                 "table_rows and n_gathers must be in [1, 2^31)");
  HPSPMM_REQUIRE(ctx, ctas_per_sm >= 1 && ctas_per_sm <= 3 && repeats >= 1 && repeats <= 1000,
                 "ctas_per_sm must be 1..3 and repeats 1..1000");
  hpspmm_device_guard guard(ctx->device);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult found;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found);
  if (e != cudaSuccess || fn == nullptr || found != cudaDriverEntryPointSuccess)
    return hpspmm_set_err(ctx, HPSPMM_ERR_UNSUPPORTED, "the driver offers no cuTensorMapEncodeTiled", e);
  const int row_floats = row_bytes / 4;
  const int rows_per_stage = kTmaStageBytes / row_bytes;
  const int grid = ctx->sm_count * ctas_per_sm;
  const int iters = (int)((n_gathers + (int64_t)grid * rows_per_stage - 1) / ((int64_t)grid * rows_per_stage));
  const int64_t done = (int64_t)grid * iters * rows_per_stage;
  HPSPMM_REQUIRE(ctx, done <= 0xffffffffll, "too many gathers for the 32-bit gather counter");
  const int threads = (kTmaConsumerWarps + 4) * 32;
  float* table = nullptr;
  float* sums = nullptr;
  int* err = nullptr;
  cudaEvent_t a = nullptr, b = nullptr;
  const size_t table_bytes = (size_t)table_rows * (size_t)row_bytes;
  e = hpspmm_device_malloc((void**)&table, table_bytes);
  if (e == cudaSuccess) e = hpspmm_device_malloc((void**)&sums, (size_t)grid * threads * 4);
  if (e == cudaSuccess) e = hpspmm_device_malloc((void**)&err, 4);
  if (e == cudaSuccess) e = cudaMemset(err, 0, 4);
  if (e == cudaSuccess) e = cudaEventCreate(&a);
  if (e == cudaSuccess) e = cudaEventCreate(&b);
  float ms = 0.f;
  int waited_out = 0;
  double checksum = 0.0;
  bool encoded = true;
  if (e == cudaSuccess) {
    cudaStream_t s = 0;
    probe_fill_rows_kernel<<<ctx->sm_count * 8, 256, 0, s>>>(table, table_rows, row_floats);
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)row_floats, (cuuint64_t)table_rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)row_floats, 1};   // gather4: one row per box, four boxes per operation
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = ((tensor_map_encode_fn)fn)(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, table, gdim, gstride, box,
                                                  estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    encoded = r == CUDA_SUCCESS;
    for (int it = 0; encoded && it < 3 + repeats && e == cudaSuccess && !waited_out; ++it) {
      if (it == 3) e = cudaEventRecord(a, s);
      if (e != cudaSuccess) break;
      if (row_bytes == 128)
        e = launch_tma_probe<32>(tmap, (unsigned)table_rows, grid, iters, sums, err, s);
      else if (row_bytes == 256)
        e = launch_tma_probe<64>(tmap, (unsigned)table_rows, grid, iters, sums, err, s);
      else
        e = launch_tma_probe<128>(tmap, (unsigned)table_rows, grid, iters, sums, err, s);
      ctx->launches++;
      if (it == 0 && e == cudaSuccess) {   // a protocol fault is caught after the first launch, not after thirteen
        e = cudaStreamSynchronize(s);
        if (e == cudaSuccess) e = cudaMemcpy(&waited_out, err, 4, cudaMemcpyDeviceToHost);
      }
    }
    if (encoded && e == cudaSuccess && !waited_out) e = cudaEventRecord(b, s);
    if (encoded && e == cudaSuccess && !waited_out) e = cudaEventSynchronize(b);
    if (encoded && e == cudaSuccess && !waited_out) e = cudaEventElapsedTime(&ms, a, b);
    if (encoded && e == cudaSuccess && !waited_out) e = cudaMemcpy(&waited_out, err, 4, cudaMemcpyDeviceToHost);
    if (encoded && e == cudaSuccess && !waited_out && checksum_out) {
      const size_t n_sums = (size_t)grid * threads;
      float* host = (float*)malloc(n_sums * 4);
      if (host) {
        e = cudaMemcpy(host, sums, n_sums * 4, cudaMemcpyDeviceToHost);
        for (size_t i = 0; i < n_sums; ++i) checksum += (double)host[i];
        free(host);
      } else {
        checksum = -1.0;
      }
    }
  }
  if (a) cudaEventDestroy(a);
  if (b) cudaEventDestroy(b);
  if (table) cudaFree(table);
  if (sums) cudaFree(sums);
  if (err) cudaFree(err);
  if (e != cudaSuccess)
    return hpspmm_set_err(ctx, e == cudaErrorMemoryAllocation ? HPSPMM_ERR_OOM : HPSPMM_ERR_CUDA, "TMA gather probe", e);
  if (!encoded) return hpspmm_set_err(ctx, HPSPMM_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled refused the table", cudaSuccess);
  if (waited_out)
    return hpspmm_set_err(ctx, HPSPMM_ERR_CUDA,
                          waited_out == 1 ? "TMA gather probe: a producer's bounded wait ran out"
                                          : "TMA gather probe: a consumer's bounded wait ran out",
                          cudaSuccess);
  ms /= (float)repeats;
  *gbs_out = (double)done * (double)row_bytes / ((double)ms * 1e-3) / 1e9;
  if (ms_out) *ms_out = ms;
  if (checksum_out) *checksum_out = checksum;
  if (gathers_done_out) *gathers_done_out = done;
  return HPSPMM_OK;
}

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
