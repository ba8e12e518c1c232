// Device / memory / stream / event layer and the dense factories of the C ABI.
// Stands where the reference has starml::Matrix, its allocators, handles and copy
// operators (include/starml/basic/matrix.h:14-77, spmm/starml/basic/allocator_cuda.cpp:5-24,
// spmm/starml/basic/handle_cuda.cpp:4-23, spmm/starml/operators/cuda/copy_kernel.cu:7-41).
#include <atomic>
#include <new>

#include "hpspmm_internal.h"

// Allocation-failure seam for tests: g_fail_skip allocations still succeed, then g_fail_count fail.
static std::atomic<int64_t> g_fail_skip{0};
static std::atomic<int64_t> g_fail_count{0};

cudaError_t hpspmm_device_malloc(void** out, size_t bytes) {
  if (g_fail_count.load(std::memory_order_relaxed) > 0) {
    if (g_fail_skip.load(std::memory_order_relaxed) > 0) {
      g_fail_skip.fetch_sub(1, std::memory_order_relaxed);
    } else {
      g_fail_count.fetch_sub(1, std::memory_order_relaxed);
      if (out) *out = nullptr;
      return cudaErrorMemoryAllocation;
    }
  }
  return cudaMalloc(out, bytes);
}

extern "C" {

int hpspmm_debug_fail_device_alloc(int64_t nth, int64_t count) {
  if (nth < 0 || count < 0) return HPSPMM_ERR_INVALID;
  g_fail_count.store(0, std::memory_order_relaxed);
  g_fail_skip.store(nth > 0 ? nth - 1 : 0, std::memory_order_relaxed);
  g_fail_count.store(nth > 0 ? count : 0, std::memory_order_relaxed);
  return HPSPMM_OK;
}

const char* hpspmm_status_string(int status) {
  switch (status) {
    case HPSPMM_OK: return "ok";
    case HPSPMM_ERR_INVALID: return "invalid argument";
    case HPSPMM_ERR_OOM: return "out of memory";
    case HPSPMM_ERR_CUDA: return "CUDA runtime error";
    case HPSPMM_ERR_TIMEOUT: return "device-side wait timed out";
    case HPSPMM_ERR_UNSUPPORTED: return "unsupported size";
    case HPSPMM_ERR_BAD_CSR: return "malformed CSR";
    default: return "unknown status";
  }
}

const char* hpspmm_version(void) { return "hpspmm 0.1 (sm_100a)"; }

int hpspmm_ctx_create(int device_ordinal, hpspmm_ctx** out) {
  if (!out) return HPSPMM_ERR_INVALID;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return HPSPMM_ERR_CUDA;
  if (device_ordinal < 0 || device_ordinal >= count) return HPSPMM_ERR_INVALID;
  hpspmm_ctx* ctx = new (std::nothrow) hpspmm_ctx();
  if (!ctx) return HPSPMM_ERR_OOM;
  memset(ctx, 0, sizeof(*ctx));
  ctx->device = device_ordinal;
  hpspmm_device_guard guard(device_ordinal);
  int v = 0;
  cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device_ordinal);
  ctx->sm_count = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, device_ordinal);
  ctx->l2_bytes = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, device_ordinal);
  ctx->max_smem_optin = v;
  e = hpspmm_device_malloc((void**)&ctx->flag, 256);
  if (e != cudaSuccess) {
    delete ctx;
    return e == cudaErrorMemoryAllocation ? HPSPMM_ERR_OOM : HPSPMM_ERR_CUDA;
  }
  cudaMemset(ctx->flag, 0, 256);
  *out = ctx;
  return HPSPMM_OK;
}

int hpspmm_ctx_destroy(hpspmm_ctx* ctx) {
  if (!ctx) return HPSPMM_OK;
  hpspmm_device_guard guard(ctx->device);
  cudaDeviceSynchronize();
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->stage) cudaFree(ctx->stage);
  if (ctx->flag) cudaFree(ctx->flag);
  for (int i = 0; i < 3; ++i)
    if (ctx->pipe_streams[i]) cudaStreamDestroy(ctx->pipe_streams[i]);
  for (int i = 0; i < 8; ++i)
    if (ctx->pipe_events[i]) cudaEventDestroy(ctx->pipe_events[i]);
  delete ctx;
  return HPSPMM_OK;
}

const char* hpspmm_last_error(const hpspmm_ctx* ctx) { return ctx ? ctx->err : ""; }
int hpspmm_ctx_tma_fallbacks(hpspmm_ctx* ctx, int64_t* count) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr && count != nullptr, "null context or output");
  hpspmm_device_guard guard(ctx->device);
  int n = 0;
  HPSPMM_CUDA_TRY(ctx, cudaDeviceSynchronize());
  HPSPMM_CUDA_TRY(ctx, cudaMemcpy(&n, ctx->flag + HPSPMM_FLAG_TMA_FALLBACKS, sizeof(int), cudaMemcpyDeviceToHost));
  *count = n;
  return HPSPMM_OK;
}

int hpspmm_ctx_device(const hpspmm_ctx* ctx) { return ctx ? ctx->device : -1; }
int hpspmm_ctx_sm_count(const hpspmm_ctx* ctx) { return ctx ? ctx->sm_count : 0; }
int64_t hpspmm_ctx_l2_bytes(const hpspmm_ctx* ctx) { return ctx ? ctx->l2_bytes : 0; }
int64_t hpspmm_ctx_launch_count(const hpspmm_ctx* ctx) { return ctx ? ctx->launches : 0; }

int hpspmm_dev_alloc(hpspmm_ctx* ctx, size_t bytes, void** out) {
  HPSPMM_REQUIRE(ctx, ctx && out, "null context or output");
  *out = nullptr;
  if (bytes == 0) return HPSPMM_OK;
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, hpspmm_device_malloc(out, bytes));
  return HPSPMM_OK;
}

int hpspmm_dev_free(hpspmm_ctx* ctx, void* ptr) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  if (!ptr) return HPSPMM_OK;
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, cudaFree(ptr));
  return HPSPMM_OK;
}

int hpspmm_host_alloc_pinned(hpspmm_ctx* ctx, size_t bytes, void** out) {
  HPSPMM_REQUIRE(ctx, ctx && out, "null context or output");
  *out = nullptr;
  if (bytes == 0) return HPSPMM_OK;
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, cudaHostAlloc(out, bytes, cudaHostAllocDefault));
  return HPSPMM_OK;
}

int hpspmm_host_free_pinned(hpspmm_ctx* ctx, void* ptr) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  if (!ptr) return HPSPMM_OK;
  HPSPMM_CUDA_TRY(ctx, cudaFreeHost(ptr));
  return HPSPMM_OK;
}

static int copy_async(hpspmm_ctx* ctx, void* dst, const void* src, size_t bytes,
                      cudaMemcpyKind kind, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  if (bytes == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, dst && src, "null pointer");
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, kind, (cudaStream_t)stream));
  return HPSPMM_OK;
}

int hpspmm_memcpy_h2d(hpspmm_ctx* ctx, void* dst, const void* src, size_t bytes,
                      hpspmm_stream stream) {
  return copy_async(ctx, dst, src, bytes, cudaMemcpyHostToDevice, stream);
}
int hpspmm_memcpy_d2h(hpspmm_ctx* ctx, void* dst, const void* src, size_t bytes,
                      hpspmm_stream stream) {
  return copy_async(ctx, dst, src, bytes, cudaMemcpyDeviceToHost, stream);
}
int hpspmm_memcpy_d2d(hpspmm_ctx* ctx, void* dst, const void* src, size_t bytes,
                      hpspmm_stream stream) {
  return copy_async(ctx, dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
}

int hpspmm_memset(hpspmm_ctx* ctx, void* dst, int byte_value, size_t bytes,
                  hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  if (bytes == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, dst, "null pointer");
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, cudaMemsetAsync(dst, byte_value, bytes, (cudaStream_t)stream));
  return HPSPMM_OK;
}

int hpspmm_stream_create(hpspmm_ctx* ctx, hpspmm_stream* out) {
  HPSPMM_REQUIRE(ctx, ctx && out, "null context or output");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s;
  HPSPMM_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *out = (hpspmm_stream)s;
  return HPSPMM_OK;
}

int hpspmm_stream_sync(hpspmm_ctx* ctx, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, cudaStreamSynchronize((cudaStream_t)stream));
  return HPSPMM_OK;
}

int hpspmm_stream_destroy(hpspmm_ctx* ctx, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  if (!stream) return HPSPMM_OK;
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, cudaStreamDestroy((cudaStream_t)stream));
  return HPSPMM_OK;
}

int hpspmm_event_create(hpspmm_ctx* ctx, hpspmm_event* out) {
  HPSPMM_REQUIRE(ctx, ctx && out, "null context or output");
  hpspmm_device_guard guard(ctx->device);
  cudaEvent_t ev;
  HPSPMM_CUDA_TRY(ctx, cudaEventCreate(&ev));
  *out = (hpspmm_event)ev;
  return HPSPMM_OK;
}

int hpspmm_event_record(hpspmm_ctx* ctx, hpspmm_event ev, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx && ev, "null context or event");
  hpspmm_device_guard guard(ctx->device);
  HPSPMM_CUDA_TRY(ctx, cudaEventRecord((cudaEvent_t)ev, (cudaStream_t)stream));
  return HPSPMM_OK;
}

int hpspmm_event_sync(hpspmm_ctx* ctx, hpspmm_event ev) {
  HPSPMM_REQUIRE(ctx, ctx && ev, "null context or event");
  HPSPMM_CUDA_TRY(ctx, cudaEventSynchronize((cudaEvent_t)ev));
  return HPSPMM_OK;
}

int hpspmm_event_elapsed_ms(hpspmm_ctx* ctx, hpspmm_event start, hpspmm_event stop,
                            float* ms_out) {
  HPSPMM_REQUIRE(ctx, ctx && start && stop && ms_out, "null argument");
  HPSPMM_CUDA_TRY(ctx, cudaEventSynchronize((cudaEvent_t)stop));
  HPSPMM_CUDA_TRY(ctx, cudaEventElapsedTime(ms_out, (cudaEvent_t)start, (cudaEvent_t)stop));
  return HPSPMM_OK;
}

int hpspmm_event_destroy(hpspmm_ctx* ctx, hpspmm_event ev) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  if (!ev) return HPSPMM_OK;
  HPSPMM_CUDA_TRY(ctx, cudaEventDestroy((cudaEvent_t)ev));
  return HPSPMM_OK;
}

}  // extern "C"

int hpspmm_ensure_scratch(hpspmm_ctx* ctx, size_t bytes) {
  if (bytes <= ctx->scratch_bytes) return HPSPMM_OK;
  // grow-only; the old buffer may still be in use by queued kernels
  HPSPMM_CUDA_TRY(ctx, cudaDeviceSynchronize());
  if (ctx->scratch) cudaFree(ctx->scratch);
  ctx->scratch = nullptr;
  ctx->scratch_bytes = 0;
  size_t want = bytes + bytes / 4 + 4096;
  cudaError_t e = hpspmm_device_malloc(&ctx->scratch, want);
  if (e != cudaSuccess) {
    want = bytes;
    e = hpspmm_device_malloc(&ctx->scratch, want);
  }
  if (e != cudaSuccess) return hpspmm_set_err(ctx, HPSPMM_ERR_OOM, "scratch cudaMalloc", e);
  ctx->scratch_bytes = want;
  return HPSPMM_OK;
}

int hpspmm_ensure_stage(hpspmm_ctx* ctx, size_t bytes) {
  if (bytes <= ctx->stage_bytes) return HPSPMM_OK;
  HPSPMM_CUDA_TRY(ctx, cudaDeviceSynchronize());
  if (ctx->stage) cudaFree(ctx->stage);
  ctx->stage = nullptr;
  ctx->stage_bytes = 0;
  cudaError_t e = hpspmm_device_malloc(&ctx->stage, bytes);
  if (e != cudaSuccess) return hpspmm_set_err(ctx, HPSPMM_ERR_OOM, "stage cudaMalloc", e);
  ctx->stage_bytes = bytes;
  return HPSPMM_OK;
}

// ---- dense factories -------------------------------------------------------------------

__global__ void fill_f32_kernel(float* __restrict__ x, int64_t n, float v) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = v;
}

__global__ void fill_uniform_f32_kernel(float* __restrict__ x, int64_t n, uint64_t seed,
                                        uint64_t stream_id, float lo, float span) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    x[i] = __fmaf_rn(span, hpspmm_u01(hpspmm_rand64(seed, stream_id, (uint64_t)i)), lo);
}

extern "C" {

int hpspmm_fill_f32(hpspmm_ctx* ctx, float* dev_ptr, int64_t count, float value,
                    hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  HPSPMM_REQUIRE(ctx, count >= 0, "negative count");
  if (count == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, dev_ptr, "null pointer");
  hpspmm_device_guard guard(ctx->device);
  int64_t blocks = (count + 1023) / 1024;
  const int64_t cap = (int64_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  fill_f32_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(dev_ptr, count, value);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

int hpspmm_fill_uniform_f32(hpspmm_ctx* ctx, float* dev_ptr, int64_t count, uint64_t seed,
                            uint64_t stream_id, float lo, float hi, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx, "null context");
  HPSPMM_REQUIRE(ctx, count >= 0, "negative count");
  if (count == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, dev_ptr, "null pointer");
  hpspmm_device_guard guard(ctx->device);
  int64_t blocks = (count + 1023) / 1024;
  const int64_t cap = (int64_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  fill_uniform_f32_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      dev_ptr, count, seed, stream_id, lo, hi - lo);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

}  // extern "C"
