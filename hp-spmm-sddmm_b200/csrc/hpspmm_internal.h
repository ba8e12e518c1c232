// Internal declarations shared by the translation units of libhpspmm.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "hpspmm.h"

// Context: device ordinal, cached device properties, grow-only scratch and the text
// of the last CUDA error.  Takes the place of starml's allocator and handle
// registries (spmm/starml/basic/allocator.cpp:21-48, spmm/starml/basic/handle.cpp:11-17).
struct hpspmm_ctx {
  int device;
  int sm_count;
  int64_t l2_bytes;
  int max_smem_optin;
  int64_t launches;
  // scratch for plan-less calls: chunk table and carries
  void* scratch;
  size_t scratch_bytes;
  // staging for the host-buffer entry point
  void* stage;
  size_t stage_bytes;
  int* flag;  // 64 device ints: [0] validation and plan building, [HPSPMM_FLAG_TMA_FALLBACKS] see below
  // streams of the host-buffer entry point: uploads, kernels, downloads (created on first use)
  cudaStream_t pipe_streams[3];
  cudaEvent_t pipe_events[8];   // "A has landed" and, per buffer, slab uploaded / multiplied / downloaded
  char err[256];
};

// ctx->flag[HPSPMM_FLAG_TMA_FALLBACKS] counts the warps of spmm_tma_kernel whose bounded wait for a TMA copy
// ran out (they finish their chunk with ordinary loads); hpspmm_ctx_tma_fallbacks reads it.
#define HPSPMM_FLAG_TMA_FALLBACKS 16

// Chunk table of one sparsity structure.
//   chunk_start[c]  first nnz of chunk c (n_chunks + 1 entries)
//   chunk_row[c]    row holding nnz chunk_start[c]
//   carry_row[c]    row whose partial sum chunk c hands on, or -1
//   carry_val[c*K..] that partial sum
struct hpspmm_plan {
  int device;
  int64_t M, nnz;
  int32_t chunk_nnz;
  int64_t n_chunks;
  int64_t n_split_chunks;  // chunks that end inside a row
  int64_t max_K;
  int32_t* chunk_start;
  int32_t* chunk_row;
  int32_t* chunk_order;  // chunk ids, most rows first: the order in which warps take chunks
  int32_t* carry_row;
  float* carry_val;
  int32_t* run_counter;  // one per chunk, zero between launches: pieces of a split row that have finished
  // rows that hold entries: ids (ascending, then the sentinel M), their ends in the entry array, and
  // for every chunk the position in this list of the row holding its first entry
  int32_t* nz_id;
  int32_t* nz_end;
  int32_t* chunk_ri;
  size_t bytes;
};

static inline int hpspmm_set_err(hpspmm_ctx* ctx, int status, const char* what, cudaError_t e) {
  if (ctx) snprintf(ctx->err, sizeof(ctx->err), "%s: %s", what, cudaGetErrorString(e));
  return status;
}

#define HPSPMM_CUDA_TRY(ctx, call)                                               \
  do {                                                                           \
    cudaError_t e__ = (call);                                                    \
    if (e__ != cudaSuccess)                                                      \
      return hpspmm_set_err((ctx), e__ == cudaErrorMemoryAllocation ? HPSPMM_ERR_OOM \
                                                                   : HPSPMM_ERR_CUDA, \
                            #call, e__);                                         \
  } while (0)

#define HPSPMM_REQUIRE(ctx, cond, msg)                                     \
  do {                                                                     \
    if (!(cond)) {                                                         \
      if (ctx) snprintf((ctx)->err, sizeof((ctx)->err), "invalid argument: %s", msg); \
      return HPSPMM_ERR_INVALID;                                           \
    }                                                                      \
  } while (0)

// Makes the context's device current for the calling thread for the duration of a call.
struct hpspmm_device_guard {
  int prev;
  bool switched;
  explicit hpspmm_device_guard(int dev) : prev(-1), switched(false) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
      cudaSetDevice(dev);
      switched = true;
    }
  }
  ~hpspmm_device_guard() {
    if (switched) cudaSetDevice(prev);
  }
};

// Every device allocation of the library goes through here: cudaMalloc, unless a test has armed
// hpspmm_debug_fail_device_alloc, in which case the chosen allocation reports cudaErrorMemoryAllocation
// without touching the device.
cudaError_t hpspmm_device_malloc(void** out, size_t bytes);
template <typename T>
static inline cudaError_t hpspmm_device_malloc(T** out, size_t bytes) {
  return hpspmm_device_malloc(reinterpret_cast<void**>(out), bytes);
}

// A named range around an entry point for timeline tools (NVTX 3, header-only: nothing to link, and a call is a
// null-pointer test when no tool is attached).  The reference has no tracing beyond its event timer
// (include/spmm/utils/timer_cuda.h:6-40).
#include <nvtx3/nvToolsExt.h>
struct hpspmm_trace_range {
  explicit hpspmm_trace_range(const char* name) { nvtxRangePushA(name); }
  ~hpspmm_trace_range() { nvtxRangePop(); }
  hpspmm_trace_range(const hpspmm_trace_range&) = delete;
  hpspmm_trace_range& operator=(const hpspmm_trace_range&) = delete;
};
#define HPSPMM_TRACE(name) hpspmm_trace_range hpspmm_trace_range__(name)

int hpspmm_ensure_scratch(hpspmm_ctx* ctx, size_t bytes);
int hpspmm_ensure_stage(hpspmm_ctx* ctx, size_t bytes);

// nominal chunk size for a dense width and a matrix of nnz entries
int32_t hpspmm_default_chunk_nnz(int64_t K, int64_t nnz);

// Builds chunk_start / chunk_row for (M, nnz, row_ptr) into the given arrays (device).
// split_count (device int, may be null) receives the number of chunks ending mid-row.
// run_counter (n_chunks + 1 ints, may be null) is zeroed.
int hpspmm_launch_chunk_table(hpspmm_ctx* ctx, int64_t M, int64_t nnz, const int32_t* row_ptr,
                              int32_t chunk_nnz, int64_t n_chunks, int32_t* chunk_start,
                              int32_t* chunk_row, int* split_count, cudaStream_t stream,
                              int32_t* run_counter);

// Processing order of the chunks: chunk ids sorted by estimated cost (entries / 8 + rows / 2),
// most expensive first (stable 8-bit counting-sort passes on the device).  Chunks full of short
// rows started last leave the GPU draining; started first they overlap with the others.
// With col_idx (may be null) the chunks that lie inside one row come last, in ascending order
// of their first column, so that pieces of different heavy rows running together read the same
// band of B.  `scratch` needs hpspmm_order_scratch_bytes(n_chunks) bytes.
size_t hpspmm_order_scratch_bytes(int64_t n_chunks);
int hpspmm_order_chunks_by_cost(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t n_chunks,
                                const int32_t* row_ptr, const int32_t* col_idx, const int32_t* chunk_start,
                                const int32_t* chunk_row, int32_t* order_out, void* scratch,
                                cudaStream_t stream);

// The rows that hold entries, as the product kernels of a plan walk them: nz_id / nz_end need M + 1
// ints each, chunk_ri n_chunks; scratch needs hpspmm_row_list_scratch_bytes(M) bytes.
size_t hpspmm_row_list_scratch_bytes(int64_t M);
int hpspmm_build_row_list(hpspmm_ctx* ctx, int64_t M, int64_t n_chunks, const int32_t* row_ptr,
                          const int32_t* chunk_row, int32_t* nz_id, int32_t* nz_end, int32_t* chunk_ri,
                          void* scratch, cudaStream_t stream);

// ---- counter-based PRNG shared by host and device --------------------------------------
// splitmix64 finaliser over (seed, stream, index); 24 high bits -> [0, 1).
#if defined(__CUDACC__)
#define HPSPMM_HD __host__ __device__ __forceinline__
#else
#define HPSPMM_HD static inline
#endif

HPSPMM_HD uint64_t hpspmm_mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

HPSPMM_HD uint64_t hpspmm_rand64(uint64_t seed, uint64_t stream, uint64_t index) {
  uint64_t k = hpspmm_mix64(seed * 0x9E3779B97F4A7C15ull + stream + 0x632BE59BD9B4E019ull);
  return hpspmm_mix64(k + index * 0x9E3779B97F4A7C15ull);
}

// u in [0,1) on a 2^-24 grid: exact in fp32, so host and device agree bit for bit.
HPSPMM_HD float hpspmm_u01(uint64_t bits) { return (float)(uint32_t)(bits >> 40) * (1.0f / 16777216.0f); }
