/*
 * hpspmm.h -- C ABI of the B200 (sm_100a) FP32 CSR SpMM / SDDMM library.
 *
 * This is the drop-in boundary for the sparse x dense hot path of
 * fan1997/HP-SpMM-SDDMM.  Every entry point takes plain pointers and sizes,
 * returns an int status (0 = ok), never aborts, never throws, and -- unless
 * stated otherwise -- only enqueues work on the caller's stream without
 * synchronising.  Element counts and offsets are 64-bit; CSR indices are
 * 32-bit as in the reference.  Reference citations (file:line) are paths
 * inside the reference project.
 *
 * Dense operands are row-major, contiguous, leading dimension K.
 */
#ifndef HPSPMM_H_
#define HPSPMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define HPSPMM_API
#else
#define HPSPMM_API __attribute__((visibility("default")))
#endif

typedef struct hpspmm_ctx hpspmm_ctx;   /* one per (process, device)            */
typedef struct hpspmm_plan hpspmm_plan; /* cached nnz-balanced chunk table of A */
typedef void* hpspmm_stream;            /* a cudaStream_t; NULL = default stream */
typedef void* hpspmm_event;             /* a cudaEvent_t                         */

/* Status codes.  Replace the reference's STARML_CHECK -> abort() behaviour
 * (include/starml/utils/loguru.h:1526-1568) and its unchecked CUDA calls. */
enum {
  HPSPMM_OK = 0,
  HPSPMM_ERR_INVALID = 1,     /* bad argument (null pointer, negative size, K <= 0 ...) */
  HPSPMM_ERR_OOM = 2,         /* device or pinned-host allocation failed                */
  HPSPMM_ERR_CUDA = 3,        /* a CUDA runtime call failed; see hpspmm_last_error      */
  HPSPMM_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out                     */
  HPSPMM_ERR_UNSUPPORTED = 5, /* size beyond what an entry point supports               */
  HPSPMM_ERR_BAD_CSR = 6      /* CSR structure failed validation                        */
};

/* Algorithm selectors for hpspmm_opts.algo. */
enum {
  HPSPMM_ALGO_AUTO = 0,      /* nnz-balanced chunks, heavy rows split (the default)     */
  HPSPMM_ALGO_BALANCED = 1,  /* same as AUTO                                            */
  HPSPMM_ALGO_ROW_SPLIT = 2, /* one sub-warp per row; the shape of the reference's
                                GESpMM kernels (spmm/mm/spmm_kernel.cu:247-370)          */
  HPSPMM_ALGO_TMA = 3        /* BALANCED with the rows of B fetched by TMA (tile::gather4
                                into shared memory) instead of per-lane loads.  Taken at
                                K = 128 with a plan of nominal chunk size up to 256;
                                any other call runs as BALANCED.  Same order of additions,
                                hence the same bits, as BALANCED.                        */
};

/* Runtime options; zero-initialise for defaults.  Replace the reference's
 * in-code heuristics (spmm/mm/spmm_kernel.cu:749-750, :406-420). */
typedef struct hpspmm_opts {
  int32_t algo;        /* HPSPMM_ALGO_*                                              */
  int32_t chunk_nnz;   /* nominal nnz per chunk; 0 = chosen from K; multiple of 32   */
  int32_t b_l2_hint;   /* L2 evict-last policy on the gathers of B: 0 = auto (on for
                          K >= 64: +6 % at 128 columns, neutral at 64; off below,
                          where it costs a little), 1 = off, 2 = on                  */
  int32_t reserved;
} hpspmm_opts;

HPSPMM_API const char* hpspmm_status_string(int status);
HPSPMM_API const char* hpspmm_version(void);

/* ---- device / memory / stream / event layer ---------------------------------
 * Replaces starml's Allocator / Handle / copy operators:
 * include/starml/basic/allocator.h:18-66, spmm/starml/basic/allocator_cuda.cpp:5-24,
 * spmm/starml/basic/handle_cuda.cpp:4-23, spmm/starml/operators/cuda/copy_kernel.cu:7-41,
 * include/spmm/utils/timer_cuda.h:6-40 (GpuTimer). */
HPSPMM_API int hpspmm_ctx_create(int device_ordinal, hpspmm_ctx** out);
HPSPMM_API int hpspmm_ctx_destroy(hpspmm_ctx* ctx);
HPSPMM_API const char* hpspmm_last_error(const hpspmm_ctx* ctx);
HPSPMM_API int hpspmm_ctx_device(const hpspmm_ctx* ctx);
HPSPMM_API int hpspmm_ctx_sm_count(const hpspmm_ctx* ctx);
HPSPMM_API int64_t hpspmm_ctx_l2_bytes(const hpspmm_ctx* ctx);
/* Number of this library's kernels launched through ctx since creation. */
HPSPMM_API int64_t hpspmm_ctx_launch_count(const hpspmm_ctx* ctx);

HPSPMM_API int hpspmm_dev_alloc(hpspmm_ctx* ctx, size_t bytes, void** out);
HPSPMM_API int hpspmm_dev_free(hpspmm_ctx* ctx, void* ptr);
HPSPMM_API int hpspmm_host_alloc_pinned(hpspmm_ctx* ctx, size_t bytes, void** out);
HPSPMM_API int hpspmm_host_free_pinned(hpspmm_ctx* ctx, void* ptr);
HPSPMM_API int hpspmm_memcpy_h2d(hpspmm_ctx* ctx, void* dst, const void* src, size_t bytes,
                                 hpspmm_stream stream);
HPSPMM_API int hpspmm_memcpy_d2h(hpspmm_ctx* ctx, void* dst, const void* src, size_t bytes,
                                 hpspmm_stream stream);
HPSPMM_API int hpspmm_memcpy_d2d(hpspmm_ctx* ctx, void* dst, const void* src, size_t bytes,
                                 hpspmm_stream stream);
HPSPMM_API int hpspmm_memset(hpspmm_ctx* ctx, void* dst, int byte_value, size_t bytes,
                             hpspmm_stream stream);
HPSPMM_API int hpspmm_stream_create(hpspmm_ctx* ctx, hpspmm_stream* out);
HPSPMM_API int hpspmm_stream_sync(hpspmm_ctx* ctx, hpspmm_stream stream);
HPSPMM_API int hpspmm_stream_destroy(hpspmm_ctx* ctx, hpspmm_stream stream);
HPSPMM_API int hpspmm_event_create(hpspmm_ctx* ctx, hpspmm_event* out);
HPSPMM_API int hpspmm_event_record(hpspmm_ctx* ctx, hpspmm_event ev, hpspmm_stream stream);
HPSPMM_API int hpspmm_event_sync(hpspmm_ctx* ctx, hpspmm_event ev);
HPSPMM_API int hpspmm_event_elapsed_ms(hpspmm_ctx* ctx, hpspmm_event start, hpspmm_event stop,
                                       float* ms_out);
HPSPMM_API int hpspmm_event_destroy(hpspmm_ctx* ctx, hpspmm_event ev);

/* ---- factories ---------------------------------------------------------------
 * fill: replaces fill_matrix / fill_cuda (spmm/mm/spmm_kernel.cu:23-34) and
 * `full` (spmm/starml/operators/cuda/factories_kernel.cu:8-17).
 * fill_uniform: replaces `rand` (spmm/starml/operators/cpu/factories_kernel.cpp:14-28),
 * which is unseeded in the reference; here element i of stream `stream_id` is a
 * pure function of (seed, stream_id, i), identical on host and device. */
HPSPMM_API int hpspmm_fill_f32(hpspmm_ctx* ctx, float* dev_ptr, int64_t count, float value,
                               hpspmm_stream stream);
HPSPMM_API int hpspmm_fill_uniform_f32(hpspmm_ctx* ctx, float* dev_ptr, int64_t count,
                                       uint64_t seed, uint64_t stream_id, float lo, float hi,
                                       hpspmm_stream stream);
HPSPMM_API int hpspmm_host_fill_uniform_f32(float* host_ptr, int64_t count, uint64_t seed,
                                            uint64_t stream_id, float lo, float hi);

/* ---- CSR SpMM: C = A * B ---------------------------------------------------------
 * Replaces GESpMM (include/spmm/mm/spmm_kernel.h:19, spmm/mm/spmm_kernel.cu:389-426) and
 * the kernels it dispatches to (:247-387).  Argument order follows the reference's
 * kernels: (m, k, row_ptr, col_idx, values, B, C), with N and nnz added.  Overwrites C;
 * empty rows become zeros.  All pointers are device pointers.  K >= 1; K = 32/64/128
 * take the specialised kernels, every other multiple of 32 up to 512 runs them over
 * column slabs of 128, 64 and 32, any other K a generic kernel.
 *
 * plan may be NULL: the chunk table is then rebuilt into context-owned scratch on
 * every call (one extra small kernel).  The first call that needs more scratch than
 * the context holds allocates it (cudaMalloc, synchronising); later calls do not.
 * With a plan the call only enqueues kernels (no allocation, no synchronisation), so it can
 * be recorded into a CUDA graph and replayed.
 * Calls that share a context or a plan must not overlap on the GPU. */
HPSPMM_API int hpspmm_spmm_csr_f32(hpspmm_ctx* ctx, const hpspmm_plan* plan, int64_t M,
                                   int64_t N, int64_t K, int64_t nnz, const int32_t* row_ptr,
                                   const int32_t* col_idx, const float* vals, const float* B,
                                   float* C, const hpspmm_opts* opts, hpspmm_stream stream);

/* Chunk table of A, the order in which chunks are scheduled, and the list of rows that
 * hold entries, for repeated products with the same sparsity structure (a GNN reuses
 * them across layers and epochs).  Reads row_ptr on the device, synchronises
 * the stream once.  col_idx may be NULL (N is then ignored); when given, the pieces
 * of rows longer than a chunk are scheduled in ascending order of the column band
 * they read, which raises the L2 hit rate of the gathers by a few per cent.  The
 * results do not depend on it.  No counterpart in the reference, whose LBSpMM recomputes its
 * grid from nnz alone (spmm/mm/spmm_kernel.cu:749-751) because its COO input
 * carries an explicit row index per entry. */
HPSPMM_API int hpspmm_plan_create(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz,
                                  const int32_t* row_ptr, const int32_t* col_idx,
                                  int64_t max_K, const hpspmm_opts* opts,
                                  hpspmm_stream stream, hpspmm_plan** out);
HPSPMM_API int hpspmm_plan_destroy(hpspmm_ctx* ctx, hpspmm_plan* plan);
/* chunks, rows split across chunks (heavy rows), nominal chunk size, scratch bytes. */
HPSPMM_API int hpspmm_plan_info(const hpspmm_plan* plan, int64_t* n_chunks,
                                int64_t* n_split_chunks, int64_t* chunk_nnz,
                                int64_t* scratch_bytes);
/* Name and template arguments of the kernel hpspmm_spmm_csr_f32 launches for width K with this
 * plan (plan may be NULL) and L2 hint setting, as a string: profiler captures are filed under it. */
HPSPMM_API int hpspmm_spmm_kernel_signature(const hpspmm_plan* plan, int64_t K, int32_t b_l2_hint,
                                            char* buf, size_t len);
/* Device pointers to the plan's tables, for inspection: chunk_start[n_chunks + 1] (first
 * entry of every chunk), chunk_row[n_chunks] (row holding that entry), chunk_order[n_chunks]
 * (the chunk ids in the order in which warps take them: a permutation of 0..n_chunks-1). */
HPSPMM_API int hpspmm_plan_tables(const hpspmm_plan* plan, const int32_t** chunk_start,
                                  const int32_t** chunk_row, const int32_t** chunk_order);
/* Device pointers to the plan's list of rows that hold entries, for inspection: nz_id (row
 * ids, ascending, followed by the sentinel M), nz_end (row_ptr[id + 1] of those rows; the
 * sentinel's is INT32_MAX), chunk_ri[n_chunks] (position in the list of the row that holds
 * a chunk's first entry).  The kernels step through this list and never visit an empty row. */
HPSPMM_API int hpspmm_plan_row_list(const hpspmm_plan* plan, const int32_t** nz_id,
                                    const int32_t** nz_end, const int32_t** chunk_ri);

/* The same product for callers that cannot allocate device memory when they need it.
 * (No counterpart in the reference, whose entry points allocate nothing because its
 * kernels need no scratch.)  Typical callers: the enqueue hook of an inference-runtime
 * plugin, which is forbidden to allocate; a process whose framework allocator has already
 * reserved the whole device, so that cudaMalloc would fail; a latency-critical loop that
 * cannot take the device-wide synchronisation an allocation may bring.
 *
 * This entry point calls no cudaMalloc, cudaFree or allocating library routine, and needs
 * no context.  The chunk table, the carry slots and the per-row counters of the nnz-balanced
 * kernel live in one 16 MiB array inside the library image, so every GPU that loads the library gives up
 * 16 MiB until the process exits.  A matrix whose scratch would not fit -- more than
 * (16 MiB - 1.25 KiB) / (16 + 4 K) chunks (of 128 / 160 / 256 nnz at K = 32 / 64 / 128):
 * about 15 M nnz at K = 32, 10 M at K = 64, 8 M at K = 128 -- is refused with HPSPMM_ERR_UNSUPPORTED and a message in
 * err_buf; use hpspmm_spmm_csr_f32 for it.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress,
 * once per device, with that device current).  Make that first call at start-up, before
 * any stream capture begins.  All calls on one device share the array: two calls that
 * overlap on the GPU (different streams, or different host threads) race on it, so
 * serialise them.  Nothing has to be cleared between calls: each call rewrites everything
 * it later reads.  Pointers are device pointers on device_ordinal; results equal those of
 * hpspmm_spmm_csr_f32 within the parity tolerance, and bit for bit whenever both use the
 * same nominal chunk size (K > 64, or matrices of fewer than about 4 M entries).
 * err_buf may be NULL. */
HPSPMM_API int hpspmm_spmm_csr_f32_static_scratch(int device_ordinal, int64_t M, int64_t N,
                                                  int64_t K, int64_t nnz, const int32_t* row_ptr,
                                                  const int32_t* col_idx, const float* vals,
                                                  const float* B, float* C, hpspmm_stream stream,
                                                  char* err_buf, size_t err_len);

/* Same product with HOST buffers: copies A and B to the device, runs the product,
 * copies C back, synchronises.  When K is a multiple of 32 and at least 64 the call is
 * pipelined over 32- or 64-column slabs of B and C (uploads, products and downloads overlap on
 * three internal streams, PCIe being full duplex); each slab is a product of the slab's width, so
 * the rounding of rows split across chunks can differ from the device-pointer entry point in
 * the last bits.  The overlap needs page-locked host buffers (hpspmm_host_alloc_pinned or the
 * caller's own): from pageable memory the copies are staged and serialised by the driver and the
 * call degrades to upload, product, download one after the other.  It is what the reference's
 * driver does around GESpMM (test/test_all.cpp:44-60 upload, :91-92 product) plus the download
 * the reference only performs inside its disabled checker (spmm/utils/compare.cpp:6-7). */
HPSPMM_API int hpspmm_spmm_csr_f32_host(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t K,
                                        int64_t nnz, const int32_t* row_ptr,
                                        const int32_t* col_idx, const float* vals,
                                        const float* B, float* C, const hpspmm_opts* opts);

/* Several products that share A, with HOST buffers: C_i = A * B_i for i < n_products (at most 16),
 * B_i being N x Ks[i] and C_i M x Ks[i].  A crosses PCIe once; the column slabs of all the
 * products then follow one another through one upload / product / download pipeline, so the
 * call costs about upload(A) + upload(all B_i) + product and download of the last slab.  This
 * is the shape of the reference's driver, which uploads one graph and then runs its products
 * at K = 32, 64, 128 ... on it (test/test_all.cpp:44-60, run.sh).  Widths from 1 to 512;
 * balanced kernels only.  Synchronises.  Pinned host buffers are needed for the overlap. */
HPSPMM_API int hpspmm_spmm_csr_f32_host_multi(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz,
                                              const int32_t* row_ptr, const int32_t* col_idx,
                                              const float* vals, int32_t n_products,
                                              const int64_t* Ks, const float* const* Bs,
                                              float* const* Cs, const hpspmm_opts* opts);

/* ---- COO SpMM: C += A * B --------------------------------------------------------
 * Replaces LBSpMM (include/spmm/mm/spmm_kernel.h:20, spmm/mm/spmm_kernel.cu:733-768,
 * kernel :428-477) for callers that hold the reference's padded COO arrays.  Like the
 * reference it ACCUMULATES into C (the caller zeroes C first, test/test_all.cpp:101)
 * and accepts padded entries (row 0, col 0, value 0); unlike the reference one call is
 * one product (no 200 internal launches) and padded entries are skipped rather than
 * multiplied (a NaN in B[0,:] does not leak into C[0,:]).  nnz_padded need not be a
 * multiple of 32.  Entries of one row need not be adjacent. */
HPSPMM_API int hpspmm_spmm_coo_f32(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t K,
                                   int64_t nnz_padded, const int32_t* row_idx,
                                   const int32_t* col_idx, const float* vals, const float* B,
                                   float* C, const hpspmm_opts* opts, hpspmm_stream stream);

/* ---- SDDMM over the CSR pattern: out[j] = dot(X[row(j),:], Y[col[j],:]) -------------
 * The reference ships no SDDMM (only the unused ResInfo::sddmm_* fields,
 * include/spmm/mm/spmm_common.h:130-135).  A's values are not multiplied in. */
HPSPMM_API int hpspmm_sddmm_csr_f32(hpspmm_ctx* ctx, const hpspmm_plan* plan, int64_t M,
                                    int64_t N, int64_t K, int64_t nnz, const int32_t* row_ptr,
                                    const int32_t* col_idx, const float* X, const float* Y,
                                    float* out_vals, const hpspmm_opts* opts,
                                    hpspmm_stream stream);

/* ---- CSR transpose on the device ---------------------------------------------------
 * Stable counting sort by column: row_ptr_t[N+1], col_idx_t[nnz] (source rows,
 * ascending within each transposed row), vals_t[nnz]; perm_out (optional, may be
 * NULL) receives the source position of every transposed entry.  Deterministic.
 * No counterpart in the reference. */
HPSPMM_API int hpspmm_csr_transpose(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz,
                                    const int32_t* row_ptr, const int32_t* col_idx,
                                    const float* vals, int32_t* row_ptr_t, int32_t* col_idx_t,
                                    float* vals_t, int32_t* perm_out, hpspmm_stream stream);

/* ---- aggregation layer: forward product, both backward products, cached structure -------
 * One handle per sparse operand A of a GNN aggregation C = A * H.  It owns what a training
 * loop would otherwise rebuild every step: the chunk tables of A and of its transpose, the
 * transpose itself (built on the device), and the permutation that carries new edge
 * weights into the transpose.  row_ptr, col_idx and vals are borrowed device arrays that
 * must outlive the handle.  The reference has no counterpart: its driver issues single
 * products (test/test_all.cpp:63-107) and ships neither a transpose nor an SDDMM.
 *   forward            C  = A  * H        H is N x K, C is M x K
 *   backward_features  dH = A^T * dC      dC is M x K, dH is N x K
 *   backward_weights   dA[j] = dot(dC[row(j),:], H[col[j],:])   (nnz values, CSR order)
 *   update_values      new vals pointer; the transpose's values are re-gathered from it
 * The best chunk size depends on K, so the handle keeps one pair of plans per width class
 * (K <= 32, K <= 64, wider).  create builds the pair for max_K and synchronises the stream;
 * the first product at a width of another class builds that pair (synchronising once more);
 * every other call only enqueues.  Calls on one handle must not overlap on the GPU. */
typedef struct hpspmm_layer hpspmm_layer;
HPSPMM_API int hpspmm_layer_create(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz,
                                   const int32_t* row_ptr, const int32_t* col_idx,
                                   const float* vals, int64_t max_K, hpspmm_stream stream,
                                   hpspmm_layer** out);
HPSPMM_API int hpspmm_layer_destroy(hpspmm_ctx* ctx, hpspmm_layer* layer);
HPSPMM_API int hpspmm_layer_info(const hpspmm_layer* layer, int64_t* M, int64_t* N, int64_t* nnz,
                                 int64_t* max_K, int64_t* owned_bytes);
/* device pointers to the transpose the handle owns (row_ptr_t[N+1], col_idx_t, vals_t, perm) */
HPSPMM_API int hpspmm_layer_transposed(const hpspmm_layer* layer, const int32_t** row_ptr_t,
                                       const int32_t** col_idx_t, const float** vals_t,
                                       const int32_t** perm);
HPSPMM_API int hpspmm_layer_forward(hpspmm_ctx* ctx, hpspmm_layer* layer, int64_t K,
                                    const float* H, float* C, hpspmm_stream stream);
HPSPMM_API int hpspmm_layer_backward_features(hpspmm_ctx* ctx, hpspmm_layer* layer,
                                              int64_t K, const float* dC, float* dH,
                                              hpspmm_stream stream);
HPSPMM_API int hpspmm_layer_backward_weights(hpspmm_ctx* ctx, hpspmm_layer* layer,
                                             int64_t K, const float* dC, const float* H,
                                             float* dA, hpspmm_stream stream);
HPSPMM_API int hpspmm_layer_update_values(hpspmm_ctx* ctx, hpspmm_layer* layer,
                                          const float* vals, hpspmm_stream stream);

/* ---- CSR -> padded COO (device) ------------------------------------------------------
 * Replaces the host loops of get_coo_mat_from_smtx (spmm/mm/spmm_common.cpp:210-226):
 * row_out[j] = row of entry j, then (0, 0, 0.0f) padding up to a multiple of `padding`.
 * Output arrays hold hpspmm_padded_nnz(nnz, padding) entries. */
HPSPMM_API int64_t hpspmm_padded_nnz(int64_t nnz, int64_t padding);
HPSPMM_API int hpspmm_csr_to_coo_padded(hpspmm_ctx* ctx, int64_t M, int64_t nnz,
                                        const int32_t* row_ptr, const int32_t* col_idx,
                                        const float* vals, int64_t padding, int32_t* row_out,
                                        int32_t* col_out, float* val_out, hpspmm_stream stream);

/* ---- row reordering (device) ---------------------------------------------------------------
 * The reference reorders by emitting COO rows in the order an offline permutation file names,
 * each entry keeping its original row id (get_coo_mat_from_smtx_reorder,
 * spmm/mm/spmm_common.cpp:237-296).  row_order[i] = source row emitted i-th; it must be a
 * permutation of 0..M-1 (checked on the device; HPSPMM_ERR_INVALID otherwise).  These calls
 * are set-up work: each synchronises the stream once.
 *
 * csr_to_coo_reordered: that emission, padded like hpspmm_csr_to_coo_padded; feed the arrays
 *   to hpspmm_spmm_coo_f32.  Integer outputs are bit-exact.
 * csr_permute: the CSR form A' = P * A * Q: row i of A' is row row_order[i] of A, and column c
 *   is relabelled col_new_id[c] when col_new_id is given (NULL keeps column ids).  For a
 *   symmetric reordering pass the inverse of row_order.  Entries keep their order inside a
 *   row, so relabelled columns are in general not ascending.  No counterpart in the
 *   reference, whose CSR entry has no reordered form.
 * order_rows_by_degree: row ids by descending row length, ties by ascending id (a stable
 *   radix sort).  The reference takes its order from an offline tool; this is the built-in one.
 * invert_permutation: inverse_out[order[i]] = i.
 * gather_rows_f32: dst[i, :] = src[order[i], :] for an M x K row-major matrix (dst != src);
 *   carries B or C into and out of a reordered numbering. */
HPSPMM_API int hpspmm_csr_to_coo_reordered(hpspmm_ctx* ctx, int64_t M, int64_t nnz,
                                           const int32_t* row_ptr, const int32_t* col_idx,
                                           const float* vals, const int32_t* row_order,
                                           int64_t padding, int32_t* row_out, int32_t* col_out,
                                           float* val_out, hpspmm_stream stream);
HPSPMM_API int hpspmm_csr_permute(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz,
                                  const int32_t* row_ptr, const int32_t* col_idx,
                                  const float* vals, const int32_t* row_order,
                                  const int32_t* col_new_id, int32_t* row_ptr_out,
                                  int32_t* col_out, float* val_out, hpspmm_stream stream);
HPSPMM_API int hpspmm_order_rows_by_degree(hpspmm_ctx* ctx, int64_t M, const int32_t* row_ptr,
                                           int32_t* order_out, hpspmm_stream stream);
HPSPMM_API int hpspmm_invert_permutation(hpspmm_ctx* ctx, int64_t M, const int32_t* order,
                                         int32_t* inverse_out, hpspmm_stream stream);
HPSPMM_API int hpspmm_gather_rows_f32(hpspmm_ctx* ctx, int64_t M, int64_t K, const float* src,
                                      const int32_t* order, float* dst, hpspmm_stream stream);

/* ---- validation ------------------------------------------------------------------------
 * Checks row_ptr[0] == 0, monotone row_ptr, row_ptr[M] == nnz, 0 <= col < N on the device;
 * synchronises; returns HPSPMM_ERR_BAD_CSR and the first offending position found.
 * The reference validates nothing (include/spmm/mm/spmm_kernel.h:17-21). */
HPSPMM_API int hpspmm_validate_csr(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz,
                                   const int32_t* row_ptr, const int32_t* col_idx,
                                   int64_t* bad_pos_out, hpspmm_stream stream);

/* ---- host side: seeded synthetic CSR generator --------------------------------------------
 * Replaces the .smtx dataset loaders (spmm/mm/spmm_common.cpp:125-174) for benchmarking.
 * Two-call protocol: hpspmm_gen_* builds the graph inside an opaque handle and reports its
 * size; hpspmm_gen_export copies it into caller arrays; hpspmm_gen_free releases it. */
typedef struct hpspmm_graph hpspmm_graph;
enum { HPSPMM_VALS_ONES = 0, HPSPMM_VALS_U01 = 1, HPSPMM_VALS_UPM1 = 2 };
/* rows with degree uniform in [deg_lo, deg_hi], distinct sorted columns */
HPSPMM_API int hpspmm_gen_uniform_degree(int64_t M, int64_t N, int32_t deg_lo, int32_t deg_hi,
                                         uint64_t seed, int32_t vals_kind, hpspmm_graph** out);
/* Erdos-Renyi: Poisson(mean_degree) distinct sorted columns per row */
HPSPMM_API int hpspmm_gen_erdos_renyi(int64_t M, int64_t N, double mean_degree, uint64_t seed,
                                      int32_t vals_kind, hpspmm_graph** out);
/* R-MAT: scale, edge_factor*2^scale/2 undirected draws, both directions kept,
 * duplicates removed, self loops kept, rows sorted */
HPSPMM_API int hpspmm_gen_rmat(int32_t scale, int32_t edge_factor, double a, double b, double c,
                               uint64_t seed, int32_t vals_kind, hpspmm_graph** out);
HPSPMM_API int hpspmm_gen_shape(const hpspmm_graph* g, int64_t* M, int64_t* N, int64_t* nnz);
HPSPMM_API int hpspmm_gen_export(const hpspmm_graph* g, int32_t* row_ptr, int32_t* col_idx,
                                 float* vals);
HPSPMM_API int hpspmm_gen_free(hpspmm_graph* g);

/* ---- host side: .smtx reader ---------------------------------------------------------------
 * One-pass reader of the reference's text format (spmm/mm/spmm_common.cpp:125-174):
 * line 1 "rows,cols,nnz", line 2 rows+1 offsets, line 3 nnz column ids; values are 1.0. */
HPSPMM_API int hpspmm_read_smtx(const char* path, hpspmm_graph** out);
/* Row order file of the reference (".cugraph_reorder", spmm/mm/spmm_common.cpp:262-267): one
 * line of M row ids.  Fills order_out[M]; HPSPMM_ERR_BAD_CSR unless it is a permutation. */
HPSPMM_API int hpspmm_read_row_order(const char* path, int64_t M, int32_t* order_out);

/* ---- host side: multi-GPU row sharding ---------------------------------------------------------
 * nnz-balanced contiguous row blocks: bounds[g] = first row r with row_ptr[r] >= g*nnz/G;
 * bounds has G+1 entries.  Rows are never split across shards.  The reference is
 * single-GPU; this has no counterpart there. */
HPSPMM_API int hpspmm_shard_bounds(int64_t M, const int32_t* row_ptr_host, int32_t G,
                                   int64_t* bounds);
/* The same cut with a cost per row added to the entries: bounds[g] = first row r with
 * row_ptr[r] + row_weight * r >= g * (nnz + row_weight * M) / G.  A block of many short rows writes more
 * of C and ends more rows than a block of few heavy rows with the same entries; on the power-law
 * benchmark graph a product costs about as much per row as per two to three entries.  row_weight = 0 gives
 * hpspmm_shard_bounds. */
HPSPMM_API int hpspmm_shard_bounds_weighted(int64_t M, const int32_t* row_ptr_host, int32_t G,
                                            double row_weight, int64_t* bounds);
/* Local row_ptr of shard [row_lo, row_hi): local_row_ptr[i] = row_ptr[row_lo+i] - row_ptr[row_lo],
 * row_hi-row_lo+1 entries; *nnz_lo_out / *nnz_local_out give the slice of col_idx / vals. */
HPSPMM_API int hpspmm_shard_row_ptr(const int32_t* row_ptr_host, int64_t row_lo, int64_t row_hi,
                                    int32_t* local_row_ptr, int64_t* nnz_lo_out,
                                    int64_t* nnz_local_out);

/* Which rows of B a shard references, and the shard's columns renumbered into that list.
 * col_idx_host[nnz_local] holds global column ids in [0, N); rank s owns rows
 * [b_bounds[s], b_bounds[s+1]) of B (world + 1 ascending bounds from 0 to N).  Outputs:
 * need_rows_out (capacity min(N, nnz_local)): the distinct columns, ascending, i.e. owner after
 * owner; need_off_out[world + 1]: where every owner's part starts in that list;
 * col_compact_out[nnz_local]: position of col_idx_host[j] in the list; *n_needed_out its length.
 * Integer outputs, deterministic.  No counterpart in the reference (single GPU). */
HPSPMM_API int hpspmm_shard_needed_rows(int64_t nnz_local, const int32_t* col_idx_host, int64_t N,
                                        int32_t world, const int64_t* b_bounds,
                                        int32_t* col_compact_out, int32_t* need_rows_out,
                                        int64_t* need_off_out, int64_t* n_needed_out);

/* ---- multi-GPU: row-sharded product, rows of B exchanged over NCCL -------------------------------
 * One process per GPU.  Rank r holds rows [bounds[r], bounds[r+1]) of A and of C (hpspmm_shard_bounds)
 * and the rows [b_bounds[r], b_bounds[r+1]) of B (for a square graph the same bounds: a vertex's
 * features live where its row of A lives).  C stays row-sharded.  The reference is single-GPU
 * (test/test_all.cpp:27-109); nothing below has a counterpart there.
 *
 * comm: a communicator over NCCL (looked up at run time with dlopen; NCCL is needed only when
 *   world > 1).  hpspmm_comm_unique_id on one rank, its 128 bytes carried to the others by any
 *   means the host program has, then hpspmm_comm_create on every rank (collective).
 * shard plan (collective, synchronises): from the shard's HOST row_ptr / col_idx it lists the rows of B
 *   the shard references per owner (HPSPMM_EXCHANGE_NEEDED_ROWS, and ..._NCCL, which differs in the
 *   transport only) or takes all of them (HPSPMM_EXCHANGE_ALL_ROWS, the plain all-gather), renumbers
 *   the shard's columns into that list, tells every owner which rows to send, and keeps device copies
 *   of row_ptr and the renumbered columns.  Every rank must pass the same b_bounds, max_K and mode.
 * exchange_begin: enqueues, on the plan's own stream and after what `stream` holds now, the transfer
 *   of the rows the other ranks need: one kernel that stores them into the receivers' operands over
 *   NVLink followed by a four-byte NCCL all-reduce as the completion signal, or (the NCCL transports)
 *   a packing kernel and one grouped send / receive.  Remote rows land in this GPU's own memory
 *   before any product reads them.  A slot must not be begun again before its product has been
 *   enqueued.  If some rank cannot map another rank's buffers (no peer access, IPC not permitted),
 *   all ranks switch together to the NCCL transport.
 * product: waits (stream event) for that slot's rows, then runs the local product on `stream`.
 *   Slots 0..3 are independent buffers: begin several products, then multiply them in turn, and each
 *   exchange overlaps the previous product.  All ranks must issue their begins in the same order.
 *   The first use of a slot (or a wider K on it) allocates, is collective, and synchronises.
 * hpspmm_spmm_sharded_f32 = exchange_begin + product on slot 0.
 * destroy: collective when world > 1 and a slot was used (the ranks unmap each other's buffers, meet, then
 *   free their own); call it once the last product has completed on this rank, before hpspmm_comm_destroy.
 * vals: the shard's values (device, nnz_local); B_own: rows_own x K (device); C_local: M_local x K.
 * No kernel reads another GPU's memory and nothing waits on the device: ordering is by stream events
 * and by the completion of NCCL operations. */
typedef struct hpspmm_comm hpspmm_comm;
typedef struct hpspmm_shard_plan hpspmm_shard_plan;
enum { HPSPMM_COMM_ID_BYTES = 128 };
enum {
  HPSPMM_EXCHANGE_NEEDED_ROWS = 0,      /* referenced rows only, pushed into the receivers' operands by
                                           peer stores (CUDA IPC mappings), NCCL only as the signal      */
  HPSPMM_EXCHANGE_ALL_ROWS = 1,         /* plain all-gather of B over NCCL send / receive               */
  HPSPMM_EXCHANGE_NEEDED_ROWS_NCCL = 2  /* referenced rows only, packed and sent by ncclSend / ncclRecv */
};
HPSPMM_API int hpspmm_comm_unique_id(unsigned char* id_out);
HPSPMM_API int hpspmm_comm_create(hpspmm_ctx* ctx, int32_t world, int32_t rank,
                                  const unsigned char* id, hpspmm_comm** out);
HPSPMM_API int hpspmm_comm_destroy(hpspmm_comm* comm);
HPSPMM_API int hpspmm_comm_info(const hpspmm_comm* comm, int32_t* world, int32_t* rank);
HPSPMM_API int hpspmm_shard_plan_create(hpspmm_ctx* ctx, hpspmm_comm* comm, int64_t M_local,
                                        int64_t N, int64_t nnz_local, const int32_t* row_ptr_host,
                                        const int32_t* col_idx_host, const int64_t* b_bounds,
                                        int64_t max_K, int32_t exchange, hpspmm_stream stream,
                                        hpspmm_shard_plan** out);
HPSPMM_API int hpspmm_shard_plan_destroy(hpspmm_ctx* ctx, hpspmm_shard_plan* plan);
/* rows of the local dense operand (own + received), rows received from and sent to other ranks
 * per product, device bytes the plan holds */
HPSPMM_API int hpspmm_shard_plan_info(const hpspmm_shard_plan* plan, int64_t* rows_local,
                                      int64_t* rows_received, int64_t* rows_sent,
                                      int64_t* device_bytes);
HPSPMM_API int hpspmm_sharded_exchange_begin(hpspmm_ctx* ctx, hpspmm_shard_plan* plan, int32_t slot,
                                             int64_t K, const float* B_own, hpspmm_stream stream);
HPSPMM_API int hpspmm_sharded_product(hpspmm_ctx* ctx, hpspmm_shard_plan* plan, int32_t slot,
                                      int64_t K, const float* vals, float* C_local,
                                      const hpspmm_opts* opts, hpspmm_stream stream);
HPSPMM_API int hpspmm_spmm_sharded_f32(hpspmm_ctx* ctx, hpspmm_shard_plan* plan, int64_t K,
                                       const float* vals, const float* B_own, float* C_local,
                                       const hpspmm_opts* opts, hpspmm_stream stream);

/* ---- host side: metric -----------------------------------------------------------------------------
 * GFLOPS = 2*nnz*K / ms / 1e6 with the unpadded nnz (spmm/mm/spmm_common.cpp:24-31);
 * row-length coefficient of variation (spmm/mm/spmm_common.cpp:57-67, :349-374). */
HPSPMM_API double hpspmm_gflops(int64_t nnz, int64_t K, double ms);
HPSPMM_API double hpspmm_row_length_cv(int64_t M, const int32_t* row_ptr_host);
/* Compulsory bytes of one product: 4(M+1) + 8 nnz + 4 K N_ref + 4 K M. */
HPSPMM_API double hpspmm_spmm_algorithmic_bytes(int64_t M, int64_t N_ref, int64_t K, int64_t nnz);
HPSPMM_API double hpspmm_sddmm_algorithmic_bytes(int64_t M_ref, int64_t N_ref, int64_t K,
                                                 int64_t M, int64_t nnz);

/* ---- diagnostics: allocation-failure seam ------------------------------------------------------------
 * Test hook: starting with the nth device allocation the library makes from now on (1 = the next one),
 * `count` allocations in a row report an out-of-memory error without touching the device; nth = 0
 * disarms.  Process-wide, meant for single-threaded tests.  Lets a test see that every entry point
 * that allocates returns HPSPMM_ERR_OOM, frees what it had already taken and leaves the context usable
 * -- where the reference ignores the result of cudaMalloc altogether
 * (spmm/starml/basic/allocator_cuda.cpp:5-13). */
HPSPMM_API int hpspmm_debug_fail_device_alloc(int64_t nth, int64_t count);

/* ---- diagnostics: load-path ceilings ---------------------------------------------------------------
 * Times the gather shape of the product kernels alone (lane groups of row_bytes / 16 lanes,
 * one 16-byte load per lane, four gathers in flight per lane, no sparse stream, no stores):
 * n_gathers rows of row_bytes (128, 256 or 512) bytes from a zero-filled table of table_rows rows
 * that the call allocates and frees.  pattern 0 walks the table row after row (a stream), 1 picks
 * rows uniformly at random, 2 does the same but sends a share hot_share of the gathers to the first
 * hot_rows rows.  A table smaller than the L2 cache gives the L2 -> SM ceiling, a larger one the
 * DRAM-backed gather rate.  Returns GB/s (and ms per launch) averaged over `repeats` launches after
 * three warm-up launches; synchronises.  The reference has no counterpart (its README reports
 * kernel GFLOPS only); the number bounds what any gather-based product can reach on the GPU. */
HPSPMM_API int hpspmm_probe_gather_gbs(hpspmm_ctx* ctx, int32_t row_bytes, int64_t table_rows,
                                       int64_t n_gathers, int32_t pattern, int64_t hot_rows,
                                       double hot_share, int32_t repeats, double* gbs_out,
                                       double* ms_out);

/* Number of warps of the HPSPMM_ALGO_TMA kernel, since the context was created, whose bounded wait for a
 * TMA copy ran out; such a warp finishes its chunk with ordinary loads, so results are unaffected and the
 * count is a health check (expected: 0).  Synchronises the device. */
HPSPMM_API int hpspmm_ctx_tma_fallbacks(hpspmm_ctx* ctx, int64_t* count);

/* The same random rows through the tensor memory accelerator: producer warps fetch four rows per
 * instruction into shared memory (cp.async.bulk.tensor ... tile::gather4 on a tensor map of the table),
 * consumer warps read every delivered byte into registers.  row_bytes is 128, 256 or 512; the table is
 * allocated and filled by the probe (row r holds the value r mod 251 in every column); ctas_per_sm is 1
 * to 3 (each CTA: four producer and eight consumer warps over four 16 KB buffers).  n_gathers is rounded
 * up to whole buffers per CTA; *gathers_done_out receives the number performed and *checksum_out the sum
 * of everything the consumers read, which a caller can replay on the host (gather i reads row
 * umulhi(((h ^ (h >> 15)) * 2246822519), table_rows) with h = i * 2654435761, 32-bit arithmetic).
 * Every wait inside the kernel is bounded; one that runs out returns HPSPMM_ERR_CUDA with a message.
 * HPSPMM_ERR_UNSUPPORTED when the driver has no cuTensorMapEncodeTiled.  The reference has no
 * counterpart. */
HPSPMM_API int hpspmm_probe_tma_gather_gbs(hpspmm_ctx* ctx, int32_t row_bytes, int64_t table_rows,
                                           int64_t n_gathers, int32_t ctas_per_sm, int32_t repeats,
                                           double* gbs_out, double* ms_out, double* checksum_out,
                                           int64_t* gathers_done_out);

#ifdef __cplusplus
}
#endif
#endif /* HPSPMM_H_ */
