// Integer / structure work around the SpMM path: CSR validation, CSR -> padded COO row
// expansion (the device form of spmm/mm/spmm_common.cpp:210-226), and a deterministic CSR
// transpose (stable LSD radix sort of the entry positions by column index).  All outputs
// are integer-exact and independent of thread scheduling.
#include "hpspmm_internal.h"

namespace {

constexpr int kThreads = 256;

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// row holding entry j: last r with row_ptr[r] <= j
__device__ __forceinline__ int row_of_entry(const int* __restrict__ row_ptr, int M, int j) {
  int lo = 0, hi = M + 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(row_ptr + mid) <= j)
      lo = mid + 1;
    else
      hi = mid;
  }
  const int r = lo - 1;
  return r < 0 ? 0 : (r > M - 1 ? M - 1 : r);
}

// The same search by a whole block (every thread must call it, every thread gets the answer): each round
// probes blockDim.x evenly spaced candidates at once, so a million rows take three rounds of one load
// each instead of twenty dependent loads.
__device__ __forceinline__ int row_of_entry_by_block(const int* __restrict__ row_ptr, int M, int j) {
  int64_t lo = 0, hi = (int64_t)M + 1;           // row_ptr[lo] <= j always holds (row_ptr[0] = 0)
  while (hi - lo > 1) {
    const int64_t step = (hi - lo + blockDim.x - 1) / blockDim.x;
    const int64_t r = lo + (int64_t)threadIdx.x * step;
    const int below = __syncthreads_count(r < hi && __ldg(row_ptr + r) <= j);   // >= 1: thread 0 probes lo
    const int64_t new_lo = lo + (int64_t)(below - 1) * step;
    const int64_t new_hi = new_lo + step;
    lo = new_lo;
    hi = new_hi < hi ? new_hi : hi;
  }
  const int r = (int)lo;
  return r > M - 1 ? M - 1 : r;
}

// ---- validation ------------------------------------------------------------------------
// bad[0] = smallest offending position + 1 (rows first, then M + 1 + entry index), 0 if none
__global__ void validate_csr_kernel(int64_t M, int64_t N, int64_t nnz, const int* __restrict__ row_ptr,
                                    const int* __restrict__ col_idx, unsigned long long* bad) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M + 1 + nnz; i += stride) {
    bool ok = true;
    if (i <= M) {
      const int v = row_ptr[i];
      if (i == 0) ok = v == 0;
      if (i == M) ok = ok && v == nnz;
      if (i > 0) ok = ok && v >= row_ptr[i - 1];
      ok = ok && v >= 0 && v <= nnz;
    } else {
      const int c = col_idx[i - M - 1];
      ok = c >= 0 && c < N;
    }
    if (!ok) atomicMin(bad, (unsigned long long)(i + 1));
  }
}

// ---- CSR -> COO ------------------------------------------------------------------------
// One block per tile of 4096 entries.  The rows that begin inside the tile mark their first entry with
// their index (empty rows share a position with the row that owns it; the largest index wins, which is
// the owner); a running maximum over the tile then gives every entry its row.  Two binary searches per
// tile instead of one per entry, and every global access is coalesced.  Positions past nnz are padding
// and receive zeros.  PAIRS writes (row, value bits) as one 8-byte word per entry instead of the arrays.
constexpr int kExpandTile = 4096;
template <bool PAIRS>
__global__ void __launch_bounds__(kThreads)
expand_rows_kernel(int M, int64_t nnz, int64_t padded, const int* __restrict__ row_ptr,
                   const int* __restrict__ col_idx, const float* __restrict__ vals, int* __restrict__ row_out,
                   int* __restrict__ col_out, float* __restrict__ val_out, int2* __restrict__ pair_out) {
  constexpr int kWarpsHere = kThreads / 32;
  constexpr int kSpan = kExpandTile / kWarpsHere;     // contiguous entries per warp
  __shared__ int head[kExpandTile];
  __shared__ int warp_max[kWarpsHere];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t start = (int64_t)blockIdx.x * kExpandTile;
  const int live = (int)(nnz - start < kExpandTile ? (nnz > start ? nnz - start : 0) : kExpandTile);
  if (live > 0) {
    for (int i = threadIdx.x; i < kExpandTile; i += kThreads) head[i] = -1;
    const int r_first = row_of_entry_by_block(row_ptr, M, (int)start);
    const int r_last = row_of_entry_by_block(row_ptr, M, (int)(start + live - 1));
    for (int r = r_first + threadIdx.x; r <= r_last; r += kThreads) {
      const int64_t p = (int64_t)__ldg(row_ptr + r) - start;
      if (p < live) atomicMax(&head[p < 0 ? 0 : (int)p], r);
    }
    __syncthreads();
    int m = -1;
#pragma unroll 4
    for (int s = 0; s < kSpan / 32; ++s) m = max(m, head[warp * kSpan + s * 32 + lane]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) warp_max[warp] = m;
    __syncthreads();
  }
  int carry = -1;
  if (live > 0)
    for (int w = 0; w < warp; ++w) carry = max(carry, warp_max[w]);
  // what the tile copies is fetched before the scan, all loads in flight at once
  constexpr int kStepsHere = kSpan / 32;
  int c_in[PAIRS ? 1 : kStepsHere];
  float v_in[kStepsHere];
#pragma unroll
  for (int s = 0; s < kStepsHere; ++s) {
    const int i = warp * kSpan + s * 32 + lane;
    const int64_t j = start + i;
    v_in[s] = i < live && vals && (PAIRS || val_out) ? vals[j] : 0.f;
    if (!PAIRS) c_in[s] = i < live && col_out ? col_idx[j] : 0;
  }
#pragma unroll
  for (int s = 0; s < kStepsHere; ++s) {
    const int i = warp * kSpan + s * 32 + lane;
    const int64_t j = start + i;
    int r = i < live ? head[i] : -1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, r, o);
      if (lane >= o) r = max(r, t);
    }
    r = max(r, carry);
    carry = __shfl_sync(0xffffffffu, r, 31);
    if (j < padded) {
      const int row = i < live ? r : 0;
      if (PAIRS) {
        pair_out[j] = make_int2(row, __float_as_int(v_in[s]));
      } else {
        row_out[j] = row;
        if (col_out) col_out[j] = c_in[s];
        if (val_out) val_out[j] = v_in[s];
      }
    }
  }
}

// ---- radix sort passes -----------------------------------------------------------------
constexpr int kItems = 16;                      // keys per thread
constexpr int kTile = kThreads * kItems;        // keys per block
constexpr int kWarps = kThreads / 32;
constexpr int kWarpSpan = kTile / kWarps;       // contiguous keys per warp
constexpr int kSteps = kWarpSpan / 32;          // == kItems

// hist[d * n_tiles + tile] = number of keys of the tile with digit d
__global__ void __launch_bounds__(kThreads)
radix_hist_kernel(const int* __restrict__ keys, int64_t n, int shift, int n_tiles,
                  int* __restrict__ hist) {
  __shared__ int cnt[256];
  cnt[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kTile;
  for (int i = 0; i < kItems; ++i) {
    const int64_t idx = base + (int64_t)i * kThreads + threadIdx.x;
    if (idx < n) atomicAdd(&cnt[(keys[idx] >> shift) & 255], 1);
  }
  __syncthreads();
  hist[(int64_t)threadIdx.x * n_tiles + blockIdx.x] = cnt[threadIdx.x];
}

// Exclusive scan in three steps: per-block totals, scan of the totals by one block, rescan.
constexpr int kScanTile = 4096;
__global__ void __launch_bounds__(kThreads)
scan_block_totals_kernel(const int* __restrict__ in, int64_t n, int* __restrict__ totals) {
  __shared__ int red[kThreads];
  const int64_t base = (int64_t)blockIdx.x * kScanTile;
  int s = 0;
  for (int i = threadIdx.x; i < kScanTile; i += kThreads)
    if (base + i < n) s += in[base + i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = kThreads / 2; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = red[0];
}

// in-place exclusive scan of `n` ints by a single block
__global__ void __launch_bounds__(kThreads)
scan_single_block_kernel(int* __restrict__ data, int64_t n) {
  __shared__ int part[kThreads];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += kThreads) {
    const int64_t i = base + threadIdx.x;
    const int v = i < n ? data[i] : 0;
    part[threadIdx.x] = v;
    __syncthreads();
    for (int o = 1; o < kThreads; o <<= 1) {
      const int t = (int)threadIdx.x >= o ? part[threadIdx.x - o] : 0;
      __syncthreads();
      part[threadIdx.x] += t;
      __syncthreads();
    }
    if (i < n) data[i] = carry + part[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == kThreads - 1) carry += part[threadIdx.x];
    __syncthreads();
  }
}

// out[i] = totals_scanned[block] + exclusive prefix inside the block's tile; in-place safe
__global__ void __launch_bounds__(kThreads)
scan_rescan_kernel(int* __restrict__ data, int64_t n, const int* __restrict__ totals_scanned) {
  __shared__ int part[kThreads];
  constexpr int per = kScanTile / kThreads;
  const int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * per;
  int v[per];
  int s = 0;
  // a thread's 16 values are 64 contiguous bytes: four 16-byte accesses when the tile is full and aligned
  const bool vec = per % 4 == 0 && base + per <= n && (reinterpret_cast<uintptr_t>(data) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int i = 0; i < per; i += 4) {
      const int4 q = *reinterpret_cast<const int4*>(data + base + i);
      v[i] = q.x, v[i + 1] = q.y, v[i + 2] = q.z, v[i + 3] = q.w;
      s += q.x + q.y + q.z + q.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < per; ++i) {
      v[i] = base + i < n ? data[base + i] : 0;
      s += v[i];
    }
  }
  part[threadIdx.x] = s;
  __syncthreads();
  for (int o = 1; o < kThreads; o <<= 1) {
    const int t = (int)threadIdx.x >= o ? part[threadIdx.x - o] : 0;
    __syncthreads();
    part[threadIdx.x] += t;
    __syncthreads();
  }
  int run = totals_scanned[blockIdx.x] + part[threadIdx.x] - s;
  if (vec) {
#pragma unroll
    for (int i = 0; i < per; i += 4) {
      int4 q;
      q.x = run, run += v[i];
      q.y = run, run += v[i + 1];
      q.z = run, run += v[i + 2];
      q.w = run, run += v[i + 3];
      *reinterpret_cast<int4*>(data + base + i) = q;
    }
  } else {
#pragma unroll
    for (int i = 0; i < per; ++i) {
      if (base + i < n) data[base + i] = run;
      run += v[i];
    }
  }
}

// Stable scatter of one 8-bit digit.  Warp w of a block owns keys
// [tile + w*kWarpSpan, tile + (w+1)*kWarpSpan) and walks them 32 at a time, so that
// (warp, step, lane) order is ascending key position; ranks among equal digits follow it.
// payload_in == nullptr means the payload of key i is i itself.
// If final_* outputs are given, the pass writes the transposed matrix directly.
__global__ void __launch_bounds__(kThreads)
radix_scatter_kernel(const int* __restrict__ keys_in, const int* __restrict__ payload_in, int64_t n,
                     int shift, int n_tiles, const int* __restrict__ hist_scanned,
                     int* __restrict__ keys_out, int* __restrict__ payload_out) {
  __shared__ int cnt[kWarps][256];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kWarps * 256; i += kThreads) (&cnt[0][0])[i] = 0;
  __syncthreads();

  const int64_t wbase = (int64_t)blockIdx.x * kTile + (int64_t)warp * kWarpSpan;
  int key[kSteps], pay[kSteps], rank[kSteps];
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int64_t idx = wbase + s * 32 + lane;
    const bool valid = idx < n;
    key[s] = valid ? keys_in[idx] : 0;
    pay[s] = valid ? (payload_in ? payload_in[idx] : (int)idx) : 0;
    const int d = (key[s] >> shift) & 255;
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? d : (0x10000 | lane));
    const int leader = __ffs(peers) - 1;
    int before = 0;
    if (valid && lane == leader) {
      before = cnt[warp][d];
      cnt[warp][d] = before + __popc(peers);
    }
    before = __shfl_sync(0xffffffffu, before, leader);
    rank[s] = before + __popc(peers & ((1u << lane) - 1u));
    __syncwarp();
  }
  __syncthreads();
  {
    // digit threadIdx.x: turn per-warp counts into per-warp output offsets
    const int d = threadIdx.x;
    int run = hist_scanned[(int64_t)d * n_tiles + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int t = cnt[w][d];
      cnt[w][d] = run;
      run += t;
    }
  }
  __syncthreads();
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int64_t idx = wbase + s * 32 + lane;
    if (idx < n) {
      const int d = (key[s] >> shift) & 255;
      const int pos = cnt[warp][d] + rank[s];
      keys_out[pos] = key[s];
      payload_out[pos] = pay[s];
    }
  }
}

// ---- transpose passes: (column, entry position) pairs, digits of 8, 10 or 11 bits -------------
// The transpose sorts 64-bit (key, payload) pairs so that a pass moves one 8-byte word per entry, and
// takes digits wide enough for two passes up to 2^22 columns.  Per-warp digit counts are 16-bit (a warp
// owns kWarpSpan = 512 keys), which keeps 2048 bins x 8 warps inside the static shared-memory limit.
template <int DBITS>
__global__ void __launch_bounds__(kThreads)
pair_hist_kernel(const int* __restrict__ keys, const int2* __restrict__ pairs, int64_t n, int shift,
                 int n_tiles, int* __restrict__ hist) {
  constexpr int D = 1 << DBITS;
  __shared__ int cnt[D];
  for (int d = threadIdx.x; d < D; d += kThreads) cnt[d] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kTile;
  int k[kItems];
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const int64_t idx = base + (int64_t)i * kThreads + threadIdx.x;
    k[i] = idx < n ? (pairs ? pairs[idx].x : keys[idx]) : -1;
  }
#pragma unroll
  for (int i = 0; i < kItems; ++i)
    if (k[i] >= 0) atomicAdd(&cnt[(k[i] >> shift) & (D - 1)], 1);
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += kThreads) hist[(int64_t)d * n_tiles + blockIdx.x] = cnt[d];
}

// Stable scatter of one digit, same ranking scheme as radix_scatter_kernel.  pairs_in == nullptr is the
// first pass: key i is keys_in[i] and its payload is i.
template <int DBITS>
__global__ void __launch_bounds__(kThreads, 3)
pair_scatter_kernel(const int* __restrict__ keys_in, const int2* __restrict__ pairs_in, int64_t n, int shift,
                    int n_tiles, const int* __restrict__ hist_scanned, int2* __restrict__ pairs_out) {
  constexpr int D = 1 << DBITS;
  __shared__ unsigned short cnt[kWarps][D];
  __shared__ int tile_base[D];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kWarps * D; i += kThreads) (&cnt[0][0])[i] = 0;
  __syncthreads();

  const int64_t wbase = (int64_t)blockIdx.x * kTile + (int64_t)warp * kWarpSpan;
  // The keys are fetched up front, all loads in flight at once: the ranking loop below synchronises the
  // warp at every step, and a load issued inside it would wait out its whole latency sixteen times.
  // Payloads are not held; the scatter reads them again (the tile is 32 KB and still in cache).
  int key[kSteps];
  unsigned short rank[kSteps];
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int64_t idx = wbase + s * 32 + lane;
    key[s] = idx < n ? (pairs_in ? pairs_in[idx].x : keys_in[idx]) : 0;
  }
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int64_t idx = wbase + s * 32 + lane;
    const bool valid = idx < n;
    const int k = key[s];
    const int d = (k >> shift) & (D - 1);
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? d : (0x10000 | lane));
    const int leader = __ffs(peers) - 1;
    int before = 0;
    if (valid && lane == leader) {
      before = cnt[warp][d];
      cnt[warp][d] = (unsigned short)(before + __popc(peers));
    }
    before = __shfl_sync(0xffffffffu, before, leader);
    rank[s] = (unsigned short)(before + __popc(peers & ((1u << lane) - 1u)));
    __syncwarp();
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += kThreads) {
    // per-warp counts -> offsets of each warp's keys inside the tile's run of digit d
    int run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int t = cnt[w][d];
      cnt[w][d] = (unsigned short)run;
      run += t;
    }
    tile_base[d] = hist_scanned[(int64_t)d * n_tiles + blockIdx.x];
  }
  __syncthreads();
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int64_t idx = wbase + s * 32 + lane;
    if (idx < n) {
      const int d = (key[s] >> shift) & (D - 1);
      pairs_out[tile_base[d] + cnt[warp][d] + rank[s]] = make_int2(key[s], pairs_in ? pairs_in[idx].y : (int)idx);
    }
  }
}

// row_ptr_t[c] = number of sorted pairs with key < c
__global__ void transposed_row_ptr_pairs_kernel(const int2* __restrict__ sorted, int64_t nnz, int64_t N,
                                                int* __restrict__ row_ptr_t) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c <= N; c += stride) {
    int64_t lo = 0, hi = nnz;
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if ((int64_t)__ldg(&sorted[mid].x) < c)
        lo = mid + 1;
      else
        hi = mid;
    }
    row_ptr_t[c] = (int)lo;
  }
}

// transposed entry t comes from entry sorted[t].y of the source: its row becomes the column index
__global__ void transposed_emit_kernel(int64_t nnz, const int2* __restrict__ sorted,
                                       const int2* __restrict__ row_val, int* __restrict__ col_idx_t,
                                       float* __restrict__ vals_t, int* __restrict__ perm_out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < nnz; t += stride) {
    const int j = sorted[t].y;
    const int2 e = __ldg(row_val + j);
    col_idx_t[t] = e.x;
    if (vals_t) vals_t[t] = __int_as_float(e.y);
    if (perm_out) perm_out[t] = j;
  }
}

// one pass: histogram per tile and digit, exclusive scan of the digit-major matrix, stable scatter
template <int DBITS>
void launch_pair_pass(const int* keys_in, const int2* pairs_in, int64_t n, int shift, int n_tiles, int* hist,
                      int* totals, int2* pairs_out, cudaStream_t s) {
  const int64_t hist_n = ((int64_t)1 << DBITS) * n_tiles;
  const int64_t scan_blocks = (hist_n + kScanTile - 1) / kScanTile;
  pair_hist_kernel<DBITS><<<n_tiles, kThreads, 0, s>>>(keys_in, pairs_in, n, shift, n_tiles, hist);
  scan_block_totals_kernel<<<(unsigned)scan_blocks, kThreads, 0, s>>>(hist, hist_n, totals);
  scan_single_block_kernel<<<1, kThreads, 0, s>>>(totals, scan_blocks);
  scan_rescan_kernel<<<(unsigned)scan_blocks, kThreads, 0, s>>>(hist, hist_n, totals);
  pair_scatter_kernel<DBITS><<<n_tiles, kThreads, 0, s>>>(keys_in, pairs_in, n, shift, n_tiles, hist, pairs_out);
}

// Sort key of chunk c (ascending = earlier).  Without col_idx: 255 - cost (8 bits).  With col_idx, 16 bits:
//   Chunks that span row ends: (255 - cost) << 7 with cost = entries / 8 (gather batches) + rows / 2
//   (each row end costs a cross-group reduction, a store and a step along row_ptr), capped at 255:
//   the most expensive first.
//   Chunks that lie inside one row (pieces of heavy rows): 32768 + (first column >> col_shift), so that
//   they follow all the others and run in ascending order of the column band they gather from.  Column
//   indices ascend inside a row, so pieces of different heavy rows that run at the same time read the
//   same band of B and find it in L2.  Without col_idx these chunks sort by cost like the rest.
__global__ void chunk_cost_key_kernel(int M, int64_t n_chunks, const int* __restrict__ chunk_start,
                                      const int* __restrict__ chunk_row, const int* __restrict__ row_ptr,
                                      const int* __restrict__ col_idx, int col_shift,
                                      int* __restrict__ keys) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += stride) {
    const int next = c + 1 < n_chunks ? chunk_row[c + 1] : M;
    const int r0 = chunk_row[c];
    int rows = next - r0;
    rows = rows < 0 ? 0 : rows;
    const int n0 = chunk_start[c], n1 = chunk_start[c + 1];
    const int entries = n1 - n0;
    int cost = (entries >> 3) + (rows >> 1);
    cost = cost > 255 ? 255 : cost;
    int key = 255 - cost;
    if (col_idx != nullptr) {
      key <<= 7;
      if (entries >= 32 && r0 < M && __ldg(row_ptr + r0 + 1) >= n1)
        key = 32768 + min(32767, __ldg(col_idx + n0) >> col_shift);
    }
    keys[c] = key;
  }
}

// ---- row reordering ----------------------------------------------------------------------
// len[i] = length of row order[i]; hits[order[i]] counts how often a row is named.
// flag: bit 0 = an index outside [0, M), bit 1 = a row named twice.
__global__ void ordered_row_lengths_kernel(int M, const int* __restrict__ row_ptr, const int* __restrict__ order,
                                           int* __restrict__ len, int* __restrict__ hits, int* flag) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= M; i += stride) {
    if (i == M) {
      len[i] = 0;
      continue;
    }
    const int r = order[i];
    if (r < 0 || r >= M) {
      len[i] = 0;
      atomicOr(flag, 1);
      continue;
    }
    len[i] = row_ptr[r + 1] - row_ptr[r];
    if (atomicAdd(hits + r, 1) != 0) atomicOr(flag, 2);
  }
}

// Output entry t lies in output row i = last i with new_ptr[i] <= t; it is entry
// row_ptr[order[i]] + (t - new_ptr[i]) of the source.  row_out (optional) receives the source
// row id, col_new_id (optional) relabels columns, entries in [nnz, padded) become (0, 0, 0).
__global__ void permute_rows_kernel(int M, int64_t nnz, int64_t padded, const int* __restrict__ new_ptr,
                                    const int* __restrict__ row_ptr, const int* __restrict__ order,
                                    const int* __restrict__ col_idx, const float* __restrict__ vals,
                                    const int* __restrict__ col_new_id, int* __restrict__ row_out,
                                    int* __restrict__ col_out, float* __restrict__ val_out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < padded; t += stride) {
    if (t >= nnz) {
      if (row_out) row_out[t] = 0;
      if (col_out) col_out[t] = 0;
      if (val_out) val_out[t] = 0.f;
      continue;
    }
    const int i = row_of_entry(new_ptr, M, (int)t);
    const int r = __ldg(order + i);
    const int64_t src = (int64_t)__ldg(row_ptr + r) + (t - __ldg(new_ptr + i));
    if (row_out) row_out[t] = r;
    if (col_out) {
      const int c = col_idx[src];
      col_out[t] = col_new_id ? __ldg(col_new_id + c) : c;
    }
    if (val_out) val_out[t] = vals[src];
  }
}

__global__ void degree_key_kernel(int M, const int* __restrict__ row_ptr, int* __restrict__ keys) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < M; r += stride)
    keys[r] = 0x7fffffff - (row_ptr[r + 1] - row_ptr[r]);   // ascending key = descending degree
}

__global__ void invert_permutation_kernel(int M, const int* __restrict__ order, int* __restrict__ inv) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M; i += stride) {
    const int r = order[i];
    if (r >= 0 && r < M) inv[r] = (int)i;
  }
}

// dst[i, :] = src[order[i], :], 16 bytes per thread when K % 4 == 0
template <typename T>
__global__ void gather_rows_kernel(int64_t M, int64_t row_elems, const T* __restrict__ src,
                                   const int* __restrict__ order, T* __restrict__ dst) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t total = M * row_elems;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t i = t / row_elems, c = t - i * row_elems;
    dst[t] = src[(int64_t)__ldg(order + i) * row_elems + c];
  }
}

unsigned grid_for(const hpspmm_ctx* ctx, int64_t n) {
  int64_t b = (n + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)ctx->sm_count * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

// in-place exclusive scan of n ints; totals needs ceil(n / kScanTile) ints
void exclusive_scan_inplace(hpspmm_ctx* ctx, int* data, int64_t n, int* totals, cudaStream_t s) {
  const int64_t blocks = (n + kScanTile - 1) / kScanTile;
  scan_block_totals_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(data, n, totals);
  scan_single_block_kernel<<<1, kThreads, 0, s>>>(totals, blocks);
  scan_rescan_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(data, n, totals);
  ctx->launches += 3;
}

// new_ptr[0..M] = offsets of the rows taken in `order`; checks that order is a permutation.
// new_ptr may be caller memory (the permuted CSR's row_ptr) or context scratch.
int build_ordered_row_ptr(hpspmm_ctx* ctx, int64_t M, const int32_t* row_ptr, const int32_t* order,
                          int32_t* new_ptr, int* hits, int* totals, cudaStream_t s) {
  HPSPMM_CUDA_TRY(ctx, cudaMemsetAsync(hits, 0, (size_t)(M > 0 ? M : 1) * 4, s));
  HPSPMM_CUDA_TRY(ctx, cudaMemsetAsync(ctx->flag, 0, sizeof(int), s));
  ordered_row_lengths_kernel<<<grid_for(ctx, M + 1), kThreads, 0, s>>>((int)M, row_ptr, order, new_ptr, hits,
                                                                      ctx->flag);
  ctx->launches++;
  exclusive_scan_inplace(ctx, new_ptr, M + 1, totals, s);
  int flag = 0;
  HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(&flag, ctx->flag, sizeof(int), cudaMemcpyDeviceToHost, s));
  HPSPMM_CUDA_TRY(ctx, cudaStreamSynchronize(s));
  if (flag != 0) {
    snprintf(ctx->err, sizeof(ctx->err), "row_order is not a permutation of 0..M-1 (%s)",
             (flag & 1) ? "index out of range" : "a row is named twice");
    return HPSPMM_ERR_INVALID;
  }
  return HPSPMM_OK;
}

}  // namespace

// ---- list of the rows that hold entries -------------------------------------------------------
namespace {

__global__ void nonempty_flag_kernel(int M, const int* __restrict__ row_ptr, int* __restrict__ flags) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r <= M; r += stride)
    flags[r] = r < M ? (row_ptr[r + 1] > row_ptr[r] ? 1 : 0) : 0;
}

// rank[r] = number of rows before r that hold entries (rank[M] = their total)
__global__ void row_list_scatter_kernel(int M, const int* __restrict__ row_ptr, const int* __restrict__ rank,
                                        int* __restrict__ nz_id, int* __restrict__ nz_end) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r <= M; r += stride) {
    if (r == M) {
      // sentinel after the last row: never a row of C, an end no entry reaches
      nz_id[rank[M]] = M;
      nz_end[rank[M]] = 0x7fffffff;
    } else if (row_ptr[r + 1] > row_ptr[r]) {
      nz_id[rank[r]] = (int)r;
      nz_end[rank[r]] = row_ptr[r + 1];
    }
  }
}

__global__ void chunk_row_index_kernel(int64_t n_chunks, const int* __restrict__ chunk_row,
                                       const int* __restrict__ rank, int* __restrict__ chunk_ri) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += stride)
    chunk_ri[c] = rank[chunk_row[c]];
}

}  // namespace

size_t hpspmm_row_list_scratch_bytes(int64_t M) {
  return align_up((size_t)(M + 1) * 4, 256) + align_up((size_t)((M + 1 + kScanTile - 1) / kScanTile + 1) * 4, 256);
}

int hpspmm_build_row_list(hpspmm_ctx* ctx, int64_t M, int64_t n_chunks, const int32_t* row_ptr,
                          const int32_t* chunk_row, int32_t* nz_id, int32_t* nz_end, int32_t* chunk_ri,
                          void* scratch, cudaStream_t stream) {
  int* rank = (int*)scratch;
  int* totals = (int*)((char*)scratch + align_up((size_t)(M + 1) * 4, 256));
  nonempty_flag_kernel<<<grid_for(ctx, M + 1), kThreads, 0, stream>>>((int)M, row_ptr, rank);
  ctx->launches++;
  exclusive_scan_inplace(ctx, rank, M + 1, totals, stream);
  row_list_scatter_kernel<<<grid_for(ctx, M + 1), kThreads, 0, stream>>>((int)M, row_ptr, rank, nz_id, nz_end);
  if (n_chunks > 0)
    chunk_row_index_kernel<<<grid_for(ctx, n_chunks), kThreads, 0, stream>>>(n_chunks, chunk_row, rank, chunk_ri);
  ctx->launches += 2;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

size_t hpspmm_order_scratch_bytes(int64_t n_chunks) {
  const int64_t n = n_chunks > 0 ? n_chunks : 1;
  const int64_t n_tiles = (n + kTile - 1) / kTile;
  const int64_t hist_n = 256 * n_tiles;
  const int64_t scan_blocks = (hist_n + kScanTile - 1) / kScanTile;
  return 3 * align_up((size_t)n * 4, 256) + align_up((size_t)hist_n * 4, 256) +
         align_up((size_t)scan_blocks * 4, 256);
}

int hpspmm_order_chunks_by_cost(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t n_chunks,
                                const int32_t* row_ptr, const int32_t* col_idx, const int32_t* chunk_start,
                                const int32_t* chunk_row, int32_t* order_out, void* scratch,
                                cudaStream_t stream) {
  if (n_chunks <= 0) return HPSPMM_OK;
  const int n_tiles = (int)((n_chunks + kTile - 1) / kTile);
  const int64_t hist_n = (int64_t)256 * n_tiles;
  const int64_t scan_blocks = (hist_n + kScanTile - 1) / kScanTile;
  const size_t b_arr = align_up((size_t)n_chunks * 4, 256);
  char* base = (char*)scratch;
  int* keys = (int*)base;
  int* keys_tmp = (int*)(base + b_arr);
  int* order_tmp = (int*)(base + 2 * b_arr);
  int* hist = (int*)(base + 3 * b_arr);
  int* totals = (int*)(base + 3 * b_arr + align_up((size_t)hist_n * 4, 256));
  int col_shift = 0;
  while (((N > 0 ? N - 1 : 0) >> col_shift) > 32767) ++col_shift;
  chunk_cost_key_kernel<<<grid_for(ctx, n_chunks), kThreads, 0, stream>>>(
      (int)M, n_chunks, chunk_start, chunk_row, row_ptr, col_idx, col_shift, keys);
  ctx->launches++;
  // stable 8-bit passes, low digit first: one for the 8-bit key, two for the 16-bit key
  const int passes = col_idx ? 2 : 1;
  for (int pass = 0; pass < passes; ++pass) {
    const int* kin = pass == 0 ? keys : keys_tmp;
    const int* pin = pass == 0 ? nullptr : order_tmp;
    int* kout = pass == 0 ? keys_tmp : keys;
    int* pout = pass == passes - 1 ? order_out : order_tmp;
    radix_hist_kernel<<<n_tiles, kThreads, 0, stream>>>(kin, n_chunks, 8 * pass, n_tiles, hist);
    scan_block_totals_kernel<<<(unsigned)scan_blocks, kThreads, 0, stream>>>(hist, hist_n, totals);
    scan_single_block_kernel<<<1, kThreads, 0, stream>>>(totals, scan_blocks);
    scan_rescan_kernel<<<(unsigned)scan_blocks, kThreads, 0, stream>>>(hist, hist_n, totals);
    radix_scatter_kernel<<<n_tiles, kThreads, 0, stream>>>(kin, pin, n_chunks, 8 * pass, n_tiles, hist, kout,
                                                          pout);
    ctx->launches += 5;
  }
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

extern "C" {

int hpspmm_validate_csr(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz, const int32_t* row_ptr,
                        const int32_t* col_idx, int64_t* bad_pos_out, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0, "negative size");
  HPSPMM_REQUIRE(ctx, row_ptr != nullptr && (nnz == 0 || col_idx != nullptr), "null pointer");
  if (bad_pos_out) *bad_pos_out = -1;
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned long long* flag = (unsigned long long*)ctx->flag;
  HPSPMM_CUDA_TRY(ctx, cudaMemsetAsync(flag, 0xff, sizeof(unsigned long long), s));
  validate_csr_kernel<<<grid_for(ctx, M + 1 + nnz), kThreads, 0, s>>>(M, N, nnz, row_ptr, col_idx, flag);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  unsigned long long h = 0;
  HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(&h, flag, sizeof(h), cudaMemcpyDeviceToHost, s));
  HPSPMM_CUDA_TRY(ctx, cudaStreamSynchronize(s));
  HPSPMM_CUDA_TRY(ctx, cudaMemsetAsync(flag, 0, sizeof(unsigned long long), s));
  if (h != ~0ull) {
    if (bad_pos_out) *bad_pos_out = (int64_t)h - 1;
    snprintf(ctx->err, sizeof(ctx->err), "malformed CSR at position %lld", (long long)h - 1);
    return HPSPMM_ERR_BAD_CSR;
  }
  return HPSPMM_OK;
}

int64_t hpspmm_padded_nnz(int64_t nnz, int64_t padding) {
  if (padding <= 0 || nnz % padding == 0) return nnz;
  return nnz + padding - nnz % padding;
}

int hpspmm_csr_to_coo_padded(hpspmm_ctx* ctx, int64_t M, int64_t nnz, const int32_t* row_ptr,
                             const int32_t* col_idx, const float* vals, int64_t padding,
                             int32_t* row_out, int32_t* col_out, float* val_out,
                             hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && nnz >= 0 && padding >= 0, "negative size");
  if (M > 2147483646ll || nnz > 2147483647ll) return HPSPMM_ERR_UNSUPPORTED;
  const int64_t padded = hpspmm_padded_nnz(nnz, padding);
  if (padded == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, row_ptr && row_out, "null pointer");
  HPSPMM_REQUIRE(ctx, (!col_out || col_idx) && (!val_out || vals), "missing source array");
  hpspmm_device_guard guard(ctx->device);
  expand_rows_kernel<false><<<(unsigned)((padded + kExpandTile - 1) / kExpandTile), kThreads, 0, (cudaStream_t)stream>>>(
      (int)M, nnz, padded, row_ptr, col_idx, vals, row_out, col_out, val_out, nullptr);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

int hpspmm_csr_transpose(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz, const int32_t* row_ptr,
                         const int32_t* col_idx, const float* vals, int32_t* row_ptr_t,
                         int32_t* col_idx_t, float* vals_t, int32_t* perm_out, hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_csr_transpose");
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0, "negative size");
  if (M > 2147483646ll || N > 2147483646ll || nnz > 2147483647ll) return HPSPMM_ERR_UNSUPPORTED;
  HPSPMM_REQUIRE(ctx, row_ptr && row_ptr_t, "null pointer");
  HPSPMM_REQUIRE(ctx, nnz == 0 || (col_idx && col_idx_t), "null pointer");
  HPSPMM_REQUIRE(ctx, !vals_t || vals, "vals_t requested without vals");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  if (nnz == 0) {
    HPSPMM_CUDA_TRY(ctx, cudaMemsetAsync(row_ptr_t, 0, (size_t)(N + 1) * 4, s));
    return HPSPMM_OK;
  }
  // digits: as few passes as 11-bit digits allow, each as narrow as that number of passes permits
  int bits = 1;
  while (bits < 31 && ((int64_t)1 << bits) < N) ++bits;
  const int passes = (bits + 10) / 11;
  const int need = (bits + passes - 1) / passes;
  const int dbits = need <= 8 ? 8 : (need <= 10 ? 10 : 11);
  const int n_tiles = (int)((nnz + kTile - 1) / kTile);
  const int64_t hist_n = ((int64_t)1 << dbits) * n_tiles;
  const int64_t scan_blocks = (hist_n + kScanTile - 1) / kScanTile;
  const size_t b_pairs = align_up((size_t)nnz * 8, 256);
  const size_t b_hist = align_up((size_t)hist_n * 4, 256);
  const size_t b_tot = align_up((size_t)scan_blocks * 4, 256);
  int st = hpspmm_ensure_scratch(ctx, 3 * b_pairs + b_hist + b_tot);
  if (st != HPSPMM_OK) return st;
  char* base = (char*)ctx->scratch;
  int2* pairs[2] = {(int2*)base, (int2*)(base + b_pairs)};
  int2* row_val = (int2*)(base + 2 * b_pairs);
  int* hist = (int*)(base + 3 * b_pairs);
  int* totals = (int*)(base + 3 * b_pairs + b_hist);

  // (source row, value) of every entry as one word, so that the final gather reads one sector per entry
  expand_rows_kernel<true><<<(unsigned)((nnz + kExpandTile - 1) / kExpandTile), kThreads, 0, s>>>(
      (int)M, nnz, nnz, row_ptr, nullptr, vals, nullptr, nullptr, nullptr, row_val);
  ctx->launches++;

  const int2* pin = nullptr;
  int cur = 0;
  for (int p = 0; p < passes; ++p) {
    const int shift = dbits * p;
    if (dbits == 8)
      launch_pair_pass<8>(col_idx, pin, nnz, shift, n_tiles, hist, totals, pairs[cur], s);
    else if (dbits == 10)
      launch_pair_pass<10>(col_idx, pin, nnz, shift, n_tiles, hist, totals, pairs[cur], s);
    else
      launch_pair_pass<11>(col_idx, pin, nnz, shift, n_tiles, hist, totals, pairs[cur], s);
    ctx->launches += 5;
    HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
    pin = pairs[cur];
    cur ^= 1;
  }
  transposed_row_ptr_pairs_kernel<<<grid_for(ctx, N + 1), kThreads, 0, s>>>(pin, nnz, N, row_ptr_t);
  transposed_emit_kernel<<<grid_for(ctx, nnz), kThreads, 0, s>>>(nnz, pin, row_val, col_idx_t, vals_t, perm_out);
  ctx->launches += 2;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

// scratch for the reordering entry points: [new_ptr (M+1)] [hits (M)] [scan totals]
static int reorder_scratch(hpspmm_ctx* ctx, int64_t M, bool need_ptr, int** new_ptr, int** hits, int** totals) {
  const size_t b_ptr = need_ptr ? align_up((size_t)(M + 1) * 4, 256) : 0;
  const size_t b_hits = align_up((size_t)(M > 0 ? M : 1) * 4, 256);
  const size_t b_tot = align_up((size_t)((M + 1 + kScanTile - 1) / kScanTile + 1) * 4, 256);
  int st = hpspmm_ensure_scratch(ctx, b_ptr + b_hits + b_tot);
  if (st != HPSPMM_OK) return st;
  char* base = (char*)ctx->scratch;
  if (new_ptr) *new_ptr = (int*)base;
  *hits = (int*)(base + b_ptr);
  *totals = (int*)(base + b_ptr + b_hits);
  return HPSPMM_OK;
}

int hpspmm_csr_to_coo_reordered(hpspmm_ctx* ctx, int64_t M, int64_t nnz, const int32_t* row_ptr,
                                const int32_t* col_idx, const float* vals, const int32_t* row_order,
                                int64_t padding, int32_t* row_out, int32_t* col_out, float* val_out,
                                hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && nnz >= 0 && padding >= 0, "negative size");
  if (M > 2147483646ll || nnz > 2147483647ll) return HPSPMM_ERR_UNSUPPORTED;
  const int64_t padded = hpspmm_padded_nnz(nnz, padding);
  if (padded == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, row_ptr && row_order && row_out, "null pointer");
  HPSPMM_REQUIRE(ctx, (!col_out || col_idx) && (!val_out || vals), "missing source array");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  int *new_ptr, *hits, *totals;
  int st = reorder_scratch(ctx, M, true, &new_ptr, &hits, &totals);
  if (st != HPSPMM_OK) return st;
  st = build_ordered_row_ptr(ctx, M, row_ptr, row_order, new_ptr, hits, totals, s);
  if (st != HPSPMM_OK) return st;
  permute_rows_kernel<<<grid_for(ctx, padded), kThreads, 0, s>>>((int)M, nnz, padded, new_ptr, row_ptr, row_order,
                                                                col_idx, vals, nullptr, row_out, col_out, val_out);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

int hpspmm_csr_permute(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz, const int32_t* row_ptr,
                       const int32_t* col_idx, const float* vals, const int32_t* row_order,
                       const int32_t* col_new_id, int32_t* row_ptr_out, int32_t* col_out, float* val_out,
                       hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0, "negative size");
  if (M > 2147483646ll || nnz > 2147483647ll) return HPSPMM_ERR_UNSUPPORTED;
  HPSPMM_REQUIRE(ctx, row_ptr && row_order && row_ptr_out, "null pointer");
  HPSPMM_REQUIRE(ctx, nnz == 0 || (col_idx && col_out), "null pointer");
  HPSPMM_REQUIRE(ctx, !val_out || vals, "val_out requested without vals");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  int *hits, *totals;
  int st = reorder_scratch(ctx, M, false, nullptr, &hits, &totals);
  if (st != HPSPMM_OK) return st;
  st = build_ordered_row_ptr(ctx, M, row_ptr, row_order, row_ptr_out, hits, totals, s);
  if (st != HPSPMM_OK || nnz == 0) return st;
  permute_rows_kernel<<<grid_for(ctx, nnz), kThreads, 0, s>>>((int)M, nnz, nnz, row_ptr_out, row_ptr, row_order,
                                                             col_idx, vals, col_new_id, nullptr, col_out, val_out);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

int hpspmm_order_rows_by_degree(hpspmm_ctx* ctx, int64_t M, const int32_t* row_ptr, int32_t* order_out,
                                hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0, "negative size");
  if (M > 2147483646ll) return HPSPMM_ERR_UNSUPPORTED;
  if (M == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, row_ptr && order_out, "null pointer");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  const int n_tiles = (int)((M + kTile - 1) / kTile);
  const int64_t hist_n = (int64_t)256 * n_tiles;
  const int64_t scan_blocks = (hist_n + kScanTile - 1) / kScanTile;
  const size_t b_arr = align_up((size_t)M * 4, 256);
  const size_t b_hist = align_up((size_t)hist_n * 4, 256);
  const size_t b_tot = align_up((size_t)scan_blocks * 4, 256);
  int st = hpspmm_ensure_scratch(ctx, 3 * b_arr + b_hist + b_tot);
  if (st != HPSPMM_OK) return st;
  char* base = (char*)ctx->scratch;
  int* keys[2] = {(int*)base, (int*)(base + b_arr)};
  int* pay_tmp = (int*)(base + 2 * b_arr);
  int* hist = (int*)(base + 3 * b_arr);
  int* totals = (int*)(base + 3 * b_arr + b_hist);
  degree_key_kernel<<<grid_for(ctx, M), kThreads, 0, s>>>((int)M, row_ptr, keys[0]);
  ctx->launches++;
  // four stable 8-bit passes; payloads alternate between pay_tmp and order_out and end in order_out
  const int* pin = nullptr;
  for (int p = 0; p < 4; ++p) {
    const int* kin = keys[p & 1];
    int* kout = keys[(p & 1) ^ 1];
    int* pout = (p & 1) ? order_out : pay_tmp;
    radix_hist_kernel<<<n_tiles, kThreads, 0, s>>>(kin, M, 8 * p, n_tiles, hist);
    scan_block_totals_kernel<<<(unsigned)scan_blocks, kThreads, 0, s>>>(hist, hist_n, totals);
    scan_single_block_kernel<<<1, kThreads, 0, s>>>(totals, scan_blocks);
    scan_rescan_kernel<<<(unsigned)scan_blocks, kThreads, 0, s>>>(hist, hist_n, totals);
    radix_scatter_kernel<<<n_tiles, kThreads, 0, s>>>(kin, pin, M, 8 * p, n_tiles, hist, kout, pout);
    ctx->launches += 5;
    pin = pout;
  }
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

int hpspmm_invert_permutation(hpspmm_ctx* ctx, int64_t M, const int32_t* order, int32_t* inverse_out,
                              hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0, "negative size");
  if (M > 2147483646ll) return HPSPMM_ERR_UNSUPPORTED;
  if (M == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, order && inverse_out, "null pointer");
  hpspmm_device_guard guard(ctx->device);
  invert_permutation_kernel<<<grid_for(ctx, M), kThreads, 0, (cudaStream_t)stream>>>((int)M, order, inverse_out);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

int hpspmm_gather_rows_f32(hpspmm_ctx* ctx, int64_t M, int64_t K, const float* src, const int32_t* order,
                           float* dst, hpspmm_stream stream) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && K >= 1, "bad size");
  if (M == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, src && order && dst && src != dst, "null pointer or in-place gather");
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = (K % 4 == 0) && (((uintptr_t)src | (uintptr_t)dst) % 16 == 0);
  if (vec)
    gather_rows_kernel<float4><<<grid_for(ctx, M * (K / 4)), kThreads, 0, s>>>(
        M, K / 4, reinterpret_cast<const float4*>(src), order, reinterpret_cast<float4*>(dst));
  else
    gather_rows_kernel<float><<<grid_for(ctx, M * K), kThreads, 0, s>>>(M, K, src, order, dst);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

}  // extern "C"
