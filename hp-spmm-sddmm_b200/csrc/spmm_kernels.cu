// FP32 CSR SpMM for sm_100a: C = A * B with A in CSR, B and C dense row-major.
//
// Replaces the reference's GESpMM / LBSpMM kernel set (spmm/mm/spmm_kernel.cu:247-477).
// Scheduling: the nnz axis is cut into chunks of a nominal size S.  A cut that falls
// inside a row no longer than S is moved back to the start of that row, so short rows
// stay whole; a cut inside a longer ("heavy") row stays where it is, so heavy rows are
// split across chunks (a merge-path split restricted to heavy rows).  One warp owns one
// chunk.  The warp stages (col, val) tiles of 32 entries in shared memory with
// asynchronous copies, two tiles ahead of their use.  For K = 4*W the warp is G = 32/W
// lane groups; in every step group g takes entry G*s+g of the tile, reads its (col, val)
// pair as one shared-memory broadcast, and gathers its float4 of that row of B, so one
// warp instruction gathers G rows and no two groups ever diverge (row ends are warp-
// uniform).  Gathers are issued U steps at a time before the first FMA.  When a row
// ends, the groups' partial sums are combined with shuffles and the row is stored once,
// by plain stores.  A chunk that ends inside a heavy row hands its partial sum on through
// a carry slot, and the carries of a split row are added, in chunk order, to the row its last
// piece stored.  Who adds them depends on the width: at 32 columns a second, small kernel; at 64
// and 128 columns the pieces themselves -- each bumps a per-row counter (one atomicAdd) when its
// part is visible, and the piece that finds the counter complete sums the carries.  Either way
// the order of the additions is fixed by the chunking, so results are bit-reproducible from run
// to run.  Empty rows are zeroed by extra blocks at the end of the same grid.
// HPSPMM_ALGO_ROW_SPLIT keeps the reference's GESpMM shape (one sub-warp per row, every row
// summed in storage order), which reproduces the CPU oracle bit for bit.
#include <algorithm>
#include <mutex>
#include <new>

#include <cuda.h>   // CUtensorMap and the encode prototype; the entry point is looked up at run time

#include "device_utils.cuh"
#include "hpspmm_internal.h"

namespace {

using namespace hpspmm;

constexpr int kBlockThreads = 256;

// resident 64-thread blocks per SM the contiguous warp kernels are compiled for (20 -> 48 registers)
#ifndef HPSPMM_WARP_MINB
#define HPSPMM_WARP_MINB 20
#endif

// ---- chunk table -----------------------------------------------------------------------

__global__ void chunk_table_kernel(int M, int nnz, const int* __restrict__ row_ptr, int S,
                                   int n_chunks, int* __restrict__ chunk_start,
                                   int* __restrict__ chunk_row, int* __restrict__ split_count,
                                   int* __restrict__ run_counter) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c > n_chunks) return;
  if (run_counter != nullptr) run_counter[c] = 0;   // per-row counters of the in-kernel carry settlement
  if (c == n_chunks) {
    chunk_start[c] = nnz;
    return;
  }
  const int t = c * S;
  // first index i in [0, M] with row_ptr[i] > t
  int lo = 0, hi = M + 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(row_ptr + mid) <= t)
      lo = mid + 1;
    else
      hi = mid;
  }
  int r = lo - 1;
  r = r < 0 ? 0 : (r > M - 1 ? M - 1 : r);  // only a malformed row_ptr can need this
  const int rs = __ldg(row_ptr + r), re = __ldg(row_ptr + r + 1);
  const int start = (re - rs <= S) ? rs : t;
  chunk_start[c] = c == 0 ? 0 : start;
  chunk_row[c] = r;
  if (split_count != nullptr && c > 0 && start != rs) atomicAdd(split_count, 1);
}

// ---- empty rows ------------------------------------------------------------------------

// Blocks past the chunk blocks walk all rows and write zeros into the empty ones.
__device__ __forceinline__ void zero_empty_rows(int M, int K, const int* __restrict__ row_ptr,
                                                float* __restrict__ C, int zero_block,
                                                int n_zero_blocks, int block_threads = kBlockThreads,
                                                int64_t row_stride = 0) {
  if (row_stride == 0) row_stride = K;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_block = block_threads / 32;
  const int64_t stride = (int64_t)n_zero_blocks * warps_per_block * 32;
  for (int64_t r0 = ((int64_t)zero_block * warps_per_block + warp) * 32; r0 < M; r0 += stride) {
    const int64_t r = r0 + lane;
    bool empty = false;
    if (r < M) empty = __ldg(row_ptr + r) == __ldg(row_ptr + r + 1);
    unsigned m = __ballot_sync(0xffffffffu, empty);
    while (m) {
      const int b = __ffs(m) - 1;
      m &= m - 1;
      float* crow = C + (r0 + b) * row_stride;
      if ((K & 3) == 0) {
        for (int c = lane * 4; c < K; c += 128) st_stream(crow + c, make_float4(0.f, 0.f, 0.f, 0.f));
      } else {
        for (int c = lane; c < K; c += 32) crow[c] = 0.f;
      }
    }
  }
}

// Next non-empty row after `row`, given that entry j (< nnz) follows the end of `row`.
__device__ __forceinline__ void advance_row(const int* __restrict__ row_ptr, int M, int j,
                                            int& row, int& row_end) {
  ++row;
  int e = __ldg(row_ptr + row + 1);
  int probes = 0;
  while (e == j) {
    if (++probes == 8) {
      // a long run of empty rows: gallop (8, 16, 32, ... rows ahead) to bracket the row holding j,
      // then a binary search inside the bracket
      int lo = row + 1, step = 8, hi;
      for (;;) {
        hi = min(lo + step, M);
        if (hi == M || __ldg(row_ptr + hi) > j) break;
        lo = hi;
        step <<= 1;
      }
      ++hi;
      ++lo;
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

// ---- sub-warp kernel: one W-lane worker per chunk or per row, K = 4 * W * R ----------------

// Row that holds entry j, packed as (row_end << 32) | row.  Kept out of line: it runs once
// per row, and inlining its search at every unrolled entry bloats the hot loop.  It takes
// and returns plain integers so that the accumulators never leave registers.
__device__ __noinline__ unsigned long long next_row_packed(const int* __restrict__ row_ptr, int M,
                                                           int j, int row) {
  int row_end;
  advance_row(row_ptr, M, j, row, row_end);
  return ((unsigned long long)(unsigned)row_end << 32) | (unsigned)row;
}

template <int W, int R, int U, int MINB, bool HINT, bool ROWSPLIT>
__global__ void __launch_bounds__(kBlockThreads, MINB)
spmm_subwarp_kernel(int M, int n_chunks, int n_chunk_blocks, const int* __restrict__ row_ptr,
                     const int* __restrict__ col_idx, const float* __restrict__ vals,
                     const float* __restrict__ B, float* __restrict__ C,
                     const int* __restrict__ chunk_start, const int* __restrict__ chunk_row,
                     int* __restrict__ carry_row, float* __restrict__ carry_val) {
  constexpr int K = 4 * W * R;
  constexpr int T = 32;       // entries per staged (col, val) tile
  constexpr int RT = T / W;   // entries each lane stages per tile
  constexpr int STAGES = 2;
  __shared__ int2 tiles[kBlockThreads / W][STAGES][T];

  if ((int)blockIdx.x >= n_chunk_blocks) {
    zero_empty_rows(M, K, row_ptr, C, blockIdx.x - n_chunk_blocks, gridDim.x - n_chunk_blocks);
    return;
  }
  const int lane = threadIdx.x & (W - 1);
  const int worker = (int)(((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) / W);
  if (worker >= n_chunks) return;
  const unsigned mask = subwarp_mask<W>();
  const uint64_t policy = HINT ? policy_evict_last() : 0ull;
  int2(*my)[T] = tiles[threadIdx.x / W];

  int n0, n1, row, row_end;
  if (ROWSPLIT) {
    row = worker;
    n0 = __ldg(row_ptr + row);
    n1 = __ldg(row_ptr + row + 1);
    row_end = n1;
  } else {
    n0 = __ldg(chunk_start + worker);
    n1 = __ldg(chunk_start + worker + 1);
    row = __ldg(chunk_row + worker);
    row_end = __ldg(row_ptr + row + 1);
  }

  // (col, val) pairs travel global -> shared with 4-byte asynchronous copies, two tiles
  // ahead of their use; entries past the end of the chunk are staged as (column 0, 0.0f).
  auto stage_tile = [&](int stage, int base) {
#pragma unroll
    for (int t = 0; t < RT; ++t) {
      const int e = t * W + lane;
      const int j = base + e;
      if (j < n1) {
        cp_async_4(&my[stage][e].x, col_idx + j);
        cp_async_4(&my[stage][e].y, vals + j);
      } else {
        my[stage][e] = make_int2(0, 0);
      }
    }
    cp_async_commit();
  };
  stage_tile(0, n0);
  stage_tile(1, n0 + T);

  float4 acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* Bl = B + lane * 4;

  int stage = 0;
  for (int base = n0; base < n1; base += T) {
    cp_async_wait<STAGES - 1>();
    __syncwarp(mask);
#pragma unroll 1
    for (int u0 = 0; u0 < T; u0 += U) {
      const int j0 = base + u0;
      if (j0 >= n1) break;
      float4 b[U][R];
      float v[U];
#pragma unroll
      for (int i = 0; i < U; ++i) {
        const int2 e = my[stage][u0 + i];  // same address for the whole worker: a broadcast
        v[i] = __int_as_float(e.y);
        const float* p = Bl + (int64_t)e.x * K;
#pragma unroll
        for (int r = 0; r < R; ++r) b[i][r] = ld_gather<HINT>(p + r * W * 4, policy);
      }
      if (ROWSPLIT || (j0 + U <= n1 && row_end >= j0 + U)) {
        // no row ends inside this batch: padded entries (ROWSPLIT tail) carry value 0 and
        // are skipped below by the same test the slow path uses
        if (!ROWSPLIT || j0 + U <= n1) {
#pragma unroll
          for (int i = 0; i < U; ++i)
#pragma unroll
            for (int r = 0; r < R; ++r) fma4(acc[r], v[i], b[i][r]);
        } else {
#pragma unroll
          for (int i = 0; i < U; ++i)
            if (j0 + i < n1)
#pragma unroll
              for (int r = 0; r < R; ++r) fma4(acc[r], v[i], b[i][r]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < U; ++i) {
          if (j0 + i < n1) {
            if (j0 + i == row_end) {
              float* crow = C + (int64_t)row * K + lane * 4;
#pragma unroll
              for (int r = 0; r < R; ++r) {
                st_stream(crow + r * W * 4, acc[r]);
                acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
              const unsigned long long nr = next_row_packed(row_ptr, M, j0 + i, row);
              row = (int)(unsigned)nr;
              row_end = (int)(nr >> 32);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) fma4(acc[r], v[i], b[i][r]);
          }
        }
      }
    }
    __syncwarp(mask);
    stage_tile(stage, base + STAGES * T);
    stage ^= 1;
  }
  cp_async_wait<0>();

  if (ROWSPLIT || row_end == n1) {
    float* crow = C + (int64_t)row * K + lane * 4;
#pragma unroll
    for (int r = 0; r < R; ++r) st_stream(crow + r * W * 4, acc[r]);
    if (!ROWSPLIT && lane == 0) carry_row[worker] = -1;
  } else {
    float* slot = carry_val + (int64_t)worker * K + lane * 4;
#pragma unroll
    for (int r = 0; r < R; ++r) *reinterpret_cast<float4*>(slot + r * W * 4) = acc[r];
    if (lane == 0) carry_row[worker] = row;
  }
}

// ---- warp kernel: one warp per chunk, G = 32/W interleaved lane groups, K = 4 * W ---------

template <int W>
__device__ __forceinline__ float4 reduce_groups(float4 a) {
  if (W <= 16) {
    a.x += __shfl_xor_sync(0xffffffffu, a.x, 16);
    a.y += __shfl_xor_sync(0xffffffffu, a.y, 16);
    a.z += __shfl_xor_sync(0xffffffffu, a.z, 16);
    a.w += __shfl_xor_sync(0xffffffffu, a.w, 16);
  }
  if (W <= 8) {
    a.x += __shfl_xor_sync(0xffffffffu, a.x, 8);
    a.y += __shfl_xor_sync(0xffffffffu, a.y, 8);
    a.z += __shfl_xor_sync(0xffffffffu, a.z, 8);
    a.w += __shfl_xor_sync(0xffffffffu, a.w, 8);
  }
  return a;
}

// A finished row: add the groups' partial sums and store the row.  Instead of giving every group the whole
// sum (reduce_groups: 8 shuffles at W = 8) and letting one group store it, the groups split the work: each
// exchange hands the partner the half it will own and keeps the other, so W = 8 takes 3 shuffles and every
// lane stores one float (group g ends up with component g of each float4: 32 lanes, one 128-byte line),
// W = 16 takes 2 shuffles and every lane stores a float2.  Every kept value is own + partner at each
// step, in the same pairing as reduce_groups, so the stored bits are the same.
// ACCUM adds the row into C with reductions (the accumulating COO product) instead of storing it.
template <int W, bool ACCUM = false>
__device__ __forceinline__ void store_row_sum(float* __restrict__ crow, const float4& a, int g, int l) {
  if (W == 8) {
    const bool up2 = (g & 2) != 0, up1 = (g & 1) != 0;
    const float s0 = up2 ? a.x : a.z, s1 = up2 ? a.y : a.w;   // the pair the partner (g ^ 2) keeps
    float k0 = up2 ? a.z : a.x, k1 = up2 ? a.w : a.y;
    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    const float s = up1 ? k0 : k1;                            // the one the partner (g ^ 1) keeps
    float k = up1 ? k1 : k0;
    k += __shfl_xor_sync(0xffffffffu, s, 8);
    if (ACCUM)
      asm volatile("red.global.add.f32 [%0], %1;" ::"l"(crow + l * 4 + g), "f"(k) : "memory");
    else
      asm volatile("st.global.cs.f32 [%0], %1;" ::"l"(crow + l * 4 + g), "f"(k) : "memory");
  } else if (W == 16) {
    const bool up = (g & 1) != 0;
    const float s0 = up ? a.x : a.z, s1 = up ? a.y : a.w;
    float k0 = up ? a.z : a.x, k1 = up ? a.w : a.y;
    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    if (ACCUM)
      asm volatile("red.global.add.v2.f32 [%0], {%1,%2};" ::"l"(crow + l * 4 + g * 2), "f"(k0), "f"(k1) : "memory");
    else
      asm volatile("st.global.cs.v2.f32 [%0], {%1,%2};" ::"l"(crow + l * 4 + g * 2), "f"(k0), "f"(k1) : "memory");
  } else {
    if (ACCUM)
      red_add_v4(crow + l * 4, a);
    else
      st_stream(crow + l * 4, a);
  }
}

// In-kernel fix-up of one split row.  A row longer than S is cut at multiples of S only, so its pieces
// are the chunks first = row_ptr[r] / S .. last = (row_ptr[r+1] - 1) / S: all but the last hand a carry
// on, the last stores the row.  Every piece bumps the row's counter when its own part is visible
// device-wide; whoever bumps it last adds the carries, in chunk order, to the stored row.  The sum does
// not depend on who that is, so results stay bit-reproducible.  No piece ever waits.  Kept out of line
// so that its registers do not weigh on the gather loop of the caller.
template <int W>
__device__ __noinline__ void settle_split_row(int r, int r_end, int S, const int* __restrict__ row_ptr,
                                              const float* __restrict__ carry_val, float* __restrict__ C,
                                              int* __restrict__ run_counter, int ld) {
  const int64_t K = ld;   // row stride of C and of the carry slots (the slab is 4 * W columns wide)
  constexpr int G = 32 / W;
  const int lane = threadIdx.x & 31;
  const int g = lane / W, l = lane % W;
  const int first = __ldg(row_ptr + r) / S;
  const int last = (r_end - 1) / S;
  int seen = 0;
  if (lane == 0) seen = atomicAdd(run_counter + first, 1);
  seen = __shfl_sync(0xffffffffu, seen, 0);
  if (seen != last - first) return;
  __threadfence();
  const float* src = carry_val + (int64_t)first * K + l * 4;
  const int len = last - first;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  int i = g;
  for (; i + 7 * G < len; i += 8 * G) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)(i + u * G) * K));
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      sum.x += v[u].x;
      sum.y += v[u].y;
      sum.z += v[u].z;
      sum.w += v[u].w;
    }
  }
  for (; i < len; i += G) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)i * K));
    sum.x += v.x;
    sum.y += v.y;
    sum.z += v.z;
    sum.w += v.w;
  }
  sum = reduce_groups<W>(sum);
  if (g == 0) {
    float4* out = reinterpret_cast<float4*>(C + (int64_t)r * K + l * 4);
    float4 o = __ldcg(out);
    o.x += sum.x;
    o.y += sum.y;
    o.z += sum.z;
    o.w += sum.w;
    st_stream(reinterpret_cast<float*>(out), o);
  }
  if (lane == 0) run_counter[first] = 0;   // ready for the next launch
}

template <int W, int U, int MINB, bool HINT, int BT, bool SETTLE, bool STRIDED, bool COMPACT>
__global__ void __launch_bounds__(BT, MINB)
spmm_warp_kernel(int M, int n_chunks, int n_chunk_blocks, const int* __restrict__ row_ptr,
                 const int* __restrict__ col_idx, const float* __restrict__ vals,
                 const float* __restrict__ B, float* __restrict__ C,
                 const int* __restrict__ chunk_start, const int* __restrict__ chunk_row,
                 int* __restrict__ carry_row, float* __restrict__ carry_val,
                 const int* __restrict__ chunk_order, int S, int* __restrict__ run_counter, int ld,
                 const int* __restrict__ nz_id, const int* __restrict__ nz_end,
                 const int* __restrict__ chunk_ri) {
  // COMPACT: the plan lists the rows that hold entries (nz_id, with their ends nz_end) and the position in
  // that list of every chunk's first row (chunk_ri), so the kernel steps from one such row to the next with
  // two independent loads and never looks at an empty row.  Without the list it probes row_ptr row by row.
  // The kernel computes a slab of KW = 4 * W columns.  STRIDED: the slab is part of wider matrices, B, C
  // and the carry slots have row stride ld; otherwise the stride is the compile-time KW.
  constexpr int KW = 4 * W;
  const int64_t K = STRIDED ? (int64_t)ld : (int64_t)KW;
  constexpr int G = 32 / W;      // lane groups = entries gathered per warp instruction
  constexpr int T = 32;          // entries per staged tile
  constexpr int BATCH = U * G;   // entries per batch of gathers
  constexpr int STAGES = 2;
  static_assert(BATCH <= T && T % BATCH == 0, "batch must tile the staged tile");
  __shared__ int2 tiles[BT / 32][STAGES][T];

  if ((int)blockIdx.x >= n_chunk_blocks) {
    zero_empty_rows(M, KW, row_ptr, C, blockIdx.x - n_chunk_blocks, gridDim.x - n_chunk_blocks, BT, K);
    return;
  }
  const int lane = threadIdx.x & 31;
  const int g = lane / W;   // group
  const int l = lane % W;   // position inside the group = float4 column
  const int slot = (int)(((int64_t)blockIdx.x * BT + threadIdx.x) >> 5);
  if (slot >= n_chunks) return;
  // warps take chunks in the plan's order (chunks with many rows first), not in matrix order
  const int chunk = chunk_order != nullptr ? __ldg(chunk_order + slot) : slot;
  const uint64_t policy = HINT ? policy_evict_last() : 0ull;
  int2(*my)[T] = tiles[threadIdx.x >> 5];

  const int n0 = __ldg(chunk_start + chunk);
  const int n1 = __ldg(chunk_start + chunk + 1);
  int ri = COMPACT ? __ldg(chunk_ri + chunk) : 0;
  int row = COMPACT ? __ldg(nz_id + ri) : __ldg(chunk_row + chunk);
  int row_end = COMPACT ? __ldg(nz_end + ri) : __ldg(row_ptr + row + 1);

  auto stage_tile = [&](int stage, int base) {
    const int j = base + lane;
    if (j < n1) {
      cp_async_4(&my[stage][lane].x, col_idx + j);
      cp_async_4(&my[stage][lane].y, vals + j);
    } else {
      my[stage][lane] = make_int2(0, 0);   // past the chunk: column 0, value 0
    }
    cp_async_commit();
  };
  stage_tile(0, n0);
  stage_tile(1, n0 + T);

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* Bl = B + l * 4;

  // the row is complete: combine the groups' partial sums, store, start the next row.
  // The common case (the next row is not empty, or only a few are) stays inline; a long
  // run of empty rows falls back to a binary search.
  auto finish_row = [&](int next_entry) {
    store_row_sum<W>(C + (int64_t)row * K, acc, g, l);
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (COMPACT) {
      ++ri;
      row = __ldg(nz_id + ri);
      row_end = __ldg(nz_end + ri);
      return;
    }
    int e, probes = 0;
    do {
      ++row;
      e = __ldg(row_ptr + row + 1);
    } while (e == next_entry && ++probes < 16);
    if (e == next_entry) {
      // a long run of empty rows: gallop (16, 32, 64, ... rows ahead) to bracket the row that holds
      // next_entry, then a binary search inside the bracket
      int lo = row + 1, step = 16, hi;
      for (;;) {
        hi = min(lo + step, M);
        if (hi == M || __ldg(row_ptr + hi) > next_entry) break;
        lo = hi;
        step <<= 1;
      }
      ++hi;
      ++lo;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(row_ptr + mid) <= next_entry)
          lo = mid + 1;
        else
          hi = mid;
      }
      row = lo - 1;
      e = __ldg(row_ptr + row + 1);
    }
    row_end = e;
  };

  int stage = 0;
  for (int base = n0; base < n1; base += T) {
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const int2* tile = &my[stage][g];
    if (base + T <= n1 && row_end >= base + T) {
      // Fast tile: all 32 entries belong to the current row.  Fully unrolled, every
      // shared-memory offset is a compile-time constant, no tests between gathers.
#pragma unroll
      for (int s0 = 0; s0 < T / G; s0 += U) {
        float4 b[U];
        float v[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
          const int2 e = tile[(s0 + i) * G];   // one broadcast per group
          v[i] = __int_as_float(e.y);
          b[i] = ld_gather<HINT>(Bl + (int64_t)e.x * K, policy);
        }
#pragma unroll
        for (int i = 0; i < U; ++i) fma4(acc, v[i], b[i]);
      }
    } else {
#pragma unroll 1
      for (int u0 = 0; u0 < T; u0 += BATCH) {
        const int j0 = base + u0;
        if (j0 >= n1) break;
        float4 b[U];
        float v[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
          const int2 e = tile[u0 + i * G];
          v[i] = __int_as_float(e.y);
          b[i] = ld_gather<HINT>(Bl + (int64_t)e.x * K, policy);
        }
        if (j0 + BATCH <= n1 && row_end >= j0 + BATCH) {
#pragma unroll
          for (int i = 0; i < U; ++i) fma4(acc, v[i], b[i]);
        } else {
#pragma unroll
          for (int i = 0; i < U; ++i) {
            const int lo = j0 + i * G;
            const int hi = min(lo + G, n1);
            const int mine = lo + g;
            int cur = lo;
            while (row_end < hi) {   // warp-uniform: the current row ends inside this step
              if (mine >= cur && mine < row_end) fma4(acc, v[i], b[i]);
              cur = row_end;
              finish_row(cur);
            }
            if (mine >= cur && mine < hi) fma4(acc, v[i], b[i]);
          }
        }
      }
    }
    __syncwarp();
    stage_tile(stage, base + STAGES * T);
    stage ^= 1;
  }
  cp_async_wait<0>();

  const bool hands_on = row_end != n1;   // the chunk ends inside `row`
  if (!hands_on) {
    store_row_sum<W>(C + (int64_t)row * K, acc, g, l);
  } else {
    const float4 t = reduce_groups<W>(acc);
    if (g == 0) *reinterpret_cast<float4*>(carry_val + (int64_t)chunk * K + l * 4) = t;
  }
  if (!SETTLE) {
    // a separate kernel adds the carries
    if (lane == 0) carry_row[chunk] = hands_on ? row : -1;
    return;
  }

  // the pieces of a split row settle it among themselves (settle_split_row)
  const int r0 = __ldg(chunk_row + chunk);
  const int r0_start = __ldg(row_ptr + r0), r0_end = __ldg(row_ptr + r0 + 1);
  const bool stores_split_row = r0_start < n0 && r0_end <= n1;   // began in an earlier chunk, ends here
  if (!hands_on && !stores_split_row) return;
  __threadfence();
  __syncwarp();   // every lane's part is visible before lane 0 bumps a counter
  if (stores_split_row) settle_split_row<W>(r0, r0_end, S, row_ptr, carry_val, C, run_counter, (int)K);
  if (hands_on) settle_split_row<W>(row, row_end, S, row_ptr, carry_val, C, run_counter, (int)K);
}

// ---- K = 128 with the rows of B fetched by TMA ----------------------------------------------------
// Same chunks, same order of additions and same settlement as spmm_warp_kernel<32, ...>; what differs is
// how a row of B (512 bytes) reaches the warp.  Lane 0 names four rows at a time to the tensor memory
// accelerator (cp.async.bulk.tensor ... tile::gather4 on a tensor map of B whose box is one row), which
// writes them into a ring of kTmaRing 2 KB buffers private to the warp and signals an mbarrier per buffer;
// the warp reads each row back with one 16-byte shared-memory load per lane.  The gathers of up to
// kTmaRing groups are in flight while the warp multiplies, whatever its register budget, and they occupy
// neither the load/store unit's global path nor registers while they travel.
//
// The chunk's (column, value) pairs are staged whole (a chunk of nominal size S holds at most 2 S - 1
// entries, and the launcher takes plans up to S = kTmaMaxS).
// Every wait is bounded by a clock limit; a warp whose wait runs out counts that in *fallbacks, fetches
// the rest of its chunk with ordinary loads and, before it leaves, waits (bounded again) for the copies
// it still has in flight, so a fault in the protocol costs time and leaves a record but neither hangs
// nor changes the result.
#ifndef HPSPMM_TMA_RING
#define HPSPMM_TMA_RING 2
#endif
#ifndef HPSPMM_TMA_WARPS
#define HPSPMM_TMA_WARPS 8
#endif
#ifndef HPSPMM_TMA_BATCH
#define HPSPMM_TMA_BATCH 1
#endif
constexpr int kTmaBatch = HPSPMM_TMA_BATCH;        // groups issued per TMA instruction (one per lane)
constexpr int kTmaRing = HPSPMM_TMA_RING;          // 2 KB buffers per warp, a multiple of kTmaBatch
#ifndef HPSPMM_TMA_MAX_S
#define HPSPMM_TMA_MAX_S 256
#endif
constexpr int kTmaMaxS = HPSPMM_TMA_MAX_S;         // largest nominal chunk size taken
constexpr int kTmaMaxChunk = 2 * kTmaMaxS;         // a chunk holds at most 2 S - 1 entries (chunk_table_kernel)
constexpr int kTmaWarps = HPSPMM_TMA_WARPS;        // warps (= chunks) per block; three blocks per SM
constexpr int kTmaGroupBytes = 4 * 128 * 4;        // four rows of 128 floats
constexpr long long kTmaSpinLimit = 1000000000ll;  // clock cycles, about half a second
static_assert(kTmaRing % kTmaBatch == 0 && kTmaRing >= 2 * kTmaBatch, "ring = whole batches, at least two");
constexpr int kTmaSmemPerWarp = kTmaRing * kTmaGroupBytes + kTmaMaxChunk * 8 + kTmaRing * 8;

__device__ __forceinline__ uint32_t smem_addr_of(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// the slow side of a wait: polls until the phase completes or the clock limit passes
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  for (unsigned n = 1;; ++n) {
    if (mbar_try(bar, parity)) return true;
    if ((n & 63u) == 0 && clock64() - t0 > kTmaSpinLimit) return false;
  }
}

__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;   // the copy has usually landed: no clock read, no loop
  return mbar_wait_slow(bar, parity);
}

__global__ void __launch_bounds__(kTmaWarps * 32, 3)
spmm_tma_kernel(const __grid_constant__ CUtensorMap map_b, int M, int n_chunks, int n_chunk_blocks,
                const int* __restrict__ row_ptr, const int* __restrict__ col_idx,
                const float* __restrict__ vals, const float* __restrict__ B, float* __restrict__ C,
                const int* __restrict__ chunk_start, const int* __restrict__ chunk_row,
                float* __restrict__ carry_val, const int* __restrict__ chunk_order, int S,
                int* __restrict__ run_counter, const int* __restrict__ nz_id, const int* __restrict__ nz_end,
                const int* __restrict__ chunk_ri, int* __restrict__ fallbacks) {
  constexpr int KW = 128;
  constexpr int64_t K = KW;
  extern __shared__ __align__(1024) unsigned char tma_smem[];
  if ((int)blockIdx.x >= n_chunk_blocks) {
    zero_empty_rows(M, KW, row_ptr, C, blockIdx.x - n_chunk_blocks, gridDim.x - n_chunk_blocks, kTmaWarps * 32, K);
    return;
  }
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int slot = blockIdx.x * kTmaWarps + warp;
  if (slot >= n_chunks) return;
  const int chunk = chunk_order != nullptr ? __ldg(chunk_order + slot) : slot;

  // this warp's part of shared memory: ring buffers (1 KB aligned), staged entries, barriers
  unsigned char* ring = tma_smem + (size_t)warp * (kTmaRing * kTmaGroupBytes);
  int2* ent = reinterpret_cast<int2*>(tma_smem + (size_t)kTmaWarps * (kTmaRing * kTmaGroupBytes)) + warp * kTmaMaxChunk;
  uint64_t* full = reinterpret_cast<uint64_t*>(tma_smem + (size_t)kTmaWarps * (kTmaRing * kTmaGroupBytes + kTmaMaxChunk * 8)) +
                   warp * kTmaRing;

  const int n0 = __ldg(chunk_start + chunk);
  const int n1 = __ldg(chunk_start + chunk + 1);
  const int len = n1 - n0;                  // < kTmaMaxChunk: the launcher checks the plan's chunk size
  const int n_groups = (len + 3) >> 2;
  int ri = __ldg(chunk_ri + chunk);
  int row = __ldg(nz_id + ri);
  int row_end = __ldg(nz_end + ri);

  for (int i = lane; i < n_groups * 4; i += 32) {
    if (i < len) {
      cp_async_4(&ent[i].x, col_idx + n0 + i);
      cp_async_4(&ent[i].y, vals + n0 + i);
    } else {
      ent[i] = make_int2(0, 0);             // past the chunk: row 0 is fetched and not used
    }
  }
  cp_async_commit();
  if (lane == 0) {
#pragma unroll
    for (int b = 0; b < kTmaRing; ++b)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr_of(&full[b])), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  cp_async_wait<0>();
  __syncwarp();

  // lane 0: fetch the four rows of group g into buffer g % kTmaRing
  auto issue = [&](int g) {
    const int b = g % kTmaRing;
    const uint32_t bar = smem_addr_of(&full[b]);
    const int4 c01 = *reinterpret_cast<const int4*>(&ent[4 * g]);
    const int4 c23 = *reinterpret_cast<const int4*>(&ent[4 * g + 2]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kTmaGroupBytes) : "memory");
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(smem_addr_of(ring + (size_t)b * kTmaGroupBytes)),
        "l"(&map_b), "r"(0), "r"(c01.x), "r"(c01.z), "r"(c23.x), "r"(c23.z), "r"(bar)
        : "memory");
  };
  // One TMA instruction costs the SM about as much as five gather4 operations, so the lanes 0 .. kTmaBatch-1
  // issue one group each with a single instruction, every kTmaBatch groups.
  const int ahead = n_groups < kTmaRing ? n_groups : kTmaRing;
  for (int g0 = 0; g0 < ahead; g0 += kTmaBatch)
    if (lane < kTmaBatch && g0 + lane < ahead) issue(g0 + lane);
  int issued = ahead;                        // groups handed to the TMA so far (warp-uniform)

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  auto finish_row = [&]() {
    st_stream(C + (int64_t)row * K + lane * 4, acc);
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    ++ri;
    row = __ldg(nz_id + ri);
    row_end = __ldg(nz_end + ri);
  };

  bool by_tma = true;
  int pending_from = 0;                      // first group whose copy was never seen to land
  const uint32_t bar0 = smem_addr_of(full);
  // one group: wait for its buffer, read the four rows, hand the buffer back to the TMA, multiply
  auto do_group = [&](int g, int b, uint32_t parity) {
    float4 rows4[4];
    float v[4];
    const int4 e01 = *reinterpret_cast<const int4*>(&ent[4 * g]);       // (col, val) x 2, broadcast
    const int4 e23 = *reinterpret_cast<const int4*>(&ent[4 * g + 2]);
    v[0] = __int_as_float(e01.y), v[1] = __int_as_float(e01.w);
    v[2] = __int_as_float(e23.y), v[3] = __int_as_float(e23.w);
    if (by_tma) {
      const bool ok = mbar_wait_limited(bar0 + 8u * (uint32_t)b, parity);
      by_tma = __all_sync(0xffffffffu, ok);
      if (!by_tma) {
        pending_from = g;
        if (lane == 0) atomicAdd(fallbacks, 1);
      }
    }
    if (by_tma) {
      const float4* src = reinterpret_cast<const float4*>(ring + (size_t)b * kTmaGroupBytes) + lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) rows4[i] = src[i * 32];
      __syncwarp();                          // every lane has read the buffer before it is refilled
      if ((b + 1) % kTmaBatch == 0 && issued < n_groups) {
        // the kTmaBatch buffers of groups g - kTmaBatch + 1 .. g are free: refill them with the next groups
        // (the warp's reads of these buffers are ordered before this point by the __syncwarp above; the
        // refill is ordered after it by program order, as in any mbarrier-released TMA ring)
        const int n_new = min(kTmaBatch, n_groups - issued);
        if (lane < n_new) issue(issued + lane);
        issued += n_new;
      }
    } else {
      const int cols[4] = {e01.x, e01.z, e23.x, e23.z};
#pragma unroll
      for (int i = 0; i < 4; ++i) rows4[i] = ld_gather_plain(B + (int64_t)cols[i] * K + lane * 4);
    }
    const int j0 = n0 + 4 * g;
    if (j0 + 4 <= n1 && row_end >= j0 + 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) fma4(acc, v[i], rows4[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = j0 + i;
        if (j < n1) {
          while (row_end <= j) finish_row();   // warp-uniform
          fma4(acc, v[i], rows4[i]);
        }
      }
    }
  };
  // the ring is walked in whole turns so that a group's buffer index is a compile-time constant
  for (int turn = 0; turn * kTmaRing < n_groups; ++turn) {
    const uint32_t parity = (uint32_t)turn & 1u;
#pragma unroll
    for (int b = 0; b < kTmaRing; ++b) {
      const int g = turn * kTmaRing + b;
      if (g < n_groups) do_group(g, b, parity);
    }
  }
  if (!by_tma) {
    // copies still in flight target this block's shared memory: let them land before the warp leaves
    for (int g = pending_from; g < issued; ++g)
      mbar_wait_limited(smem_addr_of(&full[g % kTmaRing]), (uint32_t)(g / kTmaRing) & 1u);
  }

  const bool hands_on = row_end != n1;   // the chunk ends inside `row`
  if (!hands_on)
    st_stream(C + (int64_t)row * K + lane * 4, acc);
  else
    *reinterpret_cast<float4*>(carry_val + (int64_t)chunk * K + lane * 4) = acc;
  const int r0 = __ldg(chunk_row + chunk);
  const int r0_start = __ldg(row_ptr + r0), r0_end = __ldg(row_ptr + r0 + 1);
  const bool stores_split_row = r0_start < n0 && r0_end <= n1;   // began in an earlier chunk, ends here
  if (!hands_on && !stores_split_row) return;
  __threadfence();
  __syncwarp();
  if (stores_split_row) settle_split_row<32>(r0, r0_end, S, row_ptr, carry_val, C, run_counter, KW);
  if (hands_on) settle_split_row<32>(row, row_end, S, row_ptr, carry_val, C, run_counter, KW);
}

// ---- generic kernel: any K -------------------------------------------------------------
// One warp per chunk; lane l owns columns kb + (s*32 + l)*VEC .. +VEC-1 for s < NS, where
// kb = blockIdx.y * (32*VEC*NS).  VEC = 4 needs K % 4 == 0.
template <int VEC, int NS, bool ROWSPLIT>
__global__ void __launch_bounds__(kBlockThreads)
spmm_generic_kernel(int M, int K, int n_chunks, int n_chunk_blocks, const int* __restrict__ row_ptr,
                    const int* __restrict__ col_idx, const float* __restrict__ vals,
                    const float* __restrict__ B, float* __restrict__ C,
                    const int* __restrict__ chunk_start, const int* __restrict__ chunk_row,
                    int* __restrict__ carry_row, float* __restrict__ carry_val,
                    const int* __restrict__ chunk_order) {
  if ((int)blockIdx.x >= n_chunk_blocks) {
    if (blockIdx.y == 0)
      zero_empty_rows(M, K, row_ptr, C, blockIdx.x - n_chunk_blocks, gridDim.x - n_chunk_blocks);
    return;
  }
  const int lane = threadIdx.x & 31;
  const int slot = (int)(((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) >> 5);
  if (slot >= n_chunks) return;
  const int worker = (!ROWSPLIT && chunk_order != nullptr) ? __ldg(chunk_order + slot) : slot;
  const int kb = blockIdx.y * (32 * VEC * NS);

  int n0, n1, row, row_end;
  if (ROWSPLIT) {
    row = worker;
    n0 = __ldg(row_ptr + row);
    n1 = __ldg(row_ptr + row + 1);
    row_end = n1;
  } else {
    n0 = __ldg(chunk_start + worker);
    n1 = __ldg(chunk_start + worker + 1);
    row = __ldg(chunk_row + worker);
    row_end = __ldg(row_ptr + row + 1);
  }

  float acc[NS][VEC];
  int colbase[NS];
  bool live[NS];
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    colbase[s] = kb + (s * 32 + lane) * VEC;
    live[s] = colbase[s] < K;  // VEC == 4 implies K % 4 == 0, so the whole vector is inside
#pragma unroll
    for (int x = 0; x < VEC; ++x) acc[s][x] = 0.f;
  }

  auto store_acc = [&](float* dst) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (!live[s]) continue;
      if (VEC == 4) {
        *reinterpret_cast<float4*>(dst + colbase[s]) =
            make_float4(acc[s][0], acc[s][1], acc[s][2], acc[s][3]);
      } else {
#pragma unroll
        for (int x = 0; x < VEC; ++x) dst[colbase[s] + x] = acc[s][x];
      }
    }
  };

  for (int base = n0; base < n1; base += 32) {
    const int jj = base + lane;
    int mycol = 0;
    float myval = 0.f;
    if (jj < n1) {
      mycol = ld_stream(col_idx + jj);
      myval = ld_stream(vals + jj);
    }
    const int cnt = min(32, n1 - base);
    for (int i = 0; i < cnt; ++i) {
      const int c = __shfl_sync(0xffffffffu, mycol, i);
      const float v = __shfl_sync(0xffffffffu, myval, i);
      const float* brow = B + (int64_t)c * K;
      float bv[NS][VEC];
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        if (live[s]) {
          if (VEC == 4) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(brow + colbase[s]));
            bv[s][0] = t.x;
            bv[s][1] = t.y;
            bv[s][2] = t.z;
            bv[s][3] = t.w;
          } else {
#pragma unroll
            for (int x = 0; x < VEC; ++x) bv[s][x] = __ldg(brow + colbase[s] + x);
          }
        } else {
#pragma unroll
          for (int x = 0; x < VEC; ++x) bv[s][x] = 0.f;
        }
      }
      if (!ROWSPLIT && base + i == row_end) {
        store_acc(C + (int64_t)row * K);
#pragma unroll
        for (int s = 0; s < NS; ++s)
#pragma unroll
          for (int x = 0; x < VEC; ++x) acc[s][x] = 0.f;
        advance_row(row_ptr, M, base + i, row, row_end);
      }
#pragma unroll
      for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int x = 0; x < VEC; ++x) acc[s][x] = fmaf(v, bv[s][x], acc[s][x]);
    }
  }

  if (ROWSPLIT || row_end == n1) {
    store_acc(C + (int64_t)row * K);
    if (!ROWSPLIT && lane == 0 && blockIdx.y == 0) carry_row[worker] = -1;
  } else {
    store_acc(carry_val + (int64_t)worker * K);
    if (lane == 0 && blockIdx.y == 0) carry_row[worker] = row;
  }
}

// ---- carries ---------------------------------------------------------------------------
// Fix-up for K = 4*W in {32, 64, 128} when the nominal chunk size S is known.  A block takes
// CB = 256 / W consecutive chunks, one group of W lanes per chunk, each lane owning four columns.
// A row longer than S is cut at multiples of S only, so the carries of row r sit in chunks
// first = row_ptr[r] / S .. last - 1 with last = (row_ptr[r+1] - 1) / S: the group of chunk `first`
// needs two loads to know the whole run, where a scan of carry_row would take one round trip per
// 32 chunks.  Short runs (a row of 300 entries has one or two carries) are summed by that group;
// tens of thousands of such independent walks hide each other's latency.  A run longer than
// kLongRun (a row of many thousand entries; at most one can start in a block, since it covers every
// later chunk of the block) is summed by the whole block: group g takes carries g, g + CB, ..., and
// the groups are combined pairwise in shared memory in a fixed order.
// The order of additions depends only on the chunking, never on timing.
constexpr int kLongRun = 32;

template <int W>
__global__ void __launch_bounds__(kBlockThreads)
carry_fixup_grouped_kernel(int n_chunks, int S, const int* __restrict__ row_ptr,
                           const int* __restrict__ carry_row, const float* __restrict__ carry_val,
                           float* __restrict__ C, int ld) {
  const int64_t K = ld;   // row stride of C and of the carry slots; the slab is 4 * W columns wide
  constexpr int CB = kBlockThreads / W;
  __shared__ int long_head, long_len, long_row;
  __shared__ float4 part[CB][W];
  const int g = threadIdx.x / W, l = threadIdx.x % W;
  const int64_t c = (int64_t)blockIdx.x * CB + g;
  if (threadIdx.x == 0) long_len = 0;
  __syncthreads();

  const int row = c < n_chunks ? carry_row[c] : -1;
  if (row >= 0) {
    const int first = __ldg(row_ptr + row) / S;
    if (c == first) {
      const int len = (__ldg(row_ptr + row + 1) - 1) / S - first;
      if (len > kLongRun) {
        if (l == 0) {
          long_head = g;
          long_len = len;
          long_row = row;
        }
      } else {
        const float* src = carry_val + c * K + l * 4;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        int i = 0;
        for (; i + 4 <= len; i += 4) {
          float4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float4*>(src + (int64_t)(i + u) * K);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            s.x += v[u].x;
            s.y += v[u].y;
            s.z += v[u].z;
            s.w += v[u].w;
          }
        }
        for (; i < len; ++i) {
          const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)i * K);
          s.x += v.x;
          s.y += v.y;
          s.z += v.z;
          s.w += v.w;
        }
        float4* out = reinterpret_cast<float4*>(C + (int64_t)row * K + l * 4);
        float4 o = *out;
        o.x += s.x;
        o.y += s.y;
        o.z += s.z;
        o.w += s.w;
        *out = o;
      }
    }
  }
  __syncthreads();
  const int len = long_len;
  if (len == 0) return;   // block-uniform

  const float* src = carry_val + ((int64_t)blockIdx.x * CB + long_head) * K + l * 4;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  int i = g;
  for (; i + 3 * CB < len; i += 4 * CB) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float4*>(src + (int64_t)(i + u * CB) * K);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s.x += v[u].x;
      s.y += v[u].y;
      s.z += v[u].z;
      s.w += v[u].w;
    }
  }
  for (; i < len; i += CB) {
    const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)i * K);
    s.x += v.x;
    s.y += v.y;
    s.z += v.z;
    s.w += v.w;
  }
  part[g][l] = s;
  __syncthreads();
#pragma unroll
  for (int o = CB / 2; o > 0; o >>= 1) {
    if (g < o) {
      const float4 a = part[g][l], b = part[g + o][l];
      part[g][l] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
    }
    __syncthreads();
  }
  if (g == 0) {
    const float4 t = part[0][l];
    float4* out = reinterpret_cast<float4*>(C + (int64_t)long_row * K + l * 4);
    float4 o = *out;
    o.x += t.x;
    o.y += t.y;
    o.z += t.z;
    o.w += t.w;
    *out = o;
  }
}

// Fix-up for any other K: one lane per chunk finds the first carry of each split row; the warp then
// counts that row's carries (32 at a time) and sums them in chunk order, lanes owning columns.
__global__ void __launch_bounds__(kBlockThreads)
carry_fixup_kernel(int K, int n_chunks, const int* __restrict__ carry_row,
                   const float* __restrict__ carry_val, float* __restrict__ C) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) >> 5;
  const int64_t c0 = warp * 32;
  if (c0 >= n_chunks) return;
  const int64_t c = c0 + lane;
  const int row = c < n_chunks ? carry_row[c] : -1;
  const int prev = (c > 0 && c < n_chunks) ? carry_row[c - 1] : -1;
  unsigned m = __ballot_sync(0xffffffffu, row >= 0 && row != prev);
  while (m) {
    const int bpos = __ffs(m) - 1;
    m &= m - 1;
    const int hr = __shfl_sync(0xffffffffu, row, bpos);
    const int64_t first = c0 + bpos;
    // length of the run of carries that belong to row hr
    int64_t len = 0;
    for (int64_t w = first;; w += 32) {
      const int64_t cc = w + lane;
      const bool same = cc < n_chunks && carry_row[cc] == hr;
      const unsigned bm = __ballot_sync(0xffffffffu, same);
      if (bm == 0xffffffffu) {
        len += 32;
        continue;
      }
      len += __ffs(~bm) - 1;
      break;
    }
    float* crow = C + (int64_t)hr * K;
    const float* src = carry_val + first * K;
    if ((K & 3) == 0) {
      for (int col = lane * 4; col < K; col += 128) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int64_t i = 0; i < len; ++i) {
          const float4 t = *reinterpret_cast<const float4*>(src + i * K + col);
          s.x += t.x;
          s.y += t.y;
          s.z += t.z;
          s.w += t.w;
        }
        float4 o = *reinterpret_cast<float4*>(crow + col);
        o.x += s.x;
        o.y += s.y;
        o.z += s.z;
        o.w += s.w;
        *reinterpret_cast<float4*>(crow + col) = o;
      }
    } else {
      for (int col = lane; col < K; col += 32) {
        float s = 0.f;
        for (int64_t i = 0; i < len; ++i) s += src[i * K + col];
        crow[col] += s;
      }
    }
  }
}

// ---- COO, accumulate -------------------------------------------------------------------
// ---- COO warp kernel: K = 4 * W in {32, 64, 128} --------------------------------------------
// C += A * B from (row, col, val) triples in any order; zero-valued entries (the padding) are
// skipped.  Same machinery as the CSR warp kernel: one warp per S consecutive triples, G = 32 / W
// lane groups that each gather a whole row of B per step, tiles of 32 triples staged global ->
// shared with cp.async two tiles ahead, U steps of gathers in flight, an unrolled path for tiles
// that lie inside one row.  Row boundaries come from the staged row ids (one ballot per tile)
// instead of row_ptr; every run of equal row ids ends in one cross-group reduction and one
// 16-byte vector reduction per lane of group 0 into C.
template <int W, int U, int BT, bool STRIDED>
__global__ void __launch_bounds__(BT, 16)
spmm_coo_warp_kernel(int64_t nnz, int S, const int* __restrict__ row_idx, const int* __restrict__ col_idx,
                     const float* __restrict__ vals, const float* __restrict__ B, float* __restrict__ C, int ld) {
  // a slab of 4 * W columns; STRIDED: part of wider B and C with row stride ld
  const int64_t K = STRIDED ? (int64_t)ld : (int64_t)(4 * W);
  constexpr int G = 32 / W;
  constexpr int T = 32;
  constexpr int BATCH = U * G;
  constexpr int STAGES = 2;
  static_assert(BATCH <= T && T % BATCH == 0, "batch must tile the staged tile");
  __shared__ int2 cv_tiles[BT / 32][STAGES][T];
  __shared__ int row_tiles[BT / 32][STAGES][T];

  const int lane = threadIdx.x & 31;
  const int g = lane / W, l = lane % W;
  const int64_t worker = ((int64_t)blockIdx.x * BT + threadIdx.x) >> 5;
  const int64_t n0 = worker * S;
  if (n0 >= nnz) return;
  const int64_t n1 = min(nnz, n0 + (int64_t)S);
  int2(*cv)[T] = cv_tiles[threadIdx.x >> 5];
  int(*rw)[T] = row_tiles[threadIdx.x >> 5];

  auto stage_tile = [&](int stage, int64_t base) {
    const int64_t j = base + lane;
    if (j < n1) {
      cp_async_4(&cv[stage][lane].x, col_idx + j);
      cp_async_4(&cv[stage][lane].y, vals + j);
      cp_async_4(&rw[stage][lane], row_idx + j);
    } else {
      cv[stage][lane] = make_int2(0, 0);   // past the chunk: column 0, value 0 (skipped)
      rw[stage][lane] = -1;
    }
    cp_async_commit();
  };
  stage_tile(0, n0);
  stage_tile(1, n0 + T);

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* Bl = B + l * 4;
  int cur_row = -1;   // row of the run being accumulated

  auto flush = [&]() {
    if (cur_row >= 0) {   // warp-uniform
      if (W == 16) {
        // the groups split the sum and every lane adds a float2: 0.378 -> 0.365 ms at K = 64 on the R-MAT
        // bench graph.  At K = 32 thirty-two scalar reductions per row cost more than eight 16-byte ones
        // save in shuffles (0.233 -> 0.236 ms), so that width keeps the full reduction.
        store_row_sum<W, true>(C + (int64_t)cur_row * K, acc, g, l);
      } else {
        const float4 t = reduce_groups<W>(acc);
        if (g == 0) red_add_v4(C + (int64_t)cur_row * K + l * 4, t);
      }
    }
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
  };

  int stage = 0;
  for (int64_t base = n0; base < n1; base += T) {
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    // bit e: triple e of the tile starts a new run (its row differs from its predecessor's);
    // triples past the chunk carry row -1 and never match, which ends the last run
    const int my_row = rw[stage][lane];
    const int prev_row = lane == 0 ? cur_row : rw[stage][lane - 1];
    unsigned bnd = __ballot_sync(0xffffffffu, my_row != prev_row);
    const int2* tile = &cv[stage][g];
    if (bnd == 0u) {
      // the whole tile continues the current run
#pragma unroll
      for (int s0 = 0; s0 < T / G; s0 += U) {
        float4 b[U];
        float v[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
          const int2 e = tile[(s0 + i) * G];
          v[i] = __int_as_float(e.y);
          b[i] = ld_gather<false>(Bl + (int64_t)e.x * K, 0ull);
        }
#pragma unroll
        for (int i = 0; i < U; ++i)
          if (v[i] != 0.f) fma4(acc, v[i], b[i]);
      }
    } else {
      const int limit = (int)min((int64_t)T, n1 - base);   // triples of this tile inside the chunk
#pragma unroll 1
      for (int u0 = 0; u0 < T; u0 += BATCH) {
        if (u0 >= limit) break;
        float4 b[U];
        float v[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
          const int2 e = tile[u0 + i * G];
          v[i] = __int_as_float(e.y);
          b[i] = ld_gather<false>(Bl + (int64_t)e.x * K, 0ull);
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
          const int lo = u0 + i * G;
          const int hi = min(lo + G, limit);
          const int mine = lo + g;
          int cur = lo;
          // warp-uniform: runs that start inside this step
          unsigned m = hi > lo ? (bnd >> lo) & ((1u << (hi - lo)) - 1u) : 0u;
          while (m) {
            const int p = lo + __ffs(m) - 1;
            m &= m - 1;
            if (mine >= cur && mine < p && v[i] != 0.f) fma4(acc, v[i], b[i]);
            flush();
            cur_row = rw[stage][p];
            cur = p;
          }
          if (mine >= cur && mine < hi && v[i] != 0.f) fma4(acc, v[i], b[i]);
        }
      }
    }
    // the last triple's row carries into the next tile's first comparison
    __syncwarp();
    stage_tile(stage, base + STAGES * T);
    stage ^= 1;
  }
  cp_async_wait<0>();
  flush();
}

// C += A * B from (row, col, val) triples in any order; zero-valued padding is skipped.
// One warp per run of S entries; a lane owns columns (s*32 + lane)*VEC of a 128*VEC-wide
// column block.  Partial sums leave through vector reductions on every row change.
template <int VEC, int NS>
__global__ void __launch_bounds__(kBlockThreads)
spmm_coo_kernel(int K, int64_t nnz, int S, const int* __restrict__ row_idx,
                const int* __restrict__ col_idx, const float* __restrict__ vals,
                const float* __restrict__ B, float* __restrict__ C) {
  const int lane = threadIdx.x & 31;
  const int64_t worker = ((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) >> 5;
  const int64_t n0 = worker * S;
  if (n0 >= nnz) return;
  const int64_t n1 = min(nnz, n0 + S);
  const int kb = blockIdx.y * (32 * VEC * NS);

  float acc[NS][VEC];
  int colbase[NS];
  bool live[NS];
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    colbase[s] = kb + (s * 32 + lane) * VEC;
    live[s] = colbase[s] < K;
#pragma unroll
    for (int x = 0; x < VEC; ++x) acc[s][x] = 0.f;
  }
  int cur_row = -1;
  bool dirty = false;

  auto flush = [&]() {
    if (!dirty) return;
    float* crow = C + (int64_t)cur_row * K;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (live[s]) {
        if (VEC == 4) {
          red_add_v4(crow + colbase[s], make_float4(acc[s][0], acc[s][1], acc[s][2], acc[s][3]));
        } else {
#pragma unroll
          for (int x = 0; x < VEC; ++x) atomicAdd(crow + colbase[s] + x, acc[s][x]);
        }
      }
#pragma unroll
      for (int x = 0; x < VEC; ++x) acc[s][x] = 0.f;
    }
    dirty = false;
  };

  for (int64_t base = n0; base < n1; base += 32) {
    const int64_t jj = base + lane;
    int myrow = 0, mycol = 0;
    float myval = 0.f;
    if (jj < n1) {
      myrow = ld_stream(row_idx + jj);
      mycol = ld_stream(col_idx + jj);
      myval = ld_stream(vals + jj);
    }
    const int cnt = (int)min((int64_t)32, n1 - base);
    for (int i = 0; i < cnt; ++i) {
      const int r = __shfl_sync(0xffffffffu, myrow, i);
      const int c = __shfl_sync(0xffffffffu, mycol, i);
      const float v = __shfl_sync(0xffffffffu, myval, i);
      if (v == 0.f) continue;  // padding (and explicit zeros) contribute nothing
      if (r != cur_row) {
        flush();
        cur_row = r;
      }
      const float* brow = B + (int64_t)c * K;
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        if (!live[s]) continue;
        if (VEC == 4) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(brow + colbase[s]));
          acc[s][0] = fmaf(v, t.x, acc[s][0]);
          acc[s][1] = fmaf(v, t.y, acc[s][1]);
          acc[s][2] = fmaf(v, t.z, acc[s][2]);
          acc[s][3] = fmaf(v, t.w, acc[s][3]);
        } else {
#pragma unroll
          for (int x = 0; x < VEC; ++x) acc[s][x] = fmaf(v, __ldg(brow + colbase[s] + x), acc[s][x]);
        }
      }
      dirty = true;
    }
  }
  flush();
}

template <int W, int R, int U, int MINB>
int launch_balanced(hpspmm_ctx* ctx, bool hint, bool rowsplit, int M, int n_chunks,
                    const int32_t* row_ptr, const int32_t* col_idx, const float* vals,
                    const float* B, float* C, const int32_t* chunk_start, const int32_t* chunk_row,
                    int32_t* carry_row, float* carry_val, cudaStream_t stream) {
  const int workers_per_block = kBlockThreads / W;
  const int n_chunk_blocks = (n_chunks + workers_per_block - 1) / workers_per_block;
  int n_zero_blocks = 0;
  if (!rowsplit) {
    n_zero_blocks = (M + kBlockThreads - 1) / kBlockThreads;
    const int cap = ctx->sm_count * 2;
    if (n_zero_blocks > cap) n_zero_blocks = cap;
  }
  const unsigned grid = (unsigned)(n_chunk_blocks + n_zero_blocks);
  if (grid == 0) return HPSPMM_OK;
#define HPSPMM_LAUNCH(H, RS)                                                                   \
  spmm_subwarp_kernel<W, R, U, MINB, H, RS><<<grid, kBlockThreads, 0, stream>>>(                    \
      M, n_chunks, n_chunk_blocks, row_ptr, col_idx, vals, B, C, chunk_start, chunk_row,       \
      carry_row, carry_val)
  if (rowsplit) {
    if (hint) HPSPMM_LAUNCH(true, true); else HPSPMM_LAUNCH(false, true);
  } else {
    if (hint) HPSPMM_LAUNCH(true, false); else HPSPMM_LAUNCH(false, false);
  }
#undef HPSPMM_LAUNCH
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

// rows that hold entries, as a plan lists them (all null without a plan)
struct row_list {
  const int32_t* nz_id;
  const int32_t* nz_end;
  const int32_t* chunk_ri;
};

template <int W, int U, int MINB, int BT = kBlockThreads, bool STRIDED = false>
int launch_warp(hpspmm_ctx* ctx, bool hint, int M, int n_chunks, const int32_t* row_ptr,
                const int32_t* col_idx, const float* vals, const float* B, float* C,
                const int32_t* chunk_start, const int32_t* chunk_row, int32_t* carry_row,
                float* carry_val, const int32_t* chunk_order, int S, int* run_counter, cudaStream_t stream,
                int ld = 4 * W, row_list rows = row_list{nullptr, nullptr, nullptr}) {
  const int chunks_per_block = BT / 32;
  const int n_chunk_blocks = (n_chunks + chunks_per_block - 1) / chunks_per_block;
  int n_zero_blocks = (M + BT - 1) / BT;
  const int cap = ctx->sm_count * 2 * (kBlockThreads / BT);
  if (n_zero_blocks > cap) n_zero_blocks = cap;
  const unsigned grid = (unsigned)(n_chunk_blocks + n_zero_blocks);
  if (grid == 0) return HPSPMM_OK;
#define HPSPMM_LAUNCH_WARP(H, ST, CP)                                                           \
  spmm_warp_kernel<W, U, MINB, H, BT, ST, STRIDED, CP><<<grid, BT, 0, stream>>>(                   \
      M, n_chunks, n_chunk_blocks, row_ptr, col_idx, vals, B, C, chunk_start, chunk_row, carry_row, \
      carry_val, chunk_order, S, run_counter, ld, rows.nz_id, rows.nz_end, rows.chunk_ri)
  const bool compact = rows.nz_id != nullptr;
  if (run_counter != nullptr) {
    if (hint) { if (compact) HPSPMM_LAUNCH_WARP(true, true, true); else HPSPMM_LAUNCH_WARP(true, true, false); }
    else { if (compact) HPSPMM_LAUNCH_WARP(false, true, true); else HPSPMM_LAUNCH_WARP(false, true, false); }
  } else {
    if (hint) { if (compact) HPSPMM_LAUNCH_WARP(true, false, true); else HPSPMM_LAUNCH_WARP(true, false, false); }
    else { if (compact) HPSPMM_LAUNCH_WARP(false, false, true); else HPSPMM_LAUNCH_WARP(false, false, false); }
  }
#undef HPSPMM_LAUNCH_WARP
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

template <int VEC>
int launch_generic(hpspmm_ctx* ctx, bool rowsplit, int M, int K, int n_chunks,
                   const int32_t* row_ptr, const int32_t* col_idx, const float* vals,
                   const float* B, float* C, const int32_t* chunk_start, const int32_t* chunk_row,
                   int32_t* carry_row, float* carry_val, const int32_t* chunk_order,
                   cudaStream_t stream) {
  constexpr int NS = 4;
  const int kblock = 32 * VEC * NS;
  const int n_kblocks = (K + kblock - 1) / kblock;
  const int n_chunk_blocks = (n_chunks + kBlockThreads / 32 - 1) / (kBlockThreads / 32);
  int n_zero_blocks = 0;
  if (!rowsplit) {
    n_zero_blocks = (M + kBlockThreads - 1) / kBlockThreads;
    const int cap = ctx->sm_count * 2;
    if (n_zero_blocks > cap) n_zero_blocks = cap;
  }
  const dim3 grid((unsigned)(n_chunk_blocks + n_zero_blocks), (unsigned)n_kblocks, 1);
  if (grid.x == 0) return HPSPMM_OK;
  if (n_kblocks > 65535) return HPSPMM_ERR_UNSUPPORTED;
  if (rowsplit)
    spmm_generic_kernel<VEC, NS, true><<<grid, kBlockThreads, 0, stream>>>(
        M, K, n_chunks, n_chunk_blocks, row_ptr, col_idx, vals, B, C, chunk_start, chunk_row,
        carry_row, carry_val, nullptr);
  else
    spmm_generic_kernel<VEC, NS, false><<<grid, kBlockThreads, 0, stream>>>(
        M, K, n_chunks, n_chunk_blocks, row_ptr, col_idx, vals, B, C, chunk_start, chunk_row,
        carry_row, carry_val, chunk_order);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

typedef CUresult (*tensor_map_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

tensor_map_encode_fn tensor_map_encoder() {
  static std::once_flag once;
  static tensor_map_encode_fn fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &found) == cudaSuccess &&
        found == cudaDriverEntryPointSuccess)
      fn = (tensor_map_encode_fn)p;
  });
  return fn;
}

// The K = 128 product with B fetched by TMA.  Returns 1 when this path cannot take the call (no encoder in
// the driver, a chunk size beyond what the kernel stages, a B the tensor map refuses): the caller then runs
// the ordinary kernel.  0 = launched, negative = error.
int launch_spmm_tma(hpspmm_ctx* ctx, int m, int nc, int64_t rows_b, const int32_t* row_ptr, const int32_t* col_idx,
                    const float* vals, const float* B, float* C, const int32_t* chunk_start,
                    const int32_t* chunk_row, float* carry_val, const int32_t* chunk_order, int S,
                    int* run_counter, row_list rows, cudaStream_t stream) {
  if (S <= 0 || S > kTmaMaxS || run_counter == nullptr || rows.nz_id == nullptr || rows_b <= 0) return 1;
  tensor_map_encode_fn enc = tensor_map_encoder();
  if (!enc) return 1;
  CUtensorMap map_b;
  const cuuint64_t gdim[2] = {128, (cuuint64_t)rows_b};
  const cuuint64_t gstride[1] = {512};
  const cuuint32_t box[2] = {128, 1};   // gather4: one row per box, four boxes per operation
  const cuuint32_t estride[2] = {1, 1};
  if (enc(&map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(B), gdim, gstride, box, estride,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return 1;
  constexpr int smem = kTmaWarps * kTmaSmemPerWarp;
  // per call: the attribute belongs to the current device's context, and a process may drive several GPUs
  if (cudaFuncSetAttribute(spmm_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    cudaGetLastError();
    return 1;
  }
  const int n_chunk_blocks = (nc + kTmaWarps - 1) / kTmaWarps;
  int n_zero_blocks = (m + kTmaWarps * 32 - 1) / (kTmaWarps * 32);
  const int cap = ctx->sm_count * 4;
  if (n_zero_blocks > cap) n_zero_blocks = cap;
  const unsigned grid = (unsigned)(n_chunk_blocks + n_zero_blocks);
  if (grid == 0) return 0;
  spmm_tma_kernel<<<grid, kTmaWarps * 32, smem, stream>>>(map_b, m, nc, n_chunk_blocks, row_ptr, col_idx, vals, B, C,
                                                          chunk_start, chunk_row, carry_val, chunk_order, S,
                                                          run_counter, rows.nz_id, rows.nz_end, rows.chunk_ri,
                                                          ctx->flag + HPSPMM_FLAG_TMA_FALLBACKS);
  ctx->launches++;
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "spmm_tma_kernel launch", e);
    return -1;
  }
  return 0;
}

}  // namespace

// Nominal chunk size of the kernels that probe row_ptr or reduce into C (the allocation-free entry, the COO
// product): measured best on B200 (R-MAT scale 20) at 128 / 160 / 256 entries for K = 32 / 64 / 128.
static int32_t probing_chunk_nnz(int64_t K) {
  if (K <= 32) return 128;
  if (K <= 64) return 160;
  return 256;
}

int32_t hpspmm_default_chunk_nnz(int64_t K, int64_t nnz) {
  // With the list of non-empty rows a row end costs two loads, and larger chunks amortise the per-chunk
  // prologue (table loads, pipeline fill) and leave fewer carries.  Measured on B200 (R-MAT scale 20, product
  // time in ms at S = 128 / 256 / 320 / 512 / 1024): K = 32: 0.240 / 0.217 / 0.208 / 0.199 / 0.193;
  // K = 64: 0.356 / 0.314 / 0.307 / 0.310 / 0.306; K = 128: 0.630 / 0.563 / 0.563 / 0.595 / 0.592.
  // Small matrices keep smaller chunks so that there are still several waves of them
  // (148 SMs x 40 resident warps x 4).
  // Re-measured at K = 32 after the row-store exchange (S = 384 / 512 / 640 / 768 / 1024 / 1280 / 1536):
  // 0.195 / 0.189 / 0.186 / 0.185 / 0.182 / 0.193 / 0.212 ms.  The default stays at 512 all the same: plans are
  // shared with the SDDMM, which on the same graph takes 0.193 / 0.230 / 0.271 / 0.333 ms at S = 512 / 640 /
  // 768 / 1024.  A caller that builds a plan for products only can ask for 1024 (hpspmm_opts.chunk_nnz).
  const int32_t floor_s = probing_chunk_nnz(K);
  const int32_t best = K <= 32 ? 512 : (K <= 64 ? 320 : 256);
  const int64_t want = nnz / 24000 / 32 * 32;
  int64_t s = want < floor_s ? floor_s : want;
  if (s > best) s = best;
  return (int32_t)s;
}

int hpspmm_launch_chunk_table(hpspmm_ctx* ctx, int64_t M, int64_t nnz, const int32_t* row_ptr,
                              int32_t chunk_nnz, int64_t n_chunks, int32_t* chunk_start,
                              int32_t* chunk_row, int* split_count, cudaStream_t stream,
                              int32_t* run_counter) {
  const unsigned blocks = (unsigned)((n_chunks + 1 + 255) / 256);
  chunk_table_kernel<<<blocks, 256, 0, stream>>>((int)M, (int)nnz, row_ptr, chunk_nnz, (int)n_chunks,
                                                 chunk_start, chunk_row, split_count, run_counter);
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

namespace {

int check_spmm_args(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t K, int64_t nnz,
                    const void* row_ptr, const void* col_idx, const void* vals, const void* B,
                    const void* C) {
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0, "negative size");
  HPSPMM_REQUIRE(ctx, K >= 1, "K must be >= 1");
  // entry positions are 32-bit and the kernels look up to one tile past a chunk's end
  if (M > 2147483646ll || N > 2147483647ll || nnz > 2147483647ll - 4096 || K > (1 << 20)) {
    snprintf(ctx->err, sizeof(ctx->err), "sizes beyond 32-bit CSR indices");
    return HPSPMM_ERR_UNSUPPORTED;
  }
  HPSPMM_REQUIRE(ctx, row_ptr != nullptr, "null row_ptr");
  HPSPMM_REQUIRE(ctx, nnz == 0 || (col_idx && vals && B), "null operand");
  HPSPMM_REQUIRE(ctx, M == 0 || C != nullptr, "null output");
  if ((K & 3) == 0 && (((uintptr_t)B & 15u) || ((uintptr_t)C & 15u))) {
    snprintf(ctx->err, sizeof(ctx->err), "dense operands must be 16-byte aligned");
    return HPSPMM_ERR_INVALID;
  }
  return HPSPMM_OK;
}

// One slab of 4 * W columns with the warp kernel, then its carries.  STRIDED: the slab is part of wider
// matrices (B, C and the carry slots have row stride ld, the pointers already point at the slab's first
// column).  With a counter array, slabs of 64 or 128 columns add the carries themselves.  Measured on the
// R-MAT bench graph against the separate fix-up launch: -6 % at 128 columns, -2 % at 64, but +7 % at 32,
// where chunks are short and the device-wide fence every piece of a split row takes weighs more than the
// launch saved.
// Tuning on B200 (R-MAT scale 20): 64-thread blocks, U = 4 gather steps in flight per lane and at most
// 51 registers (20 blocks per SM) beat 128/256-thread blocks, U = 2/8/16 and the 32/40/64/80-register
// builds at every width.
template <int W, bool STRIDED>
int run_slab(hpspmm_ctx* ctx, bool hint, int m, int nc, const int32_t* row_ptr, const int32_t* col_idx,
             const float* vals, const float* B, float* C, const int32_t* chunk_start,
             const int32_t* chunk_row, int32_t* carry_row, float* carry_val, const int32_t* chunk_order,
             bool need_fixup, cudaStream_t stream, int S, int* run_counter, int ld, row_list rows) {
  const bool settle = run_counter != nullptr && W >= 16;
  // strided slabs carry two more live values (the stride) and spill at 48 registers: 16 blocks per SM
  // (64 registers) took the K = 256 product from 1.44 to 1.20 ms
  constexpr int MINB = STRIDED ? 16 : HPSPMM_WARP_MINB;
  int st = launch_warp<W, 4, MINB, 64, STRIDED>(ctx, hint, m, nc, row_ptr, col_idx, vals, B, C, chunk_start,
                                                chunk_row, carry_row, carry_val, chunk_order, S,
                                                settle ? run_counter : nullptr, stream, ld, rows);
  if (st != HPSPMM_OK) return st;
  if (need_fixup && nc > 0 && !settle) {
    if (S > 0) {
      const unsigned gblocks = (unsigned)(((int64_t)nc * W + kBlockThreads - 1) / kBlockThreads);
      carry_fixup_grouped_kernel<W><<<gblocks, kBlockThreads, 0, stream>>>(nc, S, row_ptr, carry_row, carry_val,
                                                                         C, ld);
    } else {
      const unsigned blocks = (unsigned)((nc + kBlockThreads - 1) / kBlockThreads);
      carry_fixup_kernel<<<blocks, kBlockThreads, 0, stream>>>(4 * W, nc, carry_row, carry_val, C);
    }
    ctx->launches++;
    HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  }
  return HPSPMM_OK;
}

int run_spmm(hpspmm_ctx* ctx, bool hint, bool rowsplit, int64_t M, int64_t K, int64_t n_chunks,
             const int32_t* row_ptr, const int32_t* col_idx, const float* vals, const float* B,
             float* C, const int32_t* chunk_start, const int32_t* chunk_row, int32_t* carry_row,
             float* carry_val, const int32_t* chunk_order, bool need_fixup, cudaStream_t stream,
             int S = 0, int* run_counter = nullptr, row_list rows = row_list{nullptr, nullptr, nullptr},
             int64_t tma_rows_b = 0) {
  int st;
  const int m = (int)M, nc = (int)n_chunks;
  if (!rowsplit && K == 128 && tma_rows_b > 0) {
    // B through the tensor memory accelerator (HPSPMM_ALGO_TMA); falls through when that path declines
    const int r = launch_spmm_tma(ctx, m, nc, tma_rows_b, row_ptr, col_idx, vals, B, C, chunk_start, chunk_row,
                                  carry_val, chunk_order, S, run_counter, rows, stream);
    if (r == 0) return HPSPMM_OK;
    if (r < 0) return HPSPMM_ERR_CUDA;   // the launcher has recorded the message
  }
#define HPSPMM_ARGS ctx, hint, rowsplit, m, nc, row_ptr, col_idx, vals, B, C, chunk_start, chunk_row, carry_row, carry_val, stream
#define HPSPMM_SLAB(W, STRIDED, off) \
  run_slab<W, STRIDED>(ctx, hint, m, nc, row_ptr, col_idx, vals, B + (off), C + (off), chunk_start, chunk_row, \
                       carry_row, carry_val + (off), chunk_order, need_fixup, stream, S, run_counter, (int)K, rows)
  if (rowsplit && (K == 32 || K == 64 || K == 128)) {
    st = K == 32 ? launch_balanced<8, 1, 8, 4>(HPSPMM_ARGS)
                 : (K == 64 ? launch_balanced<16, 1, 8, 4>(HPSPMM_ARGS) : launch_balanced<32, 1, 8, 4>(HPSPMM_ARGS));
    return st;
  }
  if (!rowsplit && K == 32) return HPSPMM_SLAB(8, false, 0);
  if (!rowsplit && K == 64) return HPSPMM_SLAB(16, false, 0);
  if (!rowsplit && K == 128) return HPSPMM_SLAB(32, false, 0);
  if (!rowsplit && K % 32 == 0 && S > 0 && K <= 512) {
    // any other multiple of 32 up to 512: column slabs of 128, then 64 and/or 32, each a strided run of the
    // warp kernel (the sparse stream is read once per slab, as the reference's K / 32 grid rows read it).
    // Measured on the R-MAT bench graph against the generic kernel: K = 96 0.73 vs 1.33 ms, 160 0.95 vs 1.49,
    // 256 1.20 vs 1.61, 512 2.42 vs 2.51; beyond that the generic kernel's 2 KB contiguous gathers win.
    int64_t off = 0;
    while (K - off >= 128) {
      st = HPSPMM_SLAB(32, true, off);
      if (st != HPSPMM_OK) return st;
      off += 128;
    }
    if (K - off >= 64) {
      st = HPSPMM_SLAB(16, true, off);
      if (st != HPSPMM_OK) return st;
      off += 64;
    }
    if (K - off >= 32) {
      st = HPSPMM_SLAB(8, true, off);
      if (st != HPSPMM_OK) return st;
    }
    return HPSPMM_OK;
  }
#undef HPSPMM_ARGS
#undef HPSPMM_SLAB
  if ((K & 3) == 0)
    st = launch_generic<4>(ctx, rowsplit, m, (int)K, nc, row_ptr, col_idx, vals, B, C, chunk_start,
                           chunk_row, carry_row, carry_val, chunk_order, stream);
  else
    st = launch_generic<1>(ctx, rowsplit, m, (int)K, nc, row_ptr, col_idx, vals, B, C, chunk_start,
                           chunk_row, carry_row, carry_val, chunk_order, stream);
  if (st != HPSPMM_OK) return st;
  if (!rowsplit && need_fixup && n_chunks > 0) {
    const unsigned blocks = (unsigned)((n_chunks + kBlockThreads - 1) / kBlockThreads);
    carry_fixup_kernel<<<blocks, kBlockThreads, 0, stream>>>((int)K, nc, carry_row, carry_val, C);
    ctx->launches++;
    HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  }
  return HPSPMM_OK;
}

}  // namespace

extern "C" {

int hpspmm_plan_create(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz, const int32_t* row_ptr,
                       const int32_t* col_idx, int64_t max_K, const hpspmm_opts* opts,
                       hpspmm_stream stream, hpspmm_plan** out) {
  HPSPMM_TRACE("hpspmm_plan_create");
  HPSPMM_REQUIRE(ctx, ctx != nullptr && out != nullptr, "null context or output");
  *out = nullptr;
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0 && max_K >= 1, "bad size");
  HPSPMM_REQUIRE(ctx, row_ptr != nullptr, "null row_ptr");
  if (M > 2147483646ll || nnz > 2147483647ll - 4096) return HPSPMM_ERR_UNSUPPORTED;
  int32_t S = (opts && opts->chunk_nnz > 0) ? opts->chunk_nnz : hpspmm_default_chunk_nnz(max_K, nnz);
  S = (S + 31) / 32 * 32;
  hpspmm_device_guard guard(ctx->device);
  hpspmm_plan* p = new (std::nothrow) hpspmm_plan();
  if (!p) return HPSPMM_ERR_OOM;
  memset(p, 0, sizeof(*p));
  p->device = ctx->device;
  p->M = M;
  p->nnz = nnz;
  p->chunk_nnz = S;
  p->max_K = max_K;
  p->n_chunks = (nnz + S - 1) / S;
  const size_t b_start = align_up((size_t)(p->n_chunks + 1) * 4, 256);
  const size_t b_row = align_up((size_t)(p->n_chunks + 1) * 4, 256);
  const size_t b_crow = align_up((size_t)(p->n_chunks + 1) * 4, 256);
  const size_t b_cval = align_up((size_t)(p->n_chunks + 1) * (size_t)max_K * 4, 256);
  const size_t b_order = align_up((size_t)(p->n_chunks + 1) * 4, 256);
  const size_t b_count = align_up((size_t)(p->n_chunks + 1) * 4, 256);
  const size_t b_nz = align_up((size_t)(M + 2) * 4, 256);          // nz_id, nz_end: one slot per row + sentinel
  const size_t b_ri = align_up((size_t)(p->n_chunks + 1) * 4, 256);
  const size_t b_sort = hpspmm_order_scratch_bytes(p->n_chunks);   // only needed while building
  p->bytes = b_start + b_row + b_crow + b_cval + b_order + b_count + 2 * b_nz + b_ri + b_sort;
  char* base = nullptr;
  cudaError_t e = hpspmm_device_malloc((void**)&base, p->bytes);
  if (e != cudaSuccess) {
    delete p;
    return hpspmm_set_err(ctx, HPSPMM_ERR_OOM, "plan cudaMalloc", e);
  }
  p->chunk_start = (int32_t*)base;
  p->chunk_row = (int32_t*)(base + b_start);
  p->carry_row = (int32_t*)(base + b_start + b_row);
  p->carry_val = (float*)(base + b_start + b_row + b_crow);
  p->chunk_order = (int32_t*)(base + b_start + b_row + b_crow + b_cval);
  p->run_counter = (int32_t*)(base + b_start + b_row + b_crow + b_cval + b_order);
  p->nz_id = (int32_t*)(base + b_start + b_row + b_crow + b_cval + b_order + b_count);
  p->nz_end = (int32_t*)(base + b_start + b_row + b_crow + b_cval + b_order + b_count + b_nz);
  p->chunk_ri = (int32_t*)(base + b_start + b_row + b_crow + b_cval + b_order + b_count + 2 * b_nz);
  void* sort_scratch = base + b_start + b_row + b_crow + b_cval + b_order + b_count + 2 * b_nz + b_ri;
  cudaStream_t s = (cudaStream_t)stream;
  int st = HPSPMM_OK;
  int split = 0;
  e = cudaMemsetAsync(ctx->flag, 0, sizeof(int), s);
  if (e == cudaSuccess) e = cudaMemsetAsync(p->run_counter, 0, b_count, s);
  if (e == cudaSuccess && M > 0)
    st = hpspmm_launch_chunk_table(ctx, M, nnz, row_ptr, S, p->n_chunks, p->chunk_start,
                                   p->chunk_row, ctx->flag, s, nullptr);
  if (e == cudaSuccess && st == HPSPMM_OK && M > 0)
    st = hpspmm_order_chunks_by_cost(ctx, M, N, p->n_chunks, row_ptr, col_idx, p->chunk_start, p->chunk_row,
                                     p->chunk_order, sort_scratch, s);
  if (e == cudaSuccess && st == HPSPMM_OK && M > 0) {
    // the list of rows that hold entries (its scratch lives in the context and is free again afterwards)
    st = hpspmm_ensure_scratch(ctx, hpspmm_row_list_scratch_bytes(M));
    if (st == HPSPMM_OK)
      st = hpspmm_build_row_list(ctx, M, p->n_chunks, row_ptr, p->chunk_row, p->nz_id, p->nz_end, p->chunk_ri,
                                 ctx->scratch, s);
  }
  if (e == cudaSuccess && st == HPSPMM_OK)
    e = cudaMemcpyAsync(&split, ctx->flag, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess && st == HPSPMM_OK) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess || st != HPSPMM_OK) {
    cudaFree(base);
    delete p;
    return e != cudaSuccess ? hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "plan build", e) : st;
  }
  p->n_split_chunks = split;
  *out = p;
  return HPSPMM_OK;
}

int hpspmm_plan_destroy(hpspmm_ctx* ctx, hpspmm_plan* plan) {
  if (!plan) return HPSPMM_OK;
  hpspmm_device_guard guard(plan->device);
  if (plan->chunk_start) cudaFree(plan->chunk_start);
  delete plan;
  (void)ctx;
  return HPSPMM_OK;
}

int hpspmm_plan_info(const hpspmm_plan* plan, int64_t* n_chunks, int64_t* n_split_chunks,
                     int64_t* chunk_nnz, int64_t* scratch_bytes) {
  if (!plan) return HPSPMM_ERR_INVALID;
  if (n_chunks) *n_chunks = plan->n_chunks;
  if (n_split_chunks) *n_split_chunks = plan->n_split_chunks;
  if (chunk_nnz) *chunk_nnz = plan->chunk_nnz;
  if (scratch_bytes) *scratch_bytes = (int64_t)plan->bytes;
  return HPSPMM_OK;
}

int hpspmm_spmm_kernel_signature(const hpspmm_plan* plan, int64_t K, int32_t b_l2_hint, char* buf, size_t len) {
  if (!buf || len == 0 || K < 1) return HPSPMM_ERR_INVALID;
  const bool hint = b_l2_hint == 2 || (b_l2_hint == 0 && K >= 64);
  if (K == 32 || K == 64 || K == 128) {
    const int W = (int)K / 4;
    // the template arguments of spmm_warp_kernel as run_slab / launch_warp choose them
    snprintf(buf, len, "spmm_warp_kernel<%d,4,%d,%d,64,%d,0,1> chunk_nnz=%d", W, HPSPMM_WARP_MINB, hint ? 1 : 0,
             W >= 16 ? 1 : 0, plan ? (int)plan->chunk_nnz : (int)hpspmm_default_chunk_nnz(K, plan ? plan->nnz : 0));
  } else if (K % 32 == 0 && K <= 512) {
    snprintf(buf, len, "spmm_warp_kernel slabs of 128/64/32 columns, strided, K=%lld", (long long)K);
  } else {
    snprintf(buf, len, "spmm_generic_kernel<%d,4,0> K=%lld", (K & 3) == 0 ? 4 : 1, (long long)K);
  }
  return HPSPMM_OK;
}

int hpspmm_plan_tables(const hpspmm_plan* plan, const int32_t** chunk_start, const int32_t** chunk_row,
                       const int32_t** chunk_order) {
  if (!plan) return HPSPMM_ERR_INVALID;
  if (chunk_start) *chunk_start = plan->chunk_start;
  if (chunk_row) *chunk_row = plan->chunk_row;
  if (chunk_order) *chunk_order = plan->chunk_order;
  return HPSPMM_OK;
}

int hpspmm_plan_row_list(const hpspmm_plan* plan, const int32_t** nz_id, const int32_t** nz_end,
                         const int32_t** chunk_ri) {
  if (!plan) return HPSPMM_ERR_INVALID;
  if (nz_id) *nz_id = plan->nz_id;
  if (nz_end) *nz_end = plan->nz_end;
  if (chunk_ri) *chunk_ri = plan->chunk_ri;
  return HPSPMM_OK;
}

int hpspmm_spmm_csr_f32(hpspmm_ctx* ctx, const hpspmm_plan* plan, int64_t M, int64_t N, int64_t K,
                        int64_t nnz, const int32_t* row_ptr, const int32_t* col_idx,
                        const float* vals, const float* B, float* C, const hpspmm_opts* opts,
                        hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_spmm_csr_f32");
  int st = check_spmm_args(ctx, M, N, K, nnz, row_ptr, col_idx, vals, B, C);
  if (st != HPSPMM_OK) return st;
  if (M == 0) return HPSPMM_OK;
  hpspmm_device_guard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  const int hint_mode = opts ? opts->b_l2_hint : 0;
  // evict-last on the gathers of B, R-MAT bench graph, on / off, one width timed alone: K = 128 0.555 / 0.591 ms,
  // K = 64 0.307 / 0.304, K = 32 0.189 / 0.1885.  Inside a step of three products run back to back K = 64 measures
  // the other way round (0.311 on, 0.313 off), so 64 columns stay on.
  const bool hint = hint_mode == 2 || (hint_mode == 0 && K >= 64);
  const int algo = opts ? opts->algo : HPSPMM_ALGO_AUTO;
  if (algo == HPSPMM_ALGO_ROW_SPLIT) {
    return run_spmm(ctx, hint, true, M, K, M, row_ptr, col_idx, vals, B, C, nullptr, nullptr,
                    nullptr, nullptr, nullptr, false, s);
  }
  HPSPMM_REQUIRE(ctx, algo == HPSPMM_ALGO_AUTO || algo == HPSPMM_ALGO_BALANCED || algo == HPSPMM_ALGO_TMA,
                 "unknown algo");
  if (plan) {
    HPSPMM_REQUIRE(ctx, plan->M == M && plan->nnz == nnz, "plan built for another matrix");
    HPSPMM_REQUIRE(ctx, K <= plan->max_K, "K exceeds the plan's max_K");
    HPSPMM_REQUIRE(ctx, plan->device == ctx->device, "plan built on another device");
    return run_spmm(ctx, hint, false, M, K, plan->n_chunks, row_ptr, col_idx, vals, B, C,
                    plan->chunk_start, plan->chunk_row, plan->carry_row, plan->carry_val,
                    plan->chunk_order, plan->n_split_chunks > 0, s, plan->chunk_nnz, plan->run_counter,
                    row_list{plan->nz_id, plan->nz_end, plan->chunk_ri}, algo == HPSPMM_ALGO_TMA ? N : 0);
  }
  int32_t S = (opts && opts->chunk_nnz > 0) ? opts->chunk_nnz : hpspmm_default_chunk_nnz(K, nnz);
  S = (S + 31) / 32 * 32;
  const int64_t n_chunks = (nnz + S - 1) / S;
  const size_t b_int = align_up((size_t)(n_chunks + 1) * 4, 256);
  const size_t b_cval = align_up((size_t)(n_chunks + 1) * (size_t)K * 4, 256);
  const size_t b_sort = hpspmm_order_scratch_bytes(n_chunks);
  const size_t b_nz = align_up((size_t)(M + 2) * 4, 256);
  const size_t b_list = hpspmm_row_list_scratch_bytes(M);
  const size_t b_tmp = b_sort > b_list ? b_sort : b_list;   // the two builders run one after the other
  st = hpspmm_ensure_scratch(ctx, 6 * b_int + b_cval + 2 * b_nz + b_tmp);
  if (st != HPSPMM_OK) return st;
  char* base = (char*)ctx->scratch;
  int32_t* chunk_start = (int32_t*)base;
  int32_t* chunk_row = (int32_t*)(base + b_int);
  int32_t* carry_row = (int32_t*)(base + 2 * b_int);
  int32_t* chunk_order = (int32_t*)(base + 3 * b_int);
  int32_t* run_counter = (int32_t*)(base + 4 * b_int);
  int32_t* chunk_ri = (int32_t*)(base + 5 * b_int);
  float* carry_val = (float*)(base + 6 * b_int);
  int32_t* nz_id = (int32_t*)(base + 6 * b_int + b_cval);
  int32_t* nz_end = (int32_t*)(base + 6 * b_int + b_cval + b_nz);
  void* tmp = base + 6 * b_int + b_cval + 2 * b_nz;
  // the table kernel also zeroes the counters of the in-kernel carry settlement
  st = hpspmm_launch_chunk_table(ctx, M, nnz, row_ptr, S, n_chunks, chunk_start, chunk_row,
                                 nullptr, s, run_counter);
  if (st != HPSPMM_OK) return st;
  // cost order only: the second sort pass of the column-band order costs more per call than it saves
  st = hpspmm_order_chunks_by_cost(ctx, M, N, n_chunks, row_ptr, nullptr, chunk_start, chunk_row, chunk_order,
                                   tmp, s);
  if (st != HPSPMM_OK) return st;
  // the list of rows that hold entries: a few small launches per call, but without it a chunk in a very
  // sparse region (entries separated by dozens of empty rows) can outlast the rest of the product
  st = hpspmm_build_row_list(ctx, M, n_chunks, row_ptr, chunk_row, nz_id, nz_end, chunk_ri, tmp, s);
  if (st != HPSPMM_OK) return st;
  return run_spmm(ctx, hint, false, M, K, n_chunks, row_ptr, col_idx, vals, B, C, chunk_start,
                  chunk_row, carry_row, carry_val, chunk_order, true, s, S, run_counter,
                  row_list{nz_id, nz_end, chunk_ri});
}

// Host-buffer products, pipelined over column slabs: C[:, s] = A * B[:, s] needs only slab s of B,
// so slab s+1 is uploaded (strided 2-D copy) while slab s is multiplied (as a contiguous product of
// the slab's width) and slab s-1 is downloaded.  PCIe is full duplex: the downloads hide behind the
// uploads.  A is uploaded once, in front; the slabs of several products that share A follow one
// another through the same pipeline, so the whole call costs about
// upload(A) + upload(all B) + product and download of the last slab.
namespace {
struct host_slab {
  const float* B;   // host, first column of the slab
  float* C;         // host, first column of the slab
  int64_t K;        // row stride of the host matrices
  int64_t width;    // 32 or 64 (or K itself for widths that are not multiples of 32)
};
}  // namespace

static int host_products_pipelined(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz, const int32_t* row_ptr,
                                   const int32_t* col_idx, const float* vals, const host_slab* slabs, int n_slabs,
                                   const hpspmm_opts* opts) {
  constexpr int NBUF = 2;
  for (int i = 0; i < 3; ++i)
    if (!ctx->pipe_streams[i])
      HPSPMM_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->pipe_streams[i], cudaStreamNonBlocking));
  // the events live in the context: created once, never leaked by an error path of a call
  for (int i = 0; i < 1 + 3 * NBUF; ++i)
    if (!ctx->pipe_events[i])
      HPSPMM_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->pipe_events[i], cudaEventDisableTiming));
  cudaStream_t s_in = ctx->pipe_streams[0], s_run = ctx->pipe_streams[1], s_out = ctx->pipe_streams[2];
  cudaEvent_t ev_a = ctx->pipe_events[0];
  cudaEvent_t* ev_b = ctx->pipe_events + 1;
  cudaEvent_t* ev_run = ctx->pipe_events + 1 + NBUF;
  cudaEvent_t* ev_out = ctx->pipe_events + 1 + 2 * NBUF;
  int64_t wmax = 1;
  for (int i = 0; i < n_slabs; ++i) wmax = slabs[i].width > wmax ? slabs[i].width : wmax;
  const size_t b_rp = align_up((size_t)(M + 1) * 4, 256);
  const size_t b_nz = align_up((size_t)(nnz > 0 ? nnz : 1) * 4, 256);
  const size_t b_Bs = align_up((size_t)(N > 0 ? N : 1) * wmax * 4, 256);
  const size_t b_Cs = align_up((size_t)M * wmax * 4, 256);
  int st = hpspmm_ensure_stage(ctx, b_rp + 2 * b_nz + NBUF * (b_Bs + b_Cs));
  if (st != HPSPMM_OK) return st;
  // size the kernel scratch before anything is queued (growing it synchronises the device)
  {
    size_t need = 0;
    for (int i = 0; i < n_slabs; ++i) {
      const int64_t w = slabs[i].width;
      const int32_t S = (opts && opts->chunk_nnz > 0) ? (opts->chunk_nnz + 31) / 32 * 32 : hpspmm_default_chunk_nnz(w, nnz);
      const int64_t n_chunks = (nnz + S - 1) / S;
      const size_t b_int = align_up((size_t)(n_chunks + 1) * 4, 256);
      const size_t b_sort = hpspmm_order_scratch_bytes(n_chunks), b_list = hpspmm_row_list_scratch_bytes(M);
      const size_t want = 6 * b_int + align_up((size_t)(n_chunks + 1) * w * 4, 256) +
                          2 * align_up((size_t)(M + 2) * 4, 256) + (b_sort > b_list ? b_sort : b_list);
      need = want > need ? want : need;
    }
    st = hpspmm_ensure_scratch(ctx, need);
    if (st != HPSPMM_OK) return st;
  }
  char* base = (char*)ctx->stage;
  int32_t* d_rp = (int32_t*)base;
  int32_t* d_col = (int32_t*)(base + b_rp);
  float* d_val = (float*)(base + b_rp + b_nz);
  float* d_Bs[NBUF];
  float* d_Cs[NBUF];
  for (int i = 0; i < NBUF; ++i) {
    d_Bs[i] = (float*)(base + b_rp + 2 * b_nz + i * b_Bs);
    d_Cs[i] = (float*)(base + b_rp + 2 * b_nz + NBUF * b_Bs + i * b_Cs);
  }
  int rc = HPSPMM_OK;
  cudaError_t e = cudaSuccess;
#define PIPE_TRY(call)                      \
  if (rc == HPSPMM_OK && e == cudaSuccess) { \
    e = (call);                             \
  }
  PIPE_TRY(cudaMemcpyAsync(d_rp, row_ptr, (size_t)(M + 1) * 4, cudaMemcpyHostToDevice, s_in));
  if (nnz > 0) {
    PIPE_TRY(cudaMemcpyAsync(d_col, col_idx, (size_t)nnz * 4, cudaMemcpyHostToDevice, s_in));
    PIPE_TRY(cudaMemcpyAsync(d_val, vals, (size_t)nnz * 4, cudaMemcpyHostToDevice, s_in));
  }
  PIPE_TRY(cudaEventRecord(ev_a, s_in));
  PIPE_TRY(cudaStreamWaitEvent(s_run, ev_a, 0));
  for (int s = 0; s < n_slabs; ++s) {
    const int buf = s % NBUF;
    const host_slab& sl = slabs[s];
    // upload slab s once the product that last read this buffer is done
    if (s >= NBUF) PIPE_TRY(cudaStreamWaitEvent(s_in, ev_run[buf], 0));
    if (nnz > 0 && N > 0)
      PIPE_TRY(cudaMemcpy2DAsync(d_Bs[buf], sl.width * 4, sl.B, (size_t)sl.K * 4, sl.width * 4, (size_t)N,
                                 cudaMemcpyHostToDevice, s_in));
    PIPE_TRY(cudaEventRecord(ev_b[buf], s_in));
    // multiply once the slab has landed and the previous download from this C buffer is done
    PIPE_TRY(cudaStreamWaitEvent(s_run, ev_b[buf], 0));
    if (s >= NBUF) PIPE_TRY(cudaStreamWaitEvent(s_run, ev_out[buf], 0));
    if (rc == HPSPMM_OK && e == cudaSuccess)
      rc = hpspmm_spmm_csr_f32(ctx, nullptr, M, N, sl.width, nnz, d_rp, d_col, d_val, d_Bs[buf], d_Cs[buf], opts,
                               (hpspmm_stream)s_run);
    PIPE_TRY(cudaEventRecord(ev_run[buf], s_run));
    // download
    PIPE_TRY(cudaStreamWaitEvent(s_out, ev_run[buf], 0));
    PIPE_TRY(cudaMemcpy2DAsync(sl.C, (size_t)sl.K * 4, d_Cs[buf], sl.width * 4, sl.width * 4, (size_t)M,
                               cudaMemcpyDeviceToHost, s_out));
    PIPE_TRY(cudaEventRecord(ev_out[buf], s_out));
  }
#undef PIPE_TRY
  // drain all three streams whatever happened
  cudaError_t e1 = cudaStreamSynchronize(s_in), e2 = cudaStreamSynchronize(s_run), e3 = cudaStreamSynchronize(s_out);
  if (rc != HPSPMM_OK) return rc;
  if (e == cudaSuccess) e = e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3);
  if (e != cudaSuccess) return hpspmm_set_err(ctx, HPSPMM_ERR_CUDA, "host-buffer product pipeline", e);
  return HPSPMM_OK;
}

// Width of the column slabs a product of width K travels in.  64 columns when they divide K and leave at
// least two slabs: with both directions busy this link moves 256-byte rows at 50 GB/s each way and 128-byte
// rows at 36.  `others_overlap` (several products in one call): a 64-column product then travels whole, as
// one contiguous copy, and overlaps with its neighbours instead of with itself.  Else 32; a width that is
// no multiple of 32 travels whole.
static int64_t host_slab_width(int64_t K, bool others_overlap) {
  if (K % 32 != 0) return K;
  return (K % 64 == 0 && (K >= 128 || others_overlap)) ? 64 : 32;
}

static int append_slabs(host_slab* out, int cap, int n, const float* B, float* C, int64_t K,
                        bool others_overlap = false) {
  if (K % 32 != 0) {
    if (n >= cap) return -1;
    out[n++] = host_slab{B, C, K, K};
    return n;
  }
  const int64_t w = host_slab_width(K, others_overlap);
  for (int64_t off = 0; off < K; off += w) {
    if (n >= cap) return -1;
    out[n++] = host_slab{B + off, C + off, K, w};
  }
  return n;
}

static int host_product_slabs(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t K, int64_t nnz,
                              const int32_t* row_ptr, const int32_t* col_idx, const float* vals,
                              const float* B, float* C, const hpspmm_opts* opts) {
  host_slab slabs[64];
  const int n = append_slabs(slabs, 64, 0, B, C, K);
  if (n < 0) return HPSPMM_ERR_UNSUPPORTED;
  return host_products_pipelined(ctx, M, N, nnz, row_ptr, col_idx, vals, slabs, n, opts);
}

int hpspmm_spmm_csr_f32_host_multi(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t nnz, const int32_t* row_ptr,
                                   const int32_t* col_idx, const float* vals, int32_t n_products, const int64_t* Ks,
                                   const float* const* Bs, float* const* Cs, const hpspmm_opts* opts) {
  HPSPMM_TRACE("hpspmm_spmm_csr_f32_host_multi");
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0, "bad size");
  HPSPMM_REQUIRE(ctx, n_products >= 0 && n_products <= 16, "between 0 and 16 products per call");
  HPSPMM_REQUIRE(ctx, n_products == 0 || (Ks && Bs && Cs), "null product list");
  HPSPMM_REQUIRE(ctx, row_ptr != nullptr, "null row_ptr");
  HPSPMM_REQUIRE(ctx, nnz == 0 || (col_idx && vals), "null operand");
  if (M == 0 || n_products == 0) return HPSPMM_OK;
  const int algo = opts ? opts->algo : HPSPMM_ALGO_AUTO;
  HPSPMM_REQUIRE(ctx, algo != HPSPMM_ALGO_ROW_SPLIT, "the multi-product entry runs the balanced kernels only");
  host_slab slabs[16 * 16];
  int n = 0;
  for (int i = 0; i < n_products; ++i) {
    HPSPMM_REQUIRE(ctx, Ks[i] >= 1 && Ks[i] <= 512, "K must be between 1 and 512");
    HPSPMM_REQUIRE(ctx, Cs[i] != nullptr && (nnz == 0 || Bs[i] != nullptr), "null dense operand");
  }
  // Order of the products.  Downloads can start only after the first slab has been uploaded and multiplied, and the
  // download of the very last slab overlaps nothing, so the pipeline should begin AND end on a narrow slab: the
  // product with the narrowest slabs goes last, the next narrowest first, the others between them, widest first.
  const bool several = n_products >= 2;
  auto slab_width = [&](int i) { return host_slab_width(Ks[i], several); };
  int order[16];
  for (int i = 0; i < n_products; ++i) order[i] = i;
  std::stable_sort(order, order + n_products, [&](int a, int b) {
    return slab_width(a) != slab_width(b) ? slab_width(a) > slab_width(b) : Ks[a] > Ks[b];
  });
  if (n_products >= 3) {
    // order is now widest .. narrowest; bring the second narrowest to the front
    const int second = order[n_products - 2];
    for (int i = n_products - 2; i > 0; --i) order[i] = order[i - 1];
    order[0] = second;
  }
  for (int i = 0; i < n_products; ++i) {
    n = append_slabs(slabs, 16 * 16, n, Bs[order[i]], Cs[order[i]], Ks[order[i]], several);
    if (n < 0) return HPSPMM_ERR_UNSUPPORTED;
  }
  hpspmm_device_guard guard(ctx->device);
  return host_products_pipelined(ctx, M, N, nnz, row_ptr, col_idx, vals, slabs, n, opts);
}

int hpspmm_spmm_csr_f32_host(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t K, int64_t nnz,
                             const int32_t* row_ptr, const int32_t* col_idx, const float* vals,
                             const float* B, float* C, const hpspmm_opts* opts) {
  HPSPMM_TRACE("hpspmm_spmm_csr_f32_host");
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz >= 0 && K >= 1, "bad size");
  HPSPMM_REQUIRE(ctx, row_ptr != nullptr, "null row_ptr");
  HPSPMM_REQUIRE(ctx, nnz == 0 || (col_idx && vals && B), "null operand");
  HPSPMM_REQUIRE(ctx, M == 0 || C != nullptr, "null output");
  if (M == 0) return HPSPMM_OK;
  hpspmm_device_guard guard(ctx->device);
  const int algo = opts ? opts->algo : HPSPMM_ALGO_AUTO;
  if (nnz > 0 && N > 0 && K >= 64 && K % 32 == 0 && algo != HPSPMM_ALGO_ROW_SPLIT)
    return host_product_slabs(ctx, M, N, K, nnz, row_ptr, col_idx, vals, B, C, opts);
  const size_t b_rp = align_up((size_t)(M + 1) * 4, 256);
  const size_t b_nz = align_up((size_t)nnz * 4, 256);
  const size_t b_B = align_up((size_t)N * (size_t)K * 4, 256);
  const size_t b_C = align_up((size_t)M * (size_t)K * 4, 256);
  int st = hpspmm_ensure_stage(ctx, b_rp + 2 * b_nz + b_B + b_C);
  if (st != HPSPMM_OK) return st;
  char* base = (char*)ctx->stage;
  int32_t* d_rp = (int32_t*)base;
  int32_t* d_col = (int32_t*)(base + b_rp);
  float* d_val = (float*)(base + b_rp + b_nz);
  float* d_B = (float*)(base + b_rp + 2 * b_nz);
  float* d_C = (float*)(base + b_rp + 2 * b_nz + b_B);
  cudaStream_t s = 0;
  HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(d_rp, row_ptr, (size_t)(M + 1) * 4, cudaMemcpyHostToDevice, s));
  if (nnz > 0) {
    HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(d_col, col_idx, (size_t)nnz * 4, cudaMemcpyHostToDevice, s));
    HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(d_val, vals, (size_t)nnz * 4, cudaMemcpyHostToDevice, s));
    HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(d_B, B, (size_t)N * (size_t)K * 4, cudaMemcpyHostToDevice, s));
  }
  st = hpspmm_spmm_csr_f32(ctx, nullptr, M, N, K, nnz, d_rp, d_col, d_val, d_B, d_C, opts,
                           (hpspmm_stream)s);
  if (st != HPSPMM_OK) return st;
  HPSPMM_CUDA_TRY(ctx, cudaMemcpyAsync(C, d_C, (size_t)M * (size_t)K * 4, cudaMemcpyDeviceToHost, s));
  HPSPMM_CUDA_TRY(ctx, cudaStreamSynchronize(s));
  return HPSPMM_OK;
}

int hpspmm_spmm_coo_f32(hpspmm_ctx* ctx, int64_t M, int64_t N, int64_t K, int64_t nnz_padded,
                        const int32_t* row_idx, const int32_t* col_idx, const float* vals,
                        const float* B, float* C, const hpspmm_opts* opts, hpspmm_stream stream) {
  HPSPMM_TRACE("hpspmm_spmm_coo_f32");
  HPSPMM_REQUIRE(ctx, ctx != nullptr, "null context");
  HPSPMM_REQUIRE(ctx, M >= 0 && N >= 0 && nnz_padded >= 0 && K >= 1, "bad size");
  if (nnz_padded == 0 || M == 0) return HPSPMM_OK;
  HPSPMM_REQUIRE(ctx, row_idx && col_idx && vals && B && C, "null operand");
  if ((K & 3) == 0 && (((uintptr_t)B & 15u) || ((uintptr_t)C & 15u))) {
    snprintf(ctx->err, sizeof(ctx->err), "dense operands must be 16-byte aligned");
    return HPSPMM_ERR_INVALID;
  }
  hpspmm_device_guard guard(ctx->device);
  int32_t S = (opts && opts->chunk_nnz > 0) ? opts->chunk_nnz : 128;
  S = (S + 31) / 32 * 32;
  const int64_t n_workers = (nnz_padded + S - 1) / S;
  const int64_t blocks = (n_workers + kBlockThreads / 32 - 1) / (kBlockThreads / 32);
  if (blocks > 2147483647ll) return HPSPMM_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (K % 32 == 0 && K <= 512) {
    // 32/64/128 directly, other multiples of 32 as column slabs of 128, 64 and 32 (every slab accumulates into
    // its own columns of C, so the slabs are independent)
    int32_t Sw = (opts && opts->chunk_nnz > 0) ? opts->chunk_nnz : probing_chunk_nnz(K);
    Sw = (Sw + 31) / 32 * 32;
    constexpr int BT = 64;
    const int64_t n_w = (nnz_padded + Sw - 1) / Sw;
    const int64_t nb = (n_w + BT / 32 - 1) / (BT / 32);
    if (nb > 2147483647ll) return HPSPMM_ERR_UNSUPPORTED;
    const bool whole = K == 32 || K == 64 || K == 128;
    int64_t off = 0;
    while (off < K) {
      const int64_t w = K - off >= 128 ? 128 : (K - off >= 64 ? 64 : 32);
#define HPSPMM_COO(WW, ST) \
  spmm_coo_warp_kernel<WW, 4, BT, ST><<<(unsigned)nb, BT, 0, s>>>(nnz_padded, Sw, row_idx, col_idx, vals, B + off, \
                                                                 C + off, (int)K)
      if (w == 128) { if (whole) HPSPMM_COO(32, false); else HPSPMM_COO(32, true); }
      else if (w == 64) { if (whole) HPSPMM_COO(16, false); else HPSPMM_COO(16, true); }
      else { if (whole) HPSPMM_COO(8, false); else HPSPMM_COO(8, true); }
#undef HPSPMM_COO
      ctx->launches++;
      off += w;
    }
    HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
    return HPSPMM_OK;
  }
  if ((K & 3) == 0) {
    // narrow K keeps one column slab per lane so no lane idles on dead slabs
    if (K <= 128) {
      const dim3 grid((unsigned)blocks, 1, 1);
      spmm_coo_kernel<4, 1><<<grid, kBlockThreads, 0, s>>>((int)K, nnz_padded, S, row_idx, col_idx,
                                                           vals, B, C);
    } else {
      const int kblock = 32 * 4 * 4;
      const dim3 grid((unsigned)blocks, (unsigned)((K + kblock - 1) / kblock), 1);
      if (grid.y > 65535) return HPSPMM_ERR_UNSUPPORTED;
      spmm_coo_kernel<4, 4><<<grid, kBlockThreads, 0, s>>>((int)K, nnz_padded, S, row_idx, col_idx,
                                                           vals, B, C);
    }
  } else {
    const int kblock = 32 * 4;
    const dim3 grid((unsigned)blocks, (unsigned)((K + kblock - 1) / kblock), 1);
    if (grid.y > 65535) return HPSPMM_ERR_UNSUPPORTED;
    spmm_coo_kernel<1, 4><<<grid, kBlockThreads, 0, s>>>((int)K, nnz_padded, S, row_idx, col_idx,
                                                         vals, B, C);
  }
  ctx->launches++;
  HPSPMM_CUDA_TRY(ctx, cudaGetLastError());
  return HPSPMM_OK;
}

}  // extern "C"

// ---- CSR SpMM with its scratch in a static device array -----------------------------------
// Some callers must not allocate device memory at the moment they need a product: the
// enqueue hook of an inference-runtime plugin, a step inside a serving loop whose framework
// allocator already owns every byte of the device, or code on a latency budget that cannot
// afford the device-wide synchronisation an allocation may cause.  For them the chunk table
// and the carry slots live in the array below instead of in context-owned scratch.  The
// array is part of the library image: every GPU that loads the library holds these bytes
// until the process exits, which is why the limit is modest.
#define HPSPMM_STATIC_SCRATCH_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[HPSPMM_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxStaticDevices = 64;
struct static_scratch_state {
  bool ready;
  unsigned char* base;  // device address of g_static_scratch on this device
  int sm_count;
};
static_scratch_state g_static_state[kMaxStaticDevices];
std::mutex g_static_mutex;

void write_err(char* buf, size_t len, const char* msg) {
  if (buf && len) snprintf(buf, len, "%s", msg);
}

}  // namespace

extern "C" int hpspmm_spmm_csr_f32_static_scratch(int device_ordinal, int64_t M, int64_t N,
                                                  int64_t K, int64_t nnz, const int32_t* row_ptr,
                                                  const int32_t* col_idx, const float* vals,
                                                  const float* B, float* C, hpspmm_stream stream,
                                                  char* err_buf, size_t err_len) {
  if (err_buf && err_len) err_buf[0] = 0;
  if (device_ordinal < 0 || device_ordinal >= kMaxStaticDevices) {
    write_err(err_buf, err_len, "device ordinal out of range");
    return HPSPMM_ERR_INVALID;
  }
  {
    // a device the process cannot see must be refused here: making it current below would fail
    // silently and the array's address would be looked up on whichever device happens to be current
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device_ordinal >= count) {
      char msg[128];
      snprintf(msg, sizeof(msg), "device ordinal %d does not exist (%d visible)", device_ordinal, count);
      write_err(err_buf, err_len, msg);
      return HPSPMM_ERR_INVALID;
    }
  }
  hpspmm_ctx local;  // a stack stand-in for a context: no allocation behind it
  memset(&local, 0, sizeof(local));
  local.device = device_ordinal;
  int st = check_spmm_args(&local, M, N, K, nnz, row_ptr, col_idx, vals, B, C);
  if (st != HPSPMM_OK) {
    write_err(err_buf, err_len, local.err);
    return st;
  }
  if (M == 0) return HPSPMM_OK;

  const int32_t S = probing_chunk_nnz(K);
  const int64_t n_chunks = (nnz + S - 1) / S;
  const size_t b_int = align_up((size_t)(n_chunks + 1) * 4, 256);
  const size_t b_cval = align_up((size_t)(n_chunks + 1) * (size_t)K * 4, 256);
  const size_t need = 4 * b_int + b_cval;
  if (need > (size_t)HPSPMM_STATIC_SCRATCH_BYTES) {
    char msg[256];
    const long long max_chunks = (long long)(HPSPMM_STATIC_SCRATCH_BYTES - 5 * 256) / (16 + 4 * K) - 1;
    snprintf(msg, sizeof(msg),
             "matrix too large for the static scratch: nnz = %lld at K = %lld needs %zu bytes, the "
             "array holds %u (about %lld nnz at this K); use hpspmm_spmm_csr_f32 instead",
             (long long)nnz, (long long)K, need, (unsigned)HPSPMM_STATIC_SCRATCH_BYTES,
             max_chunks > 0 ? max_chunks * S : 0ll);
    write_err(err_buf, err_len, msg);
    return HPSPMM_ERR_UNSUPPORTED;
  }

  hpspmm_device_guard guard(device_ordinal);  // the device is current from here on
  static_scratch_state& state = g_static_state[device_ordinal];
  {
    // Once per device: the array's name is a host-side handle, not a device address, so ask
    // the runtime where the array lives on the current device.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!state.ready) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        char msg[200];
        snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        write_err(err_buf, err_len, msg);
        return HPSPMM_ERR_CUDA;
      }
      int sms = 0;
      e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_ordinal);
      if (e != cudaSuccess || sms <= 0) {
        write_err(err_buf, err_len, "cudaDeviceGetAttribute(multiprocessor count) failed");
        return HPSPMM_ERR_CUDA;
      }
      state.base = (unsigned char*)p;
      state.sm_count = sms;
      state.ready = true;
    }
  }
  local.sm_count = state.sm_count;

  // Every call rewrites the whole chunk table, zeroes the per-row counters (the table kernel does
  // both) and rewrites every carry_row entry it later reads, and a carry_val slot is read only
  // where this call hands a carry on, so nothing left over from an earlier call is ever consumed.
  int32_t* chunk_start = (int32_t*)state.base;
  int32_t* chunk_row = (int32_t*)(state.base + b_int);
  int32_t* carry_row = (int32_t*)(state.base + 2 * b_int);
  int32_t* run_counter = (int32_t*)(state.base + 3 * b_int);
  float* carry_val = (float*)(state.base + 4 * b_int);
  cudaStream_t s = (cudaStream_t)stream;
  st = hpspmm_launch_chunk_table(&local, M, nnz, row_ptr, S, n_chunks, chunk_start, chunk_row,
                                 nullptr, s, run_counter);
  if (st == HPSPMM_OK)
    st = run_spmm(&local, K >= 64, false, M, K, n_chunks, row_ptr, col_idx, vals, B, C, chunk_start,
                  chunk_row, carry_row, carry_val, /*chunk_order=*/nullptr, true, s, S, run_counter);
  if (st != HPSPMM_OK) write_err(err_buf, err_len, local.err);
  return st;
}
