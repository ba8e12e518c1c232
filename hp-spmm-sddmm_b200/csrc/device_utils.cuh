// Small device helpers: cache-hinted loads / stores and vector reductions (sm_100a PTX).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hpspmm {

// L2 policy that asks the cache to keep the gathered rows of the dense operand.
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// 16-byte read-only gather of a dense row fragment with an L2 residency policy attached.
__device__ __forceinline__ float4 ld_gather_keep(const float* p, uint64_t policy) {
  float4 v;
  asm("ld.global.nc.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
      : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
      : "l"(p), "l"(policy));
  return v;
}

__device__ __forceinline__ float4 ld_gather_plain(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}

template <bool HINT>
__device__ __forceinline__ float4 ld_gather(const float* p, uint64_t policy) {
  if (HINT) return ld_gather_keep(p, policy);
  return ld_gather_plain(p);
}

// Streaming (read-once) scalar loads of the sparse operand: do not pollute L1.
__device__ __forceinline__ int ld_stream(const int* p) {
  int v;
  asm("ld.global.nc.L1::no_allocate.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_stream(const float* p) {
  float v;
  asm("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// 4-byte asynchronous copy global -> shared (completion tracked per thread in commit groups).
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Streaming 16-byte store of an output row fragment.
__device__ __forceinline__ void st_stream(float* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

// 16-byte vector reduction into global memory (no return value).
__device__ __forceinline__ void red_add_v4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

__device__ __forceinline__ void fma4(float4& acc, float a, const float4& b) {
  acc.x = fmaf(a, b.x, acc.x);
  acc.y = fmaf(a, b.y, acc.y);
  acc.z = fmaf(a, b.z, acc.z);
  acc.w = fmaf(a, b.w, acc.w);
}

// Lanes of the calling thread's W-wide sub-warp, as a shuffle mask.
template <int W>
__device__ __forceinline__ unsigned subwarp_mask() {
  if (W == 32) return 0xffffffffu;
  const unsigned lane = threadIdx.x & 31u;
  return ((1u << W) - 1u) << (lane & ~(unsigned)(W - 1));
}

}  // namespace hpspmm
