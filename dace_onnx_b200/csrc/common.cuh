// Shared host/device helpers of libb200ops: error reporting across the C ABI, launch checks,
// warp reductions and 128-bit vector access.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "b200_ops.h"

namespace b200 {

// Thread-local message behind b200_last_error_string().
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

// Device status word: kernels with bounded waits OR a code in here when a wait expires.
unsigned *device_status_ptr();

inline int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return B200_OK;
}

constexpr int kNumSMs = 148;

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Streaming 128-bit accesses: row-wise and elementwise kernels touch every byte exactly once,
// so loads bypass L1 allocation and stores are marked evict-first.
__device__ __forceinline__ float4 ld_stream4(const float *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream4(float *p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// erf-based Gelu exactly as the exported node chain computes it:
// Div(x, sqrt2) -> Erf -> Add 1 -> Mul x -> Mul 0.5.
// The division by sqrt(2) is a multiplication by 1/sqrt(2) (<= 1 ulp apart): an IEEE division per
// element would dominate the GEMM epilogue that calls this 128 times per thread and tile.
__device__ __forceinline__ float gelu_erf(float x) {
  float t = erff(x * 0.70710678118654752440f);
  return (x * (t + 1.0f)) * 0.5f;
}

}  // namespace b200
