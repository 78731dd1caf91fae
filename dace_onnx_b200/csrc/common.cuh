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

// erf for the fused Gelu: Abramowitz & Stegun 7.1.26, erf(|x|) = 1 - (a1 t + ... + a5 t^5) exp(-x^2) with
// t = 1 / (1 + p |x|). Absolute error below 6e-7 in fp32 (checked against float64 over [-8, 8]), about a dozen
// instructions with two special-function operations, against ~35 for erff(): the Gelu epilogue runs 32768 times
// per 128 x 256 tile next to the thread that issues the MMAs, and with erff() it slowed that GEMM by 10-25 %.
// The standalone Erf node keeps erff().
__device__ __forceinline__ float erf_fast(float x) {
  const float ax = fabsf(x);
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.0f)));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  p *= t;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(ax * ax * -1.4426950408889634f));
  return copysignf(fmaf(-p, e, 1.0f), x);
}

// erf-based Gelu as the exported node chain computes it: Div(x, sqrt2) -> Erf -> Add 1 -> Mul x -> Mul 0.5
// (the division as a multiplication by 1/sqrt(2), <= 1 ulp apart; erf as above: |Gelu error| < 5e-7 + rounding,
// inside the 1e-5 absolute tolerance of the fp32 parity bar).
__device__ __forceinline__ float gelu_erf(float x) {
  const float t = erf_fast(x * 0.70710678118654752440f);
  return (x * (t + 1.0f)) * 0.5f;
}

}  // namespace b200
