// Row-wise kernels: Softmax, LogSoftmax, ReduceMean and the fused LayerNormalization chain.
//
// All of them are HBM-bound: the algorithmic traffic is one read and one write of the tensor
// (4 B + 4 B per element). Every kernel therefore touches each element of global memory exactly
// once: a row is loaded with 128-bit streaming loads into registers (one warp per row, rows up to
// 2048 elements) or into shared memory (one CTA per row, rows up to 48K elements), reduced with
// warp shuffles, and written back with 128-bit streaming stores. Arithmetic follows the node
// order of the reference's pure expansions (max, subtract, exp, sum, divide; mean, centred
// second moment, sqrt, divide) with IEEE expf/logf/sqrtf and true division (no fast-math).
#include <math.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace b200 {
namespace {

constexpr int kWarpsPerCta = 8;

enum class RowOp { Softmax, LogSoftmax };

// ---------------------------------------------------------------------------------------------
// Warp-per-row softmax / logsoftmax, row resident in registers as VPT float4 per lane.
// Requires len % 4 == 0 and 16-byte aligned x / y.
// ---------------------------------------------------------------------------------------------
template <int VPT, RowOp OP>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
softmax_warp_vec_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int len) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float *xr = x + row * len;
  float *yr = y + row * len;
  const int nvec = len >> 2;

  float4 v[VPT];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      v[i] = ld_stream4(xr + 4 * c);
      m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    }
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      v[i].x -= m; v[i].y -= m; v[i].z -= m; v[i].w -= m;
      if (OP == RowOp::Softmax) {
        v[i].x = expf(v[i].x); v[i].y = expf(v[i].y); v[i].z = expf(v[i].z); v[i].w = expf(v[i].w);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      } else {
        s += (expf(v[i].x) + expf(v[i].y)) + (expf(v[i].z) + expf(v[i].w));
      }
    }
  }
  s = warp_sum(s);
  const float ls = (OP == RowOp::LogSoftmax) ? logf(s) : 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float4 o;
      if (OP == RowOp::Softmax) {
        o.x = v[i].x / s; o.y = v[i].y / s; o.z = v[i].z / s; o.w = v[i].w / s;
      } else {
        o.x = v[i].x - ls; o.y = v[i].y - ls; o.z = v[i].z - ls; o.w = v[i].w - ls;
      }
      st_stream4(yr + 4 * c, o);
    }
  }
}

// Warp-per-row, scalar accesses, row resident in registers (len <= 32*EPT). Any alignment.
template <int EPT, RowOp OP>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
softmax_warp_scalar_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int len) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float *xr = x + row * len;
  float *yr = y + row * len;
  float v[EPT];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int c = lane + 32 * i;
    if (c < len) { v[i] = xr[c]; m = fmaxf(m, v[i]); }
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int c = lane + 32 * i;
    if (c < len) {
      v[i] -= m;
      if (OP == RowOp::Softmax) { v[i] = expf(v[i]); s += v[i]; } else { s += expf(v[i]); }
    }
  }
  s = warp_sum(s);
  const float ls = (OP == RowOp::LogSoftmax) ? logf(s) : 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int c = lane + 32 * i;
    if (c < len) yr[c] = (OP == RowOp::Softmax) ? v[i] / s : v[i] - ls;
  }
}

__device__ __forceinline__ float block_reduce(float v, float *red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();  // protects `red` against the previous reduction's readers
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int i = 0; i < nwarp; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

// CTA-per-row; the row is staged once in shared memory when it fits (cached == true), otherwise
// re-read from global (three passes) for rows beyond the shared-memory capacity.
template <RowOp OP>
__global__ void __launch_bounds__(512)
softmax_block_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t len, bool cached) {
  extern __shared__ float srow[];
  __shared__ float red[32];
  const float *xr = x + (int64_t)blockIdx.x * len;
  float *yr = y + (int64_t)blockIdx.x * len;
  float m = -INFINITY;
  for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
    float t = xr[c];
    if (cached) srow[c] = t;
    m = fmaxf(m, t);
  }
  m = block_reduce(m, red, true);
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
    float t = (cached ? srow[c] : xr[c]) - m;
    float e = expf(t);
    if (cached) srow[c] = (OP == RowOp::Softmax) ? e : t;
    s += e;
  }
  s = block_reduce(s, red, false);
  const float ls = (OP == RowOp::LogSoftmax) ? logf(s) : 0.f;
  for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
    float t;
    if (cached) t = srow[c];
    else { t = xr[c] - m; if (OP == RowOp::Softmax) t = expf(t); }
    yr[c] = (OP == RowOp::Softmax) ? t / s : t - ls;
  }
}

// Reduced axis is not the last one: one thread per (outer, inner) column, consecutive threads on
// consecutive `inner` so every access is coalesced. Three passes over the column.
template <RowOp OP>
__global__ void softmax_strided_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t outer,
                                       int64_t len, int64_t inner) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= outer * inner) return;
  const int64_t base = (t / inner) * len * inner + (t % inner);
  float m = -INFINITY;
  for (int64_t k = 0; k < len; ++k) m = fmaxf(m, x[base + k * inner]);
  float s = 0.f;
  for (int64_t k = 0; k < len; ++k) s += expf(x[base + k * inner] - m);
  const float ls = logf(s);
  for (int64_t k = 0; k < len; ++k) {
    float d = x[base + k * inner] - m;
    y[base + k * inner] = (OP == RowOp::Softmax) ? expf(d) / s : d - ls;
  }
}

// ---------------------------------------------------------------------------------------------
// LayerNormalization chain, warp-per-row, row resident in registers.
// ---------------------------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
layernorm_warp_vec_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                          const float *__restrict__ beta, float *__restrict__ y, int64_t rows, int len,
                          float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float *xr = x + row * len;
  float *yr = y + row * len;
  const int nvec = len >> 2;
  float4 v[VPT];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      v[i] = ld_stream4(xr + 4 * c);
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  const float mean = warp_sum(s) / (float)len;  // ReduceMean
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;      // Sub
      q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);  // Pow 2
    }
  }
  const float var = warp_sum(q) / (float)len;  // ReduceMean
  const float sd = sqrtf(var + eps);           // Add eps, Sqrt
  // Div: one IEEE reciprocal per row, then a multiply per element. x * (1/sd) differs from x / sd by
  // at most one ulp; a per-element IEEE division would make this kernel instruction-bound.
  const float inv = 1.0f / sd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float4 o;
      o.x = v[i].x * inv; o.y = v[i].y * inv; o.z = v[i].z * inv; o.w = v[i].w * inv;
      if (gamma) {
        const float4 g = *reinterpret_cast<const float4 *>(gamma + 4 * c);
        o.x *= g.x; o.y *= g.y; o.z *= g.z; o.w *= g.w;  // Mul
      }
      if (beta) {
        const float4 b = *reinterpret_cast<const float4 *>(beta + 4 * c);
        o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;  // Add
      }
      st_stream4(yr + 4 * c, o);
    }
  }
}

// The same arithmetic with the rows staged in shared memory by the bulk-copy engine. One persistent CTA per SM,
// 16 warps; every warp owns a ring of `depth` row buffers in shared memory and keeps `depth` rows of loads in
// flight with cp.async.bulk (a row is one contiguous block of global memory, so one instruction by one lane moves
// it and signals an mbarrier): ~190 KiB in flight per SM regardless of what the warps are doing, where register
// staging keeps only what the resident warps have issued. gamma / beta live in registers for the whole kernel.
// Rows are walked from the last to the first, with plain (not evict-first) stores: a tensor this size is usually
// the output of a GEMM whose last tiles are still in L2 when this kernel starts, and the GEMM that follows reads
// this kernel's output from row 0 up (measured inside the encoder step: 27.6 -> 25.3 ms per 960 launches).
constexpr int kBulkWarps = 16;

__device__ __forceinline__ void bulk_load_row(uint32_t dst, const float *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <int VPT>
__global__ void __launch_bounds__(kBulkWarps * 32, 1)
layernorm_bulk_kernel(const float *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                      float *__restrict__ y, int64_t rows, int len, float eps, int depth, unsigned *status) {
  extern __shared__ __align__(128) uint8_t ln_smem[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row_bytes = (uint32_t)len * 4;
  uint64_t *bars = reinterpret_cast<uint64_t *>(ln_smem + (size_t)kBulkWarps * depth * row_bytes);
  const uint32_t my_bar = tc::smem_u32(bars + warp * depth);
  const uint32_t my_buf = tc::smem_u32(ln_smem + (size_t)warp * depth * row_bytes);
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kBulkWarps * depth; ++i) tc::mbar_init(tc::smem_u32(bars + i), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  volatile int *abort_flag = &s_abort;
  const int64_t nwarps = (int64_t)gridDim.x * kBulkWarps;
  const int64_t first = (int64_t)blockIdx.x * kBulkWarps + warp;
  const int nvec = len >> 2;

  float4 g[VPT], b[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    g[i] = (gamma && c < nvec) ? __ldg(reinterpret_cast<const float4 *>(gamma + 4 * c)) : make_float4(1.f, 1.f, 1.f, 1.f);
    b[i] = (beta && c < nvec) ? __ldg(reinterpret_cast<const float4 *>(beta + 4 * c)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (lane == 0) {
    for (int j = 0; j < depth; ++j) {
      const int64_t r = first + j * nwarps;
      if (r < rows) {
        tc::mbar_expect_tx(my_bar + 8 * j, row_bytes);
        bulk_load_row(my_buf + j * row_bytes, x + (rows - 1 - r) * len, row_bytes, my_bar + 8 * j);
      }
    }
  }
  int slot = 0;
  uint32_t ph = 0;
  for (int64_t row = first; row < rows; row += nwarps) {
    if (!tc::mbar_wait(my_bar + 8 * slot, ph, abort_flag, status, 128u)) break;
    const float4 *src = reinterpret_cast<const float4 *>(ln_smem + ((size_t)warp * depth + slot) * row_bytes);
    float4 v[VPT];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        v[i] = src[c];
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    // the row is in registers: refill this buffer with the row `depth` iterations ahead
    __syncwarp();
    if (lane == 0) {
      const int64_t next = row + (int64_t)depth * nwarps;
      if (next < rows) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc::mbar_expect_tx(my_bar + 8 * slot, row_bytes);
        bulk_load_row(my_buf + slot * row_bytes, x + (rows - 1 - next) * len, row_bytes, my_bar + 8 * slot);
      }
    }
    const float mean = warp_sum(s) / (float)len;  // ReduceMean
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (lane + 32 * i < nvec) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;                   // Sub
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);  // Pow 2
      }
    }
    const float var = warp_sum(q) / (float)len;  // ReduceMean
    const float inv = 1.0f / sqrtf(var + eps);   // Add eps, Sqrt; Div as one reciprocal per row (see above)
    float *yr = y + (rows - 1 - row) * len;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        float4 o;
        o.x = v[i].x * inv; o.y = v[i].y * inv; o.z = v[i].z * inv; o.w = v[i].w * inv;
        if (gamma) { o.x *= g[i].x; o.y *= g[i].y; o.z *= g[i].z; o.w *= g[i].w; }  // Mul
        if (beta) { o.x += b[i].x; o.y += b[i].y; o.z += b[i].z; o.w += b[i].w; }    // Add
        *reinterpret_cast<float4 *>(yr + 4 * c) = o;
      }
    }
    if (++slot == depth) { slot = 0; ph ^= 1; }
  }
  // an aborting warp may still have copies in flight into this CTA's shared memory: give them time to land
  __syncthreads();
  if (s_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
}

// CTA-per-row fallback for any length / alignment (row cached in shared memory when it fits).
__global__ void __launch_bounds__(512)
layernorm_block_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                       const float *__restrict__ beta, float *__restrict__ y, int64_t len, float eps,
                       bool cached) {
  extern __shared__ float srow[];
  __shared__ float red[32];
  const float *xr = x + (int64_t)blockIdx.x * len;
  float *yr = y + (int64_t)blockIdx.x * len;
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
    float t = xr[c];
    if (cached) srow[c] = t;
    s += t;
  }
  const float mean = block_reduce(s, red, false) / (float)len;
  float q = 0.f;
  for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
    float d = (cached ? srow[c] : xr[c]) - mean;
    q += d * d;
  }
  const float sd = sqrtf(block_reduce(q, red, false) / (float)len + eps);
  for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
    float o = ((cached ? srow[c] : xr[c]) - mean) / sd;
    if (gamma) o *= gamma[c];
    if (beta) o += beta[c];
    yr[c] = o;
  }
}

// ---------------------------------------------------------------------------------------------
// ReduceMean over [outer, len, inner].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerCta * 32)
reduce_mean_last_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int64_t len,
                        bool vec) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float *xr = x + row * len;
  float s = 0.f;
  if (vec) {
    for (int64_t c = lane; c < (len >> 2); c += 32) {
      float4 v = ld_stream4(xr + 4 * c);
      s += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (int64_t c = lane; c < len; c += 32) s += xr[c];
  }
  s = warp_sum(s);
  if (lane == 0) y[row] = s / (float)len;
}

__global__ void reduce_mean_strided_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t outer,
                                           int64_t len, int64_t inner) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= outer * inner) return;
  const int64_t base = (t / inner) * len * inner + (t % inner);
  float s = 0.f;
  for (int64_t k = 0; k < len; ++k) s += x[base + k * inner];
  y[t] = s / (float)len;
}

constexpr int kMaxSmemRow = 48 * 1024;  // floats cached per CTA-per-row kernel (192 KiB)

template <RowOp OP>
int launch_softmax(cudaStream_t st, const float *x, float *y, int64_t outer, int64_t len, int64_t inner) {
  if (outer < 0 || len < 0 || inner < 0) return fail(B200_EINVAL, "softmax: negative extent");
  if (outer == 0 || len == 0 || inner == 0) return B200_OK;
  if (!x || !y) return fail(B200_EINVAL, "softmax: null pointer");
  if (inner > 1) {
    const int64_t cols = outer * inner;
    softmax_strided_kernel<OP><<<(unsigned)((cols + 255) / 256), 256, 0, st>>>(x, y, outer, len, inner);
    return check_launch("softmax_strided");
  }
  const int64_t rows = outer;
  const unsigned grid_w = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
  const bool vec_ok = (len % 4 == 0) && aligned16(x) && aligned16(y);
  if (vec_ok && len <= 2048) {
    const int nvec = (int)(len >> 2);
#define B200_SM_VEC(V)                                                                           \
  softmax_warp_vec_kernel<V, OP><<<grid_w, kWarpsPerCta * 32, 0, st>>>(x, y, rows, (int)len)
    if (nvec <= 32) B200_SM_VEC(1);
    else if (nvec <= 64) B200_SM_VEC(2);
    else if (nvec <= 96) B200_SM_VEC(3);
    else if (nvec <= 128) B200_SM_VEC(4);
    else if (nvec <= 256) B200_SM_VEC(8);
    else B200_SM_VEC(16);
#undef B200_SM_VEC
    return check_launch("softmax_warp_vec");
  }
  if (len <= 1024) {
#define B200_SM_SC(E)                                                                            \
  softmax_warp_scalar_kernel<E, OP><<<grid_w, kWarpsPerCta * 32, 0, st>>>(x, y, rows, (int)len)
    if (len <= 32) B200_SM_SC(1);
    else if (len <= 128) B200_SM_SC(4);
    else if (len <= 512) B200_SM_SC(16);
    else B200_SM_SC(32);
#undef B200_SM_SC
    return check_launch("softmax_warp_scalar");
  }
  if (rows > 0x7fffffffLL) return fail(B200_EUNSUPPORTED, "softmax: more than 2^31-1 long rows");
  const bool cached = len <= kMaxSmemRow;
  const size_t smem = cached ? (size_t)len * sizeof(float) : 0;
  // Per-device function attribute; setting it on every call of this rare path keeps the library
  // free of per-process state.
  if (cudaFuncSetAttribute(softmax_block_kernel<OP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kMaxSmemRow * (int)sizeof(float)) != cudaSuccess)
    return fail(B200_ECUDA, "softmax: cannot raise the dynamic shared memory limit");
  softmax_block_kernel<OP><<<(unsigned)rows, 512, smem, st>>>(x, y, len, cached);
  return check_launch("softmax_block");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" B200_API int b200_softmax_f32(void *stream, const float *x, float *y, int64_t outer, int64_t len,
                                int64_t inner) {
  return launch_softmax<RowOp::Softmax>((cudaStream_t)stream, x, y, outer, len, inner);
}

extern "C" B200_API int b200_logsoftmax_f32(void *stream, const float *x, float *y, int64_t outer, int64_t len,
                                   int64_t inner) {
  return launch_softmax<RowOp::LogSoftmax>((cudaStream_t)stream, x, y, outer, len, inner);
}

extern "C" B200_API int b200_reduce_mean_f32(void *stream, const float *x, float *y, int64_t outer, int64_t len,
                                    int64_t inner) {
  cudaStream_t st = (cudaStream_t)stream;
  if (outer < 0 || len <= 0 || inner < 0) return fail(B200_EINVAL, "reduce_mean: bad extent");
  if (outer == 0 || inner == 0) return B200_OK;
  if (!x || !y) return fail(B200_EINVAL, "reduce_mean: null pointer");
  if (inner > 1) {
    const int64_t cols = outer * inner;
    reduce_mean_strided_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, st>>>(x, y, outer, len, inner);
    return check_launch("reduce_mean_strided");
  }
  const bool vec = (len % 4 == 0) && aligned16(x);
  reduce_mean_last_kernel<<<(unsigned)((outer + kWarpsPerCta - 1) / kWarpsPerCta), kWarpsPerCta * 32, 0, st>>>(
      x, y, outer, len, vec);
  return check_launch("reduce_mean_last");
}

extern "C" B200_API int b200_layernorm_f32(void *stream, const float *x, const float *gamma, const float *beta,
                                  float *y, int64_t rows, int64_t len, float eps) {
  cudaStream_t st = (cudaStream_t)stream;
  if (rows < 0 || len <= 0) return fail(B200_EINVAL, "layernorm: bad extent");
  if (rows == 0) return B200_OK;
  if (!x || !y) return fail(B200_EINVAL, "layernorm: null pointer");
  const bool vec_ok = (len % 4 == 0) && aligned16(x) && aligned16(y) && (!gamma || aligned16(gamma)) &&
                      (!beta || aligned16(beta));
  // Large tensors of BERT-width rows: the persistent bulk-copy kernel (measured inside the encoder step it sustains
  // 0.85 of the HBM copy rate where the one-row-per-warp kernel reaches 0.78); small ones: one warp per row.
  if (vec_ok && len <= 1024 && len >= 256 && rows >= 4 * kBulkWarps * kNumSMs) {
    const int nvec = (int)(len >> 2);
    int depth = (int)((200 * 1024) / ((size_t)kBulkWarps * len * 4));
    if (depth > 8) depth = 8;
    const size_t smem = (size_t)kBulkWarps * depth * len * 4 + (size_t)kBulkWarps * depth * 8;
    unsigned *status = device_status_ptr();
    if (!status) return fail(B200_ECUDA, "layernorm: device status word unavailable");
#define B200_LN_BULK(V)                                                                                              \
  do {                                                                                                               \
    if (cudaFuncSetAttribute(layernorm_bulk_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024) !=   \
        cudaSuccess)                                                                                                 \
      return fail(B200_ECUDA, "layernorm: cannot raise the dynamic shared memory limit");                           \
    layernorm_bulk_kernel<V><<<kNumSMs, kBulkWarps * 32, smem, st>>>(x, gamma, beta, y, rows, (int)len, eps, depth,  \
                                                                     status);                                        \
  } while (0)
    if (nvec <= 128) B200_LN_BULK(4);
    else if (nvec <= 192) B200_LN_BULK(6);
    else B200_LN_BULK(8);
#undef B200_LN_BULK
    return check_launch("layernorm_bulk");
  }
  if (vec_ok && len <= 2048) {
    const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
    const int nvec = (int)(len >> 2);
#define B200_LN_VEC(V)                                                                           \
  layernorm_warp_vec_kernel<V><<<grid, kWarpsPerCta * 32, 0, st>>>(x, gamma, beta, y, rows, (int)len, eps)
    if (nvec <= 32) B200_LN_VEC(1);
    else if (nvec <= 64) B200_LN_VEC(2);
    else if (nvec <= 128) B200_LN_VEC(4);
    else if (nvec <= 192) B200_LN_VEC(6);
    else if (nvec <= 256) B200_LN_VEC(8);
    else B200_LN_VEC(16);
#undef B200_LN_VEC
    return check_launch("layernorm_warp_vec");
  }
  if (rows > 0x7fffffffLL) return fail(B200_EUNSUPPORTED, "layernorm: more than 2^31-1 long rows");
  const bool cached = len <= kMaxSmemRow;
  const size_t smem = cached ? (size_t)len * sizeof(float) : 0;
  if (cudaFuncSetAttribute(layernorm_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kMaxSmemRow * (int)sizeof(float)) != cudaSuccess)
    return fail(B200_ECUDA, "layernorm: cannot raise the dynamic shared memory limit");
  layernorm_block_kernel<<<(unsigned)rows, 512, smem, st>>>(x, gamma, beta, y, len, eps, cached);
  return check_launch("layernorm_block");
}
