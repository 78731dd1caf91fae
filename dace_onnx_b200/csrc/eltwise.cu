// Elementwise nodes: Add / Sub / Mul / Div / Pow with numpy broadcasting, Sqrt / Erf / Relu and the
// fused Gelu chain, plus the two layout permutations used either side of attention.
//
// All HBM-bound: 12 B per element for a binary op on two full operands, 8 B with a broadcast
// operand or for a unary op. The host collapses the broadcast shape to the smallest rank that
// still describes both operands, then picks a 128-bit vector kernel (flat, or rows x columns with
// the broadcast operand indexed per row / per column) or the generic strided kernel.
#include <math.h>

#include "common.cuh"

namespace b200 {
namespace {

template <int OP>
__device__ __forceinline__ float apply_binary(float a, float b) {
  if (OP == B200_ADD) return a + b;
  if (OP == B200_SUB) return a - b;
  if (OP == B200_MUL) return a * b;
  if (OP == B200_DIV) return a / b;
  return powf(a, b);
}

template <int OP>
__device__ __forceinline__ float apply_unary(float x) {
  if (OP == B200_SQRT) return sqrtf(x);
  if (OP == B200_ERF) return erff(x);
  if (OP == B200_RELU) return fmaxf(x, 0.f);
  return gelu_erf(x);
}

template <int OP>
__device__ __forceinline__ float4 apply_binary4(float4 a, float4 b) {
  return make_float4(apply_binary<OP>(a.x, b.x), apply_binary<OP>(a.y, b.y), apply_binary<OP>(a.z, b.z),
                     apply_binary<OP>(a.w, b.w));
}

// rows x cols view; each operand advances by (rs, cs) elements per (row, column) with cs in {0,1}.
// One float4 of output per thread per iteration; requires cols % 4 == 0 and 16-byte alignment of
// every operand that is read as a vector.
template <int OP, int RU>
__global__ void __launch_bounds__(256)
binary_rc_vec_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ c,
                     int64_t rows, int64_t cols4, int64_t a_rs, int a_cs, int64_t b_rs, int b_cs) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  if (RU == 1) {
    if (rows == 1 && gridDim.y == 1) {
      // one long row (flattened tensors): every block walks chunks of 4 x 256 consecutive vectors, four
      // independent groups of loads in flight per thread, all in the same 16 KiB
      const int64_t chunks = cols4 / (4 * 256);
      for (int64_t ch = blockIdx.x; ch < chunks; ch += gridDim.x) {
        const int64_t base = ch * (4 * 256) + threadIdx.x;
        float4 va[4], vb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t j = base + u * 256;
          if (a_cs) va[u] = ld_stream4(a + 4 * j);
          else { float t = __ldg(a); va[u] = make_float4(t, t, t, t); }
          if (b_cs) vb[u] = ld_stream4(b + 4 * j);
          else { float t = __ldg(b); vb[u] = make_float4(t, t, t, t); }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) st_stream4(c + 4 * (base + u * 256), apply_binary4<OP>(va[u], vb[u]));
      }
      for (int64_t j = chunks * (4 * 256) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < cols4; j += step) {
        float4 va, vb;
        if (a_cs) va = ld_stream4(a + 4 * j);
        else { float t = __ldg(a); va = make_float4(t, t, t, t); }
        if (b_cs) vb = ld_stream4(b + 4 * j);
        else { float t = __ldg(b); vb = make_float4(t, t, t, t); }
        st_stream4(c + 4 * j, apply_binary4<OP>(va, vb));
      }
      return;
    }
    // few (long) rows: one column group per thread and iteration
    for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
      const float *ar = a + r * a_rs;
      const float *br = b + r * b_rs;
      float *cr = c + r * cols4 * 4;
      for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < cols4; j += step) {
        float4 va, vb;
        if (a_cs) va = ld_stream4(ar + 4 * j);
        else { float t = __ldg(ar); va = make_float4(t, t, t, t); }
        if (b_cs) vb = ld_stream4(br + 4 * j);
        else { float t = __ldg(br); vb = make_float4(t, t, t, t); }
        st_stream4(cr + 4 * j, apply_binary4<OP>(va, vb));
      }
    }
    return;
  }
  // Many rows (activations [tokens, hidden] with a bias or scale row, or a per-row scalar): columns outside, rows
  // inside, RU rows per iteration, i.e. up to 2 RU independent 16-byte loads in flight per thread. An operand that
  // is the same for every row (row stride 0) stays in L1; everything else streams past it.
  const int64_t rstep = gridDim.y;
  const bool a_keep = a_rs == 0, b_keep = b_rs == 0;
  for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < cols4; j += step) {
    for (int64_t r0 = blockIdx.y; r0 < rows; r0 += RU * rstep) {
      float4 va[RU], vb[RU];
#pragma unroll
      for (int u = 0; u < RU; ++u) {
        const int64_t r = r0 + u * rstep;
        if (r < rows) {
          const float *ar = a + r * a_rs;
          const float *br = b + r * b_rs;
          if (a_cs) va[u] = a_keep ? __ldg(reinterpret_cast<const float4 *>(ar + 4 * j)) : ld_stream4(ar + 4 * j);
          else { float t = __ldg(ar); va[u] = make_float4(t, t, t, t); }
          if (b_cs) vb[u] = b_keep ? __ldg(reinterpret_cast<const float4 *>(br + 4 * j)) : ld_stream4(br + 4 * j);
          else { float t = __ldg(br); vb[u] = make_float4(t, t, t, t); }
        }
      }
#pragma unroll
      for (int u = 0; u < RU; ++u) {
        const int64_t r = r0 + u * rstep;
        if (r < rows) st_stream4(c + (r * cols4 + j) * 4, apply_binary4<OP>(va[u], vb[u]));
      }
    }
  }
}

struct StridedArgs {
  int rank;
  int64_t shape[8];
  int64_t as[8];
  int64_t bs[8];
};

template <int OP>
__global__ void __launch_bounds__(256)
binary_strided_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ c,
                      int64_t numel, StridedArgs args) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, ao = 0, bo = 0;
#pragma unroll 1
    for (int d = args.rank - 1; d >= 0; --d) {
      const int64_t q = rem / args.shape[d];
      const int64_t idx = rem - q * args.shape[d];
      rem = q;
      ao += idx * args.as[d];
      bo += idx * args.bs[d];
    }
    c[i] = apply_binary<OP>(a[ao], b[bo]);
  }
}

template <int OP>
__global__ void __launch_bounds__(256)
unary_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t numel, bool vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nth = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = numel >> 2;
    // Each block walks chunks of 4 x 256 consecutive vectors: four independent 16-byte loads in flight per thread,
    // all in the same 16 KiB of memory.
    const int64_t chunks = n4 / (4 * 256);
    for (int64_t ch = blockIdx.x; ch < chunks; ch += gridDim.x) {
      const int64_t base = ch * (4 * 256) + threadIdx.x;
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ld_stream4(x + 4 * (base + u * 256));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[u].x = apply_unary<OP>(v[u].x); v[u].y = apply_unary<OP>(v[u].y);
        v[u].z = apply_unary<OP>(v[u].z); v[u].w = apply_unary<OP>(v[u].w);
        st_stream4(y + 4 * (base + u * 256), v[u]);
      }
    }
    for (int64_t i = chunks * (4 * 256) + tid; i < n4; i += nth) {
      float4 v = ld_stream4(x + 4 * i);
      v.x = apply_unary<OP>(v.x); v.y = apply_unary<OP>(v.y);
      v.z = apply_unary<OP>(v.z); v.w = apply_unary<OP>(v.w);
      st_stream4(y + 4 * i, v);
    }
    for (int64_t i = (n4 << 2) + tid; i < numel; i += nth) y[i] = apply_unary<OP>(x[i]);
  } else {
    for (int64_t i = tid; i < numel; i += nth) y[i] = apply_unary<OP>(x[i]);
  }
}

// out[a,c,b,:] = in[a,b,c,:], rows of d3 floats moved as float4 (d3 % 4 == 0) or scalars.
__global__ void __launch_bounds__(256)
transpose_0213_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t d0, int64_t d1, int64_t d2,
                      int64_t d3v, bool vec) {
  const int64_t total = d0 * d1 * d2 * d3v;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = i % d3v;
    int64_t r = i / d3v;
    const int64_t b = r % d1;  // output order [d0, d2, d1, d3]: fastest after e is the old axis 1
    r /= d1;
    const int64_t cc = r % d2;
    const int64_t aa = r / d2;
    const int64_t src = ((aa * d1 + b) * d2 + cc) * d3v + e;
    if (vec) st_stream4(y + 4 * i, ld_stream4(x + 4 * src));
    else y[i] = x[src];
  }
}

__global__ void __launch_bounds__(256)
transpose_2d_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t batch, int64_t rows, int64_t cols) {
  __shared__ float tile[32][33];
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int64_t b = blockIdx.z; b < batch; b += gridDim.z) {  // grid.z is capped at 65535
    const float *xb = x + b * rows * cols;
    float *yb = y + b * rows * cols;
    for (int k = ty; k < 32; k += 8)
      if (r0 + k < rows && c0 + tx < cols) tile[k][tx] = xb[(r0 + k) * cols + c0 + tx];
    __syncthreads();
    for (int k = ty; k < 32; k += 8)
      if (c0 + k < cols && r0 + tx < rows) yb[(c0 + k) * rows + r0 + tx] = tile[tx][k];
    __syncthreads();
  }
}

// Same, 64 x 64 tiles moved with 128-bit accesses on both sides (rows % 4 == 0, cols % 4 == 0,
// 16-byte aligned pointers): the NCHW -> NHWC pre-pass of the tensor-core convolution runs on this.
__global__ void __launch_bounds__(256)
transpose_2d_vec_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t batch, int64_t rows, int64_t cols) {
  __shared__ float tile[64][65];
  const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
  const int q = (threadIdx.x & 15) * 4, l = threadIdx.x >> 4;  // 16 float4 per tile row, 16 rows per pass
  for (int64_t b = blockIdx.z; b < batch; b += gridDim.z) {  // grid.z is capped at 65535
    const float *xb = x + b * rows * cols;
    float *yb = y + b * rows * cols;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = l + 16 * i;
      if (r0 + r < rows && c0 + q < cols) {
        const float4 v = ld_stream4(xb + (r0 + r) * cols + c0 + q);
        tile[r][q + 0] = v.x; tile[r][q + 1] = v.y; tile[r][q + 2] = v.z; tile[r][q + 3] = v.w;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = l + 16 * i;  // input column = output row
      if (c0 + c < cols && r0 + q < rows)
        st_stream4(yb + (c0 + c) * rows + r0 + q, make_float4(tile[q + 0][c], tile[q + 1][c], tile[q + 2][c], tile[q + 3][c]));
    }
    __syncthreads();
  }
}

// ONNXMaxPool, 2-D, no padding, floor mode: one thread per output element; the kh x kw window is read
// through L1 (neighbouring threads share its cache lines), so every input byte leaves HBM once.
__global__ void __launch_bounds__(256)
maxpool2d_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t planes, int H, int W, int OH, int OW,
                 int kh, int kw, int sh, int sw) {
  const int64_t total = planes * OH * OW;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int ow = (int)(i % OW);
    const int64_t r = i / OW;
    const int oh = (int)(r % OH);
    const int64_t plane = r / OH;
    const float *src = x + (plane * H + (int64_t)oh * sh) * W + (int64_t)ow * sw;
    float m = -3.402823466e+38f;  // lowest finite float: the initial value of the pure expansion
    for (int a = 0; a < kh; ++a)
      for (int b = 0; b < kw; ++b) m = fmaxf(m, __ldg(src + (int64_t)a * W + b));
    y[i] = m;
  }
}

inline unsigned grid_for(int64_t work_items, int threads) {
  int64_t g = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)kNumSMs * 16;  // grid-stride loops cover the rest
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (unsigned)g;
}

template <int OP>
int launch_binary(cudaStream_t st, const float *a, const float *b, float *c, int rank, const int64_t *shape,
                  const int64_t *as, const int64_t *bs) {
  // Drop size-1 axes and merge adjacent axes that both operands traverse contiguously.
  int64_t sh[8], sa[8], sb[8];
  int n = 0;
  int64_t numel = 1;
  for (int d = 0; d < rank; ++d) {
    if (shape[d] < 0) return fail(B200_EINVAL, "binary: negative extent");
    numel *= shape[d];
  }
  if (numel == 0) return B200_OK;
  for (int d = 0; d < rank; ++d) {
    if (shape[d] == 1) continue;
    if (n > 0 && sa[n - 1] == as[d] * shape[d] && sb[n - 1] == bs[d] * shape[d]) {
      sh[n - 1] *= shape[d];
      sa[n - 1] = as[d];
      sb[n - 1] = bs[d];
    } else {
      sh[n] = shape[d]; sa[n] = as[d]; sb[n] = bs[d];
      ++n;
    }
  }
  if (n == 0) { sh[0] = 1; sa[0] = 0; sb[0] = 0; n = 1; }

  // rows x cols forms: rank 1 (one row) or rank 2 with unit/zero column strides.
  int64_t rows = 1, cols = sh[n - 1], a_rs = 0, b_rs = 0;
  bool rc = false;
  if (n == 1) rc = true;
  else if (n == 2) { rc = true; rows = sh[0]; a_rs = sa[0]; b_rs = sb[0]; }
  const int64_t a_cs = sa[n - 1], b_cs = sb[n - 1];
  if (rc && (a_cs == 0 || a_cs == 1) && (b_cs == 0 || b_cs == 1) && cols % 4 == 0 && aligned16(c) &&
      (a_cs == 0 || (aligned16(a) && a_rs % 4 == 0)) && (b_cs == 0 || (aligned16(b) && b_rs % 4 == 0)) &&
      (rows == 1 || cols >= 64)) {
    const int64_t cols4 = cols / 4;
    unsigned gx = (unsigned)((cols4 + 255) / 256);
    if (gx > (unsigned)kNumSMs * 16) gx = kNumSMs * 16;
    int64_t gy = rows;
    const int64_t want = ((int64_t)kNumSMs * 16 + gx - 1) / gx;
    if (gy > want) gy = want;
    if (gy > 65535) gy = 65535;
    if (rows >= 4 * gy)
      binary_rc_vec_kernel<OP, 4><<<dim3(gx, (unsigned)gy), 256, 0, st>>>(a, b, c, rows, cols4, a_rs, (int)a_cs, b_rs,
                                                                         (int)b_cs);
    else
      binary_rc_vec_kernel<OP, 1><<<dim3(gx, (unsigned)gy), 256, 0, st>>>(a, b, c, rows, cols4, a_rs, (int)a_cs, b_rs,
                                                                         (int)b_cs);
    return check_launch("binary_rc_vec");
  }
  StridedArgs args;
  args.rank = n;
  for (int d = 0; d < n; ++d) { args.shape[d] = sh[d]; args.as[d] = sa[d]; args.bs[d] = sb[d]; }
  binary_strided_kernel<OP><<<grid_for(numel, 256), 256, 0, st>>>(a, b, c, numel, args);
  return check_launch("binary_strided");
}

template <int OP>
int launch_unary(cudaStream_t st, const float *x, float *y, int64_t numel) {
  const bool vec = aligned16(x) && aligned16(y);
  unary_kernel<OP><<<grid_for(vec ? (numel + 3) / 4 : numel, 256), 256, 0, st>>>(x, y, numel, vec);
  return check_launch("unary");
}

}  // namespace

int transpose_2d(cudaStream_t st, const float *x, float *y, int64_t batch, int64_t rows, int64_t cols) {
  if ((rows + 31) / 32 > 65535) return fail(B200_EUNSUPPORTED, "transpose: more than 65535 x 32 rows");
  if (batch < 1 || rows < 1 || cols < 1) return B200_OK;
  const unsigned gz = (unsigned)(batch < 65535 ? batch : 65535);  // larger batches loop inside the kernel
  if (rows % 4 == 0 && cols % 4 == 0 && aligned16(x) && aligned16(y)) {
    dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64), gz);
    transpose_2d_vec_kernel<<<grid, 256, 0, st>>>(x, y, batch, rows, cols);
    return check_launch("transpose_2d_vec");
  }
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), gz);
  transpose_2d_kernel<<<grid, 256, 0, st>>>(x, y, batch, rows, cols);
  return check_launch("transpose_2d");
}

}  // namespace b200

using namespace b200;

extern "C" B200_API int b200_binary_f32(void *stream, int op, const float *a, const float *b, float *c, int rank,
                               const int64_t *shape, const int64_t *a_strides, const int64_t *b_strides) {
  cudaStream_t st = (cudaStream_t)stream;
  if (rank < 0 || rank > 8) return fail(B200_EUNSUPPORTED, "binary: rank %d > 8", rank);
  if (rank > 0 && (!shape || !a_strides || !b_strides)) return fail(B200_EINVAL, "binary: null shape/strides");
  if (!a || !b || !c) {
    int64_t numel = 1;
    for (int d = 0; d < rank; ++d) numel *= shape[d];
    if (numel == 0) return B200_OK;
    return fail(B200_EINVAL, "binary: null pointer");
  }
  switch (op) {
    case B200_ADD: return launch_binary<B200_ADD>(st, a, b, c, rank, shape, a_strides, b_strides);
    case B200_SUB: return launch_binary<B200_SUB>(st, a, b, c, rank, shape, a_strides, b_strides);
    case B200_MUL: return launch_binary<B200_MUL>(st, a, b, c, rank, shape, a_strides, b_strides);
    case B200_DIV: return launch_binary<B200_DIV>(st, a, b, c, rank, shape, a_strides, b_strides);
    case B200_POW: return launch_binary<B200_POW>(st, a, b, c, rank, shape, a_strides, b_strides);
  }
  return fail(B200_EINVAL, "binary: unknown op %d", op);
}

extern "C" B200_API int b200_unary_f32(void *stream, int op, const float *x, float *y, int64_t numel) {
  cudaStream_t st = (cudaStream_t)stream;
  if (numel < 0) return fail(B200_EINVAL, "unary: negative extent");
  if (numel == 0) return B200_OK;
  if (!x || !y) return fail(B200_EINVAL, "unary: null pointer");
  switch (op) {
    case B200_SQRT: return launch_unary<B200_SQRT>(st, x, y, numel);
    case B200_ERF: return launch_unary<B200_ERF>(st, x, y, numel);
    case B200_RELU: return launch_unary<B200_RELU>(st, x, y, numel);
    case B200_GELU: return launch_unary<B200_GELU>(st, x, y, numel);
  }
  return fail(B200_EINVAL, "unary: unknown op %d", op);
}

extern "C" B200_API int b200_transpose_0213_f32(void *stream, const float *x, float *y, int64_t d0, int64_t d1,
                                       int64_t d2, int64_t d3) {
  cudaStream_t st = (cudaStream_t)stream;
  if (d0 < 0 || d1 < 0 || d2 < 0 || d3 < 0) return fail(B200_EINVAL, "transpose: negative extent");
  if (d0 * d1 * d2 * d3 == 0) return B200_OK;
  if (!x || !y) return fail(B200_EINVAL, "transpose: null pointer");
  const bool vec = (d3 % 4 == 0) && aligned16(x) && aligned16(y);
  const int64_t d3v = vec ? d3 / 4 : d3;
  transpose_0213_kernel<<<grid_for(d0 * d1 * d2 * d3v, 256), 256, 0, st>>>(x, y, d0, d1, d2, d3v, vec);
  return check_launch("transpose_0213");
}

extern "C" B200_API int b200_transpose_2d_f32(void *stream, const float *x, float *y, int64_t batch, int64_t rows,
                                     int64_t cols) {
  cudaStream_t st = (cudaStream_t)stream;
  if (batch < 0 || rows < 0 || cols < 0) return fail(B200_EINVAL, "transpose: negative extent");
  if (batch * rows * cols == 0) return B200_OK;
  if (!x || !y) return fail(B200_EINVAL, "transpose: null pointer");
  return transpose_2d(st, x, y, batch, rows, cols);
}

extern "C" B200_API int b200_maxpool2d_f32(void *stream, const float *x, float *y, int64_t planes, int64_t H, int64_t W,
                                  int64_t kh, int64_t kw, int64_t sh, int64_t sw) {
  cudaStream_t st = (cudaStream_t)stream;
  if (planes < 0 || H < 0 || W < 0) return fail(B200_EINVAL, "maxpool: negative extent");
  if (kh < 1 || kw < 1 || sh < 1 || sw < 1) return fail(B200_EINVAL, "maxpool: kernel and strides must be positive");
  if (H > 0x7fffffffLL || W > 0x7fffffffLL || kh > H || kw > W) {
    if (planes == 0 || H == 0 || W == 0) return B200_OK;
    return fail(B200_EINVAL, "maxpool: window larger than the image");
  }
  const int64_t OH = (H - kh) / sh + 1, OW = (W - kw) / sw + 1;
  if (planes * OH * OW == 0) return B200_OK;
  if (!x || !y) return fail(B200_EINVAL, "maxpool: null pointer");
  maxpool2d_kernel<<<grid_for(planes * OH * OW, 256), 256, 0, st>>>(x, y, planes, (int)H, (int)W, (int)OH, (int)OW,
                                                                   (int)kh, (int)kw, (int)sh, (int)sw);
  return check_launch("maxpool2d");
}
