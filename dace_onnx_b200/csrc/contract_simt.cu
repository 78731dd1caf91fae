// CUDA-core fp32 contraction kernels (B200_MATH_FP32): a register-tiled GEMM and a direct
// convolution that accept every shape, stride and alignment the C ABI allows. They serve the
// shapes the tensor-core path cannot address with TMA (row strides that are not multiples of
// 16 bytes, K < 8, C1's 10/32/120-wide layers) and are the exact-fp32 arm of the parity tests.
#include "common.cuh"
#include "contract.cuh"

namespace b200 {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

// 256 threads, each owning a 4x4 block of the 64x64 output tile.
template <bool TRANS_B>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias,
                 const float *__restrict__ residual, float *__restrict__ Y, b200_gemm_desc d) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int64_t batch = blockIdx.z;
  const int64_t bo = batch / d.batch_inner, bi = batch % d.batch_inner;
  A += bo * d.a_stride_outer + bi * d.a_stride_inner;
  B += bo * d.b_stride_outer + bi * d.b_stride_inner;
  const int64_t yoff = bo * d.y_stride_outer + bi * d.y_stride_inner;
  const int64_t m0 = (int64_t)blockIdx.x * BM, n0 = (int64_t)blockIdx.y * BN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  // Two-level sum: `acc` holds at most kFoldK products, then folds into `tot`. A single fp32 running sum over
  // thousands of products loses ~sqrt(K) ulps to rounding; partial sums of 256 keep long-K results (K = 4096
  // in the FFN) inside the fp32 parity tolerance.
  constexpr int kFoldK = 256;
  float acc[4][4] = {}, tot[4][4] = {};
  for (int64_t k0 = 0; k0 < d.K; k0 += BK) {
    if (k0 && k0 % kFoldK == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { tot[i][j] += acc[i][j]; acc[i][j] = 0.f; }
    }
    // A tile: BM x BK, K contiguous in memory.
    for (int i = tid; i < BM * BK; i += 256) {
      const int kk = i % BK, mm = i / BK;
      const int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < d.M && k < d.K) ? A[m * d.lda + k] : 0.f;
    }
    for (int i = tid; i < BN * BK; i += 256) {
      int kk, nn;
      if (TRANS_B) { kk = i % BK; nn = i / BK; } else { nn = i % BN; kk = i / BN; }
      const int64_t n = n0 + nn, k = k0 + kk;
      float v = 0.f;
      if (n < d.N && k < d.K) v = TRANS_B ? B[n * d.ldb + k] : B[k * d.ldb + n];
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= d.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= d.N) continue;
      const int64_t o = yoff + m * d.ldy + n;
      Y[o] = apply_epilogue(d.epilogue, tot[i][j] + acc[i][j], bias ? bias[n] : 0.f, residual ? residual[o] : 0.f, d.scale);
    }
  }
}

// Direct NCHW convolution, one thread per output element, accumulation order (c, kh, kw).
__global__ void __launch_bounds__(256)
conv2d_simt_kernel(const float *__restrict__ X, const float *__restrict__ Wt, const float *__restrict__ bias,
                   float *__restrict__ Y, b200_conv_desc d, int64_t OH, int64_t OW) {
  const int64_t total = d.N * d.M * OH * OW;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t ow = i % OW;
    int64_t r = i / OW;
    const int64_t oh = r % OH;
    r /= OH;
    const int64_t m = r % d.M;
    const int64_t n = r / d.M;
    float acc = 0.f;
    for (int64_t c = 0; c < d.C; ++c) {
      const float *xp = X + (n * d.C + c) * d.H * d.W;
      const float *wp = Wt + (m * d.C + c) * d.KH * d.KW;
      for (int64_t kh = 0; kh < d.KH; ++kh) {
        const int64_t ih = oh * d.stride_h + kh - d.pad_h;
        if (ih < 0 || ih >= d.H) continue;
        for (int64_t kw = 0; kw < d.KW; ++kw) {
          const int64_t iw = ow * d.stride_w + kw - d.pad_w;
          if (iw < 0 || iw >= d.W) continue;
          acc = fmaf(xp[ih * d.W + iw], wp[kh * d.KW + kw], acc);
        }
      }
    }
    Y[i] = apply_epilogue(d.epilogue, acc, bias ? bias[m] : 0.f, 0.f, 1.f);
  }
}

}  // namespace

int gemm_simt(cudaStream_t st, const b200_gemm_desc &d, const float *A, const float *B, const float *bias,
              const float *residual, float *Y) {
  const int64_t batch = d.batch_outer * d.batch_inner;
  const int64_t gx = (d.M + BM - 1) / BM, gy = (d.N + BN - 1) / BN;
  if (batch > 65535 || gy > 65535 || gx > 0x7fffffffLL)
    return fail(B200_EUNSUPPORTED, "gemm(fp32): batch %lld or N-tiles %lld exceed the grid limit", (long long)batch,
                (long long)gy);
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batch);
  if (d.trans_b) gemm_simt_kernel<true><<<grid, 256, 0, st>>>(A, B, bias, residual, Y, d);
  else gemm_simt_kernel<false><<<grid, 256, 0, st>>>(A, B, bias, residual, Y, d);
  return check_launch("gemm_simt");
}

int conv2d_simt(cudaStream_t st, const b200_conv_desc &d, const float *X, const float *W, const float *bias,
                float *Y, int64_t OH, int64_t OW) {
  const int64_t total = d.N * d.M * OH * OW;
  int64_t g = (total + 255) / 256;
  if (g > (int64_t)kNumSMs * 32) g = (int64_t)kNumSMs * 32;
  conv2d_simt_kernel<<<(unsigned)g, 256, 0, st>>>(X, W, bias, Y, d, OH, OW);
  return check_launch("conv2d_simt");
}

}  // namespace b200
