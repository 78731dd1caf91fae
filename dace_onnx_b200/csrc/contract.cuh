// Declarations shared by the contraction kernels (CUDA-core and tcgen05 paths) and their C ABI.
#pragma once

#include "common.cuh"

namespace b200 {

// Fused epilogue applied to one accumulator value; node order of the chains it replaces:
//   BIAS          MatMul/Gemm/Conv -> Add(bias)
//   BIAS_RELU     ... -> Relu
//   BIAS_GELU     ... -> Div(sqrt2) -> Erf -> Add 1 -> Mul x -> Mul 0.5
//   BIAS_RESIDUAL ... -> Add(residual)
//   SCALE         MatMul -> Mul(constant)
__device__ __forceinline__ float apply_epilogue(int epi, float acc, float bias, float residual, float scale) {
  switch (epi) {
    case B200_EPI_BIAS: return acc + bias;
    case B200_EPI_BIAS_RELU: return fmaxf(acc + bias, 0.f);
    case B200_EPI_BIAS_GELU: return gelu_erf(acc + bias);
    case B200_EPI_BIAS_RESIDUAL: return (acc + bias) + residual;
    case B200_EPI_SCALE: return acc * scale;
    default: return acc;
  }
}

// Same, with the epilogue fixed at compile time (used inside unrolled per-row loops so that the
// choice is made once per block, not once per element).
template <int EPI>
__device__ __forceinline__ float apply_epilogue_t(float acc, float bias, float residual, float scale) {
  if (EPI == B200_EPI_BIAS) return acc + bias;
  if (EPI == B200_EPI_BIAS_RELU) return fmaxf(acc + bias, 0.f);
  if (EPI == B200_EPI_BIAS_GELU) return gelu_erf(acc + bias);
  if (EPI == B200_EPI_BIAS_RESIDUAL) return (acc + bias) + residual;
  if (EPI == B200_EPI_SCALE) return acc * scale;
  return acc;
}

int gemm_simt(cudaStream_t st, const b200_gemm_desc &d, const float *A, const float *B, const float *bias,
              const float *residual, float *Y);
int conv2d_simt(cudaStream_t st, const b200_conv_desc &d, const float *X, const float *W, const float *bias,
                float *Y, int64_t OH, int64_t OW);

// tcgen05 path. `can_*` say whether the operands meet the TMA addressing rules (16-byte aligned
// bases and row strides, K a multiple of 4); the launchers assume they do.
bool gemm_tc_supported(const b200_gemm_desc &d, const float *A, const float *B, const float *Y);
// `workspace` (optional, may be null): gemm_tc_workspace_bytes(d) bytes of device scratch; with it the 3xTF32
// mode pre-splits B and runs the CTA-pair kernel.
size_t gemm_tc_workspace_bytes(const b200_gemm_desc &d);
int gemm_tc(cudaStream_t st, const b200_gemm_desc &d, const float *A, const float *B, const float *bias,
            const float *residual, float *Y, void *workspace = nullptr, size_t workspace_bytes = 0);

// Tensor-core convolution (stride 1, channel counts that are multiples of 4 and >= 16, 16-byte aligned X).
// The filter is prepared once (repacked to [M][tap][Cp]; in 3xTF32 mode also split into hi / lo) into
// conv2d_filter_bytes(d) bytes; conv2d_run then takes NCHW or NHWC tensors (flags B200_CONV_X_NHWC /
// B200_CONV_Y_NHWC; NHWC only where conv2d_nhwc_supported) and needs conv2d_run_workspace_bytes(d, flags)
// bytes of scratch (the NHWC copy of an NCHW input). Shapes the tensor cores cannot take run on conv2d_simt.
bool conv2d_tc_supported(const b200_conv_desc &d, const float *X);
size_t conv2d_filter_bytes(const b200_conv_desc &d);
int conv2d_prepare_filter(cudaStream_t st, const b200_conv_desc &d, const float *W, void *filter, size_t filter_bytes);
bool conv2d_nhwc_supported(const b200_conv_desc &d);
size_t conv2d_run_workspace_bytes(const b200_conv_desc &d, int flags);
int conv2d_run(cudaStream_t st, const b200_conv_desc &d, int flags, const float *X, const void *filter,
               const float *bias, float *Y, int64_t OH, int64_t OW, void *workspace, size_t workspace_bytes);
// the general implicit-GEMM kernel (any output-channel count; NHWC copy in, NCHW out)
int conv2d_tc_gemm(cudaStream_t st, const b200_conv_desc &d, const float *xt, const float *wt, const float *bias,
                   float *Y, int64_t OH, int64_t OW);

bool attention_tc_supported(const b200_attention_desc &d, const float *Q, const float *K, const float *V,
                            const float *out);
int attention_tc(cudaStream_t st, const b200_attention_desc &d, const float *Q, const float *K, const float *V,
                 float *out);

// out[b][c][r] = in[b][r][c]
int transpose_2d(cudaStream_t st, const float *x, float *y, int64_t batch, int64_t rows, int64_t cols);

}  // namespace b200
