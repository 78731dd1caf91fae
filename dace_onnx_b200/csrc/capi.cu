// C ABI glue: error reporting, the device status word, and dispatch of the contraction entry
// points to the tensor-core (tcgen05) or CUDA-core kernels.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"
#include "contract.cuh"

namespace b200 {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

// One status word per device, written by kernels whose bounded waits expire.
__device__ unsigned g_device_status = 0;

unsigned *device_status_ptr() {
  constexpr int kMaxDevices = 64;
  static unsigned *cache[kMaxDevices] = {};  // address of the symbol on each device; never changes
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!cache[dev]) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<unsigned *>(ptr);
  }
  return cache[dev];
}

}  // namespace b200

using namespace b200;

extern "C" B200_API int b200_version(void) { return 100; }

extern "C" B200_API const char *b200_last_error_string(void) { return g_error; }

extern "C" B200_API int b200_device_status(void) {
  unsigned v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(B200_ECUDA, "device_status: synchronize failed");
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(v)) != cudaSuccess)
    return fail(B200_ECUDA, "device_status: read failed");
  if (v != 0) {
    cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
    return fail(B200_EDEVICE, "a kernel wait expired (role mask 0x%x)", v);
  }
  return B200_OK;
}

namespace {
// numpy-style "[batch..., M, K] @ [K, N]" with a dense batch is one tall GEMM.
void flatten_dense_batch(b200_gemm_desc &d) {
  const int64_t batch = d.batch_outer * d.batch_inner;
  if (batch > 1 && d.b_stride_outer == 0 && d.b_stride_inner == 0 && d.a_stride_inner == d.M * d.lda &&
      d.y_stride_inner == d.M * d.ldy && (d.batch_outer == 1 || (d.a_stride_outer == d.batch_inner * d.a_stride_inner &&
                                                                  d.y_stride_outer == d.batch_inner * d.y_stride_inner))) {
    d.M *= batch;
    d.batch_outer = d.batch_inner = 1;
  }
}

int gemm_entry(void *stream, const b200_gemm_desc *desc, const float *A, const float *B, const float *bias,
               const float *residual, float *Y, void *workspace, size_t workspace_bytes) {
  cudaStream_t st = (cudaStream_t)stream;
  if (!desc) return fail(B200_EINVAL, "gemm: null descriptor");
  b200_gemm_desc d = *desc;
  if (d.M < 0 || d.N < 0 || d.K < 0 || d.batch_outer < 0 || d.batch_inner < 0)
    return fail(B200_EINVAL, "gemm: negative extent");
  if (d.M == 0 || d.N == 0 || d.batch_outer == 0 || d.batch_inner == 0) return B200_OK;
  if (!A || !B || !Y) return fail(B200_EINVAL, "gemm: null pointer");
  if (d.lda < d.K || d.ldy < d.N || (d.trans_b ? d.ldb < d.K : d.ldb < d.N))
    return fail(B200_EINVAL, "gemm: leading dimension smaller than the row length");
  switch (d.epilogue) {
    case B200_EPI_NONE: case B200_EPI_SCALE: break;
    case B200_EPI_BIAS: case B200_EPI_BIAS_RELU: case B200_EPI_BIAS_GELU:
      if (!bias) return fail(B200_EINVAL, "gemm: epilogue %d needs a bias", d.epilogue);
      break;
    case B200_EPI_BIAS_RESIDUAL:
      if (!bias || !residual) return fail(B200_EINVAL, "gemm: epilogue needs bias and residual");
      break;
    default: return fail(B200_EINVAL, "gemm: unknown epilogue %d", d.epilogue);
  }
  if (d.epilogue != B200_EPI_BIAS_RESIDUAL) residual = nullptr;
  if (d.epilogue == B200_EPI_NONE || d.epilogue == B200_EPI_SCALE) bias = nullptr;
  if (d.math_mode != B200_MATH_FP32X3 && d.math_mode != B200_MATH_TF32 && d.math_mode != B200_MATH_FP32)
    return fail(B200_EINVAL, "gemm: unknown math mode %d", d.math_mode);

  flatten_dense_batch(d);

  // Tensor-core path whenever TMA can address the operands; the CUDA-core kernel otherwise
  // (and when the caller asks for plain fp32 arithmetic).
  if (d.math_mode != B200_MATH_FP32 && gemm_tc_supported(d, A, B, Y))
    return gemm_tc(st, d, A, B, bias, residual, Y, workspace, workspace_bytes);
  return gemm_simt(st, d, A, B, bias, residual, Y);
}
}  // namespace

extern "C" B200_API int b200_gemm_f32(void *stream, const b200_gemm_desc *desc, const float *A, const float *B,
                             const float *bias, const float *residual, float *Y) {
  return gemm_entry(stream, desc, A, B, bias, residual, Y, nullptr, 0);
}

extern "C" B200_API size_t b200_gemm_workspace_bytes(const b200_gemm_desc *desc) {
  if (!desc || desc->M <= 0 || desc->N <= 0 || desc->K <= 0 || desc->batch_outer <= 0 || desc->batch_inner <= 0) return 0;
  b200_gemm_desc d = *desc;
  flatten_dense_batch(d);
  return gemm_tc_workspace_bytes(d);
}

extern "C" B200_API int b200_gemm_ws_f32(void *stream, const b200_gemm_desc *desc, const float *A, const float *B,
                                const float *bias, const float *residual, float *Y, void *workspace,
                                size_t workspace_bytes) {
  return gemm_entry(stream, desc, A, B, bias, residual, Y, workspace, workspace_bytes);
}

extern "C" B200_API int b200_attention_supported(const b200_attention_desc *desc, const float *Q, const float *K,
                                                 const float *V, const float *out) {
  return desc && Q && K && V && out && desc->scale > 0.f && attention_tc_supported(*desc, Q, K, V, out) ? 1 : 0;
}

extern "C" B200_API int b200_attention_f32(void *stream, const b200_attention_desc *desc, const float *Q,
                                           const float *K, const float *V, float *out) {
  if (!desc) return fail(B200_EINVAL, "attention: null descriptor");
  if (desc->batch < 0 || desc->heads < 0 || desc->seq < 0 || desc->head_dim < 1)
    return fail(B200_EINVAL, "attention: negative extent");
  if (desc->batch == 0 || desc->heads == 0 || desc->seq == 0) return B200_OK;
  if (!Q || !K || !V || !out) return fail(B200_EINVAL, "attention: null pointer");
  if (!b200_attention_supported(desc, Q, K, V, out))
    return fail(B200_EUNSUPPORTED,
                "attention: fused kernel needs TF32 mode, head_dim 64, seq %% 32 == 0 and <= 384, aligned strides "
                "(got mode %d, head_dim %lld, seq %lld); run the unfused nodes instead",
                desc->math_mode, (long long)desc->head_dim, (long long)desc->seq);
  return attention_tc((cudaStream_t)stream, *desc, Q, K, V, out);
}

static bool conv_out_shape(const b200_conv_desc &d, int64_t *oh, int64_t *ow) {
  if (d.stride_h < 1 || d.stride_w < 1 || d.KH < 1 || d.KW < 1 || d.pad_h < 0 || d.pad_w < 0) return false;
  const int64_t eh = d.H + 2 * d.pad_h - d.KH, ew = d.W + 2 * d.pad_w - d.KW;
  if (eh < 0 || ew < 0) return false;
  *oh = eh / d.stride_h + 1;
  *ow = ew / d.stride_w + 1;
  return true;
}

extern "C" B200_API size_t b200_conv2d_workspace_bytes(const b200_conv_desc *desc) {
  if (!desc) return 0;
  // alignment of X is unknown here; the tensor-core path needs this much whenever the shape allows it
  static const float *const kAligned = nullptr;
  return conv2d_tc_supported(*desc, kAligned) ? conv2d_tc_workspace_bytes(*desc) : 0;
}

extern "C" B200_API int b200_conv2d_f32(void *stream, const b200_conv_desc *desc, const float *X, const float *W,
                               const float *bias, float *Y, void *workspace, size_t workspace_bytes) {
  cudaStream_t st = (cudaStream_t)stream;
  if (!desc) return fail(B200_EINVAL, "conv: null descriptor");
  b200_conv_desc d = *desc;
  if (d.N < 0 || d.C < 1 || d.H < 1 || d.W < 1 || d.M < 0) return fail(B200_EINVAL, "conv: bad extent");
  int64_t OH, OW;
  if (!conv_out_shape(d, &OH, &OW)) return fail(B200_EINVAL, "conv: bad kernel/pad/stride");
  if (d.N == 0 || d.M == 0) return B200_OK;
  if (!X || !W || !Y) return fail(B200_EINVAL, "conv: null pointer");
  if (d.epilogue != B200_EPI_NONE && d.epilogue != B200_EPI_BIAS && d.epilogue != B200_EPI_BIAS_RELU)
    return fail(B200_EINVAL, "conv: unsupported epilogue %d", d.epilogue);
  if (d.epilogue != B200_EPI_NONE && !bias) return fail(B200_EINVAL, "conv: epilogue %d needs a bias", d.epilogue);
  if (d.epilogue == B200_EPI_NONE) bias = nullptr;
  if (d.math_mode != B200_MATH_FP32X3 && d.math_mode != B200_MATH_TF32 && d.math_mode != B200_MATH_FP32)
    return fail(B200_EINVAL, "conv: unknown math mode %d", d.math_mode);
  // Tensor-core implicit GEMM when TMA can address the NHWC copy; the CUDA-core kernel otherwise
  // (strided convolutions, channel counts that are not multiples of 4, plain fp32 arithmetic).
  if (conv2d_tc_supported(d, X)) return conv2d_tc(st, d, X, W, bias, Y, OH, OW, workspace, workspace_bytes);
  return conv2d_simt(st, d, X, W, bias, Y, OH, OW);
}
