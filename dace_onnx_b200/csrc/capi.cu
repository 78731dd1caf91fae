// C ABI glue: error reporting, the device status word, and dispatch of the contraction entry
// points to the tensor-core (tcgen05) or CUDA-core kernels.
#include <stdarg.h>
#include <string.h>

#include <atomic>

#include "common.cuh"
#include "contract.cuh"
#include "tc_common.cuh"

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
  // address of the symbol on each device; never changes. Atomic, so that host threads making their first calls
  // concurrently race benignly (they store the same value).
  static std::atomic<unsigned *> cache[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  unsigned *p = cache[dev].load(std::memory_order_relaxed);
  if (!p) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
    p = static_cast<unsigned *>(ptr);
    cache[dev].store(p, std::memory_order_relaxed);
  }
  return p;
}

// Self-test of the bounded wait every tensor-core kernel uses: one CTA, one mbarrier that nothing ever arrives at,
// no copies in flight, no TMEM. The wait gives up after `budget` cycles, records `code` in the status word and the
// kernel returns normally.
__global__ void __launch_bounds__(32)
wait_expiry_selftest_kernel(unsigned *status, long long budget, unsigned code) {
  __shared__ uint64_t bar;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    tc::mbar_init(tc::smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (threadIdx.x == 0) tc::mbar_wait_budget(tc::smem_u32(&bar), 0, &s_abort, status, code, budget);
}

}  // namespace b200

using namespace b200;

extern "C" B200_API int b200_version(void) { return 100; }

extern "C" B200_API int b200_selftest_wait_expiry(void *stream, int64_t budget_cycles) {
  if (budget_cycles < 1 || budget_cycles > 100000000LL)
    return fail(B200_EINVAL, "selftest: the budget must be between 1 and 1e8 cycles");
  unsigned *status = device_status_ptr();
  if (!status) return fail(B200_ECUDA, "selftest: device status word unavailable");
  wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (long long)budget_cycles, 0x8000u);
  return check_launch("wait_expiry_selftest");
}

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
  if (d.math_mode != B200_MATH_FP32X3 && d.math_mode != B200_MATH_TF32 && d.math_mode != B200_MATH_FP32 &&
      d.math_mode != B200_MATH_BF16)
    return fail(B200_EINVAL, "gemm: unknown math mode %d", d.math_mode);

  flatten_dense_batch(d);

  // Tensor-core path whenever TMA can address the operands; the CUDA-core kernel otherwise
  // (and when the caller asks for plain fp32 arithmetic).
  // (BF16 copies its operands into the workspace, so the TMA addressing rules do not bind its inputs.)
  const bool bf16_dense = d.math_mode == B200_MATH_BF16 && d.batch_outer * d.batch_inner == 1 && d.M <= 0x7fffffffLL &&
                          d.N <= 0x7fffffffLL && d.K >= 1 && d.K <= 0x7fffffffLL;
  if (d.math_mode != B200_MATH_FP32 && (bf16_dense || gemm_tc_supported(d, A, B, Y)))
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
  if (!desc || !Q || !K || !V || !out || !(desc->scale > 0.f)) return 0;
  b200_attention_desc d = *desc;
  if (d.math_mode == B200_MATH_BF16) d.math_mode = B200_MATH_TF32;  // the fused kernel computes a BF16 request in TF32
  return attention_tc_supported(d, Q, K, V, out) ? 1 : 0;
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
                "attention: fused kernel needs the TF32 (or BF16) mode, head_dim 64, seq %% 32 == 0, aligned strides "
                "(got mode %d, head_dim %lld, seq %lld); run the unfused nodes instead",
                desc->math_mode, (long long)desc->head_dim, (long long)desc->seq);
  b200_attention_desc d = *desc;
  if (d.math_mode == B200_MATH_BF16) d.math_mode = B200_MATH_TF32;
  return attention_tc((cudaStream_t)stream, d, Q, K, V, out);
}

static bool conv_out_shape(const b200_conv_desc &d, int64_t *oh, int64_t *ow) {
  if (d.stride_h < 1 || d.stride_w < 1 || d.KH < 1 || d.KW < 1 || d.pad_h < 0 || d.pad_w < 0) return false;
  const int64_t eh = d.H + 2 * d.pad_h - d.KH, ew = d.W + 2 * d.pad_w - d.KW;
  if (eh < 0 || ew < 0) return false;
  *oh = eh / d.stride_h + 1;
  *ow = ew / d.stride_w + 1;
  return true;
}

namespace {
inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

// Argument checks shared by the convolution entry points; on success *bias is null unless the epilogue uses it.
int conv_check(const char *who, b200_conv_desc &d, const float *X, const void *W, const float **bias,
               const float *Y, int64_t *OH, int64_t *OW, bool *empty) {
  if (d.N < 0 || d.C < 1 || d.H < 1 || d.W < 1 || d.M < 0) return fail(B200_EINVAL, "%s: bad extent", who);
  if (!conv_out_shape(d, OH, OW)) return fail(B200_EINVAL, "%s: bad kernel/pad/stride", who);
  *empty = d.N == 0 || d.M == 0;
  if (*empty) return B200_OK;
  if (!X || !W || !Y) return fail(B200_EINVAL, "%s: null pointer", who);
  if (d.epilogue != B200_EPI_NONE && d.epilogue != B200_EPI_BIAS && d.epilogue != B200_EPI_BIAS_RELU)
    return fail(B200_EINVAL, "%s: unsupported epilogue %d", who, d.epilogue);
  if (d.epilogue != B200_EPI_NONE && !*bias) return fail(B200_EINVAL, "%s: epilogue %d needs a bias", who, d.epilogue);
  if (d.epilogue == B200_EPI_NONE) *bias = nullptr;
  if (d.math_mode != B200_MATH_FP32X3 && d.math_mode != B200_MATH_TF32 && d.math_mode != B200_MATH_FP32 &&
      d.math_mode != B200_MATH_BF16)
    return fail(B200_EINVAL, "%s: unknown math mode %d", who, d.math_mode);
  if (d.math_mode == B200_MATH_BF16) d.math_mode = B200_MATH_TF32;  // no bf16 convolution kernel: TF32 is more accurate
  return B200_OK;
}
}  // namespace

// b200_conv2d_f32 = prepare + run on the caller's workspace: [NHWC copy of X | prepared filter]
// the descriptor as the kernels see it: a BF16 request runs in TF32
static b200_conv_desc conv_effective(const b200_conv_desc *desc) {
  b200_conv_desc d = *desc;
  if (d.math_mode == B200_MATH_BF16) d.math_mode = B200_MATH_TF32;
  return d;
}

extern "C" B200_API size_t b200_conv2d_workspace_bytes(const b200_conv_desc *desc) {
  if (!desc) return 0;
  const b200_conv_desc d = conv_effective(desc);
  // alignment of X is unknown here; the tensor-core path needs this much whenever the shape allows it
  if (!conv2d_tc_supported(d, nullptr)) return 0;
  return up256(conv2d_run_workspace_bytes(d, 0)) + conv2d_filter_bytes(d);
}

extern "C" B200_API int b200_conv2d_f32(void *stream, const b200_conv_desc *desc, const float *X, const float *W,
                               const float *bias, float *Y, void *workspace, size_t workspace_bytes) {
  cudaStream_t st = (cudaStream_t)stream;
  if (!desc) return fail(B200_EINVAL, "conv: null descriptor");
  b200_conv_desc d = *desc;
  int64_t OH, OW;
  bool empty;
  if (int rc = conv_check("conv", d, X, W, &bias, Y, &OH, &OW, &empty)) return rc;
  if (empty) return B200_OK;
  // Tensor-core implicit GEMM when TMA can address the NHWC copy; the CUDA-core kernel otherwise
  // (strided convolutions, channel counts that are not multiples of 4, plain fp32 arithmetic).
  if (!conv2d_tc_supported(d, X)) return conv2d_simt(st, d, X, W, bias, Y, OH, OW);
  const size_t xt_bytes = up256(conv2d_run_workspace_bytes(d, 0)), f_bytes = conv2d_filter_bytes(d);
  if (!workspace || workspace_bytes < xt_bytes + f_bytes)
    return fail(B200_EWORKSPACE, "conv: workspace of %zu bytes needed, %zu given", xt_bytes + f_bytes, workspace_bytes);
  if (!aligned16(workspace)) return fail(B200_EINVAL, "conv: workspace must be 16-byte aligned");
  void *filter = static_cast<char *>(workspace) + xt_bytes;
  if (int rc = conv2d_prepare_filter(st, d, W, filter, f_bytes)) return rc;
  return conv2d_run(st, d, 0, X, filter, bias, Y, OH, OW, workspace, xt_bytes);
}

extern "C" B200_API size_t b200_conv2d_filter_bytes(const b200_conv_desc *desc) {
  if (!desc || desc->M < 1 || desc->C < 1 || desc->KH < 1 || desc->KW < 1) return 0;
  return conv2d_filter_bytes(conv_effective(desc));
}

extern "C" B200_API int b200_conv2d_prepare_filter_f32(void *stream, const b200_conv_desc *desc, const float *W,
                                                       void *filter, size_t filter_bytes) {
  if (!desc) return fail(B200_EINVAL, "conv(prepare): null descriptor");
  if (desc->C < 1 || desc->M < 0 || desc->KH < 1 || desc->KW < 1) return fail(B200_EINVAL, "conv(prepare): bad extent");
  if (desc->M == 0) return B200_OK;
  if (!W) return fail(B200_EINVAL, "conv(prepare): null pointer");
  if (desc->math_mode != B200_MATH_FP32X3 && desc->math_mode != B200_MATH_TF32 && desc->math_mode != B200_MATH_FP32 &&
      desc->math_mode != B200_MATH_BF16)
    return fail(B200_EINVAL, "conv(prepare): unknown math mode %d", desc->math_mode);
  b200_conv_desc d = *desc;
  if (d.math_mode == B200_MATH_BF16) d.math_mode = B200_MATH_TF32;
  return conv2d_prepare_filter((cudaStream_t)stream, d, W, filter, filter_bytes);
}

extern "C" B200_API int b200_conv2d_nhwc_supported(const b200_conv_desc *desc) {
  return desc && desc->C >= 1 && desc->M >= 1 && desc->KH >= 1 && desc->KW >= 1 &&
                 conv2d_nhwc_supported(conv_effective(desc))
             ? 1
             : 0;
}

extern "C" B200_API size_t b200_conv2d_prepared_workspace_bytes(const b200_conv_desc *desc, int flags) {
  if (!desc || desc->N < 1 || desc->C < 1 || desc->H < 1 || desc->W < 1) return 0;
  return conv2d_run_workspace_bytes(conv_effective(desc), flags);
}

extern "C" B200_API int b200_conv2d_prepared_f32(void *stream, const b200_conv_desc *desc, int flags, const float *X,
                                                 const void *filter, const float *bias, float *Y, void *workspace,
                                                 size_t workspace_bytes) {
  if (!desc) return fail(B200_EINVAL, "conv(prepared): null descriptor");
  if (flags & ~(B200_CONV_X_NHWC | B200_CONV_Y_NHWC)) return fail(B200_EINVAL, "conv(prepared): unknown flags 0x%x", flags);
  b200_conv_desc d = *desc;
  int64_t OH, OW;
  bool empty;
  if (int rc = conv_check("conv(prepared)", d, X, filter, &bias, Y, &OH, &OW, &empty)) return rc;
  if (empty) return B200_OK;
  return conv2d_run((cudaStream_t)stream, d, flags, X, filter, bias, Y, OH, OW, workspace, workspace_bytes);
}
