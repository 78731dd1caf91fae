// b200_conv2d_static_f32: the convolution entry point for callers that cannot allocate.
//
// The tensor-core convolution needs device scratch (an NHWC copy of the input and the repacked
// filter). b200_conv2d_f32 takes it from the caller, which means the caller must be able to
// cudaMalloc it somewhere: DaCeML does that in an environment's init hook. Some hosts have no such
// place. Examples are generated code that is handed nothing but its input and output pointers
// (no per-program state, no init / finalize callbacks), and long-running services that size their
// device memory once at start-up and treat any later cudaMalloc as an error because it
// synchronises the device and can fail when memory is fragmented. For them this file keeps the
// scratch in a fixed array that is part of the library image.
//
// Cost and limits: every GPU on which the library's module is loaded holds
// B200_CONV_STATIC_SCRATCH_BYTES of memory until the process exits, whether or not this entry
// point is ever called, and a convolution whose scratch does not fit is refused. All calls share
// the one array per device: two calls whose kernels can overlap on the GPU (different streams,
// different host threads) race on it. The array keeps whatever the previous call left there;
// nothing in it has to start at zero, because each call overwrites every byte it later reads
// (the transpose writes the whole NHWC copy, the repack writes the whole padded filter).
#include <mutex>

#include "common.cuh"
#include "contract.cuh"

namespace b200 {
namespace {

// File-scope scratch. In host code this name is only a stand-in for the symbol: it is not a device
// address and must never be passed to a kernel. The address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_conv_static_scratch[B200_CONV_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices] = {};  // device address of the array, per device, filled on first use

// Set-up, once per device, with that device current: resolve the symbol to its device address.
int scratch_for_current_device(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200_ECUDA, "conv(static): cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(B200_EUNSUPPORTED, "conv(static): device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    void *ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_conv_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(B200_ECUDA, "conv(static): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" B200_API size_t b200_conv2d_static_scratch_bytes(void) { return B200_CONV_STATIC_SCRATCH_BYTES; }

extern "C" B200_API int b200_conv2d_static_f32(void *stream, const b200_conv_desc *desc, const float *X,
                                               const float *W, const float *bias, float *Y) {
  cudaStream_t st = (cudaStream_t)stream;
  if (!desc) return fail(B200_EINVAL, "conv(static): null descriptor");
  b200_conv_desc d = *desc;
  if (d.N < 0 || d.C < 1 || d.H < 1 || d.W < 1 || d.M < 0) return fail(B200_EINVAL, "conv(static): bad extent");
  if (d.stride_h < 1 || d.stride_w < 1 || d.KH < 1 || d.KW < 1 || d.pad_h < 0 || d.pad_w < 0)
    return fail(B200_EINVAL, "conv(static): bad kernel/pad/stride");
  const int64_t eh = d.H + 2 * d.pad_h - d.KH, ew = d.W + 2 * d.pad_w - d.KW;
  if (eh < 0 || ew < 0) return fail(B200_EINVAL, "conv(static): filter larger than the padded input");
  const int64_t OH = eh / d.stride_h + 1, OW = ew / d.stride_w + 1;
  if (d.N == 0 || d.M == 0) return B200_OK;
  if (!X || !W || !Y) return fail(B200_EINVAL, "conv(static): null pointer");
  if (d.epilogue != B200_EPI_NONE && d.epilogue != B200_EPI_BIAS && d.epilogue != B200_EPI_BIAS_RELU)
    return fail(B200_EINVAL, "conv(static): unsupported epilogue %d", d.epilogue);
  if (d.epilogue != B200_EPI_NONE && !bias) return fail(B200_EINVAL, "conv(static): epilogue %d needs a bias", d.epilogue);
  if (d.epilogue == B200_EPI_NONE) bias = nullptr;
  if (d.math_mode != B200_MATH_FP32X3 && d.math_mode != B200_MATH_TF32 && d.math_mode != B200_MATH_FP32 &&
      d.math_mode != B200_MATH_BF16)
    return fail(B200_EINVAL, "conv(static): unknown math mode %d", d.math_mode);
  if (d.math_mode == B200_MATH_BF16) d.math_mode = B200_MATH_TF32;  // as in b200_conv2d_f32

  // Shapes the tensor cores cannot take run on the CUDA-core kernel, which uses no scratch at all.
  if (!conv2d_tc_supported(d, X)) return conv2d_simt(st, d, X, W, bias, Y, OH, OW);

  // scratch layout as in b200_conv2d_f32: [NHWC copy of X | prepared filter]
  const size_t xt_bytes = (conv2d_run_workspace_bytes(d, 0) + 255) & ~(size_t)255, f_bytes = conv2d_filter_bytes(d);
  const size_t need = xt_bytes + f_bytes;
  if (need > (size_t)B200_CONV_STATIC_SCRATCH_BYTES)
    return fail(B200_EWORKSPACE,
                "conv(static): this convolution needs %zu bytes of scratch, the built-in array holds %zu; "
                "use b200_conv2d_f32 with a caller-allocated workspace",
                need, (size_t)B200_CONV_STATIC_SCRATCH_BYTES);
  void *scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  void *filter = static_cast<char *>(scratch) + xt_bytes;
  if (int rc = conv2d_prepare_filter(st, d, W, filter, f_bytes)) return rc;
  return conv2d_run(st, d, 0, X, filter, bias, Y, OH, OW, scratch, xt_bytes);
}
