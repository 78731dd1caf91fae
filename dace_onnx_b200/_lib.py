"""ctypes binding of libb200ops.so (the C ABI declared in include/b200_ops.h).

Loading fails loudly: there is no CPU or library fallback behind these entry points.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200ops.so")

OK, EINVAL, EUNSUPPORTED, ECUDA, EWORKSPACE, EDEVICE = 0, -1, -2, -3, -4, -5
MATH_FP32X3, MATH_TF32, MATH_FP32, MATH_BF16 = 0, 1, 2, 3
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_SCALE = range(6)
ADD, SUB, MUL, DIV, POW = range(5)
SQRT, ERF, RELU, GELU = range(4)
CONV_X_NHWC, CONV_Y_NHWC = 1, 2

MATH_MODES = {"fp32x3": MATH_FP32X3, "tf32": MATH_TF32, "fp32": MATH_FP32, "bf16": MATH_BF16}


class B200Error(RuntimeError):
    """Raised when an entry point of libb200ops returns a negative status."""

    def __init__(self, code, message):
        super().__init__("libb200ops error %d: %s" % (code, message))
        self.code = code


class GemmDesc(Structure):
    _fields_ = [(n, c_int64) for n in (
        "batch_outer", "batch_inner", "M", "N", "K", "lda", "ldb", "ldy",
        "a_stride_outer", "a_stride_inner", "b_stride_outer", "b_stride_inner",
        "y_stride_outer", "y_stride_inner")] + [
        ("trans_b", c_int32), ("epilogue", c_int32), ("scale", c_float), ("math_mode", c_int32)]


class AttentionDesc(Structure):
    _fields_ = [(n, c_int64) for n in (
        "batch", "heads", "seq", "head_dim", "q_row", "q_head", "q_batch", "k_row", "k_head", "k_batch",
        "v_row", "v_head", "v_batch", "o_row", "o_head", "o_batch")] + [("scale", c_float), ("math_mode", c_int32)]


class ConvDesc(Structure):
    _fields_ = [(n, c_int64) for n in (
        "N", "C", "H", "W", "M", "KH", "KW", "pad_h", "pad_w", "stride_h", "stride_w")] + [
        ("epilogue", c_int32), ("math_mode", c_int32)]


# name -> (restype, argtypes); mirrors include/b200_ops.h one to one.
SIGNATURES = {
    "b200_version": (c_int, []),
    "b200_last_error_string": (c_char_p, []),
    "b200_device_status": (c_int, []),
    "b200_selftest_wait_expiry": (c_int, [c_void_p, c_int64]),
    "b200_gemm_f32": (c_int, [c_void_p, POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_gemm_workspace_bytes": (c_size_t, [POINTER(GemmDesc)]),
    "b200_gemm_ws_f32": (c_int, [c_void_p, POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_size_t]),
    "b200_attention_supported": (c_int, [POINTER(AttentionDesc), c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_attention_f32": (c_int, [c_void_p, POINTER(AttentionDesc), c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_conv2d_workspace_bytes": (c_size_t, [POINTER(ConvDesc)]),
    "b200_conv2d_f32": (c_int, [c_void_p, POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_size_t]),
    "b200_conv2d_filter_bytes": (c_size_t, [POINTER(ConvDesc)]),
    "b200_conv2d_prepare_filter_f32": (c_int, [c_void_p, POINTER(ConvDesc), c_void_p, c_void_p, c_size_t]),
    "b200_conv2d_nhwc_supported": (c_int, [POINTER(ConvDesc)]),
    "b200_conv2d_prepared_workspace_bytes": (c_size_t, [POINTER(ConvDesc), c_int]),
    "b200_conv2d_prepared_f32": (c_int, [c_void_p, POINTER(ConvDesc), c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_size_t]),
    "b200_conv2d_static_scratch_bytes": (c_size_t, []),
    "b200_conv2d_static_f32": (c_int, [c_void_p, POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_softmax_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "b200_logsoftmax_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "b200_reduce_mean_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "b200_layernorm_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float]),
    "b200_binary_f32": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, POINTER(c_int64),
                                POINTER(c_int64), POINTER(c_int64)]),
    "b200_unary_f32": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64]),
    "b200_transpose_0213_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64]),
    "b200_maxpool2d_f32": (c_int, [c_void_p, c_void_p, c_void_p] + [c_int64] * 7),
    "b200_transpose_2d_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
}

_lib = None


def load():
    """Load libb200ops.so and type every entry point. Raises if the library is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "%s is missing: build it with `python -m dace_onnx_b200.build` (needs nvcc); "
            "there is no fallback implementation" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status):
    """Turn a negative status into B200Error carrying the library's message."""
    if status != 0:
        msg = load().b200_last_error_string()
        raise B200Error(status, msg.decode() if msg else "")


def device_status():
    """Synchronise and raise if any kernel reported an expired wait since the last check."""
    check(load().b200_device_status())
