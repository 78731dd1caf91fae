"""The C-ABI library loads and exports every symbol include/b200_ops.h declares (no GPU needed)."""
import ctypes
import os
import re

from dace_onnx_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_ops.h")).read()
    return sorted(set(re.findall(r"B200_API[^;(]*?\b(b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ["b200_gemm_f32", "b200_conv2d_f32", "b200_softmax_f32", "b200_logsoftmax_f32", "b200_layernorm_f32",
              "b200_reduce_mean_f32", "b200_binary_f32", "b200_unary_f32", "b200_last_error_string"]:
        assert s in syms


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for s in declared_symbols():
        assert hasattr(lib, s), "libb200ops.so does not export %s" % s


def test_ctypes_signatures_cover_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_constants_match_the_header():
    text = open(os.path.join(ROOT, "include", "b200_ops.h")).read()
    consts = {k: int(v.strip("()")) for k, v in re.findall(r"#define\s+(B200_\w+)\s+(\(?-?\d+\)?)", text)}
    assert consts["B200_MATH_FP32X3"] == _lib.MATH_FP32X3 and consts["B200_MATH_TF32"] == _lib.MATH_TF32
    assert consts["B200_MATH_FP32"] == _lib.MATH_FP32 and consts["B200_MATH_BF16"] == _lib.MATH_BF16
    assert [consts[k] for k in ("B200_EPI_NONE", "B200_EPI_BIAS", "B200_EPI_BIAS_RELU", "B200_EPI_BIAS_GELU",
                                "B200_EPI_BIAS_RESIDUAL", "B200_EPI_SCALE")] == list(range(6))
    assert [consts[k] for k in ("B200_ADD", "B200_SUB", "B200_MUL", "B200_DIV", "B200_POW")] == list(range(5))
    assert consts["B200_EINVAL"] == _lib.EINVAL and consts["B200_EDEVICE"] == _lib.EDEVICE


def test_argument_errors_are_reported_without_a_gpu():
    lib = _lib.load()
    assert lib.b200_version() >= 100
    # argument validation happens before any CUDA call
    assert lib.b200_gemm_f32(None, None, None, None, None, None, None) == _lib.EINVAL
    assert b"null descriptor" in lib.b200_last_error_string()
    assert lib.b200_softmax_f32(None, None, None, -1, 4, 1) == _lib.EINVAL
    arr = (ctypes.c_int64 * 9)(*([1] * 9))
    assert lib.b200_binary_f32(None, 0, None, None, None, 9, arr, arr, arr) == _lib.EUNSUPPORTED
    d = _lib.GemmDesc(1, 1, 4, 4, 4, 2, 4, 4, 0, 0, 0, 0, 0, 0, 0, 0, 1.0, 0)  # lda < K
    one = ctypes.c_void_p(16)
    assert lib.b200_gemm_f32(None, ctypes.byref(d), one, one, None, None, one) == _lib.EINVAL


def test_prepared_conv_argument_errors_without_a_gpu():
    lib = _lib.load()
    d = _lib.ConvDesc(2, 64, 8, 8, 64, 3, 3, 1, 1, 1, 1, 0, _lib.MATH_TF32)
    one = ctypes.c_void_p(256)
    assert lib.b200_conv2d_nhwc_supported(ctypes.byref(d)) == 1
    assert lib.b200_conv2d_filter_bytes(ctypes.byref(d)) == 64 * 9 * 64 * 4
    assert lib.b200_conv2d_prepared_workspace_bytes(ctypes.byref(d), 0) == 2 * 64 * 8 * 8 * 4
    assert lib.b200_conv2d_prepared_workspace_bytes(ctypes.byref(d), _lib.CONV_X_NHWC) == 0
    assert lib.b200_conv2d_prepared_f32(None, ctypes.byref(d), 4, one, one, None, one, None, 0) == _lib.EINVAL
    assert lib.b200_conv2d_prepared_f32(None, ctypes.byref(d), 0, one, one, None, one, None, 0) == _lib.EWORKSPACE
    assert lib.b200_conv2d_prepare_filter_f32(None, ctypes.byref(d), one, one, 16) == _lib.EWORKSPACE
    d3 = _lib.ConvDesc(2, 64, 8, 8, 64, 3, 3, 1, 1, 1, 1, 0, _lib.MATH_FP32X3)
    assert lib.b200_conv2d_filter_bytes(ctypes.byref(d3)) == 3 * 64 * 9 * 64 * 4     # raw, hi, lo
    wide = _lib.ConvDesc(2, 64, 8, 8, 128, 3, 3, 1, 1, 1, 1, 0, _lib.MATH_TF32)       # 128 output channels
    assert lib.b200_conv2d_nhwc_supported(ctypes.byref(wide)) == 0
    assert lib.b200_conv2d_prepared_f32(None, ctypes.byref(wide), _lib.CONV_Y_NHWC, one, one, None, one, one,
                                        1 << 30) == _lib.EUNSUPPORTED
    big = _lib.ConvDesc(2, 512, 8, 8, 64, 3, 3, 1, 1, 1, 1, 0, _lib.MATH_TF32)        # filter half beyond shared memory
    assert lib.b200_conv2d_nhwc_supported(ctypes.byref(big)) == 0
    # the one-call entry point still sizes its workspace as [NHWC copy | prepared filter]
    assert lib.b200_conv2d_workspace_bytes(ctypes.byref(d)) == 2 * 64 * 8 * 8 * 4 + 64 * 9 * 64 * 4


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from dace_onnx_b200 import ops
    with pytest.raises(ValueError, match="no CPU path"):
        ops.softmax(torch.zeros(2, 3))
