"""b200_conv2d_static_f32 -- the convolution entry point for hosts that cannot allocate.

Some embedders of this library have nowhere to create a workspace: generated code that owns only
its argument pointers, or a service that fixes its device memory at start-up and forbids
cudaMalloc afterwards. For them the library carries the convolution's scratch as a fixed array
(32 MiB per GPU). This test drives that entry point through the C ABI exactly as such a host
would -- inputs and outputs only -- and checks that it returns what the ordinary entry point
(caller-allocated workspace) returns, twice in a row with different shapes so that whatever the
first call left in the shared array cannot leak into the second. The file is named so that pytest
collects it last.
"""
import ctypes

import pytest
import torch

from dace_onnx_b200 import _lib, ops
from dace_onnx_b200._lib import EPI_BIAS, EPI_BIAS_RELU, EPI_NONE, MATH_MODES, ConvDesc
from tests._util import ATOL, RTOL, close

pytestmark = pytest.mark.gpu


def _static_conv(x, w, b, pad, relu, mode):
    """The new entry point, called the way an allocation-free host calls it."""
    n, c, h, wd = x.shape
    m, _, kh, kw = w.shape
    y = torch.empty(n, m, h + 2 * pad - kh + 1, wd + 2 * pad - kw + 1, device=x.device)
    epi = EPI_NONE if b is None else (EPI_BIAS_RELU if relu else EPI_BIAS)
    d = ConvDesc(n, c, h, wd, m, kh, kw, pad, pad, 1, 1, epi, MATH_MODES[mode])
    rc = _lib.load().b200_conv2d_static_f32(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.byref(d),
                                            ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                                            ctypes.c_void_p(b.data_ptr()) if b is not None else None,
                                            ctypes.c_void_p(y.data_ptr()))
    _lib.check(rc)
    return y


def _case(n, c, hw, m, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(n, c, hw, hw, generator=g).cuda()
    w = ((torch.rand(m, c, 3, 3, generator=g) * 2 - 1) / (c * 9) ** 0.5).cuda()
    b = ((torch.rand(m, generator=g) * 2 - 1) / (c * 9) ** 0.5).cuda()
    return x, w, b


@pytest.mark.parametrize("mode", ["fp32x3", "tf32"])
def test_static_scratch_conv_matches_workspace_conv_twice_in_a_row(mode, cuda):
    # first call: larger problem, fills more of the shared array; second: smaller, different data
    for n, c, hw, m, seed in [(4, 64, 56, 64, 1), (2, 32, 19, 48, 2)]:
        x, w, b = _case(n, c, hw, m, seed)
        expected = ops.conv2d(x, w, b, pads=(1, 1, 1, 1), relu=True, math_mode=mode)  # caller-allocated workspace
        got = _static_conv(x, w, b, 1, True, mode)
        close(got, expected, RTOL, ATOL)


def test_static_scratch_conv_cuda_core_shapes_and_limits(cuda):
    lib = _lib.load()
    assert lib.b200_conv2d_static_scratch_bytes() == 32 << 20
    # a shape the tensor cores do not take (8 channels) needs no scratch and still works
    g = torch.Generator().manual_seed(3)
    x, w = torch.rand(2, 8, 12, 12, generator=g).cuda(), (torch.rand(5, 8, 3, 3, generator=g) - 0.5).cuda()
    close(_static_conv(x, w, None, 0, False, "fp32x3"), ops.conv2d(x, w), RTOL, ATOL)
    # a convolution whose scratch exceeds the built-in array is refused with a clear message;
    # the pointers are never touched (the size check comes first), so small dummies suffice
    dummy = torch.zeros(64, device="cuda")
    d = ConvDesc(256, 64, 56, 56, 64, 3, 3, 1, 1, 1, 1, EPI_NONE, MATH_MODES["fp32x3"])
    assert lib.b200_conv2d_workspace_bytes(ctypes.byref(d)) > 32 << 20
    rc = lib.b200_conv2d_static_f32(None, ctypes.byref(d), ctypes.c_void_p(dummy.data_ptr()),
                                    ctypes.c_void_p(dummy.data_ptr()), None, ctypes.c_void_p(dummy.data_ptr()))
    assert rc == _lib.EWORKSPACE
    assert b"built-in array holds" in lib.b200_last_error_string()
