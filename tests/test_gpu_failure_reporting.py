"""The failure-reporting path of the tensor-core kernels, exercised without making any real kernel fail: a
one-warp diagnostic kernel waits (with the library's bounded wait) on a barrier nothing signals; the wait
expires after ~1e5 cycles, the kernel returns, and the device status word reports it exactly once."""
import ctypes

import pytest
import torch

from dace_onnx_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_once_and_the_context_stays_usable(cuda):
    lib = _lib.load()
    _lib.device_status()                                           # clean before
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200_selftest_wait_expiry(stream, 100000) == 0
    with pytest.raises(_lib.B200Error) as e:
        _lib.device_status()
    assert e.value.code == _lib.EDEVICE and "0x8000" in str(e.value)
    _lib.device_status()                                           # reading the status cleared it
    # the context is intact: kernels run and give right answers afterwards
    x = torch.randn(64, 512, device="cuda")
    assert torch.allclose(ops.softmax(x, -1).sum(-1), torch.ones(64, device="cuda"), atol=1e-5)
    a, b = torch.randn(256, 128, device="cuda"), torch.randn(128, 64, device="cuda")
    assert torch.allclose(ops.matmul(a, b), a @ b, rtol=1e-4, atol=1e-4)
    _lib.device_status()


def test_selftest_rejects_unbounded_budgets(cuda):
    lib = _lib.load()
    assert lib.b200_selftest_wait_expiry(None, 0) == _lib.EINVAL
    assert lib.b200_selftest_wait_expiry(None, 10 ** 9) == _lib.EINVAL
