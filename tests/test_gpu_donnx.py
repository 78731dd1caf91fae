"""The `donnx.ONNX<Op>(connector=..., output=...)` call form of the reference's node tests
(tests/test_python_frontend.py:12-22, tests/pure_expansions/test_expansions.py) on the b200 kernels:
connector names as keywords, outputs written in place."""
import numpy as np
import pytest
import torch

from dace_onnx_b200 import donnx
from oracle import pure_oracle as po
from tests._util import close

pytestmark = pytest.mark.gpu


def _r(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale)


def test_matmul_like_the_python_frontend_test(cuda):
    # tests/test_python_frontend.py:12-22: donnx.ONNXMatMul(A=X, B=Z, Y=Y) with [5,8,2,3] @ [3,4]-style operands
    A, B = _r(5, 8, 2, 3, seed=1), _r(3, 4, seed=2)
    Y = torch.empty(5, 8, 2, 4, device="cuda")
    assert donnx.ONNXMatMul(A=A.cuda(), B=B.cuda(), Y=Y) is Y
    close(Y, po.MatMul(A, B))
    with pytest.raises(NotImplementedError):
        donnx.ONNXMatMul(A=A.cuda()[0, 0, 0], B=B.cuda(), Y=torch.empty(4, device="cuda"))
    with pytest.raises(ValueError):
        donnx.ONNXMatMul(A=A.cuda(), B=B.cuda(), Y=torch.empty(5, 8, 2, 5, device="cuda"))
    with pytest.raises(TypeError):
        donnx.ONNXMatMul(A=A.cuda(), B=B.cuda(), Y=None)


def test_gemm_conv_and_rowwise_nodes(cuda):
    A, B, C = _r(33, 120, seed=3), _r(32, 120, seed=4, scale=0.1), _r(32, seed=5)
    Y = torch.empty(33, 32, device="cuda")
    donnx.ONNXGemm(A=A.cuda(), B=B.cuda(), C=C.cuda(), Y=Y, alpha=1.0, beta=1.0, transA=0, transB=1)
    close(Y, po.Gemm(A, B, C))
    with pytest.raises(NotImplementedError):
        donnx.ONNXGemm(A=A.cuda(), B=B.cuda(), Y=Y, transB=0)
    X, W, Bc = torch.rand(2, 16, 9, 9), torch.rand(8, 16, 3, 3) - 0.5, torch.rand(8)
    Yc = torch.empty(2, 8, 9, 9, device="cuda")
    donnx.ONNXConv(X=X.cuda(), W=W.cuda(), B=Bc.cuda(), Y=Yc, pads=[1, 1, 1, 1], strides=[1, 1], kernel_shape=[3, 3])
    close(Yc, po.Conv(X, W, Bc, pads=(1, 1, 1, 1)))
    with pytest.raises(NotImplementedError):
        donnx.ONNXConv(X=X.cuda(), W=W.cuda(), Y=Yc, auto_pad="SAME_UPPER")
    x = _r(2, 4, 10, seed=6, scale=10.0)
    for axis in (0, -1):
        out = torch.empty(2, 4, 10, device="cuda")
        donnx.ONNXSoftmax(input=x.cuda(), output=out, axis=axis)
        close(out, po.Softmax(x, axis))
        donnx.ONNXLogSoftmax(input=x.cuda(), output=out, axis=axis)
        close(out, po.LogSoftmax(x, axis))
    red = torch.empty(2, 4, 1, device="cuda")
    donnx.ONNXReduceMean(data=x.cuda(), reduced=red, axes=[-1], keepdims=1)
    close(red, po.ReduceMean(x, [-1], 1), rtol=1e-5, atol=1e-5)


def test_elementwise_nodes_and_non_contiguous_outputs(cuda):
    a, b = _r(6, 40, seed=7), _r(40, seed=8) + 3.0
    for name, ref in (("ONNXAdd", po.Add), ("ONNXSub", po.Sub), ("ONNXMul", po.Mul), ("ONNXDiv", po.Div)):
        out = torch.empty(6, 40, device="cuda")
        getattr(donnx, name)(A=a.cuda(), B=b.cuda(), C=out)
        close(out, ref(a, b))
    z = torch.empty(6, 40, device="cuda")
    donnx.ONNXPow(X=a.cuda(), Y=torch.tensor(2.0).cuda(), Z=z)
    close(z, po.Pow(a, np.float32(2.0)))
    base = torch.zeros(6, 80, device="cuda")
    view = base[:, ::2]                                   # an output connector that is not contiguous
    donnx.ONNXRelu(X=a.cuda(), Y=view)
    close(view, po.Relu(a))
    assert (base[:, 1::2] == 0).all()
    y = torch.empty(6, 40, device="cuda")
    donnx.ONNXSqrt(X=a.abs().cuda(), Y=y)
    close(y, po.Sqrt(a.abs()))
    donnx.ONNXErf(input=a.cuda(), output=y)
    close(y, po.Erf(a), atol=1e-6)
    t = torch.empty(2, 5, 3, 4, device="cuda")
    x4 = _r(2, 3, 5, 4, seed=9)
    donnx.ONNXTranspose(data=x4.cuda(), transposed=t, perm=[0, 2, 1, 3])
    assert torch.equal(t.cpu(), x4.permute(0, 2, 1, 3).contiguous())
    with pytest.raises(NotImplementedError):
        donnx.ONNXTranspose(data=x4.cuda(), transposed=t, perm=[3, 2, 1, 0])
