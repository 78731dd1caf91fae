"""ONNXConv through the C ABI against the oracle."""
import numpy as np
import pytest
import torch

from dace_onnx_b200 import ops
from oracle import pure_oracle as po
from tests._util import ATOL, RTOL, TF32_ATOL, TF32_RTOL, close, dev, golden, golden_names

pytestmark = pytest.mark.gpu

MODES = [("fp32x3", RTOL, ATOL), ("fp32", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)]


@pytest.mark.parametrize("mode,rtol,atol", MODES)
@pytest.mark.parametrize("name", golden_names("conv_"))
def test_conv_golden(name, mode, rtol, atol, cuda):
    g = golden(name)
    pad = int(g["pad"])
    B = dev(g["B"]) if "B" in g else None
    close(ops.conv2d(dev(g["X"]), dev(g["W"]), B, pads=(pad,) * 4, math_mode=mode), g["Y"], rtol, atol)


@pytest.mark.parametrize("cin,k,cout,bias", [(1, 3, 8, True), (8, 3, 3, False), (8, 5, 3, True), (8, 4, 3, False)])
def test_conv_reference_test_cases(cin, k, cout, bias, cuda):
    # tests/pure_expansions/test_conv_expansion.py:9-66: batch 8, 32x32, rand inputs, vs F.conv2d
    rng = np.random.default_rng(51)
    X = rng.random((8, cin, 32, 32), dtype=np.float32)
    W = rng.random((cout, cin, k, k), dtype=np.float32)
    B = rng.random(cout, dtype=np.float32) if bias else None
    ref = torch.nn.functional.conv2d(torch.tensor(X), torch.tensor(W), None if B is None else torch.tensor(B))
    out = ops.conv2d(dev(X), dev(W), None if B is None else dev(B))
    close(out, ref, rtol=1e-5, atol=1e-5)
    close(out, po.Conv(X, W, B), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("mode,rtol,atol", MODES)
@pytest.mark.parametrize("n,c,hw,m,relu", [(3, 64, 56, 64, True), (2, 64, 14, 64, False), (1, 32, 9, 128, True),
                                           (2, 96, 20, 40, True)])
def test_conv3x3_pad1_vs_oracle(n, c, hw, m, relu, mode, rtol, atol, cuda):
    g = torch.Generator().manual_seed(61)
    x = torch.rand(n, c, hw, hw, generator=g)
    (w, b), = po.make_conv_params(seed=62, channels=c, layers=1)
    w, b = w[:m] if m <= c else torch.cat([w] * (m // c + 1))[:m], (b[:m] if m <= c else torch.cat([b] * (m // c + 1))[:m])
    ref = po.Conv(x, w, b, pads=(1, 1, 1, 1))
    if relu:
        ref = po.Relu(ref)
    close(ops.conv2d(x.cuda(), w.cuda(), b.cuda(), pads=(1, 1, 1, 1), relu=relu, math_mode=mode), ref, rtol, atol)


def test_conv_stride_and_errors(cuda):
    g = torch.Generator().manual_seed(71)
    x, w = torch.rand(2, 4, 13, 13, generator=g), torch.rand(5, 4, 3, 3, generator=g) - 0.5
    ref = torch.nn.functional.conv2d(x, w, stride=2, padding=1)
    close(ops.conv2d(x.cuda(), w.cuda(), pads=(1, 1, 1, 1), strides=(2, 2)), ref, rtol=1e-5, atol=1e-5)
    with pytest.raises(NotImplementedError):
        ops.conv2d(x.cuda(), w.cuda(), pads=(1, 0, 0, 0))
    with pytest.raises(NotImplementedError):
        ops.conv2d(x.cuda(), w.cuda(), group=2)
    with pytest.raises(ValueError):
        ops.conv2d(x.cuda(), torch.rand(5, 3, 3, 3).cuda())
