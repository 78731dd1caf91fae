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


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
@pytest.mark.parametrize("n,c,h,w,m,k,pad", [(3, 64, 56, 56, 64, 3, 1), (2, 32, 20, 13, 48, 3, 1), (1, 16, 9, 9, 16, 1, 0),
                                             (5, 64, 7, 7, 24, 3, 0), (2, 32, 17, 30, 32, 5, 2), (3, 128, 33, 18, 64, 3, 1), (1, 96, 12, 12, 33, 3, 1),
                                             # k-block counts 2, 3, 9 and 50 per tile (the 3xTF32 issuers take every fourth k-block of
                                             # a count that runs on across tiles; accumulators are handed over every <= 20 k-blocks)
                                             (2, 64, 10, 10, 64, 1, 0), (2, 96, 10, 10, 48, 1, 0), (4, 32, 40, 40, 64, 3, 1),
                                             (1, 64, 12, 12, 16, 5, 2)])
def test_prepared_conv_layouts(n, c, h, w, m, k, pad, mode, rtol, atol, cuda):
    """b200_conv2d_prepared_f32 in all four layout combinations against the oracle (NCHW) -- odd image sizes
    (8x8 block tails), output-channel counts that are not multiples of 16 or 32, 1x1 / 5x5 filters."""
    g = torch.Generator().manual_seed(n * 100 + c + m)
    x = torch.rand(n, c, h, w, generator=g)
    wt = (torch.rand(m, c, k, k, generator=g) * 2 - 1) / (c * k * k) ** 0.5
    b = torch.rand(m, generator=g) - 0.5
    ref = po.Relu(po.Conv(x, wt, b, pads=(pad,) * 4))
    conv = ops.PreparedConv(wt.cuda(), b.cuda(), pads=(pad,) * 4, relu=True, math_mode=mode)
    xd = x.cuda()
    if not conv.nhwc_ok:
        # the split filter (hi + lo) of the widest cases does not fit in shared memory in the fp32x3 mode
        assert mode == "fp32x3" and c >= 96
        close(conv(xd), ref, rtol, atol)
        return
    xn = xd.permute(0, 2, 3, 1).contiguous()
    close(conv(xd), ref, rtol, atol)
    close(conv(xd, y_nhwc=True).permute(0, 3, 1, 2), ref, rtol, atol)
    close(conv(xn, x_nhwc=True), ref, rtol, atol)
    close(conv(xn, x_nhwc=True, y_nhwc=True).permute(0, 3, 1, 2), ref, rtol, atol)
    # no bias, no relu
    conv0 = ops.PreparedConv(wt.cuda(), None, pads=(pad,) * 4, math_mode=mode)
    close(conv0(xn, x_nhwc=True, y_nhwc=True).permute(0, 3, 1, 2), po.Conv(x, wt, None, pads=(pad,) * 4), rtol, atol)


def test_prepared_conv_outside_the_resident_filter_kernel(cuda):
    g = torch.Generator().manual_seed(81)
    # 128 output channels: general tensor-core kernel, NCHW only
    x, w, b = torch.rand(2, 32, 10, 10, generator=g), torch.rand(128, 32, 3, 3, generator=g) - 0.5, torch.rand(128, generator=g)
    conv = ops.PreparedConv(w.cuda(), b.cuda(), pads=(1, 1, 1, 1))
    assert not conv.nhwc_ok
    close(conv(x.cuda()), po.Conv(x, w, b, pads=(1, 1, 1, 1)))
    with pytest.raises(ops._lib.B200Error) as e:
        conv(x.cuda().permute(0, 2, 3, 1).contiguous(), x_nhwc=True)
    assert e.value.code == ops._lib.EUNSUPPORTED
    # strided, 3 input channels: CUDA-core kernel behind the same entry points
    x, w = torch.rand(2, 3, 13, 13, generator=g), torch.rand(5, 3, 3, 3, generator=g) - 0.5
    conv = ops.PreparedConv(w.cuda(), None, pads=(1, 1, 1, 1), strides=(2, 2))
    close(conv(x.cuda()), torch.nn.functional.conv2d(x, w, stride=2, padding=1), rtol=1e-5, atol=1e-5)
    # 48 input channels: not whole 32-channel blocks, so the general tensor-core kernel (NCHW only)
    x, w = torch.rand(2, 48, 17, 30, generator=g), (torch.rand(64, 48, 3, 3, generator=g) - 0.5) / 20
    conv = ops.PreparedConv(w.cuda(), None, pads=(1, 1, 1, 1))
    assert not conv.nhwc_ok
    close(conv(x.cuda()), po.Conv(x, w, None, pads=(1, 1, 1, 1)))
    # the plain fp32 mode
    x, w = torch.rand(2, 64, 9, 9, generator=g), torch.rand(64, 64, 3, 3, generator=g) - 0.5
    conv = ops.PreparedConv(w.cuda(), None, pads=(1, 1, 1, 1), math_mode="fp32")
    assert not conv.nhwc_ok
    close(conv(x.cuda()), po.Conv(x, w, None, pads=(1, 1, 1, 1)))


def test_conv_stack_keeps_nhwc_between_layers(cuda):
    from dace_onnx_b200 import graphs
    params = po.make_conv_params(3, channels=64, layers=3)
    x = torch.rand(5, 64, 28, 28, generator=torch.Generator().manual_seed(82))
    layers = graphs.prepare_conv_stack([(w.cuda(), b.cuda()) for w, b in params])
    assert all(c.nhwc_ok for c in layers)
    out = graphs.conv_stack_forward(x.cuda(), layers)
    close(out, po.conv_stack_forward(x, params))
    assert torch.equal(out, graphs.conv_stack_forward(x.cuda(), layers))  # prepared filters are reusable


def test_transpose_batch_beyond_grid_limit(cuda):
    x = torch.randn(70000, 4, 8, generator=torch.Generator().manual_seed(83)).cuda()
    assert torch.equal(ops.transpose_last2(x), x.transpose(1, 2).contiguous())
