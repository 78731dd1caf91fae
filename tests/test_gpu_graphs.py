"""BASELINE configurations 1 (MLP) and 2 (conv stack) through the C ABI against the oracle."""
import pytest
import torch

from dace_onnx_b200 import graphs
from oracle import pure_oracle as po
from tests._util import ATOL, RTOL, TF32_ATOL, TF32_RTOL, close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", RTOL, ATOL), ("fp32", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
def test_config1_mlp_full_size(mode, rtol, atol, cuda):
    # Linear 784 -> 120 -> 32 -> 10 + LogSoftmax, batch 4096, x ~ N(0,1), default nn.Linear init, seed 0
    params = po.make_mlp_params(0)
    x = torch.randn(4096, 784, generator=torch.Generator().manual_seed(0))
    ref = po.mlp_forward(x, params)
    out = graphs.mlp_forward(x.cuda(), [(w.cuda(), b.cuda()) for w, b in params], math_mode=mode)
    close(out, ref, rtol, atol)
    assert torch.allclose(out.exp().sum(1).cpu(), torch.ones(4096), atol=1e-5)


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
def test_config2_conv_stack_reduced_batch(mode, rtol, atol, cuda):
    # two 3x3 convs 64 -> 64, pad 1, bias + ReLU, 56x56; batch 16 of the configuration's 256
    params = po.make_conv_params(0, channels=64, layers=2)
    x = torch.rand(16, 64, 56, 56, generator=torch.Generator().manual_seed(0))
    ref = po.conv_stack_forward(x, params)
    out = graphs.conv_stack_forward(x.cuda(), [(w.cuda(), b.cuda()) for w, b in params], math_mode=mode)
    close(out, ref, rtol, atol)


def test_config2_full_batch_properties(cuda):
    # batch 256: per-image independence (image i of the batch == image i run alone) and agreement of
    # the fp32-accurate tensor-core path with the CUDA-core path on a slice
    params = [(w.cuda(), b.cuda()) for w, b in po.make_conv_params(0, channels=64, layers=2)]
    x = torch.rand(256, 64, 56, 56, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    full = graphs.conv_stack_forward(x, params)
    assert full.shape == (256, 64, 56, 56) and (full >= 0).all()
    assert torch.equal(full[200:203], graphs.conv_stack_forward(x[200:203].contiguous(), params))
    close(full[7:9], graphs.conv_stack_forward(x[7:9].contiguous(), params, math_mode="fp32"))
