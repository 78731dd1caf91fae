"""Softmax / LogSoftmax / ReduceMean / LayerNorm kernels against the oracle (through the C ABI)."""
import numpy as np
import pytest
import torch

from dace_onnx_b200 import ops
from oracle import pure_oracle as po
from tests._util import close, dev, golden, golden_names

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", golden_names("softmax_"))
def test_softmax_golden(name, cuda):
    g = golden(name)
    close(ops.softmax(dev(g["x"]), int(g["axis"])), g["y"])
    close(ops.logsoftmax(dev(g["x"]), int(g["axis"])), g["ylog"])


@pytest.mark.parametrize("axis", [0, -1])
def test_softmax_reference_test_criterion(axis, cuda):
    # tests/pure_expansions/test_expansions.py:343-418: [2,4,10], N(0,10^2), ||delta||_2 < 1e-5
    X = np.random.default_rng(11).normal(scale=10, size=(2, 4, 10)).astype(np.float32)
    ref = torch.nn.functional.softmax(torch.tensor(X), dim=axis).numpy()
    assert np.linalg.norm(ref - ops.softmax(dev(X), axis).cpu().numpy()) < 1e-5
    refl = torch.nn.functional.log_softmax(torch.tensor(X), dim=axis).numpy()
    assert np.linalg.norm(refl - ops.logsoftmax(dev(X), axis).cpu().numpy()) < 1e-5


@pytest.mark.parametrize("shape,axis", [((64, 512), -1), ((33, 384), -1), ((17, 10), -1), ((5, 2048), -1),
                                        ((3, 2052), -1), ((2, 50000), -1), ((2, 60001), -1), ((4, 1023), -1),
                                        ((2, 3, 4, 384), 3), ((6, 7, 9), 1), ((5, 8), 0), ((1, 1), -1),
                                        ((3, 12, 128, 128), 3)])
def test_softmax_vs_oracle(shape, axis, cuda):
    x = torch.randn(shape, generator=torch.Generator().manual_seed(5)) * 2
    close(ops.softmax(x.cuda(), axis), po.Softmax(x, axis))
    close(ops.logsoftmax(x.cuda(), axis), po.LogSoftmax(x, axis))


def test_softmax_empty_and_unaligned(cuda):
    assert ops.softmax(torch.empty(0, 8, device="cuda"), -1).shape == (0, 8)
    base = torch.randn(1 + 7 * 512, generator=torch.Generator().manual_seed(6))
    x = base[1:].view(7, 512)  # 4-byte aligned only
    xd = base.cuda()[1:].view(7, 512)
    out = torch.empty(1 + 7 * 512, device="cuda")[1:].view(7, 512)
    ops._lib.check(ops._lib.load().b200_softmax_f32(ops._stream(), ops._ptr(xd), ops._ptr(out), 7, 512, 1))
    close(out, po.Softmax(x, -1))


def test_softmax_rows_sum_to_one_at_full_size(cuda):
    # size-independent property on the microbenchmark shape [768,512,512] (axis -1)
    x = torch.randn(768, 512, 512, device="cuda", generator=torch.Generator("cuda").manual_seed(0)) * 2
    y = ops.softmax(x, -1)
    s = y.sum(-1)
    assert torch.allclose(s, torch.ones_like(s), rtol=0, atol=1e-5)
    assert (y >= 0).all() and torch.equal(y.argmax(-1), x.argmax(-1))
    # shift invariance: softmax(x + c) == softmax(x)
    y2 = ops.softmax(x[:8] + 3.0, -1)
    assert torch.allclose(y2, y[:8], rtol=1e-4, atol=1e-7)


@pytest.mark.parametrize("name", golden_names("layernorm_"))
def test_layernorm_golden(name, cuda):
    g = golden(name)
    close(ops.layernorm(dev(g["x"]), dev(g["gamma"]), dev(g["beta"]), float(g["eps"])), g["y"])
    close(ops.reduce_mean(dev(g["x"]), [-1], 1), g["mean"])


@pytest.mark.parametrize("rows,length", [(129, 768), (64, 1024), (7, 4), (5, 2048), (3, 2500), (2, 50001), (9, 127)])
def test_layernorm_vs_oracle(rows, length, cuda):
    g = torch.Generator().manual_seed(7)
    x = torch.randn(rows, length, generator=g) * 3 + 1
    gamma, beta = torch.randn(length, generator=g), torch.randn(length, generator=g)
    close(ops.layernorm(x.cuda(), gamma.cuda(), beta.cuda(), 1e-12), po.LayerNormChain(x, gamma, beta, 1e-12))
    close(ops.layernorm(x.cuda(), None, None, 1e-5), po.LayerNormChain(x, None, None, 1e-5))


def test_layernorm_node_chain_equals_fused(cuda):
    # The nine nodes run one by one through the C ABI give what the fused kernel gives.
    g = torch.Generator().manual_seed(8)
    x = torch.randn(37, 768, generator=g).cuda()
    gamma, beta = torch.randn(768, generator=g).cuda(), torch.randn(768, generator=g).cuda()
    mean = ops.reduce_mean(x, [-1], 1)
    d = ops.sub(x, mean)
    var = ops.reduce_mean(ops.pow(d, 2.0), [-1], 1)
    y = ops.add(ops.mul(ops.div(d, ops.sqrt(ops.add(var, 1e-12))), gamma), beta)
    close(y, ops.layernorm(x, gamma, beta, 1e-12))
    close(y, po.LayerNormChain(x.cpu(), gamma.cpu(), beta.cpu(), 1e-12))


def test_layernorm_full_size_properties(cuda):
    # [65536,1024], gamma=1, beta=0: every row has mean 0 and second moment 1
    x = torch.randn(65536, 1024, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    y = ops.layernorm(x, None, None, 1e-12)
    assert y.mean(-1).abs().max() < 1e-5
    assert ((y * y).mean(-1) - 1).abs().max() < 1e-4


@pytest.mark.parametrize("shape,axes,keepdims", [((2, 4, 10), [0], 1), ((2, 4, 10), [-1], 0), ((2, 4, 10), [0, 1], 0),
                                                 ((2, 4, 10), [1, 2], 1), ((300, 768), [-1], 1), ((6, 1001), [1], 1)])
def test_reduce_mean_vs_oracle(shape, axes, keepdims, cuda):
    # tests/pure_expansions/test_expansions.py:180-230 uses rtol = atol = 1e-5
    x = torch.randn(shape, generator=torch.Generator().manual_seed(9)) * 10
    out = ops.reduce_mean(x.cuda(), axes, keepdims)
    ref = po.ReduceMean(x, axes, keepdims)
    assert out.shape == ref.shape
    close(out, ref, rtol=1e-5, atol=1e-5)
