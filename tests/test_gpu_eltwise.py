"""Elementwise nodes with numpy broadcasting, unary nodes and layout helpers against the oracle."""
import numpy as np
import pytest
import torch

from dace_onnx_b200 import ops
from oracle import pure_oracle as po
from tests._util import close, dev, golden

pytestmark = pytest.mark.gpu


def test_eltwise_golden(cuda):
    g = golden("eltwise")
    x, row, col, pos = dev(g["x"]), dev(g["row"]), dev(g["col"]), dev(g["pos"])
    close(ops.add(x, row), g["add_row"])
    close(ops.sub(x, col), g["sub_col"])
    close(ops.mul(x, pos), g["mul_full"])
    close(ops.div(x, pos), g["div_full"])
    close(ops.pow(x, 2.0), g["pow2"])
    close(ops.pow(pos, x), g["pow_full"])
    close(ops.sqrt(pos), g["sqrt"])
    close(ops.erf(x), g["erf"])
    close(ops.relu(x), g["relu"])
    close(ops.gelu(x), g["gelu"])
    close(ops.add(col, 1e-12), g["add_scalar"])


BCAST = [((64, 768), (768,)), ((64, 768), (64, 1)), ((64, 768), (64, 768)), ((64, 768), ()), ((3, 1, 5), (4, 1)),
         ((2, 3, 4, 5), (3, 1, 5)), ((7,), (7,)), ((2, 12, 64, 64), ()), ((5, 10), (10,)), ((1, 768), (33, 768)),
         ((4, 1, 6, 1, 2), (1, 3, 1, 5, 2)), ((1000, 260), (260,))]


@pytest.mark.parametrize("sa,sb", BCAST)
def test_binary_broadcast_vs_oracle(sa, sb, cuda):
    g = torch.Generator().manual_seed(12)
    a = torch.randn(sa, generator=g)
    b = torch.rand(sb, generator=g) + 0.5
    for gpu_fn, ref_fn in [(ops.add, po.Add), (ops.sub, po.Sub), (ops.mul, po.Mul), (ops.div, po.Div)]:
        close(gpu_fn(a.cuda(), b.cuda()), ref_fn(a, b))
        close(gpu_fn(b.cuda(), a.cuda()), ref_fn(b, a))
    close(ops.pow(b.cuda(), a.cuda()), po.Pow(b, a))


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096, 100003])
def test_unary_vs_oracle(n, cuda):
    x = torch.randn(n, generator=torch.Generator().manual_seed(13)) * 3
    close(ops.erf(x.cuda()), po.Erf(x), atol=1e-6)
    close(ops.relu(x.cuda()), po.Relu(x), rtol=0, atol=0)
    close(ops.sqrt(x.abs().cuda()), po.Sqrt(x.abs()), rtol=1e-6, atol=0)
    close(ops.gelu(x.cuda()), po.GeluChain(x))
    # the five nodes of the Gelu chain one by one
    xd = x.cuda()
    t = ops.erf(ops.div(xd, float(po.SQRT2)))
    close(ops.mul(ops.mul(xd, ops.add(t, 1.0)), 0.5), po.GeluChain(x))


def test_unary_unaligned_and_empty(cuda):
    base = torch.randn(1030, generator=torch.Generator().manual_seed(14))
    xd = base.cuda()[1:]
    out = torch.empty(1033, device="cuda")[3:1032]
    ops._lib.check(ops._lib.load().b200_unary_f32(ops._stream(), ops._lib.ERF, ops._ptr(xd), ops._ptr(out), 1029))
    close(out, po.Erf(base[1:]), atol=1e-6)
    assert ops.relu(torch.empty(0, device="cuda")).numel() == 0


def test_transposes(cuda):
    x = torch.randn(3, 17, 4, 64, generator=torch.Generator().manual_seed(15))
    assert torch.equal(ops.transpose_0213(x.cuda()).cpu(), x.permute(0, 2, 1, 3).contiguous())
    x = torch.randn(2, 5, 3, 7, generator=torch.Generator().manual_seed(16))
    assert torch.equal(ops.transpose_0213(x.cuda()).cpu(), x.permute(0, 2, 1, 3).contiguous())
    w = torch.randn(3, 70, 45, generator=torch.Generator().manual_seed(17))
    assert torch.equal(ops.transpose_last2(w.cuda()).cpu(), w.transpose(-1, -2).contiguous())
    # multiples of four take the 64 x 64 vectorised tiles: ragged tile edges and exact tiles
    for shape, seed in (((3, 68, 44), 18), ((2, 128, 192), 19), ((5, 4, 260), 20), ((1, 1000, 8), 21)):
        w = torch.randn(*shape, generator=torch.Generator().manual_seed(seed))
        assert torch.equal(ops.transpose_last2(w.cuda()).cpu(), w.transpose(-1, -2).contiguous())


def test_binary_linearity_at_full_size(cuda):
    # (a + b) - b == a up to one rounding, on a BERT-sized activation
    a = torch.randn(32768, 768, device="cuda", generator=torch.Generator("cuda").manual_seed(2))
    b = torch.randn(768, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    assert torch.allclose(ops.sub(ops.add(a, b), b), a, rtol=1e-5, atol=1e-6)
    assert torch.equal(ops.add(a, b), a + b)
