"""MatMul / Gemm through the C ABI against the oracle, in every math mode.

fp32x3 (3xTF32 on tcgen05, the default) and fp32 (CUDA cores) must meet the fp32 parity bar
rtol 1e-4 / atol 1e-5; single-pass tf32 is checked against its stated wider tolerance.
"""
import numpy as np
import pytest
import torch

from dace_onnx_b200 import ops
from dace_onnx_b200._lib import EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RELU, EPI_BIAS_RESIDUAL, EPI_SCALE
from oracle import pure_oracle as po
from tests._util import ATOL, RTOL, TF32_ATOL, TF32_RTOL, close, dev, golden, golden_names

pytestmark = pytest.mark.gpu

MODES = [("fp32x3", RTOL, ATOL), ("fp32", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)]


@pytest.mark.parametrize("mode,rtol,atol", MODES)
@pytest.mark.parametrize("name", golden_names("matmul_"))
def test_matmul_golden(name, mode, rtol, atol, cuda):
    g = golden(name)
    close(ops.matmul(dev(g["A"]), dev(g["B"]), math_mode=mode), g["Y"], rtol, atol)


@pytest.mark.parametrize("mode,rtol,atol", MODES)
@pytest.mark.parametrize("name", golden_names("gemm_"))
def test_gemm_golden(name, mode, rtol, atol, cuda):
    g = golden(name)
    close(ops.gemm(dev(g["A"]), dev(g["B"]), dev(g["C"]), math_mode=mode), g["Y"], rtol, atol)


def test_matmul_reference_test_criterion(cuda):
    # tests/pure_expansions/test_expansions.py:18-56: [2,4]@[4,3], np.allclose defaults
    rng = np.random.default_rng(21)
    X, Z = rng.random((2, 4), dtype=np.float32), rng.random((4, 3), dtype=np.float32)
    assert np.allclose(ops.matmul(dev(X), dev(Z)).cpu().numpy(), X @ Z)
    with pytest.raises(ValueError):
        ops.matmul(dev(X), dev(Z[:, 0]))


SHAPES = [  # (M, N, K) incl. tile tails in every dimension and K tails of the 32-wide k-block
    (128, 256, 32), (128, 128, 64), (256, 64, 96), (1, 8, 4), (127, 255, 100), (129, 257, 36), (300, 72, 8),
    (512, 768, 768), (384, 384, 64), (384, 64, 384), (1000, 3072, 768), (64, 1000, 260),
]


@pytest.mark.parametrize("mode,rtol,atol", MODES)
@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_matmul_shapes(M, N, K, trans_b, mode, rtol, atol, cuda):
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(N, K, generator=g) / (K ** 0.5) if trans_b else torch.randn(K, N, generator=g) / (K ** 0.5)
    ref = po.MatMul(a, b.t().contiguous() if trans_b else b)
    close(ops.matmul(a.cuda(), b.cuda(), trans_b=trans_b, math_mode=mode), ref, rtol, atol)


@pytest.mark.parametrize("mode,rtol,atol", MODES)
def test_matmul_epilogues(mode, rtol, atol, cuda):
    g = torch.Generator().manual_seed(31)
    M, N, K = 200, 320, 128
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) / (K ** 0.5)
    bias, res = torch.randn(N, generator=g), torch.randn(M, N, generator=g)
    y = po.MatMul(a, w.t().contiguous())
    ad, wd, bd, rd = a.cuda(), w.cuda(), bias.cuda(), res.cuda()
    kw = dict(trans_b=True, math_mode=mode)
    close(ops.matmul(ad, wd, epilogue=EPI_BIAS, bias=bd, **kw), po.Add(bias, y), rtol, atol)
    close(ops.matmul(ad, wd, epilogue=EPI_BIAS_RELU, bias=bd, **kw), po.Relu(po.Add(bias, y)), rtol, atol)
    close(ops.matmul(ad, wd, epilogue=EPI_BIAS_GELU, bias=bd, **kw), po.GeluChain(po.Add(bias, y)), rtol, atol)
    close(ops.matmul(ad, wd, epilogue=EPI_BIAS_RESIDUAL, bias=bd, residual=rd, **kw), po.Add(po.Add(bias, y), res),
          rtol, atol)
    close(ops.matmul(ad, wd, epilogue=EPI_SCALE, scale=0.125, **kw), po.Mul(y, np.float32(0.125)), rtol, atol)


@pytest.mark.parametrize("mode,rtol,atol", MODES)
def test_attention_batched_views(mode, rtol, atol, cuda):
    # Q/K/V addressed in place inside a fused [B,S,3*hidden] projection, as the encoder does.
    g = torch.Generator().manual_seed(41)
    B, S, H, D = 2, 96, 3, 64
    hid = H * D
    qkv = torch.randn(B, S, 3 * hid, generator=g)
    qkvd = qkv.cuda()
    q = qkv[..., :hid].reshape(B, S, H, D).permute(0, 2, 1, 3)
    k = qkv[..., hid:2 * hid].reshape(B, S, H, D).permute(0, 2, 1, 3)
    v = qkv[..., 2 * hid:].reshape(B, S, H, D).permute(0, 2, 1, 3)
    scores_ref = po.Mul(po.MatMul(q.contiguous(), k.transpose(-1, -2).contiguous()), np.float32(0.125))
    scores = torch.empty(B, H, S, S, device="cuda")
    ops.gemm_raw(qkvd, qkvd[..., hid:], scores, batch_outer=B, batch_inner=H, M=S, N=S, K=D, lda=3 * hid,
                 ldb=3 * hid, ldy=S, a_strides=(S * 3 * hid, D), b_strides=(S * 3 * hid, D),
                 y_strides=(H * S * S, S * S), trans_b=True, epilogue=EPI_SCALE, scale=0.125, math_mode=mode)
    close(scores, scores_ref, rtol, atol)
    probs = po.Softmax(scores_ref, 3)
    ctx_ref = po.MatMul(probs, v.contiguous()).permute(0, 2, 1, 3).reshape(B, S, hid)
    ctx = torch.empty(B, S, hid, device="cuda")
    ops.gemm_raw(probs.cuda(), qkvd[..., 2 * hid:], ctx, batch_outer=B, batch_inner=H, M=S, N=D, K=S, lda=S,
                 ldb=3 * hid, ldy=hid, a_strides=(H * S * S, S * S), b_strides=(S * 3 * hid, D),
                 y_strides=(S * hid, D), trans_b=False, math_mode=mode)
    close(ctx, ctx_ref, rtol, atol)


def test_modes_agree_and_linearity_at_bert_size(cuda):
    # size-independent properties on a BERT-base projection [4096,768]x[768,768]^T
    g = torch.Generator("cuda").manual_seed(5)
    a = torch.randn(4096, 768, device="cuda", generator=g)
    a2 = torch.randn(4096, 768, device="cuda", generator=g)
    w = torch.randn(768, 768, device="cuda", generator=g) * 0.02
    y = ops.matmul(a, w, trans_b=True)
    close(y, ops.matmul(a, w, trans_b=True, math_mode="fp32"))
    close(ops.matmul(a + a2, w, trans_b=True), y + ops.matmul(a2, w, trans_b=True), rtol=1e-4, atol=2e-5)
    close(ops.matmul(a, w, trans_b=True, math_mode="tf32"), y, TF32_RTOL, TF32_ATOL)


def test_bad_arguments_raise(cuda):
    a = torch.zeros(4, 8, device="cuda")
    with pytest.raises(ValueError):
        ops.matmul(a, torch.zeros(7, 3, device="cuda"))
    with pytest.raises(ops._lib.B200Error):
        ops.matmul(a, a, trans_b=True, epilogue=EPI_BIAS)  # missing bias
    with pytest.raises(NotImplementedError):
        ops.gemm(a, a, transB=0)
    assert ops.matmul(torch.zeros(0, 8, device="cuda"), torch.zeros(8, 3, device="cuda")).shape == (0, 3)
