"""The BF16 math mode (B200_MATH_BF16): operands rounded to bf16, fp32 accumulation. Compared with the fp32 oracle
at the stated BF16 tolerance, and -- tightly -- with an oracle fed the same bf16-rounded operands, which isolates
the kernel's arithmetic from the operand rounding."""
import ctypes

import pytest
import torch

from dace_onnx_b200 import _lib, ops
from dace_onnx_b200._lib import EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL
from dace_onnx_b200.encoder import BertEncoderB200
from oracle import pure_oracle as po
from tests._util import BF16_ATOL, BF16_RTOL, RTOL, close

pytestmark = pytest.mark.gpu


def _bf16(t):
    return t.to(torch.bfloat16).to(torch.float32)


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 72, 8), (129, 257, 36), (1000, 3072, 768), (640, 1024, 4096),
                                   (64, 1000, 260), (1, 8, 4), (512, 768, 100)])
def test_bf16_matmul_vs_oracle(M, N, K, trans_b, cuda):
    g = torch.Generator().manual_seed(M + 3 * N + 7 * K)
    a = torch.randn(M, K, generator=g)
    b = (torch.randn(N, K, generator=g) if trans_b else torch.randn(K, N, generator=g)) / K ** 0.5
    bm = b.t().contiguous() if trans_b else b
    out = ops.matmul(a.cuda(), b.cuda(), trans_b=trans_b, math_mode="bf16")
    close(out, po.MatMul(a, bm), BF16_RTOL, BF16_ATOL)
    # same rounded operands on both sides: what is left is accumulation order
    close(out, po.MatMul(_bf16(a), _bf16(bm)), RTOL, 2e-5)


def test_bf16_epilogues(cuda):
    g = torch.Generator().manual_seed(5)
    M, N, K = 400, 512, 256
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) / K ** 0.5
    bias, res = torch.randn(N, generator=g), torch.randn(M, N, generator=g)
    y = po.Add(bias, po.MatMul(_bf16(a), _bf16(w).t().contiguous()))
    kw = dict(trans_b=True, math_mode="bf16", bias=bias.cuda())
    close(ops.matmul(a.cuda(), w.cuda(), epilogue=EPI_BIAS, **kw), y, RTOL, 2e-5)
    close(ops.matmul(a.cuda(), w.cuda(), epilogue=EPI_BIAS_GELU, **kw), po.GeluChain(y), RTOL, 2e-5)
    close(ops.matmul(a.cuda(), w.cuda(), epilogue=EPI_BIAS_RESIDUAL, residual=res.cuda(), **kw), po.Add(y, res), RTOL, 2e-5)


def test_bf16_needs_the_workspace_entry_point(cuda):
    lib = _lib.load()
    a, w, y = torch.randn(256, 64, device="cuda"), torch.randn(128, 64, device="cuda"), torch.empty(256, 128, device="cuda")
    d = _lib.GemmDesc(1, 1, 256, 128, 64, 64, 64, 128, 0, 0, 0, 0, 0, 0, 1, 0, 1.0, _lib.MATH_BF16)
    assert lib.b200_gemm_workspace_bytes(ctypes.byref(d)) == 256 * 64 * 2 + 128 * 64 * 2
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200_gemm_f32(st, ctypes.byref(d), p(a), p(w), None, None, p(y)) == _lib.EWORKSPACE
    assert b"workspace" in lib.b200_last_error_string()


def test_bf16_batched_attention_and_conv_requests_run_in_tf32(cuda):
    # batched operands, the fused attention and the convolution have no bf16 kernel: the request is honoured with
    # the (more accurate) TF32 kernels, bit-identical to asking for TF32
    g = torch.Generator().manual_seed(6)
    q, k = torch.randn(2, 3, 64, 64, generator=g).cuda(), torch.randn(2, 3, 64, 64, generator=g).cuda()
    assert torch.equal(ops.matmul(q, k, trans_b=True, math_mode="bf16"), ops.matmul(q, k, trans_b=True, math_mode="tf32"))
    qkv = torch.randn(2, 128, 3, 2, 64, generator=g).cuda()
    o1, o2 = torch.empty(2, 128, 2, 64, device="cuda"), torch.empty(2, 128, 2, 64, device="cuda")
    assert ops.attention_views(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], o1, 0.125, math_mode="bf16") is True
    assert ops.attention_views(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], o2, 0.125, math_mode="tf32") is True
    assert torch.equal(o1, o2)
    x, w = torch.rand(2, 32, 9, 9, generator=g).cuda(), (torch.rand(16, 32, 3, 3, generator=g) - 0.5).cuda()
    assert torch.equal(ops.conv2d(x, w, pads=(1, 1, 1, 1), math_mode="bf16"), ops.conv2d(x, w, pads=(1, 1, 1, 1), math_mode="tf32"))


def test_bf16_bert_large_layer_vs_oracle(cuda):
    p = po.make_bert_layer_params(1024, 4096, seed=51)
    x = torch.randn(2, 384, 1024, generator=torch.Generator().manual_seed(53))
    ref = po.bert_layer_forward(x, p, heads=16)
    y = BertEncoderB200([p], heads=16, device=cuda, math_mode="bf16")(x)
    err = (y - ref).abs()
    print("\nBERT-large layer, bf16 mode vs fp32 oracle: max %.3e rms %.3e" % (err.max().item(), err.pow(2).mean().sqrt().item()))
    close(y, ref, BF16_RTOL, BF16_ATOL)
