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


# ---- the workspace entry point: 3xTF32 with B split once per call, CTA-pair kernel ----------------------------
def _gemm_call(ws_bytes, M, N, K, trans_b, epi, A, B, bias, res, mode=0):
    import ctypes
    from dace_onnx_b200 import _lib
    lib = _lib.load()
    Y = torch.empty(M, N, device="cuda")
    d = _lib.GemmDesc(1, 1, M, N, K, K, K if trans_b else N, N, 0, 0, 0, 0, 0, 0, int(trans_b), epi, 0.5, mode)
    need = lib.b200_gemm_workspace_bytes(ctypes.byref(d))
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if ws_bytes is None:
        _lib.check(lib.b200_gemm_f32(st, ctypes.byref(d), p(A), p(B), p(bias), p(res), p(Y)))
    else:
        n = need if ws_bytes == "need" else ws_bytes
        ws = torch.empty(max(n, 16), device="cuda", dtype=torch.uint8)
        _lib.check(lib.b200_gemm_ws_f32(st, ctypes.byref(d), p(A), p(B), p(bias), p(res), p(Y), p(ws) if n else None, n))
    return Y, need


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("M,N,K", [(256, 192, 32), (384, 128, 96), (1000, 260, 136), (129, 64, 32), (4096, 768, 768),
                                    (2048, 3072, 768), (513, 1024, 100), (300, 8, 40)])
def test_gemm_workspace_path(M, N, K, trans_b, cuda):
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    A = torch.randn(M, K, generator=g)
    # weights ~ N(0, 0.02^2) as in the BERT configurations: the absolute tolerance (1e-5) presumes outputs of order one
    B = torch.randn((N, K) if trans_b else (K, N), generator=g) * 0.02
    bias, res = torch.randn(N, generator=g), torch.randn(M, N, generator=g)
    ref = po.MatMul(A, B.t().contiguous() if trans_b else B)
    for epi, want in ((0, ref), (EPI_BIAS, po.Add(ref, bias)), (EPI_BIAS_RESIDUAL, po.Add(po.Add(ref, bias), res)),
                      (EPI_BIAS_GELU, po.GeluChain(po.Add(ref, bias))), (EPI_SCALE, po.Mul(ref, np.float32(0.5)))):
        # the library asks for the split workspace only where the pair kernel pays (>= 4.5e9 multiply-adds); a
        # caller that brings it anyway gets that kernel at any size, which is what these shapes exercise
        full = 2 * ((N * K * 4 + 255) // 256 * 256)
        Y, need = _gemm_call(full, M, N, K, trans_b, epi, A.cuda(), B.cuda(), bias.cuda(), res.cuda())
        assert need == (full if M * N * K >= 4.5e9 else 0)
        close(Y, want, RTOL, ATOL)


def test_gemm_workspace_is_optional(cuda):
    g = torch.Generator().manual_seed(3)
    M, N, K = 4096, 1536, 768  # large enough (>= 4.5e9 multiply-adds) for the library to ask for the workspace
    A, B, bias = torch.randn(M, K, generator=g).cuda(), torch.randn(N, K, generator=g).cuda(), torch.randn(N, generator=g).cuda()
    plain, need = _gemm_call(None, M, N, K, True, EPI_BIAS, A, B, bias, None)
    assert need > 0
    for ws in (0, need - 256):                      # absent or too small: exactly the plain entry point's result
        y, _ = _gemm_call(ws, M, N, K, True, EPI_BIAS, A, B, bias, None)
        assert torch.equal(y, plain)
    y, _ = _gemm_call("need", M, N, K, True, EPI_BIAS, A, B, bias, None)
    close(y, plain, RTOL, ATOL)                     # same 3xTF32 arithmetic, different accumulation grouping
    # no scratch is asked for where the pair kernel does not apply: other modes, single row tile, ragged B rows
    assert _gemm_call(None, M, N, K, True, EPI_BIAS, A, B, bias, None, mode=1)[1] == 0
    assert _gemm_call(None, 128, N, K, True, EPI_BIAS, A[:128].contiguous(), B, bias, None)[1] == 0
    assert _gemm_call(None, M, N, 254, True, EPI_BIAS, A[:, :254].contiguous(), B[:, :254].contiguous(), bias, None)[1] == 0
    # ... and small products, where the split kernel's launch costs more than the pair kernel saves
    assert _gemm_call(None, 640, 384, 256, True, EPI_BIAS, A[:640, :256].contiguous(), B[:384, :256].contiguous(), bias[:384].contiguous(), None)[1] == 0
