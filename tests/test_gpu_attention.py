"""Fused attention (MatMul -> Mul -> Softmax -> MatMul in one kernel, TF32 mode) against the
node-by-node oracle and against the unfused kernels."""
import math

import numpy as np
import pytest
import torch

from dace_onnx_b200 import ops
from dace_onnx_b200.encoder import BertEncoderB200
from oracle import pure_oracle as po
from tests._util import TF32_ATOL, TF32_RTOL, close

pytestmark = pytest.mark.gpu


def oracle_attention(q, k, v, scale):
    """[B,S,H,D] inputs; the four nodes as the exported graph runs them."""
    qh, kh, vh = (t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))
    scores = po.Mul(po.MatMul(qh, kh.transpose(-1, -2).contiguous()), np.float32(scale))
    ctx = po.MatMul(po.Softmax(scores, 3), vh)
    return ctx.permute(0, 2, 1, 3).contiguous()


@pytest.mark.parametrize("B,S,H", [(2, 384, 3), (1, 128, 2), (3, 32, 1), (2, 96, 4), (1, 320, 2), (2, 256, 16),
                                   (2, 512, 3), (1, 640, 2), (1, 1024, 1), (5, 160, 2)])
def test_fused_attention_vs_oracle(B, S, H, cuda):
    D = 64
    g = torch.Generator().manual_seed(S + H)
    qkv = torch.randn(B, S, 3 * H * D, generator=g)
    qkvd = qkv.cuda()
    v4 = qkvd.view(B, S, 3 * H, D)
    out = torch.empty(B, S, H * D, device="cuda")
    assert ops.attention_views(v4[:, :, :H], v4[:, :, H:2 * H], v4[:, :, 2 * H:], out.view(B, S, H, D),
                               1.0 / math.sqrt(D), math_mode="tf32")
    c4 = qkv.view(B, S, 3 * H, D)
    ref = oracle_attention(c4[:, :, :H], c4[:, :, H:2 * H], c4[:, :, 2 * H:], 1.0 / math.sqrt(D))
    close(out.view(B, S, H, D), ref, TF32_RTOL, TF32_ATOL)


def test_fused_attention_sharp_rows_and_separate_tensors(cuda):
    # large logits (one key dominates each row) and separately allocated, contiguous q / k / v
    B, S, H, D = 2, 128, 2, 64
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, S, H, D, generator=g) * s for s in (6.0, 6.0, 1.0))
    out = torch.empty(B, S, H, D, device="cuda")
    assert ops.attention_views(q.cuda(), k.cuda(), v.cuda(), out, 0.125, math_mode="tf32")
    ref = oracle_attention(q, k, v, 0.125)
    # logits of magnitude ~50 carry TF32 operand error of ~0.05 into the exponent: compare loosely
    # against fp32 and tightly against the unfused TF32 kernels that make the same operand cuts
    assert (out.cpu() - ref).abs().max() < 0.25
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    sc = ops.matmul(qd.permute(0, 2, 1, 3).contiguous(), kd.permute(0, 2, 1, 3).contiguous(), trans_b=True,
                    epilogue=ops.EPI_SCALE, scale=0.125, math_mode="tf32")
    un = ops.matmul(ops.softmax(sc, 3), vd.permute(0, 2, 1, 3).contiguous(), math_mode="tf32")
    close(out.permute(0, 2, 1, 3), un, 2e-2, 2e-2)


@pytest.mark.parametrize("S", [384, 512, 160])
def test_running_maximum_moves_between_key_blocks(S, cuda):
    # Scores that grow by 64 per block of 128 keys for the even query rows (the kernel's exponent offset must follow:
    # 64 * 0.125 * log2(e) > 8, so the partial outputs accumulated so far are rescaled at every block) and fall by
    # 64 per block for the odd rows (offset fixed by the first block) - both kinds in every warp. All scores are
    # small integers, exact in TF32, so the comparison with the fp32 oracle stays at the TF32 tolerance of P and V.
    B, H, D = 2, 2, 64
    g = torch.Generator().manual_seed(S)
    q = torch.zeros(B, S, H, D)
    q[:, 0::2, :, 0] = 1.0
    q[:, 1::2, :, 0] = -1.0
    t = torch.arange(S)
    k = torch.randn(B, S, H, D, generator=g)
    k[:, :, :, 0] = (64 * (t // 128) + (t % 7)).float()[None, :, None]
    v = torch.randn(B, S, H, D, generator=g)
    out = torch.empty(B, S, H, D, device="cuda")
    assert ops.attention_views(q.cuda(), k.cuda(), v.cuda(), out, 0.125, math_mode="tf32")
    ref = oracle_attention(q, k, v, 0.125)
    close(out, ref, TF32_RTOL, TF32_ATOL)


def test_rows_are_convex_combinations_at_bench_size(cuda):
    # V = 1 everywhere -> every output element is sum(P)/sum(P) = 1 up to the TF32 cut of P
    B, S, H, D = 128, 384, 16, 64
    g = torch.Generator("cuda").manual_seed(9)
    q = torch.randn(B, S, H, D, device="cuda", generator=g)
    k = torch.randn(B, S, H, D, device="cuda", generator=g)
    v = torch.ones(B, S, H, D, device="cuda")
    out = torch.empty(B, S, H, D, device="cuda")
    assert ops.attention_views(q, k, v, out, 0.125, math_mode="tf32")
    assert (out - 1).abs().max() < 2e-3
    # permuting the keys (and values with them) does not change the result beyond rounding: P is cut to TF32's
    # ten bits relative to an exponent offset that depends on which keys share a block (measured |diff| <= 5e-4)
    v2 = torch.randn(B, S, H, D, device="cuda", generator=g)
    perm = torch.randperm(S, device="cuda", generator=g)
    o1, o2 = torch.empty_like(out), torch.empty_like(out)
    assert ops.attention_views(q[:8], k[:8], v2[:8], o1[:8], 0.125, math_mode="tf32")
    assert ops.attention_views(q[:8], k[:8][:, perm].contiguous(), v2[:8][:, perm].contiguous(), o2[:8], 0.125,
                               math_mode="tf32")
    assert torch.allclose(o1[:8], o2[:8], rtol=1e-2, atol=2e-3)


def test_unsupported_cases_decline(cuda):
    def try_(B, S, H, D, mode):
        t = torch.zeros(B, S, H, D, device="cuda")
        return ops.attention_views(t, t, t, torch.empty_like(t), 0.125, math_mode=mode)
    assert try_(1, 100, 2, 64, "tf32") is False      # seq not a multiple of 32
    assert try_(1, 128, 2, 32, "tf32") is False      # head_dim
    assert try_(1, 128, 2, 64, "fp32x3") is False    # only the TF32 mode is fused
    lib = ops._lib.load()
    d = ops.AttentionDesc(1, 2, 100, 64, *([64] * 12), 0.125, 1)
    one = torch.zeros(8, device="cuda")
    ptr = ops._ptr(one)
    assert lib.b200_attention_f32(None, d, ptr, ptr, ptr, ptr) == ops._lib.EUNSUPPORTED


def test_encoder_fused_equals_unfused(cuda):
    p = po.make_bert_layer_params(256, 512, seed=3, std=0.05)
    x = torch.randn(3, 128, 256, generator=torch.Generator().manual_seed(4))
    fused = BertEncoderB200([p], heads=4, device=cuda, math_mode="tf32", fused_attention=True)
    unfused = BertEncoderB200([p], heads=4, device=cuda, math_mode="tf32", fused_attention=False)
    yf, yu = fused(x), unfused(x)
    assert fused.launches == 7 and unfused.launches == 9
    close(yf, yu, TF32_RTOL, TF32_ATOL)
    close(yf, po.bert_layer_forward(x, p, heads=4), TF32_RTOL, TF32_ATOL)
