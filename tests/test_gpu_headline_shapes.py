"""Parity at the shapes the benchmark numbers are quoted on: the BERT-large layer (hidden 1024,
16 heads, FFN 4096, sequence 384) through both runners, its GEMM and attention shapes, samples of
the full-size bandwidth microbenchmarks and of the full-batch convolution stack, and the measured
error of the 24-layer TF32 forward against the fp32 oracle."""
import math

import numpy as np
import pytest
import torch

from dace_onnx_b200 import graphs, ops
from dace_onnx_b200._lib import EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL
from dace_onnx_b200.encoder import BertEncoderB200
from oracle import graph_oracle
from oracle import pure_oracle as po
from tests._util import ATOL, REF_ATOL, REF_RTOL, RTOL, TF32_ATOL, TF32_RTOL, close

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, FFN, SEQ = 1024, 16, 4096, 384


def _nontrivial(p, seed):
    """Non-zero biases and non-unit LayerNorm parameters (the benchmark's zeros / ones would hide them)."""
    gen = torch.Generator().manual_seed(seed)
    for k in ("bq", "bk", "bv", "bo", "bi", "bo2", "ln1_b", "ln2_b"):
        p[k] = torch.randn(p[k].shape, generator=gen) * 0.1
    for k in ("ln1_g", "ln2_g"):
        p[k] = 1 + torch.randn(p[k].shape, generator=gen) * 0.1
    return p


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
def test_bert_large_layer_vs_oracle(mode, rtol, atol, cuda):
    p = _nontrivial(po.make_bert_layer_params(HIDDEN, FFN, seed=51), 52)
    x = torch.randn(3, SEQ, HIDDEN, generator=torch.Generator().manual_seed(53))
    ref = po.bert_layer_forward(x, p, heads=HEADS)
    y = BertEncoderB200([p], heads=HEADS, device=cuda, math_mode=mode)(x)
    close(y, ref, rtol, atol)
    if mode == "fp32x3":
        close(y, ref, REF_RTOL, REF_ATOL)  # the reference's own comparator, tests/pytorch/test_bert_encoder.py:10-34


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", REF_RTOL, REF_ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
def test_bert_large_layer_through_the_front_door(mode, rtol, atol, cuda):
    """transformers.BertLayer at the BERT-large sizes, exported and run from the graph like the reference's
    DaceModule test, against the torch module itself and the node-by-node graph oracle."""
    from transformers import BertConfig, BertLayer
    from dace_onnx_b200.torch_module import B200Module, export_onnx
    torch.manual_seed(61)
    cfg = BertConfig(hidden_size=HIDDEN, num_attention_heads=HEADS, intermediate_size=FFN, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    cfg._attn_implementation = "eager"
    layer = BertLayer(cfg).eval()
    x = torch.randn(2, SEQ, HIDDEN)
    with torch.no_grad():
        ref = layer(x)
    ref = ref[0] if isinstance(ref, (tuple, list)) else ref
    mod = B200Module(layer, math_mode=mode, sdfg_name="bert_large_layer")
    out = mod(x.cuda())
    close(out, ref, rtol, atol)
    close(out, graph_oracle.run(export_onnx(layer, (x,)), [x])[0], rtol, atol)
    hist = mod.onnx_model.plan((2, SEQ, HIDDEN)).ir.op_histogram()
    if mode == "tf32":
        assert hist == {"B200SelfAttention": 1, "B200Gemm": 3, "B200LayerNorm": 2}


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", RTOL, ATOL), ("fp32", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
@pytest.mark.parametrize("M,N,K,epi", [(640, 4096, 4096, EPI_BIAS), (768, 1024, 4096, EPI_BIAS_RESIDUAL),
                                       (768, 4096, 1024, EPI_BIAS_GELU), (768, 3072, 1024, EPI_BIAS)])
def test_bert_large_gemm_shapes(M, N, K, epi, mode, rtol, atol, cuda):
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.02
    bias, res = torch.randn(N, generator=g) * 0.1, torch.randn(M, N, generator=g)
    ref = po.Add(bias, po.MatMul(a, w.t().contiguous()))
    if epi == EPI_BIAS_RESIDUAL:
        ref = po.Add(ref, res)
    elif epi == EPI_BIAS_GELU:
        ref = po.GeluChain(ref)
    out = ops.matmul(a.cuda(), w.cuda(), trans_b=True, epilogue=epi, bias=bias.cuda(),
                     residual=res.cuda() if epi == EPI_BIAS_RESIDUAL else None, math_mode=mode)
    close(out, ref, rtol, atol)


def test_bert_large_attention_shape(cuda):
    # 16 heads at sequence 384, heads addressed inside the fused QKV projection as the encoder does
    from tests.test_gpu_attention import oracle_attention
    B, S, H, D = 3, SEQ, HEADS, 64
    qkv = torch.randn(B, S, 3 * H * D, generator=torch.Generator().manual_seed(71))
    v4 = qkv.cuda().view(B, S, 3 * H, D)
    out = torch.empty(B, S, H * D, device="cuda")
    assert ops.attention_views(v4[:, :, :H], v4[:, :, H:2 * H], v4[:, :, 2 * H:], out.view(B, S, H, D),
                               1.0 / math.sqrt(D), math_mode="tf32")
    c4 = qkv.view(B, S, 3 * H, D)
    ref = oracle_attention(c4[:, :, :H], c4[:, :, H:2 * H], c4[:, :, 2 * H:], 1.0 / math.sqrt(D))
    close(out.view(B, S, H, D), ref, TF32_RTOL, TF32_ATOL)


def test_softmax_full_size_sample_vs_oracle(cuda):
    # the microbenchmark tensor [768, 512, 512]; 256 of its 393216 rows, spread over the whole tensor
    x = torch.randn(768, 512, 512, device="cuda", generator=torch.Generator("cuda").manual_seed(0)) * 2
    y = ops.softmax(x, -1).view(-1, 512)
    rows = torch.arange(0, 768 * 512, 768 * 512 // 256, device="cuda") + 7
    close(y[rows], po.Softmax(x.view(-1, 512)[rows].cpu(), -1))


def test_layernorm_full_size_sample_vs_oracle(cuda):
    x = torch.randn(65536, 1024, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    g = torch.Generator().manual_seed(2)
    gamma, beta = 1 + 0.1 * torch.randn(1024, generator=g), 0.1 * torch.randn(1024, generator=g)
    y = ops.layernorm(x, gamma.cuda(), beta.cuda(), 1e-12)
    rows = torch.arange(0, 65536, 256, device="cuda") + 3
    close(y[rows], po.LayerNormChain(x[rows].cpu(), gamma, beta, 1e-12))
    rows = torch.arange(65536 - 8, 65536, device="cuda")  # the last CTA's rows
    close(y[rows], po.LayerNormChain(x[rows].cpu(), gamma, beta, 1e-12))


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
def test_config2_full_batch_sample_vs_oracle(mode, rtol, atol, cuda):
    # batch 256 through both layers; four images (first, two inner, last) against the oracle
    params = po.make_conv_params(0, channels=64, layers=2)
    x = torch.rand(256, 64, 56, 56, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    full = graphs.conv_stack_forward(x, [(w.cuda(), b.cuda()) for w, b in params], math_mode=mode)
    idx = [0, 101, 202, 255]
    close(full[idx], po.conv_stack_forward(x[idx].cpu(), params), rtol, atol)


def test_tf32_error_of_the_24_layer_forward(cuda, record_property):
    """The headline configuration's arithmetic (24 BERT-large layers, TF32) on two sequences against the fp32
    oracle: the error a user of the TF32 mode actually sees after 24 layers. Outputs are LayerNorm outputs
    (unit variance), so the figures are relative to values of magnitude 1."""
    from dace_onnx_b200.encoder import synthetic_layer_params
    layers = [synthetic_layer_params(HIDDEN, FFN, seed=100 + i) for i in range(24)]  # the benchmark's weights
    x = torch.randn(2, SEQ, HIDDEN, generator=torch.Generator().manual_seed(7))
    ref = po.bert_encoder_forward(x, layers, heads=HEADS)
    y = BertEncoderB200(layers, heads=HEADS, device=cuda, math_mode="tf32")(x)
    err = (y - ref).abs()
    mx, rms = err.max().item(), err.pow(2).mean().sqrt().item()
    y3 = BertEncoderB200(layers, heads=HEADS, device=cuda, math_mode="fp32x3")(x)
    err3 = (y3 - ref).abs()
    mx3, rms3 = err3.max().item(), err3.pow(2).mean().sqrt().item()
    print("\n24-layer BERT-large forward vs fp32 oracle: tf32 max %.3e rms %.3e | fp32x3 max %.3e rms %.3e"
          % (mx, rms, mx3, rms3))
    for k, v in (("tf32_max", mx), ("tf32_rms", rms), ("fp32x3_max", mx3), ("fp32x3_rms", rms3)):
        record_property(k, v)
    assert mx < 5e-2 and rms < 1e-2          # measured: max 2.3e-2, rms 4.6e-3 (stated TF32 tolerance: rtol 2e-2 / atol 1e-2)
    assert mx3 < 2e-4 and rms3 < 3e-5        # measured: max 2.9e-5, rms 5.6e-6
