"""BERT encoder layer through the C ABI (fused epilogues, in-place head addressing) against the
node-by-node CPU oracle, like tests/pytorch/test_bert_encoder.py of the reference."""
import pytest
import torch

from dace_onnx_b200.encoder import BertEncoderB200
from oracle import pure_oracle as po
from tests._util import ATOL, REF_ATOL, REF_RTOL, RTOL, TF32_ATOL, TF32_RTOL, close, dev, golden

pytestmark = pytest.mark.gpu

KEYS = ["wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "ln1_g", "ln1_b", "wi", "bi", "wo2", "bo2", "ln2_g", "ln2_b"]


def test_small_layer_golden(cuda):
    g = golden("bert_layer_small")
    p = {k: torch.tensor(g[k]) for k in KEYS}
    enc = BertEncoderB200([p], heads=4, device=cuda, math_mode="fp32x3")
    close(enc(torch.tensor(g["x"])), g["y"])
    enc32 = BertEncoderB200([p], heads=4, device=cuda, math_mode="fp32")
    close(enc32(torch.tensor(g["x"])), g["y"])


@pytest.mark.parametrize("mode,rtol,atol", [("fp32x3", RTOL, ATOL), ("tf32", TF32_RTOL, TF32_ATOL)])
def test_bert_base_layer_vs_oracle(mode, rtol, atol, cuda):
    # BertConfig() sizes: hidden 768, 12 heads, ffn 3072, seq 512 (batch 2 so the CPU oracle stays quick)
    p = po.make_bert_layer_params(768, 3072, seed=21)
    # non-trivial biases / LayerNorm parameters, unlike the benchmark's zeros and ones
    gen = torch.Generator().manual_seed(22)
    for k in ("bq", "bk", "bv", "bo", "bi", "bo2", "ln1_b", "ln2_b"):
        p[k] = torch.randn(p[k].shape, generator=gen) * 0.1
    for k in ("ln1_g", "ln2_g"):
        p[k] = 1 + torch.randn(p[k].shape, generator=gen) * 0.1
    x = torch.randn(2, 512, 768, generator=gen)
    ref = po.bert_layer_forward(x, p, heads=12)
    enc = BertEncoderB200([p], heads=12, device=cuda, math_mode=mode)
    y = enc(x)
    close(y, ref, rtol, atol)
    if mode == "fp32x3":
        close(y, ref, REF_RTOL, REF_ATOL)  # the reference's own comparator (rtol 1e-5, atol 1e-4)


def test_micro_batching_and_stacking_do_not_change_results(cuda):
    layers = [po.make_bert_layer_params(128, 256, seed=30 + i, std=0.05) for i in range(3)]
    x = torch.randn(5, 64, 128, generator=torch.Generator().manual_seed(33))
    ref = po.bert_encoder_forward(x, layers, heads=2)
    whole = BertEncoderB200(layers, heads=2, device=cuda, micro_batch=8)(x)
    pieces = BertEncoderB200(layers, heads=2, device=cuda, micro_batch=2)(x)
    close(whole, ref)
    assert torch.equal(whole, pieces)  # ragged last micro-batch, bit-identical rows


def test_host_entry_overlapped_copies_match_device_path(cuda):
    layers = [po.make_bert_layer_params(128, 256, seed=40 + i, std=0.05) for i in range(2)]
    enc = BertEncoderB200(layers, heads=2, device=cuda, micro_batch=2)
    x = torch.randn(7, 64, 128, generator=torch.Generator().manual_seed(41)).pin_memory()
    y_host = torch.empty(7, 64, 128).pin_memory()
    y_dev = torch.empty(7, 64, 128, device=cuda)
    for _ in range(2):  # second pass reuses the staging buffers and streams
        enc.forward_host(x, y_host, out_device=y_dev)
        torch.cuda.synchronize()
        ref = enc.forward_device(x.to(cuda))
        assert torch.equal(y_dev, ref) and torch.equal(y_host, ref.cpu())
    assert torch.equal(enc(x), ref.cpu())  # __call__ without a device copy of the output
    # a batch that fits one micro-batch (64..micro_batch sequences) is still moved in two halves
    big = BertEncoderB200(layers, heads=2, device=cuda, micro_batch=128)
    xb = torch.randn(70, 32, 128, generator=torch.Generator().manual_seed(42)).pin_memory()
    assert torch.equal(big(xb), big.forward_device(xb.to(cuda)).cpu())
    # two or more micro-batches of at least 64: the schedule starts and ends with a half-size one (32, 64, 22, 32)
    mid = BertEncoderB200(layers, heads=2, device=cuda, micro_batch=64)
    xm = torch.randn(150, 32, 128, generator=torch.Generator().manual_seed(43)).pin_memory()
    assert torch.equal(mid(xm), mid.forward_device(xm.to(cuda)).cpu())


def test_rejects_wrong_inputs(cuda):
    enc = BertEncoderB200([po.make_bert_layer_params(128, 256, seed=1)], heads=2, device=cuda)
    with pytest.raises(ValueError):
        enc.forward_device(torch.zeros(2, 8, 64, device=cuda))
    with pytest.raises(ValueError):
        enc.forward_device(torch.zeros(2, 8, 128))
