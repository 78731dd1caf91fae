"""Pins the CPU oracle to the comparators of the reference's own tests (same shapes, same
reference functions, same tolerances), and to the committed golden vectors."""
import numpy as np
import pytest
import torch

from oracle import pure_oracle as po
from tests._util import golden, golden_names


def test_matmul_like_reference_test():
    # tests/pure_expansions/test_expansions.py:18-56  [2,4]@[4,3], rand, np.allclose defaults
    rng = np.random.default_rng(1)
    X, Z = rng.random((2, 4), dtype=np.float32), rng.random((4, 3), dtype=np.float32)
    assert np.allclose(po.MatMul(X, Z).numpy(), X @ Z)
    with pytest.raises(ValueError):
        po.MatMul(X, Z[:, 0])  # 1-D operands are not expandable (pure_implementations.py:135-140)


@pytest.mark.parametrize("a_shape,b_shape", [((3, 5, 8), (3, 8, 6)), ((2, 3, 7, 16), (16, 12)), ((5, 8), (4, 8, 3))])
def test_matmul_broadcast_is_numpy_matmul(a_shape, b_shape):
    rng = np.random.default_rng(2)
    a, b = rng.random(a_shape, dtype=np.float32), rng.random(b_shape, dtype=np.float32)
    assert np.allclose(po.MatMul(a, b).numpy(), np.matmul(a, b))


@pytest.mark.parametrize("axis", [0, -1])
def test_softmax_like_reference_test(axis):
    # test_expansions.py:343-379  [2,4,10] N(0,10^2), ||delta||_2 < 1e-5 vs torch softmax
    X = np.random.default_rng(3).normal(scale=10, size=(2, 4, 10)).astype(np.float32)
    ref = torch.nn.functional.softmax(torch.tensor(X), dim=axis).numpy()
    assert np.linalg.norm(ref - po.Softmax(X, axis).numpy()) < 1e-5


@pytest.mark.parametrize("axis", [0, -1])
def test_logsoftmax_like_reference_test(axis):
    # test_expansions.py:382-418
    X = np.random.default_rng(4).normal(scale=10, size=(2, 4, 10)).astype(np.float32)
    ref = torch.nn.functional.log_softmax(torch.tensor(X), dim=axis).numpy()
    assert np.linalg.norm(ref - po.LogSoftmax(X, axis).numpy()) < 1e-5


@pytest.mark.parametrize("axes,keepdims", [([0], 1), ([-1], 1), ([-1], 0), ([0, 1], 0), ([1, 2], 1)])
def test_reduce_mean_like_reference_test(axes, keepdims):
    # test_expansions.py:180-230  [2,4,10], rtol = atol = 1e-5 vs numpy
    X = np.random.default_rng(5).normal(scale=10, size=(2, 4, 10)).astype(np.float32)
    ref = np.mean(X, axis=tuple(axes), keepdims=bool(keepdims))
    assert np.allclose(po.ReduceMean(X, axes, keepdims).numpy(), ref, rtol=1e-5, atol=1e-5)


def test_sqrt_like_reference_test():
    # tests/pure_expansions/test_expansion_utils.py:9-39
    X = np.random.default_rng(6).random((2, 4), dtype=np.float32)
    assert np.allclose(po.Sqrt(X).numpy(), np.sqrt(X))


@pytest.mark.parametrize("cin,k,cout,bias", [(1, 3, 8, True), (8, 3, 3, False), (8, 5, 3, True), (8, 4, 3, False)])
def test_conv_like_reference_test(cin, k, cout, bias):
    # tests/pure_expansions/test_conv_expansion.py:9-66  batch 8, 32x32, stride 1, no padding.
    # The reference compares with np.allclose defaults on rand() data, which the fp32 summation
    # order of any implementation only meets up to ~1e-6; rtol 1e-5 + atol 1e-6 is used here.
    rng = np.random.default_rng(7)
    X = rng.random((8, cin, 32, 32), dtype=np.float32)
    W = rng.random((cout, cin, k, k), dtype=np.float32)
    B = rng.random(cout, dtype=np.float32) if bias else None
    ref = torch.nn.functional.conv2d(torch.tensor(X), torch.tensor(W), None if B is None else torch.tensor(B))
    assert np.allclose(po.Conv(X, W, B).numpy(), ref.numpy(), rtol=1e-5, atol=1e-5)


def test_conv_padded_is_pad_then_conv():
    # daceml/transformation/pad_conv_fusion.py:77-95 treats Pad + Conv(pads=0) as Conv(pads=p).
    rng = np.random.default_rng(8)
    X = rng.random((2, 16, 9, 9), dtype=np.float32)
    W = (rng.random((4, 16, 3, 3), dtype=np.float32) - 0.5) / 12
    B = rng.random(4, dtype=np.float32)
    ref = torch.nn.functional.conv2d(torch.tensor(X), torch.tensor(W), torch.tensor(B), padding=1)
    assert np.allclose(po.Conv(X, W, B, pads=(1, 1, 1, 1)).numpy(), ref.numpy(), rtol=1e-5, atol=1e-6)


def test_gemm_is_linear():
    rng = np.random.default_rng(9)
    A, W, C = rng.random((5, 7), dtype=np.float32), rng.random((3, 7), dtype=np.float32), rng.random(3, dtype=np.float32)
    ref = torch.nn.functional.linear(torch.tensor(A), torch.tensor(W), torch.tensor(C)).numpy()
    assert np.allclose(po.Gemm(A, W, C).numpy(), ref, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        po.Gemm(A, W, C, transB=0)  # PureGemm.forward_can_be_applied, pure_implementations.py:438


def test_layernorm_and_gelu_chains_match_torch():
    # tests/autodiff/pytorch/test_pytorch.py:106-139 exercises nn.LayerNorm through the same chain.
    g = torch.Generator().manual_seed(10)
    x = torch.randn(4, 7, 768, generator=g)
    gamma, beta = torch.randn(768, generator=g), torch.randn(768, generator=g)
    ref = torch.nn.functional.layer_norm(x, (768,), gamma, beta, eps=1e-12)
    assert torch.allclose(po.LayerNormChain(x, gamma, beta, 1e-12), ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(po.GeluChain(x), torch.nn.functional.gelu(x), rtol=1e-5, atol=1e-6)


def test_bert_layer_matches_transformers_bertlayer():
    # tests/pytorch/test_bert_encoder.py:10-34: BertLayer(BertConfig()), seq 512, hidden 768,
    # rtol 1e-5 / atol 1e-4 (batch reduced from 8 to 1 to keep the CPU suite short).
    from transformers import BertConfig
    from transformers.models.bert.modeling_bert import BertLayer
    torch.manual_seed(0)
    cfg = BertConfig()
    cfg._attn_implementation = "eager"
    layer = BertLayer(cfg).eval()
    sd = layer.state_dict()
    p = dict(wq=sd["attention.self.query.weight"], bq=sd["attention.self.query.bias"],
             wk=sd["attention.self.key.weight"], bk=sd["attention.self.key.bias"],
             wv=sd["attention.self.value.weight"], bv=sd["attention.self.value.bias"],
             wo=sd["attention.output.dense.weight"], bo=sd["attention.output.dense.bias"],
             ln1_g=sd["attention.output.LayerNorm.weight"], ln1_b=sd["attention.output.LayerNorm.bias"],
             wi=sd["intermediate.dense.weight"], bi=sd["intermediate.dense.bias"],
             wo2=sd["output.dense.weight"], bo2=sd["output.dense.bias"],
             ln2_g=sd["output.LayerNorm.weight"], ln2_b=sd["output.LayerNorm.bias"])
    x = torch.randn(1, 512, 768)
    with torch.no_grad():
        ref = layer(x)
    ref = ref[0] if isinstance(ref, (tuple, list)) else ref
    assert torch.allclose(po.bert_layer_forward(x, p, heads=12), ref, rtol=1e-5, atol=1e-4)


def test_mlp_and_conv_stack_match_torch_modules():
    params = po.make_mlp_params(0)
    x = torch.randn(16, 784, generator=torch.Generator().manual_seed(1))
    h = x
    for i, (w, b) in enumerate(params):
        h = torch.nn.functional.linear(h, w, b)
        if i < 2:
            h = torch.relu(h)
    ref = torch.log_softmax(h, dim=1)
    assert torch.allclose(po.mlp_forward(x, params), ref, rtol=1e-5, atol=1e-5)
    cp = po.make_conv_params(0, channels=8)
    xc = torch.rand(2, 8, 10, 10, generator=torch.Generator().manual_seed(2))
    h = xc
    for w, b in cp:
        h = torch.relu(torch.nn.functional.conv2d(h, w, b, padding=1))
    assert torch.allclose(po.conv_stack_forward(xc, cp), h, rtol=1e-5, atol=1e-6)


# ---- the committed golden vectors are what this oracle produces --------------------------------
@pytest.mark.parametrize("name", golden_names("softmax_"))
def test_golden_softmax(name):
    g = golden(name)
    assert np.allclose(po.Softmax(g["x"], int(g["axis"])).numpy(), g["y"], rtol=1e-6, atol=1e-7)
    assert np.allclose(po.LogSoftmax(g["x"], int(g["axis"])).numpy(), g["ylog"], rtol=1e-6, atol=1e-6)
    # independent float64 check of the vectors themselves
    x = g["x"].astype(np.float64)
    e = np.exp(x - x.max(axis=int(g["axis"]), keepdims=True))
    assert np.allclose(g["y"], e / e.sum(axis=int(g["axis"]), keepdims=True), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("name", golden_names("layernorm_"))
def test_golden_layernorm(name):
    g = golden(name)
    assert np.allclose(po.LayerNormChain(g["x"], g["gamma"], g["beta"], g["eps"]).numpy(), g["y"], rtol=1e-6, atol=1e-6)
    x = g["x"].astype(np.float64)
    mu = x.mean(-1, keepdims=True)
    ref = (x - mu) / np.sqrt(((x - mu) ** 2).mean(-1, keepdims=True) + 1e-12) * g["gamma"] + g["beta"]
    assert np.allclose(g["y"], ref, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", golden_names("matmul_"))
def test_golden_matmul(name):
    g = golden(name)
    assert np.allclose(po.MatMul(g["A"], g["B"]).numpy(), g["Y"], rtol=1e-5, atol=1e-6)
    assert np.allclose(g["Y"], np.matmul(g["A"].astype(np.float64), g["B"].astype(np.float64)), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", golden_names("gemm_"))
def test_golden_gemm(name):
    g = golden(name)
    ref = g["A"].astype(np.float64) @ g["B"].astype(np.float64).T + g["C"]
    assert np.allclose(g["Y"], ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", golden_names("conv_"))
def test_golden_conv(name):
    g = golden(name)
    B = torch.tensor(g["B"]) if "B" in g else None
    pad = int(g["pad"])
    ref = torch.nn.functional.conv2d(torch.tensor(g["X"]).double(), torch.tensor(g["W"]).double(),
                                     None if B is None else B.double(), padding=pad)
    assert np.allclose(g["Y"], ref.numpy(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("kernel,stride,shape", [((2, 2), (2, 2), (8, 6, 30, 30)), ((3, 3), (1, 1), (2, 3, 9, 11)),
                                                 ((2, 3), (3, 2), (1, 4, 17, 13))])
def test_maxpool_matches_torch(kernel, stride, shape):
    """PureMaxPool2D (pads 0, floor mode); the reference pins it through its LeNet test
    (tests/pytorch/test_lenet.py:14-54) against F.max_pool2d."""
    x = torch.randn(*shape, generator=torch.Generator().manual_seed(40))
    assert torch.equal(po.MaxPool(x, kernel, stride), torch.nn.functional.max_pool2d(x, kernel, stride))
