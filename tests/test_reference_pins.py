"""tests/golden/ref_pins.npz holds vectors computed by the reference's own source
(daceml/onnx/op_implementations/pure_implementations.py loaded unmodified and executed with numpy
semantics by tests/golden/make_reference_pins.py). The CPU tests pin the oracle to them; the GPU
tests compare the C-ABI kernels with them directly, oracle not involved."""
import numpy as np
import pytest
import torch

from oracle import pure_oracle as po
from tests._util import ATOL, RTOL, close, dev, golden

PINS = golden("ref_pins")
TAGS = sorted({k.split(".")[0] for k in PINS})


def _case(tag):
    ins = {k.split(".", 1)[1]: v for k, v in PINS.items() if k.startswith(tag + ".") and ".attr." not in k}
    attrs = {k.split(".attr.")[1]: v for k, v in PINS.items() if k.startswith(tag + ".attr.")}
    out = ins.pop("out")
    return ins, attrs, out


def _kind(tag):
    for p in ("add", "sub", "mul", "div", "pow", "sqrt", "erf", "relu", "mean", "softmax", "logsoftmax", "matmul",
              "gemm", "ln", "gelu", "attn"):
        if tag.startswith(p + "_") or tag == p:
            return p
    raise KeyError(tag)


BINARY = {"add": "Add", "sub": "Sub", "mul": "Mul", "div": "Div"}


def _oracle(tag):
    ins, attrs, _ = _case(tag)
    k = _kind(tag)
    if k in BINARY:
        return getattr(po, BINARY[k])(ins["A"], ins["B"])
    if k == "pow":
        return po.Pow(ins["X"], ins["Y"])
    if k == "sqrt":
        return po.Sqrt(ins["X"])
    if k == "erf":
        return po.Erf(ins["input"])
    if k == "relu":
        return po.Relu(ins["X"])
    if k == "mean":
        return po.ReduceMean(ins["data"], [int(a) for a in attrs["axes"]], int(attrs["keepdims"]))
    if k == "softmax":
        return po.Softmax(ins["input"], int(attrs["axis"]))
    if k == "logsoftmax":
        return po.LogSoftmax(ins["input"], int(attrs["axis"]))
    if k == "matmul":
        return po.MatMul(ins["A"], ins["B"])
    if k == "gemm":
        return po.Gemm(ins["A"], ins["B"], ins.get("C"))
    if k == "ln":
        return po.LayerNormChain(ins["x"], ins["gamma"], ins["beta"], ins["eps"])
    if k == "gelu":
        return po.GeluChain(ins["x"])
    if k == "attn":
        s = po.Mul(po.MatMul(ins["q"], ins["kt"]), np.float32(0.125))
        return po.MatMul(po.Softmax(s, 3), ins["v"])
    raise KeyError(tag)


def test_every_hot_path_node_is_pinned():
    kinds = {_kind(t) for t in TAGS}
    assert kinds == {"add", "sub", "mul", "div", "pow", "sqrt", "erf", "relu", "mean", "softmax", "logsoftmax",
                     "matmul", "gemm", "ln", "gelu", "attn"}


@pytest.mark.parametrize("tag", TAGS)
def test_oracle_matches_reference_source(tag):
    """The restatement against the reference's statements: elementwise nodes bit for bit, reductions and
    contractions within accumulation-order noise (far inside the fp32 parity bar)."""
    _, _, ref = _case(tag)
    got = _oracle(tag).numpy()
    assert got.shape == ref.shape
    if _kind(tag) in ("add", "sub", "mul", "div", "sqrt", "relu"):
        assert np.array_equal(got, ref)
    else:
        close(got, ref, rtol=2e-6, atol=2e-6)


# ---------------------------------------------------------------------------------------------
# the CUDA kernels against the same vectors
# ---------------------------------------------------------------------------------------------
def _cuda(tag):
    from dace_onnx_b200 import ops
    ins, attrs, _ = _case(tag)
    k = _kind(tag)
    d = {n: dev(v) for n, v in ins.items()}
    if k in BINARY:
        return getattr(ops, k)(d["A"], d["B"])
    if k == "pow":
        return ops.pow(d["X"], d["Y"])
    if k == "sqrt":
        return ops.sqrt(d["X"])
    if k == "erf":
        return ops.erf(d["input"])
    if k == "relu":
        return ops.relu(d["X"])
    if k == "mean":
        return ops.reduce_mean(d["data"], [int(a) for a in attrs["axes"]], int(attrs["keepdims"]))
    if k == "softmax":
        return ops.softmax(d["input"], int(attrs["axis"]))
    if k == "logsoftmax":
        return ops.logsoftmax(d["input"], int(attrs["axis"]))
    if k == "matmul":
        return ops.matmul(d["A"], d["B"])
    if k == "gemm":
        return ops.gemm(d["A"], d["B"], d.get("C"))
    if k == "ln":
        return ops.layernorm(d["x"], d["gamma"], d["beta"], float(ins["eps"]))
    if k == "gelu":
        return ops.gelu(d["x"])
    if k == "attn":
        s = ops.matmul(d["q"], d["kt"], epilogue=ops.EPI_SCALE, scale=0.125)
        return ops.matmul(ops.softmax(s, 3), d["v"])
    raise KeyError(tag)


@pytest.mark.gpu
@pytest.mark.parametrize("tag", TAGS)
def test_kernels_match_reference_source(tag, cuda):
    """C-ABI results (default fp32-accurate mode) against the vectors the reference's source produced."""
    _, _, ref = _case(tag)
    got = _cuda(tag)
    close(got, ref, rtol=RTOL, atol=ATOL)


@pytest.mark.gpu
def test_fused_attention_matches_reference_source(cuda):
    """The fused TF32 attention kernel against the reference's MatMul-Mul-Softmax-MatMul vectors."""
    from dace_onnx_b200 import ops
    from tests._util import TF32_ATOL, TF32_RTOL
    ins, _, ref = _case("attn")
    q = dev(ins["q"]).permute(0, 2, 1, 3).contiguous()            # [b, s, h, d]
    k = dev(ins["kt"]).permute(0, 3, 1, 2).contiguous()           # kt is [b, h, d, s]
    v = dev(ins["v"]).permute(0, 2, 1, 3).contiguous()
    out = torch.empty_like(q)
    assert ops.attention_views(q, k, v, out, 0.125, math_mode="tf32") is True
    close(out.permute(0, 2, 1, 3), ref, rtol=TF32_RTOL, atol=TF32_ATOL)
