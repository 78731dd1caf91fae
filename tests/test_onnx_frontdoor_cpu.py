"""Host side of the ONNX front door: protobuf reader, shape / constant folding, fusion passes, and the
graph oracle against the exporting torch modules' own outputs (no GPU needed)."""
import os

import numpy as np
import pytest
import torch

from tests._util import GOLDEN, REF_ATOL, REF_RTOL, close, golden
from dace_onnx_b200 import fusion, onnx_wire
from dace_onnx_b200.onnx_graph import GraphIR, UnsupportedNode, specialize
from dace_onnx_b200.onnx_model import clean_name
from dace_onnx_b200.onnx_wire import Node
from oracle import graph_oracle
from oracle import pure_oracle as po

CASES = ["mlp", "conv_stack", "norm_acts", "bert_layer", "bert_layer_nofold"]


def _load(name):
    return onnx_wire.load_model(os.path.join(GOLDEN, name + ".onnx"))


def test_reader_decodes_the_exported_models():
    m = _load("bert_layer")
    assert m.opset == 12 and m.producer == "pytorch"
    assert [(vi.shape, vi.dtype) for vi in m.graph.inputs] == [((2, 32, 128), np.float32)]
    assert [vi.shape for vi in m.graph.outputs] == [(2, 32, 128)]
    ops_seen = {n.op_type for n in m.graph.nodes}
    assert {"MatMul", "Add", "Softmax", "Erf", "ReduceMean", "Pow", "Sqrt", "Div", "Transpose"} <= ops_seen
    w = [a for a in m.graph.initializers.values() if a.shape == (128, 256)]
    assert len(w) == 1 and w[0].dtype == np.float32 and np.isfinite(w[0]).all()
    sm = next(n for n in m.graph.nodes if n.op_type == "Softmax")
    assert sm.attr("axis") == 3
    perms = sorted(tuple(n.attr("perm")) for n in m.graph.nodes if n.op_type == "Transpose")
    assert perms == [(0, 2, 1, 3)] * 3 + [(0, 2, 3, 1)]
    conv = next(n for n in _load("conv_stack").graph.nodes if n.op_type == "Conv")
    assert conv.attr("pads") == [1, 1, 1, 1] and conv.attr("kernel_shape") == [3, 3] and conv.attr("group") == 1


def test_reader_rejects_damaged_input():
    with open(os.path.join(GOLDEN, "norm_acts.onnx"), "rb") as fh:
        data = fh.read()
    with pytest.raises(onnx_wire.OnnxFormatError):
        onnx_wire.parse_model(data[:len(data) // 2])
    with pytest.raises(onnx_wire.OnnxFormatError):
        onnx_wire.parse_model(b"")


@pytest.mark.parametrize("name", CASES)
def test_graph_oracle_matches_the_exporting_module(name):
    """Pins the node-by-node oracle on real exported graphs with the reference's comparator
    (daceml/testing/utils.py:6, as tests/pytorch/test_bert_encoder.py:34 uses it)."""
    g = golden("onnx_" + name)
    y = graph_oracle.run(_load(name), [g["x"]])[0]
    close(y, g["y"], rtol=REF_RTOL, atol=REF_ATOL)


def test_bert_layer_collapses_to_six_fused_nodes():
    for name in ("bert_layer", "bert_layer_nofold"):
        ir = specialize(_load(name), [(2, 32, 128)])
        assert sum(ir.op_histogram().values()) == 49
        stats = fusion.run_all(ir)
        assert stats == {"layernorm": 2, "gelu": 1, "attention": 1, "transposes": 0, "gemm_epilogues": 3,
                         "conv_relu": 0}
        assert ir.op_histogram() == {"B200SelfAttention": 1, "B200Gemm": 3, "B200LayerNorm": 2}
        epis = [n.attr("epilogue") for n in ir.nodes if n.op_type == "B200Gemm"]
        assert epis == ["bias_residual", "bias_gelu", "bias_residual"]
        at = next(n for n in ir.nodes if n.op_type == "B200SelfAttention")
        assert at.attr("heads") == 2 and at.attr("scale") == 0.125 and len(at.inputs) == 7
        ln = [n for n in ir.nodes if n.op_type == "B200LayerNorm"]
        assert all(abs(n.attr("epsilon") - 1e-12) < 1e-18 and n.inputs[1] and n.inputs[2] for n in ln)
        # the rewritten list is still in dependency order
        seen = set(ir.inputs) | set(ir.consts)
        for n in ir.nodes:
            assert all((not i) or i in seen for i in n.inputs), n.name
            seen.update(n.outputs)
        assert ir.outputs[0] in seen


def test_other_models_fuse_as_expected():
    ir = specialize(_load("mlp"), [(32, 96)])
    fusion.run_all(ir)
    assert [(n.op_type, n.attr("epilogue"), n.attr("trans_b")) for n in ir.nodes] == [
        ("B200Gemm", "bias_relu", 1), ("B200Gemm", "bias_relu", 1), ("B200Gemm", "bias", 1), ("LogSoftmax", None, None)]
    ir = specialize(_load("conv_stack"), [(2, 16, 12, 12)])
    fusion.run_all(ir)
    assert [(n.op_type, n.attr("relu")) for n in ir.nodes] == [("Conv", 1), ("Conv", 1)]
    ir = specialize(_load("norm_acts"), [(3, 20, 48)])
    fusion.run_all(ir)
    assert [n.op_type for n in ir.nodes] == ["B200LayerNorm", "B200Gelu", "Transpose", "Softmax"]
    ln = ir.nodes[0]
    assert ln.inputs[1] == "" and ln.inputs[2] == "" and abs(ln.attr("epsilon") - 1e-5) < 1e-9


def test_specialize_checks_input_shapes_and_operators():
    with pytest.raises(ValueError):
        specialize(_load("mlp"), [(16, 96)])      # the graph was exported for batch 32
    with pytest.raises(ValueError):
        specialize(_load("mlp"), [(32, 96), (1,)])
    m = _load("norm_acts")
    m.graph.nodes[-1].op_type = "Hardmax"
    with pytest.raises(UnsupportedNode):
        specialize(m, [(3, 20, 48)])


def _chain_graph(extra_consumer):
    """x -> Div(sqrt2) -> Erf -> Add 1 -> Mul x -> Mul 0.5, optionally with a second reader of the Erf output."""
    ir = GraphIR("g", ["x"], ["y"] + (["z"] if extra_consumer else []))
    ir.shapes = {"x": (4, 8)}
    ir.consts = {"c2": np.float32(np.sqrt(2.0)).reshape(()), "c1": np.ones((), np.float32),
                 "ch": np.full((), 0.5, np.float32)}
    ir.nodes = [Node("Div", "d", ["x", "c2"], ["t0"]), Node("Erf", "e", ["t0"], ["t1"]),
                Node("Add", "a", ["t1", "c1"], ["t2"]), Node("Mul", "m1", ["x", "t2"], ["t3"]),
                Node("Mul", "m2", ["t3", "ch"], ["y"])]
    if extra_consumer:
        ir.nodes.append(Node("Relu", "r", ["t1"], ["z"]))
    for n in ir.nodes:
        ir.shapes[n.outputs[0]] = (4, 8)
    return ir


def test_patterns_do_not_fire_when_an_intermediate_is_read_elsewhere():
    ir = _chain_graph(False)
    assert fusion.fuse_gelu(ir) == 1 and [n.op_type for n in ir.nodes] == ["B200Gelu"]
    ir = _chain_graph(True)
    assert fusion.fuse_gelu(ir) == 0 and len(ir.nodes) == 6
    # an intermediate that is itself a graph output blocks the rewrite too
    ir = _chain_graph(False)
    ir.outputs.append("t3")
    assert fusion.fuse_gelu(ir) == 0


def test_transpose_into_trans_b_and_scale_epilogue():
    ir = GraphIR("g", ["q", "k"], ["s"])
    ir.shapes = {"q": (2, 4, 16, 8), "k": (2, 16, 4, 8), "kt": (2, 4, 8, 16), "qk": (2, 4, 16, 16), "s": (2, 4, 16, 16)}
    ir.consts = {"c": np.full((), 0.25, np.float32)}
    ir.nodes = [Node("Transpose", "t", ["k"], ["kt"], {"perm": [0, 2, 3, 1]}), Node("MatMul", "m", ["q", "kt"], ["qk"]),
                Node("Mul", "sc", ["qk", "c"], ["s"])]
    assert fusion.fold_transposes(ir) == 1
    assert ir.nodes[0].attr("perm") == [0, 2, 1, 3] and ir.shapes["kt"] == (2, 4, 16, 8)
    assert ir.nodes[1].attr("trans_b") == 1
    assert fusion.fuse_gemm_epilogues(ir) == 1
    g = ir.nodes[-1]
    assert (g.op_type, g.attr("epilogue"), g.attr("scale"), g.attr("trans_b"), g.outputs) == \
        ("B200Gemm", "scale", 0.25, 1, ["s"])
    # a plain swap of the last two axes disappears altogether
    ir = GraphIR("g", ["a", "b"], ["y"])
    ir.shapes = {"a": (8, 4), "b": (6, 4), "bt": (4, 6), "y": (8, 6)}
    ir.nodes = [Node("Transpose", "t", ["b"], ["bt"], {"perm": [1, 0]}), Node("MatMul", "m", ["a", "bt"], ["y"])]
    assert fusion.fold_transposes(ir) == 1
    assert [n.op_type for n in ir.nodes] == ["MatMul"] and ir.nodes[0].inputs == ["a", "b"]


def test_constant_glue_is_folded_on_the_host():
    """Shape -> Gather -> Unsqueeze -> Concat -> Reshape, the exporter's idiom for x.view(x.size(0), -1)."""
    g = onnx_wire.Graph("g", [
        Node("Shape", "s", ["x"], ["sh"]),
        Node("Constant", "c0", [], ["i0"], {"value": np.asarray(0, dtype=np.int64)}),
        Node("Gather", "g", ["sh", "i0"], ["b"], {"axis": 0}),
        Node("Unsqueeze", "u", ["b"], ["b1"], {"axes": [0]}),
        Node("Constant", "c1", [], ["m1"], {"value": np.asarray([-1], dtype=np.int64)}),
        Node("Concat", "cc", ["b1", "m1"], ["tgt"], {"axis": 0}),
        Node("Reshape", "r", ["x", "tgt"], ["y"]),
        Node("Relu", "act", ["y"], ["z"]),
    ], {}, [onnx_wire.ValueInfo("x", np.float32, (None, 3, 5))], [onnx_wire.ValueInfo("z", np.float32, None)])
    ir = specialize(onnx_wire.Model(g, 12), [(7, 3, 5)])
    assert [n.op_type for n in ir.nodes] == ["Reshape", "Relu"]
    assert ir.shapes["y"] == (7, 15) and ir.shapes["z"] == (7, 15)
    assert ir.consts["tgt"].tolist() == [7, -1]


def test_clean_name():
    assert clean_name("onnx::MatMul_0") == "onnx__MatMul_0"
    assert clean_name("102") == "ONNX_102"
    assert clean_name("/attention/self/Mul_output_0") == "_attention_self_Mul_output_0"


def test_graph_oracle_is_unfused():
    """The checker evaluates exported nodes one by one: it must not see any fused node type."""
    ir = specialize(_load("bert_layer"), [(2, 32, 128)])
    assert not any(n.op_type.startswith("B200") for n in ir.nodes)
    x = torch.from_numpy(golden("onnx_bert_layer")["x"])
    y1 = graph_oracle.run(_load("bert_layer"), [x])[0]
    y2 = graph_oracle.run(_load("bert_layer_nofold"), [x])[0]
    assert y1.shape == y2.shape == (2, 32, 128)


def _tiny_model(nodes, opset, inits=None, in_shape=(2, 3, 4), out="y"):
    from dace_onnx_b200.onnx_wire import Graph, Model, ValueInfo
    return Model(Graph("g", nodes, dict(inits or {}), [ValueInfo("x", np.float32, in_shape)],
                       [ValueInfo(out, np.float32, None)]), opset)


def test_newer_opsets_are_rewritten_or_refused():
    """Nodes whose definition changed after opset 12 either run with their own opset's meaning or are refused
    when the plan is built; none is silently evaluated with opset-12 defaults."""
    x = np.random.default_rng(3).standard_normal((2, 3, 4)).astype(np.float32)
    # Softmax / LogSoftmax without an axis attribute: axis 1 up to opset 12, the last axis from opset 13 on
    for op, fn in (("Softmax", po.Softmax), ("LogSoftmax", po.LogSoftmax)):
        for opset, axis in ((12, 1), (11, 1), (13, -1), (17, -1)):
            m = _tiny_model([Node(op, "s", ["x"], ["y"])], opset)
            ir = specialize(m, [(2, 3, 4)])
            assert ir.nodes[0].attr("axis") == axis
            np.testing.assert_allclose(graph_oracle.run(m, [x])[0].numpy(), fn(x, axis).numpy(), rtol=1e-6)
        m = _tiny_model([Node(op, "s", ["x"], ["y"], {"axis": 0})], 13)      # an explicit axis is kept
        assert specialize(m, [(2, 3, 4)]).nodes[0].attr("axis") == 0
    # ReduceMean with axes as an input (opset 18): constant axes become the attribute
    m = _tiny_model([Node("ReduceMean", "r", ["x", "ax"], ["y"], {"keepdims": 1})], 18, {"ax": np.asarray([-1], np.int64)})
    ir = specialize(m, [(2, 3, 4)])
    assert ir.nodes[0].attr("axes") == [-1] and ir.nodes[0].inputs == ["x"] and ir.shapes["y"] == (2, 3, 1)
    np.testing.assert_allclose(graph_oracle.run(m, [x])[0].numpy(), x.mean(-1, keepdims=True), rtol=1e-6)
    # empty constant axes = reduce over everything; with noop_with_empty_axes it is refused
    m = _tiny_model([Node("ReduceMean", "r", ["x", "ax"], ["y"], {"keepdims": 0})], 18, {"ax": np.zeros(0, np.int64)})
    assert specialize(m, [(2, 3, 4)]).shapes["y"] == ()
    m = _tiny_model([Node("ReduceMean", "r", ["x", "ax"], ["y"], {"noop_with_empty_axes": 1})], 18,
                    {"ax": np.zeros(0, np.int64)})
    with pytest.raises(UnsupportedNode):
        specialize(m, [(2, 3, 4)])
    # runtime axes cannot be planned
    from dace_onnx_b200.onnx_wire import ValueInfo
    m = _tiny_model([Node("ReduceMean", "r", ["x", "ax"], ["y"])], 18)
    m.graph.inputs.append(ValueInfo("ax", np.int64, (1,)))
    with pytest.raises(UnsupportedNode, match="runtime tensor"):
        specialize(m, [(2, 3, 4), (1,)])
    # Squeeze / Unsqueeze with axes as an input (opset 13)
    m = _tiny_model([Node("Unsqueeze", "u", ["x", "ax"], ["t"]), Node("Squeeze", "q", ["t", "ax"], ["s"]),
                     Node("Relu", "r", ["s"], ["y"])], 13, {"ax": np.asarray([1], np.int64)})
    ir = specialize(m, [(2, 3, 4)])
    assert ir.shapes["t"] == (2, 1, 3, 4) and ir.shapes["s"] == (2, 3, 4)
    np.testing.assert_array_equal(graph_oracle.run(m, [x])[0].numpy(), np.maximum(x, 0))
    m = _tiny_model([Node("Unsqueeze", "u", ["x", "ax"], ["y"])], 13)
    m.graph.inputs.append(ValueInfo("ax", np.int64, (1,)))
    with pytest.raises(UnsupportedNode):
        specialize(m, [(2, 3, 4), (1,)])
    m = _tiny_model([Node("Unsqueeze", "u", ["x"], ["y"])], 13)              # neither attribute nor input
    with pytest.raises(UnsupportedNode):
        specialize(m, [(2, 3, 4)])
