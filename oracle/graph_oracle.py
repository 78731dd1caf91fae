"""CPU oracle for whole exported graphs: every ONNX node evaluated on its own, in graph order, with the
restated pure expansions of `pure_oracle` - what the reference does when it imports a model and expands each
node with its `pure` implementation (daceml/onnx/onnx_importer.py:95-300, onnx_op.py:646-684), with no fusion.

TEST INFRASTRUCTURE ONLY (same rule as pure_oracle): used by tests/ as the checker of the fused GPU executor.
It shares the host-side protobuf reader and shape / constant folding with the package (those move no
activations); the arithmetic on activations is pure_oracle's. Parity against the reference executed here is
unpinned; the committed fixtures additionally hold the exporting torch module's own output.
"""
import numpy as np
import torch

from dace_onnx_b200 import onnx_wire
from dace_onnx_b200.onnx_graph import specialize

from . import pure_oracle as po

_BINARY = {"Add": po.Add, "Sub": po.Sub, "Mul": po.Mul, "Div": po.Div, "Pow": po.Pow}
_UNARY = {"Sqrt": po.Sqrt, "Erf": po.Erf, "Relu": po.Relu, "Identity": lambda x: x, "Dropout": lambda x: x}


def run(model, inputs):
    """model: bytes / path / onnx_wire.Model; inputs: list of CPU tensors or arrays. Returns a list of tensors."""
    if isinstance(model, (bytes, bytearray)):
        model = onnx_wire.parse_model(model)
    elif not isinstance(model, onnx_wire.Model):
        model = onnx_wire.load_model(model)
    inputs = [po._t(x) for x in inputs]
    ir = specialize(model, [tuple(t.shape) for t in inputs])
    env = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in ir.consts.items()}
    env.update(dict(zip(ir.inputs, inputs)))
    for n in ir.nodes:
        i = [env[x] if x else None for x in n.inputs]
        op = n.op_type
        if op in _BINARY:
            y = _BINARY[op](i[0], i[1])
        elif op in _UNARY:
            y = _UNARY[op](i[0])
        elif op == "MatMul":
            y = po.MatMul(i[0], i[1])
        elif op == "Gemm":
            y = po.Gemm(i[0], i[1], i[2] if len(i) > 2 else None, n.attr("alpha", 1.0), n.attr("beta", 1.0),
                        n.attr("transA", 0), n.attr("transB", 0))
        elif op == "Conv":
            y = po.Conv(i[0], i[1], i[2] if len(i) > 2 else None, tuple(n.attr("pads", [0, 0, 0, 0])),
                        tuple(n.attr("strides", [1, 1])))
        elif op == "MaxPool":
            y = po.MaxPool(i[0], n.attr("kernel_shape"), n.attr("strides") or [1, 1])
        elif op == "Softmax":
            y = po.Softmax(i[0], n.attr("axis", 1))
        elif op == "LogSoftmax":
            y = po.LogSoftmax(i[0], n.attr("axis", 1))
        elif op == "ReduceMean":
            y = po.ReduceMean(i[0], n.attr("axes") or list(range(i[0].dim())), n.attr("keepdims", 1))
        elif op == "Transpose":
            y = i[0].permute(*(n.attr("perm") or list(range(i[0].dim()))[::-1])).contiguous()
        elif op in ("Reshape", "Flatten", "Squeeze", "Unsqueeze"):
            y = i[0].reshape(ir.shapes[n.outputs[0]])
        else:
            raise NotImplementedError(op)
        env[n.outputs[0]] = y
    return [env[o] for o in ir.outputs]
