"""Graph form of an imported ONNX model, specialised to concrete input shapes.

`specialize()` does at load time what the reference importer does before expansion
(daceml/onnx/onnx_importer.py:95-300: shape inference, then constant folding of everything that does
not depend on a runtime tensor, daceml/transformation/constant_folding.py): every value gets a static
shape, `Constant` / `Shape` / `Gather` / `Concat` ... glue and any node fed only by initializers is
evaluated once on the host with numpy, and what remains is the list of nodes that touch runtime
tensors. Host-only code; nothing here computes on activations.
"""
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .onnx_wire import Graph, Model, Node


class UnsupportedNode(NotImplementedError):
    """A node outside the set this library implements (there is no fallback runtime to hand it to)."""


class GraphIR:
    def __init__(self, name: str, inputs: List[str], outputs: List[str]):
        self.name = name
        self.inputs = inputs
        self.outputs = outputs
        self.nodes: List[Node] = []
        self.consts: Dict[str, np.ndarray] = {}
        self.shapes: Dict[str, Tuple[int, ...]] = {}

    # -- structure queries used by the fusion passes -------------------------------------------------
    def producers(self) -> Dict[str, Node]:
        return {o: n for n in self.nodes for o in n.outputs if o}

    def consumers(self) -> Dict[str, List[Node]]:
        cons: Dict[str, List[Node]] = {}
        for n in self.nodes:
            for i in n.inputs:
                if i:
                    cons.setdefault(i, []).append(n)
        return cons

    def op_histogram(self) -> Dict[str, int]:
        h: Dict[str, int] = {}
        for n in self.nodes:
            h[n.op_type] = h.get(n.op_type, 0) + 1
        return h

    def replace(self, removed: Sequence[Node], new_node: Node):
        """Put new_node where the last of `removed` stood and drop the rest (keeps the list topological:
        all inputs of the pattern are produced before its last node, all consumers come after it)."""
        ids = {id(n) for n in removed}
        last = max(i for i, n in enumerate(self.nodes) if id(n) in ids)
        out = []
        for i, n in enumerate(self.nodes):
            if i == last:
                out.append(new_node)
            elif id(n) not in ids:
                out.append(n)
        self.nodes = out


# ---------------------------------------------------------------------------------------------------
# host evaluation of constant sub-graphs (numpy; ONNX opset-12 semantics of the glue operators)
# ---------------------------------------------------------------------------------------------------
def _axes(node, rank, default=None):
    axes = node.attr("axes", default)
    return None if axes is None else [a % rank for a in axes]


def _reshape_target(shape_in, target):
    target = [int(t) for t in target]
    out = [shape_in[i] if t == 0 else t for i, t in enumerate(target)]
    if -1 in out:
        known = 1
        for t in out:
            if t != -1:
                known *= t
        total = int(np.prod(shape_in)) if len(shape_in) else 1
        out[out.index(-1)] = total // known if known else 0
    return tuple(out)


def _host_eval(node: Node, ins: List[Optional[np.ndarray]]):
    op = node.op_type
    if op in ("Identity", "Dropout"):
        return ins[0]
    if op == "Cast":
        to = {1: np.float32, 6: np.int32, 7: np.int64, 9: np.bool_, 11: np.float64, 10: np.float16}[node.attr("to")]
        return ins[0].astype(to)
    if op == "Gather":
        return np.take(ins[0], ins[1].astype(np.int64), axis=node.attr("axis", 0))
    if op == "Unsqueeze":
        out = ins[0]
        for a in sorted(node.attr("axes")):
            out = np.expand_dims(out, a)
        return out
    if op == "Squeeze":
        axes = node.attr("axes")
        return np.squeeze(ins[0], axis=tuple(axes) if axes is not None else None)
    if op == "Concat":
        return np.concatenate(ins, axis=node.attr("axis"))
    if op == "Reshape":
        return ins[0].reshape(_reshape_target(ins[0].shape, ins[1]))
    if op == "Flatten":
        ax = node.attr("axis", 1)
        return ins[0].reshape(int(np.prod(ins[0].shape[:ax], dtype=np.int64)), -1)
    if op == "Transpose":
        return np.ascontiguousarray(np.transpose(ins[0], node.attr("perm")))
    if op == "Slice":
        data, starts, ends = ins[0], ins[1], ins[2]
        axes = ins[3] if len(ins) > 3 and ins[3] is not None else np.arange(len(starts))
        steps = ins[4] if len(ins) > 4 and ins[4] is not None else np.ones(len(starts), dtype=np.int64)
        sl = [slice(None)] * data.ndim
        for s, e, a, st in zip(starts, ends, axes, steps):
            sl[int(a)] = slice(int(s), int(e), int(st))
        return data[tuple(sl)]
    if op == "ConstantOfShape":
        v = node.attr("value")
        fill = v.reshape(-1)[0] if v is not None else np.float32(0)
        return np.full(tuple(int(x) for x in ins[0]), fill)
    if op in ("Add", "Sub", "Mul", "Div", "Pow"):
        a, b = ins
        if op == "Add":
            return a + b
        if op == "Sub":
            return a - b
        if op == "Mul":
            return a * b
        if op == "Pow":
            return np.power(a, b).astype(a.dtype)
        if np.issubdtype(a.dtype, np.integer):
            return (np.trunc(a / b)).astype(a.dtype)  # ONNX integer Div truncates
        return (a / b).astype(a.dtype)
    if op == "Sqrt":
        return np.sqrt(ins[0])
    if op == "Equal":
        return np.equal(ins[0], ins[1])
    if op == "Where":
        return np.where(ins[0], ins[1], ins[2])
    if op == "Expand":
        return ins[0] * np.ones(tuple(int(x) for x in ins[1]), dtype=ins[0].dtype)
    return None


# ---------------------------------------------------------------------------------------------------
# shape rules of the nodes that stay in the graph
# ---------------------------------------------------------------------------------------------------
def _bcast(a, b):
    return tuple(np.broadcast_shapes(tuple(a), tuple(b)))


def _infer(node: Node, shp, consts):
    op = node.op_type
    s = [shp(i) if i else None for i in node.inputs]
    if op in ("Softmax", "LogSoftmax", "Sqrt", "Erf", "Relu", "Identity", "Dropout"):
        return s[0]
    if op in ("Add", "Sub", "Mul", "Div", "Pow"):
        return _bcast(s[0], s[1])
    if op == "MatMul":
        a, b = s
        if len(a) < 2 or len(b) < 2:
            raise UnsupportedNode("MatMul '%s': 1-D operands are not supported" % node.name)
        if a[-1] != b[-2]:
            raise ValueError("MatMul '%s': inner dimensions differ (%s @ %s)" % (node.name, a, b))
        return _bcast(a[:-2], b[:-2]) + (a[-2], b[-1])
    if op == "Gemm":
        a, b = s[0], s[1]
        m = a[1] if node.attr("transA", 0) else a[0]
        n = b[0] if node.attr("transB", 0) else b[1]
        return (m, n)
    if op == "Conv":
        x, w = s[0], s[1]
        if len(x) != 4:
            raise UnsupportedNode("Conv '%s': only 2-D convolutions" % node.name)
        if node.attr("auto_pad", "NOTSET") != "NOTSET":
            raise UnsupportedNode("Conv '%s': auto_pad must be NOTSET" % node.name)
        pads = node.attr("pads", [0, 0, 0, 0])
        st = node.attr("strides", [1, 1])
        dil = node.attr("dilations", [1, 1])
        oh = (x[2] + pads[0] + pads[2] - dil[0] * (w[2] - 1) - 1) // st[0] + 1
        ow = (x[3] + pads[1] + pads[3] - dil[1] * (w[3] - 1) - 1) // st[1] + 1
        return (x[0], w[0], oh, ow)
    if op == "MaxPool":
        x = s[0]
        ks = node.attr("kernel_shape")
        pads = node.attr("pads") or [0] * 4
        if len(x) != 4 or ks is None or len(ks) != 2:
            raise UnsupportedNode("MaxPool '%s': only 2-D pooling of NCHW tensors" % node.name)
        if any(pads) or node.attr("ceil_mode", 0) or node.attr("auto_pad", "NOTSET") != "NOTSET" or \
                any(d != 1 for d in (node.attr("dilations") or [1, 1])) or node.attr("storage_order", 0):
            raise UnsupportedNode("MaxPool '%s': pads, ceil_mode, dilations and auto_pad are not supported "
                                  "(as in the reference's pure expansion)" % node.name)
        st = node.attr("strides") or [1, 1]
        return (x[0], x[1], (x[2] - ks[0]) // st[0] + 1, (x[3] - ks[1]) // st[1] + 1)
    if op == "ReduceMean":
        x = s[0]
        axes = _axes(node, len(x), list(range(len(x))))
        if node.attr("keepdims", 1):
            return tuple(1 if i in axes else d for i, d in enumerate(x))
        return tuple(d for i, d in enumerate(x) if i not in axes)
    if op == "Transpose":
        perm = node.attr("perm") or list(range(len(s[0])))[::-1]
        return tuple(s[0][p] for p in perm)
    if op == "Reshape":
        if node.inputs[1] not in consts:
            raise UnsupportedNode("Reshape '%s': the target shape must be a constant" % node.name)
        return _reshape_target(s[0], consts[node.inputs[1]])
    if op == "Flatten":
        ax = node.attr("axis", 1)
        return (int(np.prod(s[0][:ax], dtype=np.int64)), int(np.prod(s[0][ax:], dtype=np.int64)))
    if op == "Unsqueeze":
        out = list(s[0])
        for a in sorted(node.attr("axes")):
            out.insert(a, 1)
        return tuple(out)
    if op == "Squeeze":
        axes = _axes(node, len(s[0]))
        return tuple(d for i, d in enumerate(s[0]) if not (d == 1 and (axes is None or i in axes)))
    raise UnsupportedNode("node '%s': ONNX operator %s is not implemented by this library" % (node.name, op))


_AXES_AS_INPUT = {"ReduceMean": 18, "Squeeze": 13, "Unsqueeze": 13}  # opset from which `axes` is an input tensor


def _to_opset12_form(node: Node, opset: int, consts) -> Node:
    """Rewrites a node of a newer opset into the opset-12 form the rest of this package reads, or refuses it.

    * Softmax / LogSoftmax without an `axis` attribute: the default is 1 up to opset 12 and -1 from opset 13 on.
      (Either way `axis` is ONE numpy axis, as in the reference's pure expansions, pure_implementations.py:352-364,
      :600-614.)
    * ReduceMean (opset 18), Squeeze / Unsqueeze (opset 13): `axes` arrives as a second input. A constant one
      becomes the attribute; a runtime one cannot be planned statically and is refused."""
    op = node.op_type
    if op in ("Softmax", "LogSoftmax") and "axis" not in node.attrs:
        return Node(op, node.name, list(node.inputs), list(node.outputs), dict(node.attrs, axis=-1 if opset >= 13 else 1),
                    node.domain)
    if op in _AXES_AS_INPUT and len(node.inputs) > 1 and node.inputs[1]:
        name = node.inputs[1]
        if name not in consts:
            raise UnsupportedNode("%s '%s': `axes` is a runtime tensor (opset >= %d form); only constant axes can "
                                  "be planned" % (op, node.name, _AXES_AS_INPUT[op]))
        axes = [int(a) for a in np.asarray(consts[name]).reshape(-1)]
        attrs = dict(node.attrs)
        if not axes:
            if op == "ReduceMean" and attrs.get("noop_with_empty_axes", 0):
                raise UnsupportedNode("ReduceMean '%s': noop_with_empty_axes is not supported" % node.name)
            axes = None  # empty axes: reduce / squeeze over everything, the attribute-less meaning
        if axes is not None:
            attrs["axes"] = axes
        return Node(op, node.name, [node.inputs[0]], list(node.outputs), attrs, node.domain)
    if op == "Unsqueeze" and node.attrs.get("axes") is None:
        raise UnsupportedNode("Unsqueeze '%s' has no axes" % node.name)
    return node


def specialize(model: Model, input_shapes: Sequence[Sequence[int]]) -> GraphIR:
    """Static-shape, constant-folded form of `model` for the given input shapes (graph input order)."""
    g: Graph = model.graph
    if len(input_shapes) != len(g.inputs):
        raise ValueError("model '%s' takes %d inputs, got %d shapes" % (g.name, len(g.inputs), len(input_shapes)))
    ir = GraphIR(g.name, [vi.name for vi in g.inputs], [vi.name for vi in g.outputs])
    ir.consts = dict(g.initializers)
    for vi, shape in zip(g.inputs, input_shapes):
        shape = tuple(int(d) for d in shape)
        if vi.shape is not None:
            if len(vi.shape) != len(shape) or any(isinstance(d, int) and d > 0 and d != s
                                                  for d, s in zip(vi.shape, shape)):
                raise ValueError("input '%s' expects shape %s, got %s" % (vi.name, vi.shape, shape))
        ir.shapes[vi.name] = shape

    def shp(name):
        if name in ir.consts:
            return tuple(ir.consts[name].shape)
        if name not in ir.shapes:
            raise ValueError("value '%s' is used before it is produced" % name)
        return ir.shapes[name]

    for node in g.nodes:
        if node.domain not in ("", "ai.onnx"):
            raise UnsupportedNode("node '%s': operator domain '%s'" % (node.name, node.domain))
        node = _to_opset12_form(node, model.opset, ir.consts)
        if node.op_type == "Constant":
            v = node.attr("value")
            if v is None:
                for key, dt in (("value_float", np.float32), ("value_int", np.int64), ("value_floats", np.float32),
                                ("value_ints", np.int64)):
                    if key in node.attrs:
                        v = np.asarray(node.attrs[key], dtype=dt)
            if v is None:
                raise UnsupportedNode("Constant '%s' without a tensor value" % node.name)
            ir.consts[node.outputs[0]] = v
            continue
        if node.op_type == "Shape":
            ir.consts[node.outputs[0]] = np.asarray(shp(node.inputs[0]), dtype=np.int64)
            continue
        if all((not i) or i in ir.consts for i in node.inputs):
            val = _host_eval(node, [ir.consts[i] if i else None for i in node.inputs])
            if val is not None:
                ir.consts[node.outputs[0]] = np.asarray(val)
                continue
        ir.shapes[node.outputs[0]] = tuple(int(d) for d in _infer(node, shp, ir.consts))
        for extra in node.outputs[1:]:
            if extra:
                raise UnsupportedNode("node '%s': secondary outputs are not supported" % node.name)
        ir.nodes.append(Node(node.op_type, node.name, list(node.inputs), list(node.outputs), dict(node.attrs)))
    for o in ir.outputs:
        if o not in ir.shapes and o not in ir.consts:
            raise ValueError("graph output '%s' is never produced" % o)
    return ir
