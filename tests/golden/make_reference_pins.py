"""Generates tests/golden/ref_pins.npz by EXECUTING the reference's own source for the hot-path nodes.

The reference (spcl/dace-onnx) states each node's arithmetic as a small numpy-style Python program
inside `daceml/onnx/op_implementations/pure_implementations.py`, which DaCe (not installable where
this repository is developed) would lower to loops. This script loads that file and
`op_implementations/utils.py` UNMODIFIED from a reference checkout, behind stand-ins for the `dace`
/ `daceml` names they import, calls every `Pure<Op>.forward(node, state, sdfg)` exactly as the
library-node expansion does (daceml/onnx/nodes/onnx_op.py:646-684), and runs what comes back:

  * expansions built with `program_for_node` (Sqrt, Pow, Add, Sub, Mul, Div, ReduceMean, Erf, Softmax,
    LogSoftmax, Gemm, Relu) hand their inner `prog` to a stand-in `DaceProgram`; `prog` is then called
    with numpy fp32 arrays, so the statements the reference wrote (`np.max`, `np.exp`, `A @ np.transpose(B) + C`
    ...) are what computes the vectors. `dace.elementwise(f, x)` applies `f` through numpy; the scalar
    functions DaCe resolves by name inside those lambdas (`sqrt`, `erf`, `log`, `max`) are bound to
    numpy / scipy.special;
  * PureMatMul builds its einsum string and an ONNXEinsum node in a nested SDFG (:151-233); the
    stand-in SDFG records the node and the vectors come from `np.einsum(<that string>, A, B, optimize=True)`
    in fp32 (numpy then contracts through its BLAS, as DaCe's einsum lowers a matrix product to a BLAS
    GEMM, :238-267 and daceml/util/utils.py:213-216).

Outputs are written through a view that takes a value of equal size but different shape (DaCe's
output-connector rule: ReduceMean with keepdims assigns a [T] mean to a [T, 1] connector, :104-107).

What this pins: the oracle against the reference's statements run with numpy semantics. What it does
not: DaCe's code generation (reduction order, libm). PureConv2D (img_op_implementations.py:246-293)
is written in DaCe's map / tasklet syntax, which is not executable Python without DaCe; it stays
pinned by the reference's own comparator (F.conv2d) in tests/test_oracle_pins.py.

Run where a reference checkout exists (it is not needed to run the tests):

    python tests/golden/make_reference_pins.py [/path/to/dace-onnx]
"""
import abc
import importlib.util
import os
import sys
import types

import numpy as np
import scipy.special

OUT = os.path.dirname(os.path.abspath(__file__))


# ---------------------------------------------------------------------------------------------
# stand-ins for the dace / daceml names the two reference files import
# ---------------------------------------------------------------------------------------------
class Desc:
    """Array descriptor: what in_desc_with_name / out_desc_with_name return."""

    def __init__(self, shape, dtype):
        self.shape = tuple(shape)
        self.dtype = dtype
        self.transient = False


class DType:
    def __init__(self, name, np_type):
        self.name, self.np_type = name, np_type

    def to_string(self):
        return self.name

    def __call__(self, v):
        return self.np_type(v)


class FakeSDFG:
    def __init__(self, name="sdfg"):
        self.name = name
        self.arrays = {}
        self.states = []
        self.program = None

    def add_state(self, *a, **k):
        st = FakeState(self)
        self.states.append(st)
        return st

    def add_datadesc(self, name, desc):
        self.arrays[name] = desc

    def make_array_memlet(self, name):
        return ("memlet", name)

    def apply_gpu_transformations(self):
        pass

    def apply_strict_transformations(self):
        pass


class FakeState:
    def __init__(self, sdfg):
        self.sdfg = sdfg
        self.nodes = []
        self.edges = []

    def add_node(self, n):
        self.nodes.append(n)

    def add_read(self, name):
        return ("read", name)

    def add_write(self, name):
        return ("write", name)

    def add_edge(self, src, src_conn, dst, dst_conn, memlet):
        self.edges.append((src, src_conn, dst, dst_conn, memlet))


class FakeDaceProgram:
    """dace.frontend.python.parser.DaceProgram as program_for_node uses it (utils.py:82-85)."""

    def __init__(self, f, args, kwargs, auto_optimize, device):
        self.f = f
        self.name = None

    def to_sdfg(self):
        s = FakeSDFG(self.name)
        s.program = self.f
        return s


class Schema:
    def __init__(self, name, inputs, outputs):
        self.name, self._in, self._out = name, list(inputs), list(outputs)

    def non_variadic_inputs(self):
        return list(self._in)

    def non_variadic_outputs(self):
        return list(self._out)

    def variadic_inputs(self):
        return []

    def variadic_outputs(self):
        return []


class ONNXOp:
    """A library node: label, schema, attributes and the descriptors on its connectors."""
    schedule = "CPU"

    def __init__(self, op, inputs, outputs, descs, **attrs):
        self.label = op
        self.schema = Schema(op, inputs, outputs)
        self.in_connectors = {n: None for n in inputs if n in descs}
        self.out_connectors = {n: None for n in outputs}
        self.descs = descs
        for k, v in attrs.items():
            setattr(self, k, v)


class ONNXEinsum:
    def __init__(self, label, equation):
        self.label, self.equation = label, equation
        self.conns = []

    def add_in_connector(self, name):
        self.conns.append(name)


REGISTRY = {}


def install_fakes():
    float32 = DType("float32", np.float32)
    dace = types.ModuleType("dace")
    dace.float16, dace.float32, dace.float64 = DType("float16", np.float16), float32, DType("float64", np.float64)
    dace.SDFG, dace.SDFGState = FakeSDFG, FakeState
    dace.DeviceType = types.SimpleNamespace(CPU="CPU", GPU="GPU")
    dace.Memlet = lambda *a, **k: ("memlet",) + a
    dace.symbolic = types.SimpleNamespace(issymbolic=lambda v: False)

    def elementwise(func, arr):
        if isinstance(func, str):  # PureRelu passes the lambda as source text (:467-468)
            func = eval(func, {"dace": dace, "max": np.maximum})
        return func(arr)
    dace.elementwise = elementwise

    nodes = types.ModuleType("dace.nodes")
    nodes.Node, nodes.LibraryNode, nodes.AccessNode = type("Node", (), {}), type("LibraryNode", (), {}), type("AccessNode", (), {})
    dtypes = types.ModuleType("dace.dtypes")
    dtypes.ScheduleType = types.SimpleNamespace(GPU_Default="GPU_Default")
    dtypes.GPU_SCHEDULES = ["GPU_Device", "GPU_ThreadBlock"]
    dace.nodes, dace.dtypes = nodes, dtypes

    mods = {"dace": dace, "dace.nodes": nodes, "dace.dtypes": dtypes}

    def mod(name, **attrs):
        m = types.ModuleType(name)
        for k, v in attrs.items():
            setattr(m, k, v)
        mods[name] = m
        return m

    mod("dace.frontend")
    mod("dace.frontend.common", create_einsum_sdfg=lambda *a, **k: None)
    mod("dace.frontend.python")
    mod("dace.frontend.python.parser", DaceProgram=FakeDaceProgram)
    mod("dace.sdfg")
    mod("dace.sdfg.nodes", Node=nodes.Node)

    def autoregister(cls, **kwargs):
        REGISTRY[(kwargs["op"], kwargs["name"])] = cls
        return cls
    mod("dace.registry", autoregister=autoregister)

    class ONNXForward(abc.ABC):
        @staticmethod
        def forward_can_be_applied(node, state, sdfg):
            return True

    onnx_op = mod("daceml.onnx.nodes.onnx_op", ONNXOp=ONNXOp, ONNXEinsum=ONNXEinsum)
    mod("daceml")
    mod("daceml.onnx", converters=mod("daceml.onnx.converters"))
    mod("daceml.onnx.nodes", onnx_op=onnx_op)
    mod("daceml.onnx.forward_implementation_abc", ONNXForward=ONNXForward)

    def parse_variadic_param(param):
        name, number = param.split("__")
        return name, int(number)
    mod("daceml.onnx.nodes.node_utils", parse_variadic_param=parse_variadic_param)
    mod("daceml.transformation", constant_folding=mod("daceml.transformation.constant_folding"))
    mod("daceml.util")
    mod("daceml.util.utils",
        in_desc_with_name=lambda node, state, sdfg, name: node.descs[name],
        out_desc_with_name=lambda node, state, sdfg, name: node.descs[name],
        in_edge_with_name=lambda node, state, name: None,
        iterables_equal=lambda a, b: len(a) == len(b) and all(x == y for x, y in zip(a, b)))
    mod("daceml.onnx.op_implementations")
    sys.modules.update(mods)
    return dace


def load_reference(root):
    def load(modname, rel):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(root, rel))
        m = importlib.util.module_from_spec(spec)
        sys.modules[modname] = m
        spec.loader.exec_module(m)
        return m
    load("daceml.onnx.op_implementations.utils", "daceml/onnx/op_implementations/utils.py")
    pure = load("daceml.onnx.op_implementations.pure_implementations",
                "daceml/onnx/op_implementations/pure_implementations.py")
    # scalar functions DaCe's frontend resolves by name inside the `dace.elementwise` lambdas
    pure.sqrt, pure.log, pure.exp, pure.erf = np.sqrt, np.log, np.exp, scipy.special.erf
    return pure


class OutView:
    """Output connector: `out[:] = value` accepts a value of equal size (DaCe's connector shape rule)."""

    def __init__(self, shape):
        self.arr = np.zeros(shape, dtype=np.float32)

    def __setitem__(self, key, value):
        value = np.asarray(value)
        assert value.dtype == np.float32, "the reference program left fp32: %s" % value.dtype
        if value.shape != self.arr.shape and value.size == self.arr.size:
            value = value.reshape(self.arr.shape)
        self.arr[key] = value


SIGNATURES = {  # ONNX opset-12 connector names (the parameter names of the reference's programs)
    "Sqrt": (["X"], ["Y"]), "Pow": (["X", "Y"], ["Z"]), "Add": (["A", "B"], ["C"]), "Sub": (["A", "B"], ["C"]),
    "Mul": (["A", "B"], ["C"]), "Div": (["A", "B"], ["C"]), "ReduceMean": (["data"], ["reduced"]),
    "Erf": (["input"], ["output"]), "MatMul": (["A", "B"], ["Y"]), "Softmax": (["input"], ["output"]),
    "LogSoftmax": (["input"], ["output"]), "Gemm": (["A", "B", "C"], ["Y"]), "Relu": (["X"], ["Y"]),
}


def run_node(dace, op, out_shape, inputs, **attrs):
    """Expand one node with the reference's `pure` implementation and execute the expansion."""
    in_names, out_names = SIGNATURES[op]
    f32 = dace.float32
    descs = {n: Desc(np.shape(v), f32) for n, v in inputs.items()}
    descs[out_names[0]] = Desc(out_shape, f32)
    node = ONNXOp(op, in_names, out_names, descs, **attrs)
    impl = REGISTRY[(op, "pure")]
    sdfg, state = FakeSDFG("parent"), None
    assert impl.forward_can_be_applied(node, state, sdfg), op
    result = impl.forward(node, state, sdfg)
    out = OutView(out_shape)
    arrays = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in inputs.items()}
    if result.program is not None:
        result.program(**arrays, **{out_names[0]: out})
    else:
        einsum = [n for st in result.states for n in st.nodes if isinstance(n, ONNXEinsum)]
        assert len(einsum) == 1, "expected PureMatMul's single ONNXEinsum node"
        out[:] = np.einsum(einsum[0].equation, arrays["A"], arrays["B"], optimize=True).astype(np.float32)
        out.equation = einsum[0].equation
    return out.arr


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_reference_pins.py <checkout of spcl/dace-onnx (daceml)>")
    root = sys.argv[1]
    dace = install_fakes()
    load_reference(root)
    r = np.random.default_rng(2024)
    f = lambda *s, scale=1.0: (r.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    out = {}

    def case(tag, op, out_shape, inputs, **attrs):
        y = run_node(dace, op, out_shape, inputs, **attrs)
        for k, v in inputs.items():
            out["%s.%s" % (tag, k)] = np.asarray(v, dtype=np.float32)
        for k, v in attrs.items():
            out["%s.attr.%s" % (tag, k)] = np.asarray(v)
        out["%s.out" % tag] = y
        return y

    # elementwise nodes with the broadcasts the BERT graph uses (row, column, scalar operands)
    a, b = f(6, 40), f(6, 40)
    for op in ("Add", "Sub", "Mul", "Div"):
        case(op.lower() + "_full", op, (6, 40), {"A": a, "B": b + (3.0 if op == "Div" else 0.0)})
        case(op.lower() + "_row", op, (6, 40), {"A": a, "B": f(40) + (3.0 if op == "Div" else 0.0)})
        case(op.lower() + "_col", op, (6, 40), {"A": a, "B": f(6, 1) + (3.0 if op == "Div" else 0.0)})
        case(op.lower() + "_scalar", op, (6, 40), {"A": a, "B": np.float32(1.4142135)})
        case(op.lower() + "_lhs_row", op, (6, 40), {"A": f(40), "B": a + (3.0 if op == "Div" else 0.0)})
    case("pow_2", "Pow", (6, 40), {"X": a, "Y": np.float32(2.0)})
    case("pow_frac", "Pow", (6, 40), {"X": np.abs(a) + 0.1, "Y": np.float32(0.5)})
    case("sqrt", "Sqrt", (5, 33), {"X": np.abs(f(5, 33)) + 1e-3})
    case("erf", "Erf", (7, 65), {"input": f(7, 65, scale=2.0)})
    case("relu", "Relu", (7, 65), {"X": f(7, 65)})
    # ReduceMean: last axis keepdims (the LayerNorm use), no keepdims, a middle axis, two axes
    x = f(4, 6, 50)
    case("mean_last_keep", "ReduceMean", (4, 6, 1), {"data": x}, axes=(2,), keepdims=1)
    case("mean_last", "ReduceMean", (4, 6), {"data": x}, axes=(2,), keepdims=0)
    case("mean_mid", "ReduceMean", (4, 50), {"data": x}, axes=(1,), keepdims=0)
    case("mean_two", "ReduceMean", (4, 1, 1), {"data": x}, axes=(1, 2), keepdims=1)
    # Softmax / LogSoftmax: the reference test's shape and axes (tests/pure_expansions/test_expansions.py:343-418)
    for op in ("Softmax", "LogSoftmax"):
        xs = f(2, 4, 10, scale=10.0)
        case(op.lower() + "_ax0", op, (2, 4, 10), {"input": xs}, axis=0)
        case(op.lower() + "_axm1", op, (2, 4, 10), {"input": xs}, axis=-1)
        case(op.lower() + "_ax1", op, (3, 5, 8), {"input": f(3, 5, 8, scale=2.0)}, axis=1)
        case(op.lower() + "_rows512", op, (9, 512), {"input": f(9, 512, scale=2.0)}, axis=1)
        case(op.lower() + "_rows1000", op, (3, 1000), {"input": f(3, 1000, scale=2.0)}, axis=-1)
    # MatMul: the reference test's operand ranks (:18-56) and the BERT attention broadcasts
    for tag, sa, sb in [("2d", (2, 4), (4, 3)), ("3d_3d", (3, 5, 8), (3, 8, 6)), ("4d_2d", (2, 3, 7, 16), (16, 12)),
                        ("2d_3d", (5, 8), (3, 8, 6)), ("heads", (2, 2, 40, 64), (2, 2, 64, 40)),
                        ("tails", (130, 72), (72, 260)), ("k4096", (4, 4096), (4096, 8))]:
        A, B = f(*sa), f(*sb, scale=0.02 if tag == "k4096" else 1.0)  # K = 4096: weight-scale B, as in the FFN
        shape = tuple(np.broadcast_shapes(sa[:-2], sb[:-2])) + (sa[-2], sb[-1])
        case("matmul_" + tag, "MatMul", shape, {"A": A, "B": B})
    # Gemm, the only accepted form (alpha = beta = 1, transA = 0, transB = 1), with and without C
    A, B, C = f(33, 120), f(32, 120, scale=0.1), f(32, scale=0.1)
    case("gemm_bias", "Gemm", (33, 32), {"A": A, "B": B, "C": C}, alpha=1.0, beta=1.0, transA=0, transB=1)
    case("gemm_nobias", "Gemm", (33, 32), {"A": A, "B": B}, alpha=1.0, beta=1.0, transA=0, transB=1)

    # The exported node chains, node by node through the reference's expansions.
    #   LayerNormalization: ReduceMean, Sub, Pow 2, ReduceMean, Add eps, Sqrt, Div, Mul gamma, Add beta
    for tag, rows, width in [("ln_768", 5, 768), ("ln_1024", 3, 1024), ("ln_10", 4, 10)]:
        x, g, be = f(rows, width), (1 + 0.1 * f(width)), 0.1 * f(width)
        eps = np.float32(1e-12)
        s = (rows, width)
        mean = run_node(dace, "ReduceMean", (rows, 1), {"data": x}, axes=(-1,), keepdims=1)
        d = run_node(dace, "Sub", s, {"A": x, "B": mean})
        p = run_node(dace, "Pow", s, {"X": d, "Y": np.float32(2.0)})
        var = run_node(dace, "ReduceMean", (rows, 1), {"data": p}, axes=(-1,), keepdims=1)
        ve = run_node(dace, "Add", (rows, 1), {"A": var, "B": eps})
        sd = run_node(dace, "Sqrt", (rows, 1), {"X": ve})
        n = run_node(dace, "Div", s, {"A": d, "B": sd})
        y = run_node(dace, "Add", s, {"A": run_node(dace, "Mul", s, {"A": n, "B": g}), "B": be})
        out.update({tag + ".x": x, tag + ".gamma": g.astype(np.float32), tag + ".beta": be.astype(np.float32),
                    tag + ".eps": eps, tag + ".out": y})
    #   Gelu: Div sqrt(2), Erf, Add 1, Mul x, Mul 0.5
    x = f(6, 96, scale=2.0)
    s = x.shape
    t = run_node(dace, "Erf", s, {"input": run_node(dace, "Div", s, {"A": x, "B": np.float32(1.4142135381698608)})})
    t = run_node(dace, "Mul", s, {"A": x, "B": run_node(dace, "Add", s, {"A": t, "B": np.float32(1.0)})})
    out.update({"gelu.x": x, "gelu.out": run_node(dace, "Mul", s, {"A": t, "B": np.float32(0.5)})})
    #   attention core: MatMul(q, k^T), Mul scale, Softmax axis 3, MatMul(p, v)
    q, kt, v = f(2, 3, 32, 64), f(2, 3, 64, 32), f(2, 3, 32, 64)
    sc = run_node(dace, "MatMul", (2, 3, 32, 32), {"A": q, "B": kt})
    sc = run_node(dace, "Mul", sc.shape, {"A": sc, "B": np.float32(0.125)})
    pr = run_node(dace, "Softmax", sc.shape, {"input": sc}, axis=3)
    out.update({"attn.q": q, "attn.kt": kt, "attn.v": v,
                "attn.out": run_node(dace, "MatMul", (2, 3, 32, 64), {"A": pr, "B": v})})

    np.savez_compressed(os.path.join(OUT, "ref_pins.npz"), **out)
    print("wrote ref_pins.npz: %d arrays, %d bytes" % (len(out), os.path.getsize(os.path.join(OUT, "ref_pins.npz"))))


if __name__ == "__main__":
    main()
