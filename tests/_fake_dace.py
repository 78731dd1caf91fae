"""A minimal stand-in for the `dace` / `daceml` names that dace_onnx_b200/b200_implementations.py touches, so that
its registration code, every forward_can_be_applied / forward and the late-registration wrapper can be EXECUTED on a
machine without DaCe (the reference tests what it cannot reach with fakes too, tests/test_input_outputs.py:25-38).

The fakes keep the contracts the plugin relies on and nothing more: the registry behind @op_implementation and
ONNXForward.registered_implementations (daceml/onnx/forward_implementation_abc.py:42-52), empty_sdfg_for_node's
return value (daceml/onnx/op_implementations/utils.py:94-128), descriptor lookup by connector name
(daceml/util/utils.py:34-56), is_cuda (:236-245), dace.library.environment, and node classes with
register_implementation / implementations (what dace.library.node gives the ONNX<Op> classes)."""
import sys
import types


class Storage:
    Default, CPU_Heap, GPU_Global = "Default", "CPU_Heap", "GPU_Global"


class Desc:
    def __init__(self, shape, dtype="float32", storage=Storage.GPU_Global, strides=None):
        self.shape, self.dtype, self.storage = tuple(shape), dtype, storage
        contiguous, acc = [], 1
        for s in reversed(self.shape):
            contiguous.append(acc)
            acc *= s if isinstance(s, int) else 1
        self.strides = tuple(strides) if strides is not None else tuple(reversed(contiguous))
        self.transient = True


class Symbol(str):
    """A symbolic extent."""


class FakeTasklet:
    def __init__(self, label, inputs, outputs, code, language):
        self.label, self.in_connectors, self.out_connectors, self.code, self.language = label, inputs, outputs, code, language


class FakeState:
    def __init__(self, sdfg):
        self.sdfg, self.tasklets, self.edges, self._nodes = sdfg, [], [], []

    def add_tasklet(self, label, inputs, outputs, code, language):
        t = FakeTasklet(label, dict(inputs), dict(outputs), code, language)
        self.tasklets.append(t)
        return t

    def add_edge(self, src, src_conn, dst, dst_conn, memlet):
        self.edges.append((src, src_conn, dst, dst_conn, memlet))

    def add_node(self, node):
        self._nodes.append(node)
        return node

    def node_id(self, node):
        return self._nodes.index(node)


class FakeSDFG:
    _next_id = 0

    def __init__(self, name):
        self.name, self.arrays, self.states = name, {}, []
        self.sdfg_id = FakeSDFG._next_id
        FakeSDFG._next_id += 1

    def add_state(self):
        st = FakeState(self)
        self.states.append(st)
        return st

    def node_id(self, state):
        return self.states.index(state)

    def make_array_memlet(self, name):
        return ("memlet", name)


class FakeNode:
    """An ONNX library node placed in a state, with descriptors on its connectors and ONNX attributes."""

    def __init__(self, op, label, descs, inputs, outputs, **attrs):
        self.op, self.label, self.name = op, label, label
        self.descs = descs
        self.in_connectors = {n: None for n in inputs if n in descs}
        self.out_connectors = {n: None for n in outputs}
        self.validated = 0
        for k, v in attrs.items():
            setattr(self, k, v)

    def validate(self, sdfg, state):
        self.validated += 1


def install():
    """Put the fake modules into sys.modules; returns a namespace with the pieces tests inspect."""
    ns = types.SimpleNamespace(environments=[], registry={}, Desc=Desc, Storage=Storage, Symbol=Symbol,
                               FakeNode=FakeNode, FakeSDFG=FakeSDFG)
    mods = {}

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        mods[name] = m
        return m

    def environment(cls):
        ns.environments.append(cls)
        cls._registered_environment = True
        return cls

    class Language:
        CPP = "CPP"

    class ScheduleType:
        CPU_Multicore, GPU_Default, FPGA_Device = "CPU_Multicore", "GPU_Default", "FPGA_Device"

    def can_access(schedule, storage):
        if schedule == ScheduleType.CPU_Multicore:
            return storage in (Storage.Default, Storage.CPU_Heap)
        if schedule == ScheduleType.GPU_Default:
            return storage == Storage.GPU_Global
        return False

    dtypes = mod("dace.dtypes", Language=Language, ScheduleType=ScheduleType, StorageType=Storage, can_access=can_access)
    library = mod("dace.library", environment=environment)
    dace = mod("dace", float32="float32", float64="float64", pointer=lambda t: ("pointer", t), dtypes=dtypes,
               library=library, symbolic=types.SimpleNamespace(issymbolic=lambda s: isinstance(s, Symbol)))
    mod("dace.libraries")
    mod("dace.libraries.standard", CUDA=type("CUDA", (), {}))

    class ExpandTransformation:
        environments = []
    mod("dace.transformation")
    mod("dace.transformation.transformation", ExpandTransformation=ExpandTransformation)

    class ONNXForward:
        @staticmethod
        def forward_can_be_applied(node, state, sdfg):
            return True

        @classmethod
        def registered_implementations(cls, op_name):
            return [(name, impl) for (op, name), impl in ns.registry.items() if op == op_name]

    def op_implementation(op, name):
        def dec(cls):
            ns.registry[(op, name)] = cls
            return cls
        return dec

    def empty_sdfg_for_node(sdfg, state, node, add_access_nodes=True):
        nsdfg = FakeSDFG(node.label + "_expansion")
        nstate = nsdfg.add_state()
        ins = {n: ("read", n) for n in node.in_connectors}
        outs = {n: ("write", n) for n in node.out_connectors}
        for n in list(ins) + list(outs):
            nsdfg.arrays[n] = node.descs[n]
        return nsdfg, nstate, ins, outs

    def is_cuda(storage):
        if can_access(ScheduleType.CPU_Multicore, storage):
            return False
        if can_access(ScheduleType.GPU_Default, storage):
            return True
        raise ValueError("Unsupported storage %s" % storage)

    def is_desc_contiguous(desc):
        expect, acc = [], 1
        for s in reversed(desc.shape):
            expect.append(acc)
            acc *= s if isinstance(s, int) else 1
        return tuple(desc.strides) == tuple(reversed(expect))

    mod("daceml")
    mod("daceml.onnx.forward_implementation_abc", ONNXForward=ONNXForward)
    mod("daceml.onnx.op_implementations")
    mod("daceml.onnx.op_implementations.utils", empty_sdfg_for_node=empty_sdfg_for_node, op_implementation=op_implementation)
    mod("daceml.util")
    mod("daceml.util.utils", in_desc_with_name=lambda node, state, sdfg, name: node.descs[name],
        out_desc_with_name=lambda node, state, sdfg, name: node.descs[name], is_desc_contiguous=is_desc_contiguous,
        is_cuda=is_cuda)

    def node_class(op):
        class NodeCls:
            implementations = {}
            default_implementation = None

            @classmethod
            def register_implementation(cls, name, transformation):
                cls.implementations[name] = transformation
        NodeCls.implementations = {}
        NodeCls.__name__ = "ONNX" + op
        return NodeCls

    donnx = mod("daceml.onnx")
    for op in ("MatMul", "Gemm", "Conv", "MaxPool", "Softmax", "LogSoftmax", "ReduceMean", "Add", "Sub", "Mul", "Div",
               "Pow", "Sqrt", "Relu", "Erf"):
        setattr(donnx, "ONNX" + op, node_class(op))
    mods["daceml"].onnx = donnx
    ns.donnx, ns.ONNXForward, ns.op_implementation = donnx, ONNXForward, op_implementation
    ns.saved = {k: sys.modules.get(k) for k in mods}
    sys.modules.update(mods)
    ns.mods = mods
    return ns


def uninstall(ns):
    for k, old in ns.saved.items():
        if old is None:
            sys.modules.pop(k, None)
        else:
            sys.modules[k] = old
