"""Executes the DaCeML-facing half of the plugin (dace_onnx_b200/b200_implementations.py) against the stand-in
`dace` / `daceml` namespace of tests/_fake_dace.py: registration, forward_can_be_applied and forward of every
expansion, the per-node environments, late registration and the hand-over to `pure`."""
import importlib
import os
import re
import subprocess
import sys
import tempfile

import pytest

from tests import _fake_dace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OPS = ["MatMul", "Gemm", "Conv", "MaxPool", "Softmax", "LogSoftmax", "ReduceMean", "Add", "Sub", "Mul", "Div", "Pow",
       "Sqrt", "Relu", "Erf"]


@pytest.fixture()
def plugin(monkeypatch):
    monkeypatch.delenv("B200_MATH_MODE", raising=False)
    ns = _fake_dace.install()
    sys.modules.pop("dace_onnx_b200.b200_implementations", None)
    mod = importlib.import_module("dace_onnx_b200.b200_implementations")   # import registers, like the in-tree use
    yield ns, mod
    _fake_dace.uninstall(ns)
    sys.modules.pop("dace_onnx_b200.b200_implementations", None)


def place(ns, op, label, descs, ins, outs, **attrs):
    """A node in state 0 of a fresh SDFG (other nodes before it, so ids are not all zero)."""
    sdfg = ns.FakeSDFG("main")
    state = sdfg.add_state()
    state.add_node(object())
    node = state.add_node(ns.FakeNode(op, label, descs, ins, outs, **attrs))
    return node, state, sdfg


CONV_ATTRS = dict(group=1, auto_pad="NOTSET", dilations=[1, 1], pads=[1, 1, 1, 1], strides=[1, 1], kernel_shape=[3, 3])


def nodes(ns):
    D = ns.Desc
    return {
        "MatMul": ("MatMul", {"A": D((8, 128, 64)), "B": D((64, 32)), "Y": D((8, 128, 32))}, ["A", "B"], ["Y"], {}),
        "Gemm": ("Gemm", {"A": D((16, 784)), "B": D((120, 784)), "C": D((120,)), "Y": D((16, 120))}, ["A", "B", "C"],
                 ["Y"], dict(alpha=1.0, beta=1.0, transA=0, transB=1)),
        "Conv": ("Conv", {"X": D((2, 64, 8, 8)), "W": D((64, 64, 3, 3)), "B": D((64,)), "Y": D((2, 64, 8, 8))},
                 ["X", "W", "B"], ["Y"], CONV_ATTRS),
        "MaxPool": ("MaxPool", {"X": D((2, 6, 30, 30)), "Y": D((2, 6, 15, 15))}, ["X"], ["Y"],
                    dict(kernel_shape=[2, 2], strides=[2, 2], pads=None, auto_pad="NOTSET", ceil_mode=0,
                         storage_order=0, dilations=None)),
        "Softmax": ("Softmax", {"input": D((4, 12, 32, 32)), "output": D((4, 12, 32, 32))}, ["input"], ["output"],
                    dict(axis=3)),
        "LogSoftmax": ("LogSoftmax", {"input": D((16, 10)), "output": D((16, 10))}, ["input"], ["output"], dict(axis=1)),
        "ReduceMean": ("ReduceMean", {"data": D((4, 32, 768)), "reduced": D((4, 32, 1))}, ["data"], ["reduced"],
                       dict(axes=[-1], keepdims=1)),
        "Add": ("Add", {"A": D((4, 32, 768)), "B": D((768,)), "C": D((4, 32, 768))}, ["A", "B"], ["C"], {}),
        "Sub": ("Sub", {"A": D((4, 32, 768)), "B": D((4, 32, 1)), "C": D((4, 32, 768))}, ["A", "B"], ["C"], {}),
        "Mul": ("Mul", {"A": D((4, 32, 768)), "B": D(()), "C": D((4, 32, 768))}, ["A", "B"], ["C"], {}),
        "Div": ("Div", {"A": D((4, 32, 768)), "B": D((4, 32, 1)), "C": D((4, 32, 768))}, ["A", "B"], ["C"], {}),
        "Pow": ("Pow", {"X": D((4, 32, 768)), "Y": D(()), "Z": D((4, 32, 768))}, ["X", "Y"], ["Z"], {}),
        "Sqrt": ("Sqrt", {"X": D((4, 32, 1)), "Y": D((4, 32, 1))}, ["X"], ["Y"], {}),
        "Relu": ("Relu", {"X": D((4, 120)), "Y": D((4, 120))}, ["X"], ["Y"], {}),
        "Erf": ("Erf", {"input": D((4, 32, 3072)), "output": D((4, 32, 3072))}, ["input"], ["output"], {}),
    }


def test_import_registers_every_expansion(plugin):
    ns, mod = plugin
    assert sorted(op for op, name in ns.registry if name == "b200") == sorted(OPS)
    for op in OPS:
        impl = ns.registry[(op, "b200")]
        assert issubclass(impl, ns.ONNXForward) and impl.__name__ == "B200" + op
        assert dict(ns.ONNXForward.registered_implementations(op))["b200"] is impl
    base = ns.environments[0]
    assert base.__name__ == "B200Ops" and base.cmake_libraries == [mod.LIB_PATH] and base.cmake_includes == [mod.INCLUDE_DIR]
    assert "b200_ops.h" in base.headers and os.path.exists(os.path.join(base.cmake_includes[0], "b200_ops.h"))


@pytest.mark.parametrize("op", OPS)
def test_forward_builds_one_cpp_tasklet_wired_to_every_connector(op, plugin):
    ns, mod = plugin
    name, descs, ins, outs, attrs = nodes(ns)[op]
    node, state, sdfg = place(ns, name, op.lower() + "_3", descs, ins, outs, **attrs)
    impl = ns.registry[(op, "b200")]
    assert impl.forward_can_be_applied(node, state, sdfg) is True
    nsdfg = impl.forward(node, state, sdfg)
    (tasklet,) = nsdfg.states[0].tasklets
    assert tasklet.language == "CPP"
    assert sorted(tasklet.in_connectors) == sorted("_" + n for n in ins if n in descs)
    assert sorted(tasklet.out_connectors) == sorted("_" + n for n in outs)
    assert all(t == ("pointer", "float32") for t in list(tasklet.in_connectors.values()) + list(tasklet.out_connectors.values()))
    wired = {(e[3] or e[1]) for e in nsdfg.states[0].edges}
    assert wired == set(tasklet.in_connectors) | set(tasklet.out_connectors)
    assert "__dace_current_stream" in tasklet.code and "b200_last_error_string" in tasklet.code
    assert set(nsdfg.arrays) == set(descs)
    (env,) = impl.environments
    assert getattr(env, "_registered_environment", False) and env.cmake_libraries == [mod.LIB_PATH]


def test_workspace_fields_are_unique_per_node_instance(plugin):
    ns, mod = plugin
    name, descs, ins, outs, attrs = nodes(ns)["Conv"]
    envs, codes = [], []
    for _ in range(2):   # the same label in two different (nested) SDFGs
        node, state, sdfg = place(ns, name, "conv", descs, ins, outs, **attrs)
        impl = ns.registry[("Conv", "b200")]
        nsdfg = impl.forward(node, state, sdfg)
        envs.append(impl.environments[0])
        codes.append(nsdfg.states[0].tasklets[0].code)
    f0, f1 = envs[0].state_fields, envs[1].state_fields
    assert len(f0) == 2 and not set(f0) & set(f1)
    field = re.match(r"void \*(\w+);", f0[0]).group(1)
    assert re.fullmatch(r"b200_ws_conv_\d+_0_1", field)          # name, sdfg id, state id, node id
    assert "__state->%s" % field in codes[0] and "__state->%s" % field not in codes[1]
    assert "cudaMalloc" in envs[0].init_code and "!= cudaSuccess" in envs[0].init_code and "abort()" in envs[0].init_code
    assert "cudaFree(__state->%s)" % field in envs[0].finalize_code
    # MatMul in the fp32-accurate mode gets a workspace field of its own kind
    name, descs, ins, outs, attrs = nodes(ns)["MatMul"]
    node, state, sdfg = place(ns, name, "mm", descs, ins, outs, **attrs)
    impl = ns.registry[("MatMul", "b200")]
    code = impl.forward(node, state, sdfg).states[0].tasklets[0].code
    assert "b200_gemm_ws_f32" in code and impl.environments[0].state_fields[0].startswith("void *b200_ws_mm_")


def test_generated_environment_and_tasklet_compile_together(plugin):
    """init_code + tasklet body + finalize_code of a Conv node, compiled as the C++ DaCe would emit around them."""
    ns, mod = plugin
    name, descs, ins, outs, attrs = nodes(ns)["Conv"]
    node, state, sdfg = place(ns, name, "conv", descs, ins, outs, **attrs)
    impl = ns.registry[("Conv", "b200")]
    code = impl.forward(node, state, sdfg).states[0].tasklets[0].code
    env = impl.environments[0]
    src = """
#include <cstdio>
#include <cstdlib>
#include <cstddef>
#include "b200_ops.h"
typedef int cudaError_t; static const cudaError_t cudaSuccess = 0;
static cudaError_t cudaMalloc(void **p, size_t n) { *p = malloc(n); return cudaSuccess; }
static void cudaFree(void *p) { free(p); }
struct state_t { %s };
void init(state_t *__state) { %s }
void run(state_t *__state, void *__dace_current_stream, const float *_X, const float *_W, const float *_B, float *_Y) { %s }
void fini(state_t *__state) { %s }
""" % (" ".join(env.state_fields), env.init_code, code, env.finalize_code)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "t.cpp")
        open(path, "w").write(src)
        r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), path],
                           capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_descriptors_the_kernels_cannot_take_are_refused(plugin):
    ns, mod = plugin
    D, S = ns.Desc, ns.Storage
    impl = ns.registry[("Softmax", "b200")]

    def can(desc_in, **attrs):
        node, state, sdfg = place(ns, "Softmax", "sm", {"input": desc_in, "output": D(desc_in.shape)}, ["input"],
                                  ["output"], axis=-1, **attrs)
        return impl.forward_can_be_applied(node, state, sdfg)
    assert can(D((4, 8)))
    assert not can(D((4, 8), storage=S.Default))           # an SDFG built with cuda=False: host pointers
    assert not can(D((4, 8), storage=S.CPU_Heap))
    assert not can(D((4, 8), storage="FPGA_Global"))       # neither host nor GPU
    assert not can(D((4, 8), dtype="float64"))
    assert not can(D((4, 8), strides=(16, 1)))             # not contiguous
    assert not can(D((ns.Symbol("N"), 8)))                 # symbolic extent
    # node-specific refusals
    mm = ns.registry[("MatMul", "b200")]
    node, state, sdfg = place(ns, "MatMul", "mm", {"A": D((64,)), "B": D((64, 32)), "Y": D((32,))}, ["A", "B"], ["Y"])
    assert not mm.forward_can_be_applied(node, state, sdfg)            # 1-D operand, as PureMatMul refuses
    gm = ns.registry[("Gemm", "b200")]
    descs = {"A": D((16, 64)), "B": D((32, 64)), "C": D((32,)), "Y": D((16, 32))}
    for bad in (dict(alpha=2.0, beta=1.0, transA=0, transB=1), dict(alpha=1.0, beta=1.0, transA=0, transB=0)):
        node, state, sdfg = place(ns, "Gemm", "g", descs, ["A", "B", "C"], ["Y"], **bad)
        assert not gm.forward_can_be_applied(node, state, sdfg)
    square = {"A": D((32, 64)), "B": D((32, 64)), "C": D((32, 1)), "Y": D((32, 32))}     # per-ROW C with M == N
    node, state, sdfg = place(ns, "Gemm", "g", square, ["A", "B", "C"], ["Y"], alpha=1.0, beta=1.0, transA=0, transB=1)
    assert not gm.forward_can_be_applied(node, state, sdfg)
    cv = ns.registry[("Conv", "b200")]
    name, descs, ins, outs, attrs = nodes(ns)["Conv"]
    for bad in (dict(group=2), dict(pads=[1, 0, 0, 0]), dict(dilations=[2, 2]), dict(auto_pad="SAME_UPPER")):
        node, state, sdfg = place(ns, name, "c", descs, ins, outs, **{**attrs, **bad})
        assert not cv.forward_can_be_applied(node, state, sdfg)
    rm = ns.registry[("ReduceMean", "b200")]
    node, state, sdfg = place(ns, "ReduceMean", "r", {"data": D((4, 5, 6)), "reduced": D((5,))}, ["data"], ["reduced"],
                              axes=[0, 2], keepdims=0)
    assert not rm.forward_can_be_applied(node, state, sdfg)            # axes not adjacent


def test_late_registration_and_hand_over_to_pure(plugin):
    ns, mod = plugin
    calls = []

    @ns.op_implementation(op="Softmax", name="pure")
    class PureSoftmax(ns.ONNXForward):
        @staticmethod
        def forward(node, state, sdfg):
            calls.append(node.label)
            return "pure-expansion"

    assert mod.register_late() == sorted(OPS)
    for op in OPS:
        exp = getattr(ns.donnx, "ONNX" + op).implementations["b200"]
        assert exp.__name__ == "B200Expansion" + op and exp.forward_impl is ns.registry[(op, "b200")]
    assert mod.register_late() == sorted(OPS)                    # idempotent
    exp = ns.donnx.ONNXSoftmax.implementations["b200"]
    D, S = ns.Desc, ns.Storage
    # a node we take
    node, state, sdfg = place(ns, "Softmax", "sm", {"input": D((4, 8)), "output": D((4, 8))}, ["input"], ["output"], axis=1)
    out = exp.expansion(node, state, sdfg)
    assert node.validated == 1 and out.states[0].tasklets[0].code.count("b200_softmax_f32") == 1
    assert exp.environments and all(getattr(e, "_registered_environment", False) for e in exp.environments)
    # a node in host storage goes to `pure`, never to ONNX Runtime
    node, state, sdfg = place(ns, "Softmax", "host_sm", {"input": D((4, 8), storage=S.Default), "output": D((4, 8))},
                              ["input"], ["output"], axis=1)
    assert exp.expansion(node, state, sdfg) == "pure-expansion" and calls == ["host_sm"]
    # no pure expansion to hand over to: refuse loudly
    exp = ns.donnx.ONNXErf.implementations["b200"]
    node, state, sdfg = place(ns, "Erf", "e", {"input": D((4,), dtype="float64"), "output": D((4,))}, ["input"], ["output"])
    with pytest.raises(NotImplementedError, match="refusing to fall back"):
        exp.expansion(node, state, sdfg)


def test_math_mode_flag_is_read_at_expansion(plugin, monkeypatch):
    ns, mod = plugin
    name, descs, ins, outs, attrs = nodes(ns)["MatMul"]
    impl = ns.registry[("MatMul", "b200")]
    monkeypatch.setenv("B200_MATH_MODE", "tf32")
    node, state, sdfg = place(ns, name, "mm", descs, ins, outs, **attrs)
    code = impl.forward(node, state, sdfg).states[0].tasklets[0].code
    assert "b200_gemm_f32(" in code and code.split("1.0f, ")[1].startswith("1}")     # math_mode 1, no workspace
    monkeypatch.setenv("B200_MATH_MODE", "bf16")       # bf16 keeps its operand copies in a workspace of the SDFG state
    node, state, sdfg = place(ns, name, "mm", descs, ins, outs, **attrs)
    code = impl.forward(node, state, sdfg).states[0].tasklets[0].code
    assert "b200_gemm_ws_f32(" in code and code.split("1.0f, ")[1].startswith("3}")
    assert "b200_gemm_workspace_bytes" in impl.environments[0].init_code
    monkeypatch.setenv("B200_MATH_MODE", "fp64")
    with pytest.raises(ValueError):
        impl.forward(node, state, sdfg)
