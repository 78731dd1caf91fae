"""The C++ tasklet bodies the DaCeML plugin emits compile against include/b200_ops.h and carry
the right shapes (DaCe itself is not needed for this)."""
import os
import subprocess
import tempfile

import pytest

from dace_onnx_b200 import b200_implementations as impl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

HEAD = """
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include "b200_ops.h"
struct State { void *ws; size_t ws_bytes; };
"""
WRAP = """
void tasklet_{i}(void *__dace_current_stream, State *__state, const float *_A, const float *_B, float *_C,
                 const float *_X, const float *_W, const float *_input, const float *_data, float *_Y, float *_Z,
                 float *_output, float *_reduced) {{
{body}
}}
"""


def bodies():
    out = [
        impl.tasklet_matmul((2, 4), (4, 3), mode=0),
        impl.tasklet_matmul((64, 512, 768), (768, 768), mode=0),
        impl.tasklet_matmul((64, 12, 512, 64), (64, 12, 64, 512), mode=1),
        impl.tasklet_matmul((4096, 784), (120, 784), trans_b=True, bias=True, mode=2),
        impl.tasklet_matmul((64, 512, 768), (768, 768), mode=0, ws="ws"),
        impl.tasklet_matmul((4096, 784), (120, 784), trans_b=True, bias=True, mode=0, ws="ws"),
        impl.tasklet_conv((256, 64, 56, 56), (64, 64, 3, 3), (1, 1, 1, 1), (1, 1), True, mode=0).replace("{ws}", "ws"),
        impl.tasklet_maxpool((8, 6, 30, 30), (2, 2), (2, 2)),
        impl.tasklet_softmax((768, 512, 512), -1),
        impl.tasklet_softmax((2, 4, 10), 0, log=True),
        impl.tasklet_reduce_mean((32768, 768), [-1]),
        impl.tasklet_binary("Sub", (32768, 768), (32768, 1)),
        impl.tasklet_binary("Add", (32768, 1), ()),
        impl.tasklet_binary("Pow", (8, 16), (), names=("_X", "_A", "_Z")),
        impl.tasklet_unary("Erf", (32768, 3072), names=("_input", "_output")),
        impl.tasklet_unary("Relu", (4096, 120)),
    ]
    assert all(b is not None for b in out)
    return out


def hooks():
    """init / finalize code of the nodes that keep a workspace in the SDFG state."""
    out = []
    for fields, init, fini in (
            impl.gemm_env_code((64, 512, 768), (768, 768), "ws", mode=0),
            impl.gemm_env_code((4096, 784), (120, 784), "ws", trans_b=True, bias=True, mode=0),
            impl.conv_env_code((256, 64, 56, 56), (64, 64, 3, 3), (1, 1, 1, 1), (1, 1), "ws", mode=0)):
        assert fields == ["void *ws;", "size_t ws_bytes;"]
        out += [init, fini]
    return out


HOOK_HEAD = """
extern "C" int cudaMalloc(void **, size_t);
extern "C" int cudaFree(void *);
static const int cudaSuccess = 0;
"""
HOOK_WRAP = """
void hook_{i}(State *__state) {{
{body}
}}
"""


def test_tasklets_compile_against_the_header():
    src = HEAD + "\n".join(WRAP.format(i=i, body=b) for i, b in enumerate(bodies())) + HOOK_HEAD + \
        "\n".join(HOOK_WRAP.format(i=i, body=b) for i, b in enumerate(hooks()))
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "tasklets.cpp")
        with open(path, "w") as f:
            f.write(src)
        r = subprocess.run(["g++", "-std=c++14", "-fsyntax-only", "-Wall", "-Werror", "-I",
                            os.path.join(ROOT, "include"), path], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def test_matmul_descriptor_fields():
    code = impl.tasklet_matmul((64, 12, 512, 64), (64, 12, 64, 512), mode=0)
    # dense batch 64 x 12 merges into one level of 768 matrices
    assert "{1, 768, 512, 512, 64, 64, 512, 512, 0, 32768, 0, 32768, 0, 262144," in code.replace("\n", " ").replace("  ", " ")
    code = impl.tasklet_matmul((64, 512, 768), (768, 768), mode=0)
    assert "{1, 64, 512, 768, 768, 768, 768, 768, 0, 393216, 0, 0, 0, 393216," in code.replace("\n", " ").replace("  ", " ")
    assert impl.tasklet_matmul((2, 3, 4, 5, 6), (3, 1, 6, 7), mode=0) is None or "b200_gemm_f32" in \
        impl.tasklet_matmul((2, 3, 4, 5, 6), (3, 1, 6, 7), mode=0)
    with_ws = impl.tasklet_matmul((64, 512, 768), (768, 768), mode=0, ws="b200_ws_n1")
    assert "b200_gemm_ws_f32(" in with_ws and "__state->b200_ws_n1_bytes" in with_ws


def test_broadcast_strides():
    assert impl._broadcast((32768, 768), (768,)) == ([32768, 768], [768, 1], [0, 1])
    assert impl._broadcast((32768, 768), (32768, 1)) == ([32768, 768], [768, 1], [1, 0])
    assert impl._broadcast((3, 1, 5), (4, 1)) == ([3, 4, 5], [5, 0, 1], [0, 1, 0])
    with pytest.raises(ValueError):
        impl._broadcast((3, 4), (5,))


def test_math_mode_env(monkeypatch):
    monkeypatch.setenv(impl.MATH_MODE_ENV, "tf32")
    assert impl.math_mode() == 1
    monkeypatch.setenv(impl.MATH_MODE_ENV, "bf16")
    assert impl.math_mode() == 3
    monkeypatch.setenv(impl.MATH_MODE_ENV, "fp64")
    with pytest.raises(ValueError):
        impl.math_mode()


def test_registration_needs_daceml():
    try:
        import dace  # noqa: F401
        import daceml  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError):
            impl._register()
    else:
        assert "MatMul" in impl._register()
