"""`@op_implementation(op=..., name="b200")` expansions for a DaCeML installation.

Drop this module into `daceml/onnx/op_implementations/` (and import it from that package's
`__init__`, next to `pure_implementations`), or import it from anywhere and call
`register_late()`. After that `donnx.default_implementation = "b200"`,
`donnx.ONNXConv.default_implementation = "b200"` or `node.implementation = "b200"` select these
expansions exactly as "pure" / "cuDNN" are selected (daceml/onnx/nodes/onnx_op.py:646-684).

Every expansion has the library-call shape of the reference's cuDNN convolution
(daceml/onnx/op_implementations/cudnn_implementations.py:209-334): an empty nested SDFG from
`empty_sdfg_for_node`, one `Language.CPP` tasklet whose connectors are `dace.pointer(float32)`
and whose body is a single call into libb200ops on `__dace_current_stream`, and a
`@dace.library.environment` class that adds the header and the shared library to the build.

The C++ text of each tasklet is produced by the `tasklet_*` functions below, which need neither
DaCe nor a GPU (tests compile their output against include/b200_ops.h). Only `_register()` and
the classes it creates import dace / daceml.
"""
import os

HERE = os.path.dirname(os.path.abspath(__file__))
INCLUDE_DIR = os.path.join(os.path.dirname(HERE), "include")
LIB_PATH = os.path.join(HERE, "libb200ops.so")

MATH_MODE_ENV = "B200_MATH_MODE"  # fp32x3 (default) | tf32 | bf16 | fp32, read when a node is expanded
_MATH = {"fp32x3": 0, "tf32": 1, "fp32": 2, "bf16": 3}
_BINARY = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3, "Pow": 4}
_UNARY = {"Sqrt": 0, "Erf": 1, "Relu": 2}

CHECK = """
    if (__b200_rc != 0) {{
        fprintf(stderr, "b200 expansion of {label}: %s\\n", b200_last_error_string());
        abort();
    }}
"""


def math_mode():
    name = os.environ.get(MATH_MODE_ENV, "fp32x3")
    if name not in _MATH:
        raise ValueError("%s must be one of %s" % (MATH_MODE_ENV, sorted(_MATH)))
    return _MATH[name]


def _prod(xs):
    n = 1
    for x in xs:
        n *= int(x)
    return n


def _contig_strides(shape):
    strides, acc = [], 1
    for s in reversed(shape):
        strides.append(acc)
        acc *= int(s)
    return list(reversed(strides))


def _broadcast(a_shape, b_shape):
    """numpy broadcast of two static shapes -> (out_shape, a_strides, b_strides) with 0 on broadcast axes."""
    n = max(len(a_shape), len(b_shape))
    a = [1] * (n - len(a_shape)) + [int(s) for s in a_shape]
    b = [1] * (n - len(b_shape)) + [int(s) for s in b_shape]
    out = []
    for x, y in zip(a, b):
        if x != y and x != 1 and y != 1:
            raise ValueError("shapes %s and %s do not broadcast" % (a_shape, b_shape))
        out.append(max(x, y))
    sa = [0 if d == 1 and o != 1 else s for d, o, s in zip(a, out, _contig_strides(a))]
    sb = [0 if d == 1 and o != 1 else s for d, o, s in zip(b, out, _contig_strides(b))]
    return out, sa, sb


def _two_level_batch(batch_shape, sa, sb, sy):
    dims = [(n, a, b, y) for n, a, b, y in zip(batch_shape, sa, sb, sy) if n != 1]
    merged = []
    for n, a, b, y in dims:
        if merged and merged[-1][1] == a * n and merged[-1][2] == b * n and merged[-1][3] == y * n:
            pn = merged[-1][0]
            merged[-1] = (pn * n, a, b, y)
        else:
            merged.append((n, a, b, y))
    if len(merged) > 2:
        return None
    while len(merged) < 2:
        merged.insert(0, (1, 0, 0, 0))
    return merged


# ---------------------------------------------------------------------------------------------
# C++ tasklet bodies (pure string builders)
# ---------------------------------------------------------------------------------------------
def _gemm_desc_init(a_shape, b_shape, trans_b, bias, mode):
    """Initializer list of the b200_gemm_desc of a MatMul / Gemm node, or None when the broadcast batch cannot
    be expressed with two strided levels."""
    M, K = int(a_shape[-2]), int(a_shape[-1])
    N = int(b_shape[-2]) if trans_b else int(b_shape[-1])
    batch, _, _ = _broadcast(a_shape[:-2], b_shape[:-2])
    ea = list(batch) + [M, K]
    eb = list(batch) + [int(s) for s in b_shape[-2:]]
    _, sa_full, _ = _broadcast(a_shape, ea)
    _, sb_full, _ = _broadcast(b_shape, eb)
    sy_full = _contig_strides(list(batch) + [M, N])
    nb = len(batch)
    levels = _two_level_batch(batch, sa_full[:nb], sb_full[:nb], sy_full[:nb])
    if levels is None:
        return None
    (bo, ao, bbo, yo), (bi, ai, bbi, yi) = levels
    return "{{{bo}, {bi}, {M}, {N}, {K}, {K}, {ldb}, {N}, {ao}, {ai}, {bbo}, {bbi}, {yo}, {yi}, {tb}, {epi}, 1.0f, {mode}}}".format(
        bo=bo, bi=bi, M=M, N=N, K=K, ldb=int(b_shape[-1]), ao=ao, ai=ai, bbo=bbo, bbi=bbi, yo=yo, yi=yi,
        tb=int(trans_b), epi=1 if bias else 0, mode=mode)


def tasklet_matmul(a_shape, b_shape, label="MatMul", trans_b=False, bias=False, mode=None, ws=None):
    """Body for MatMul (A,B -> Y) or Gemm with transB=1 (A,B[,C] -> Y). Returns C++ or None when the
    broadcast batch cannot be expressed with two strided levels. With `ws` (the name of a workspace in the SDFG
    state, see gemm_env_code) the call goes through b200_gemm_ws_f32."""
    mode = math_mode() if mode is None else mode
    init = _gemm_desc_init(a_shape, b_shape, trans_b, bias, mode)
    if init is None:
        return None
    if ws is None:
        call = "b200_gemm_f32(__dace_current_stream, &__b200_d, _A, _B, {bias}, nullptr, _Y)"
    else:
        call = ("b200_gemm_ws_f32(__dace_current_stream, &__b200_d, _A, _B, {bias}, nullptr, _Y,\n"
                "                                     __state->{ws}, __state->{ws}_bytes)")
    return ("\n    b200_gemm_desc __b200_d = " + init + ";\n    int __b200_rc = " +
            call.format(bias="_C" if bias else "nullptr", ws=ws) + ";\n") + CHECK.format(label=label)


def gemm_env_code(a_shape, b_shape, ws_name, trans_b=False, bias=False, mode=None):
    """(state_fields, init_code, finalize_code) of a MatMul / Gemm node whose call can use device scratch
    (b200_gemm_workspace_bytes > 0 for its descriptor): allocated once at SDFG initialisation, freed at exit,
    as cudnn_implementations.py:281-301 does for cuDNN's workspace."""
    mode = math_mode() if mode is None else mode
    init_list = _gemm_desc_init(a_shape, b_shape, trans_b, bias, mode)
    fields = ["void *%s;" % ws_name, "size_t %s_bytes;" % ws_name]
    init = """
    {{
        b200_gemm_desc d = {init};
        __state->{ws}_bytes = b200_gemm_workspace_bytes(&d);
        __state->{ws} = nullptr;
        if (__state->{ws}_bytes && cudaMalloc(&__state->{ws}, __state->{ws}_bytes) != cudaSuccess) {{
            fprintf(stderr, "b200: cannot allocate %zu bytes of GEMM workspace\\n", __state->{ws}_bytes);
            abort();
        }}
    }}
""".format(init=init_list, ws=ws_name)
    fini = "\n    if (__state->{ws}) cudaFree(__state->{ws});\n".format(ws=ws_name)
    return fields, init, fini


def tasklet_conv(x_shape, w_shape, pads, strides, bias, label="Conv", mode=None):
    """Body for Conv (X,W[,B] -> Y); the workspace pointer lives in the SDFG state (see conv_env_code)."""
    mode = math_mode() if mode is None else mode
    n, c, h, w = [int(s) for s in x_shape]
    m, _, kh, kw = [int(s) for s in w_shape]
    return """
    b200_conv_desc __b200_d = {{{n}, {c}, {h}, {w}, {m}, {kh}, {kw}, {ph}, {pw}, {sh}, {sw}, {epi}, {mode}}};
    int __b200_rc = b200_conv2d_f32(__dace_current_stream, &__b200_d, _X, _W, {bias}, _Y,
                                    __state->{{ws}}, __state->{{ws}}_bytes);
""".format(n=n, c=c, h=h, w=w, m=m, kh=kh, kw=kw, ph=int(pads[0]), pw=int(pads[1]), sh=int(strides[0]),
           sw=int(strides[1]), epi=1 if bias else 0, mode=mode, bias="_B" if bias else "nullptr") + \
        CHECK.format(label=label)


def conv_env_code(x_shape, w_shape, pads, strides, ws_name, mode=None):
    """(state_fields, init_code, finalize_code): the workspace is allocated once at SDFG
    initialisation and freed at exit, as cudnn_implementations.py:281-301 does for cuDNN's."""
    mode = math_mode() if mode is None else mode
    n, c, h, w = [int(s) for s in x_shape]
    m, _, kh, kw = [int(s) for s in w_shape]
    fields = ["void *%s;" % ws_name, "size_t %s_bytes;" % ws_name]
    init = """
    {{
        b200_conv_desc d = {{{n}, {c}, {h}, {w}, {m}, {kh}, {kw}, {ph}, {pw}, {sh}, {sw}, 0, {mode}}};
        __state->{ws}_bytes = b200_conv2d_workspace_bytes(&d);
        __state->{ws} = nullptr;
        if (__state->{ws}_bytes && cudaMalloc(&__state->{ws}, __state->{ws}_bytes) != cudaSuccess) {{
            fprintf(stderr, "b200: cannot allocate %zu bytes of convolution workspace\\n", __state->{ws}_bytes);
            abort();
        }}
    }}
""".format(n=n, c=c, h=h, w=w, m=m, kh=kh, kw=kw, ph=int(pads[0]), pw=int(pads[1]), sh=int(strides[0]),
           sw=int(strides[1]), mode=mode, ws=ws_name)
    fini = "\n    if (__state->{ws}) cudaFree(__state->{ws});\n".format(ws=ws_name)
    return fields, init, fini


def tasklet_maxpool(x_shape, kernel_shape, strides, label="MaxPool"):
    """Body for MaxPool (X -> Y), 2-D, pads 0, floor mode (the cases PureMaxPool2D accepts,
    img_op_implementations.py:31-61)."""
    n, c, h, w = [int(s) for s in x_shape]
    kh, kw = [int(k) for k in kernel_shape]
    sh, sw = [int(s) for s in (strides or [1, 1])]
    return """
    int __b200_rc = b200_maxpool2d_f32(__dace_current_stream, _X, _Y, {planes}, {h}, {w}, {kh}, {kw}, {sh}, {sw});
""".format(planes=n * c, h=h, w=w, kh=kh, kw=kw, sh=sh, sw=sw) + CHECK.format(label=label)


def _axis_view(shape, axis):
    nd = len(shape)
    axis = int(axis) % nd
    return _prod(shape[:axis]), int(shape[axis]), _prod(shape[axis + 1:])


def tasklet_softmax(shape, axis, log=False, label="Softmax"):
    outer, length, inner = _axis_view(shape, axis)
    return """
    int __b200_rc = b200_{fn}_f32(__dace_current_stream, _input, _output, {o}, {l}, {i});
""".format(fn="logsoftmax" if log else "softmax", o=outer, l=length, i=inner) + CHECK.format(label=label)


def tasklet_reduce_mean(shape, axes, label="ReduceMean"):
    nd = len(shape)
    ax = sorted(int(a) % nd for a in axes)
    if ax != list(range(ax[0], ax[-1] + 1)):
        return None
    return """
    int __b200_rc = b200_reduce_mean_f32(__dace_current_stream, _data, _reduced, {o}, {l}, {i});
""".format(o=_prod(shape[:ax[0]]), l=_prod(shape[ax[0]:ax[-1] + 1]), i=_prod(shape[ax[-1] + 1:])) + \
        CHECK.format(label=label)


def tasklet_binary(op, a_shape, b_shape, names=("_A", "_B", "_C")):
    out, sa, sb = _broadcast(a_shape, b_shape)
    if len(out) > 8:
        return None
    arr = lambda xs: "{" + ", ".join(str(int(x)) for x in (xs or [1])) + "}"  # noqa: E731
    return """
    const int64_t __b200_shape[] = {shape};
    const int64_t __b200_sa[] = {sa};
    const int64_t __b200_sb[] = {sb};
    int __b200_rc = b200_binary_f32(__dace_current_stream, {code}, {a}, {b}, {c}, {rank}, __b200_shape, __b200_sa,
                                    __b200_sb);
""".format(shape=arr(out), sa=arr(sa), sb=arr(sb), code=_BINARY[op], a=names[0], b=names[1], c=names[2],
           rank=len(out)) + CHECK.format(label=op)


def tasklet_unary(op, shape, names=("_X", "_Y")):
    return """
    int __b200_rc = b200_unary_f32(__dace_current_stream, {code}, {x}, {y}, {n});
""".format(code=_UNARY[op], x=names[0], y=names[1], n=_prod(shape)) + CHECK.format(label=op)


# ---------------------------------------------------------------------------------------------
# DaCeML side (needs dace + daceml)
# ---------------------------------------------------------------------------------------------
_REGISTERED = {}


def _register():
    """Define and register the expansions. Raises ImportError where DaCe / DaCeML are missing."""
    if _REGISTERED:
        return _REGISTERED
    import dace
    import dace.library
    from dace import dtypes
    from dace.libraries.standard import CUDA
    from daceml.onnx.forward_implementation_abc import ONNXForward
    from daceml.onnx.op_implementations.utils import empty_sdfg_for_node, op_implementation
    from daceml.util.utils import in_desc_with_name, is_cuda, is_desc_contiguous, out_desc_with_name

    @dace.library.environment
    class B200Ops:
        """Build environment of libb200ops (pattern: daceml/onnx/environments/cudnn.py:11-69)."""
        cmake_minimum_version = None
        cmake_packages = []
        cmake_variables = {}
        cmake_includes = [INCLUDE_DIR]
        cmake_libraries = [LIB_PATH]
        cmake_compile_flags = []
        cmake_link_flags = []
        cmake_files = []
        state_fields = []
        dependencies = [CUDA]
        headers = ["b200_ops.h", "cstdio", "cstdlib"]
        init_code = ""
        finalize_code = ""

    def on_gpu(desc):
        # The kernels take device pointers: a descriptor in host (or FPGA) storage -- an SDFG built with
        # cuda=False -- is not ours (daceml/util/utils.py:236-245 is the reference's test for a GPU array).
        try:
            return is_cuda(desc.storage)
        except ValueError:
            return False

    def static_f32(desc):
        return (desc.dtype == dace.float32 and is_desc_contiguous(desc) and on_gpu(desc)
                and not any(dace.symbolic.issymbolic(s) for s in desc.shape))

    def unique_id(node, state, sdfg):
        # one state field per node instance: node name + SDFG id + state id + node id, as the reference's cuDNN
        # expansion names its descriptors (cudnn_implementations.py:205-207); two nodes with the same label in
        # different nested SDFGs must not share a workspace field
        name = "".join(ch if ch.isalnum() else "_" for ch in str(getattr(node, "name", None) or node.label))
        return "b200_ws_%s_%s_%s_%s" % (name, sdfg.sdfg_id, sdfg.node_id(state), state.node_id(node))

    def descs(node, state, sdfg, ins, outs):
        found = {}
        for n in ins:
            if n in node.in_connectors:
                found[n] = in_desc_with_name(node, state, sdfg, n)
        for n in outs:
            found[n] = out_desc_with_name(node, state, sdfg, n)
        return found

    def emit(node, state, sdfg, code, ins, outs, env=B200Ops):
        """One CPP tasklet calling the C ABI, wired to every connector the node has."""
        nsdfg, nstate, inputs, outputs = empty_sdfg_for_node(sdfg, state, node)
        T = dace.pointer(dace.float32)
        tasklet = nstate.add_tasklet(node.label + "_b200", {"_" + n: T for n in ins if n in inputs},
                                     {"_" + n: T for n in outs}, code, dtypes.Language.CPP)
        for n in ins:
            if n in inputs:
                nstate.add_edge(inputs[n], None, tasklet, "_" + n, nsdfg.make_array_memlet(n))
        for n in outs:
            nstate.add_edge(tasklet, "_" + n, outputs[n], None, nsdfg.make_array_memlet(n))
        return nsdfg, env

    def make(op, ins, outs, can_apply, build):
        class Impl(ONNXForward):
            environments = [B200Ops]

            @staticmethod
            def forward_can_be_applied(node, state, sdfg):
                d = descs(node, state, sdfg, ins, outs)
                return all(static_f32(x) for x in d.values()) and can_apply(node, d)

            @staticmethod
            def forward(node, state, sdfg):
                d = descs(node, state, sdfg, ins, outs)
                code, env = build(node, d, unique_id(node, state, sdfg))
                nsdfg, env = emit(node, state, sdfg, code, ins, outs, env or B200Ops)
                Impl.environments = [env]
                return nsdfg

        Impl.__name__ = "B200" + op
        Impl.__doc__ = "b200 expansion of ONNX%s through libb200ops." % op
        _REGISTERED[op] = op_implementation(op=op, name="b200")(Impl)

    def gemm_build(node, d, ws, trans_b, bias):
        # fp32-accurate and bf16 modes: the node gets device scratch from the SDFG state, like the cuDNN expansion
        if math_mode() not in (0, 3):
            return tasklet_matmul(d["A"].shape, d["B"].shape, node.label, trans_b=trans_b, bias=bias), None
        fields, init, fini = gemm_env_code(d["A"].shape, d["B"].shape, ws, trans_b=trans_b, bias=bias)

        class GemmEnv(B200Ops):
            state_fields = fields
            init_code = init
            finalize_code = fini
        GemmEnv.__name__ = ws + "_environment"
        env = dace.library.environment(GemmEnv)
        return tasklet_matmul(d["A"].shape, d["B"].shape, node.label, trans_b=trans_b, bias=bias, ws=ws), env

    make("MatMul", ["A", "B"], ["Y"],
         lambda node, d: len(d["A"].shape) > 1 and len(d["B"].shape) > 1 and
         tasklet_matmul(d["A"].shape, d["B"].shape) is not None,
         lambda node, d, uid: gemm_build(node, d, uid, False, False))
    make("Gemm", ["A", "B", "C"], ["Y"],
         lambda node, d: node.alpha == 1.0 and node.beta == 1.0 and node.transA == 0 and node.transB == 1 and
         ("C" not in d or (_prod(d["C"].shape) == d["B"].shape[0] and int(d["C"].shape[-1]) == d["B"].shape[0])),
         lambda node, d, uid: gemm_build(node, d, uid, True, "C" in d))

    def conv_build(node, d, ws):
        pads = node.pads if node.pads is not None else [0, 0, 0, 0]
        strides = node.strides if node.strides is not None else [1, 1]
        fields, init, fini = conv_env_code(d["X"].shape, d["W"].shape, pads, strides, ws)

        class ConvEnv(B200Ops):
            state_fields = fields
            init_code = init
            finalize_code = fini
        ConvEnv.__name__ = ws + "_environment"
        env = dace.library.environment(ConvEnv)
        code = tasklet_conv(d["X"].shape, d["W"].shape, pads, strides, "B" in d, node.label).replace("{ws}", ws)
        return code, env

    make("Conv", ["X", "W", "B"], ["Y"],
         lambda node, d: len(d["X"].shape) == 4 and len(d["W"].shape) == 4 and node.group == 1 and
         node.auto_pad == "NOTSET" and (node.dilations is None or all(x == 1 for x in node.dilations)) and
         (node.pads is None or (node.pads[0] == node.pads[2] and node.pads[1] == node.pads[3])),
         conv_build)
    make("MaxPool", ["X"], ["Y"],
         lambda node, d: len(d["X"].shape) == 4 and len(node.kernel_shape) == 2 and
         (node.pads is None or all(p == 0 for p in node.pads)) and node.auto_pad == "NOTSET" and
         node.ceil_mode == 0 and node.storage_order == 0 and
         (node.dilations is None or all(x == 1 for x in node.dilations)),
         lambda node, d, uid: (tasklet_maxpool(d["X"].shape, node.kernel_shape, node.strides, node.label), None))
    make("Softmax", ["input"], ["output"], lambda node, d: True,
         lambda node, d, uid: (tasklet_softmax(d["input"].shape, node.axis, False, node.label), None))
    make("LogSoftmax", ["input"], ["output"], lambda node, d: True,
         lambda node, d, uid: (tasklet_softmax(d["input"].shape, node.axis, True, node.label), None))
    make("ReduceMean", ["data"], ["reduced"],
         lambda node, d: tasklet_reduce_mean(d["data"].shape, node.axes) is not None,
         lambda node, d, uid: (tasklet_reduce_mean(d["data"].shape, node.axes, node.label), None))
    for op in ("Add", "Sub", "Mul", "Div"):
        make(op, ["A", "B"], ["C"], lambda node, d, op=op: tasklet_binary(op, d["A"].shape, d["B"].shape) is not None,
             lambda node, d, uid, op=op: (tasklet_binary(op, d["A"].shape, d["B"].shape), None))
    make("Pow", ["X", "Y"], ["Z"],
         lambda node, d: tasklet_binary("Pow", d["X"].shape, d["Y"].shape, ("_X", "_Y", "_Z")) is not None,
         lambda node, d, uid: (tasklet_binary("Pow", d["X"].shape, d["Y"].shape, ("_X", "_Y", "_Z")), None))
    make("Sqrt", ["X"], ["Y"], lambda node, d: True,
         lambda node, d, uid: (tasklet_unary("Sqrt", d["X"].shape), None))
    make("Relu", ["X"], ["Y"], lambda node, d: True,
         lambda node, d, uid: (tasklet_unary("Relu", d["X"].shape), None))
    make("Erf", ["input"], ["output"], lambda node, d: True,
         lambda node, d, uid: (tasklet_unary("Erf", d["input"].shape, ("_input", "_output")), None))
    return _REGISTERED


def register_late():
    """Register the `b200` expansions on the already generated node classes.

    Node classes collect their implementations once, while `daceml.onnx.nodes.onnx_op` is imported
    (onnx_op.py:646-684). A module loaded after that must repeat what that loop does for each of its
    classes: wrap it in an ExpandTransformation and call `register_implementation`. Unlike the
    stock wrapper, a node this implementation cannot take is handed to the `pure` expansion (which
    DaCe moves to the GPU), never to ONNX Runtime.
    """
    import daceml.onnx as donnx
    from dace.transformation.transformation import ExpandTransformation
    from daceml.onnx.forward_implementation_abc import ONNXForward

    impls = _register()
    for op, impl in impls.items():
        node_cls = getattr(donnx, "ONNX" + op)
        if "b200" in node_cls.implementations:
            continue
        pure = dict(ONNXForward.registered_implementations(op)).get("pure")

        class Expansion(ExpandTransformation):
            environments = []
            forward_impl = impl
            pure_impl = pure

            @classmethod
            def expansion(cls, node, state, sdfg):
                node.validate(sdfg, state)
                if cls.forward_impl.forward_can_be_applied(node, state, sdfg):
                    result = cls.forward_impl.forward(node, state, sdfg)
                    cls.environments.extend(getattr(cls.forward_impl, "environments", []))
                    return result
                if cls.pure_impl is not None and cls.pure_impl.forward_can_be_applied(node, state, sdfg):
                    return cls.pure_impl.forward(node, state, sdfg)
                raise NotImplementedError("b200: node %s is outside this implementation and has no pure "
                                          "expansion; refusing to fall back to ONNX Runtime" % node.label)

        Expansion.__name__ = "B200Expansion" + op
        node_cls.register_implementation("b200", Expansion)
    return sorted(impls)


try:  # in-tree use: importing the module registers the classes, like the other *_implementations.py
    _register()
except ImportError:
    pass
