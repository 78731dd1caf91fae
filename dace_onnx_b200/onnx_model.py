"""ONNXModelB200: run an exported ONNX inference graph on the b200 kernels, without DaCe.

The caller-side mirror of the reference's front door (`daceml.onnx.ONNXModel`,
daceml/onnx/onnx_importer.py:59-140 construction, :444-486 `__call__`): construct from a model,
call with positional or named inputs, get torch tensors back. Where the reference lowers the graph
to an SDFG and expands every node, this class specialises the graph to the input shapes
(`onnx_graph.specialize`), applies the chain fusions (`fusion.run_all`), plans the intermediate
buffers once, and then each call only launches kernels of libb200ops on torch's current stream.

Only the node types of the hot path are executable (MatMul, Gemm, Conv, Softmax, LogSoftmax,
ReduceMean, Add/Sub/Mul/Div/Pow, Sqrt, Erf, Relu, plus MaxPool and Transpose / Reshape-style views between them);
anything else raises `UnsupportedNode` when the plan is built - there is no other runtime to fall back on,
and nothing here computes on the CPU.
"""
import re
from typing import Dict, List, Sequence

import numpy as np
import torch

from . import _lib, fusion, onnx_wire, ops
from .onnx_graph import GraphIR, UnsupportedNode, specialize

_VIEW_OPS = ("Reshape", "Flatten", "Squeeze", "Unsqueeze", "Identity", "Dropout")
_BINARY = {"Add": ops.ADD, "Sub": ops.SUB, "Mul": ops.MUL, "Div": ops.DIV, "Pow": ops.POW}
_UNARY = {"Sqrt": ops.SQRT, "Erf": ops.ERF, "Relu": ops.RELU, "B200Gelu": ops.GELU}
_EPILOGUES = {"none": ops.EPI_NONE, "bias": ops.EPI_BIAS, "bias_relu": ops.EPI_BIAS_RELU,
              "bias_gelu": ops.EPI_BIAS_GELU, "bias_residual": ops.EPI_BIAS_RESIDUAL, "scale": ops.EPI_SCALE}


def clean_name(name: str) -> str:
    """Keyword form of a graph value name ('onnx::MatMul_0' -> 'onnx__MatMul_0')."""
    s = re.sub(r"[^0-9a-zA-Z_]", "_", name)
    return "ONNX_" + s if s[:1].isdigit() else s


class _Plan:
    """One specialisation of the graph: fused node list, device constants, buffer assignment."""

    def __init__(self, model: onnx_wire.Model, shapes, device, fuse: bool, math_mode):
        self.device = device
        self.math_mode = math_mode
        self.ir: GraphIR = specialize(model, shapes)
        self.fusion_stats = fusion.run_all(self.ir) if fuse else {}
        self._consts: Dict[str, torch.Tensor] = {}
        self._scratch: Dict[str, torch.Tensor] = {}
        self._nhwc: Dict[str, tuple] = {}   # values kept in [N, H, W, C] between two convolutions -> that shape
        if fuse:
            self.fusion_stats["conv_nhwc_links"] = self._mark_conv_layouts()
        self.steps = []
        self._build()

    # -- constants -----------------------------------------------------------------------------------
    def const(self, name: str) -> torch.Tensor:
        t = self._consts.get(name)
        if t is None:
            arr = self.ir.consts[name]
            if arr.dtype != np.float32:
                raise UnsupportedNode("constant '%s' of type %s feeds a device node (only float32 is supported)" %
                                      (name, arr.dtype))
            t = torch.from_numpy(np.ascontiguousarray(arr)).to(self.device)
            self._consts[name] = t
        return t

    def scratch(self, key: str, numel: int) -> torch.Tensor:
        t = self._scratch.get(key)
        if t is None or t.numel() < numel:
            t = torch.empty(numel, device=self.device, dtype=torch.float32)
            self._scratch[key] = t
        return t

    # -- convolution layouts ---------------------------------------------------------------------------
    def _conv_geometry(self, node):
        ir = self.ir
        x, w = ir.shapes[node.inputs[0]], tuple(ir.consts[node.inputs[1]].shape)
        pads = tuple(node.attr("pads", [0, 0, 0, 0]))
        strides = tuple(node.attr("strides", [1, 1]))
        return x, w, pads, strides

    def _conv_takes_nhwc(self, node) -> bool:
        ir = self.ir
        if node.inputs[1] not in ir.consts or (len(node.inputs) > 2 and node.inputs[2] and node.inputs[2] not in ir.consts):
            return False
        x, w, pads, strides = self._conv_geometry(node)
        if len(x) != 4 or len(w) != 4 or node.attr("group", 1) != 1 or tuple(node.attr("dilations", [1, 1])) != (1, 1) or \
                pads[0] != pads[2] or pads[1] != pads[3]:
            return False
        d = ops.ConvDesc(x[0], x[1], x[2], x[3], w[0], w[2], w[3], pads[0], pads[1], strides[0], strides[1], 0,
                         ops._math(self.math_mode))
        import ctypes
        return bool(_lib.load().b200_conv2d_nhwc_supported(ctypes.byref(d)))

    def _mark_conv_layouts(self) -> int:
        """A value produced by one convolution and read only by the next stays in [N, H, W, C], the layout the
        tensor-core kernel reads and writes natively: only the first input and the last output of a chain of
        convolutions pay the NCHW <-> NHWC change. Returns the number of such links."""
        ir = self.ir
        consumers = ir.consumers()
        links = 0
        for node in ir.nodes:
            if node.op_type != "Conv":
                continue
            out = node.outputs[0]
            users = consumers.get(out, [])
            if out in ir.outputs or len(users) != 1 or users[0].op_type != "Conv" or users[0].inputs[0] != out or \
                    out in users[0].inputs[1:]:
                continue
            if not (self._conv_takes_nhwc(node) and self._conv_takes_nhwc(users[0])):
                continue
            n, m, oh, ow = ir.shapes[out]
            self._nhwc[out] = (n, oh, ow, m)
            node.attrs["y_nhwc"] = 1
            users[0].attrs["x_nhwc"] = 1
            links += 1
        return links

    # -- planning ------------------------------------------------------------------------------------
    def _build(self):
        ir = self.ir
        root: Dict[str, str] = {}

        def rt(n):
            while n in root:
                n = root[n]
            return n

        for node in ir.nodes:
            if node.op_type in _VIEW_OPS or (node.op_type == "Transpose" and self._is_identity_perm(node)):
                root[node.outputs[0]] = rt(node.inputs[0])
        self._root = rt
        # storage that backs a graph output is allocated per call (the caller keeps what it gets back)
        per_call = {rt(o) for o in ir.outputs if o not in ir.consts}
        external = set(ir.inputs) | set(ir.consts)
        last_use: Dict[str, int] = {}
        for i, node in enumerate(ir.nodes):
            for name in node.inputs:
                if name:
                    last_use[rt(name)] = i
        free: Dict[int, List[torch.Tensor]] = {}
        self.prealloc: Dict[str, torch.Tensor] = {}
        self.per_call: Dict[str, tuple] = {}
        owned: Dict[str, torch.Tensor] = {}
        allocated = 0
        for i, node in enumerate(ir.nodes):
            out = node.outputs[0]
            r = rt(out)
            if r == out and r not in external:
                shape = self._nhwc.get(out, ir.shapes[out])
                numel = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
                if r in per_call:
                    self.per_call[r] = shape
                else:
                    pool = free.get(numel)
                    if pool:
                        buf = pool.pop()
                    else:
                        buf = torch.empty(numel, device=self.device, dtype=torch.float32)
                        allocated += numel
                    owned[r] = buf
                    self.prealloc[r] = buf.view(shape)
            self.steps.append(self._step(node))
            for name in {rt(n) for n in node.inputs if n}:
                if last_use.get(name) == i and name in owned:
                    buf = owned.pop(name)
                    free.setdefault(buf.numel(), []).append(buf)
        self.buffer_bytes = 4 * allocated  # intermediates held by this plan (scratch of fused nodes not counted)

    @staticmethod
    def _is_identity_perm(node):
        perm = node.attr("perm")
        return perm is not None and list(perm) == list(range(len(perm)))

    # -- one closure per node --------------------------------------------------------------------------
    def _step(self, node):
        op, ir, mm = node.op_type, self.ir, self.math_mode
        ins, out = node.inputs, node.outputs[0]
        for name in ins:
            if name and name in ir.consts and op not in ("Reshape",):
                self.const(name)  # upload once, at plan time

        if op in _VIEW_OPS or (op == "Transpose" and self._is_identity_perm(node)):
            shape = ir.shapes[out]
            return lambda env: env.__setitem__(out, env[ins[0]].view(shape))
        if op in _BINARY:
            code = _BINARY[op]
            return lambda env: ops._binary(code, env[ins[0]], env[ins[1]], env[out])
        if op in _UNARY:
            code = _UNARY[op]
            return lambda env: ops._unary(code, env[ins[0]], env[out])
        if op in ("Softmax", "LogSoftmax"):
            fn = ops.softmax if op == "Softmax" else ops.logsoftmax
            axis = node.attr("axis", 1)
            return lambda env: fn(env[ins[0]], axis, out=env[out])
        if op == "ReduceMean":
            rank = len(ir.shapes[ins[0]])
            axes = node.attr("axes") or list(range(rank))
            keep = node.attr("keepdims", 1)
            return lambda env: ops.reduce_mean(env[ins[0]], axes, keep, out=env[out])
        if op == "B200LayerNorm":
            eps = node.attr("epsilon")
            return lambda env: ops.layernorm(env[ins[0]], env[ins[1]] if ins[1] else None,
                                             env[ins[2]] if ins[2] else None, eps, out=env[out])
        if op == "MatMul":
            tb = bool(node.attr("trans_b", 0))
            return lambda env: ops.matmul(env[ins[0]], env[ins[1]], out=env[out], trans_b=tb, math_mode=mm)
        if op == "B200Gemm":
            tb = bool(node.attr("trans_b", 0))
            epi = _EPILOGUES[node.attr("epilogue")]
            scale = node.attr("scale", 1.0)
            return lambda env: ops.matmul(env[ins[0]], env[ins[1]], out=env[out], trans_b=tb, epilogue=epi,
                                          bias=env[ins[2]] if ins[2] else None,
                                          residual=env[ins[3]] if ins[3] else None, scale=scale, math_mode=mm)
        if op == "MaxPool":
            ks, st = node.attr("kernel_shape"), node.attr("strides") or [1, 1]
            return lambda env: ops.maxpool2d(env[ins[0]], ks, st, out=env[out])
        if op == "Gemm":
            return self._gemm_step(node)
        if op == "Conv":
            return self._conv_step(node)
        if op == "Transpose":
            perm = list(node.attr("perm") or list(range(len(ir.shapes[ins[0]])))[::-1])
            rank = len(perm)
            if rank == 4 and perm == [0, 2, 1, 3]:
                return lambda env: ops.transpose_0213(env[ins[0]], out=env[out])
            if rank >= 2 and perm == list(range(rank - 2)) + [rank - 1, rank - 2]:
                return lambda env: ops.transpose_last2(env[ins[0]], out=env[out])
            return lambda env: ops.permute(env[ins[0]], perm, out=env[out])
        if op in ("B200Attention", "B200SelfAttention"):
            return self._attention_step(node)
        raise UnsupportedNode("node '%s': operator %s cannot be executed" % (node.name, op))

    def _gemm_step(self, node):
        ins, out, mm = node.inputs, node.outputs[0], self.math_mode
        if node.attr("alpha", 1.0) != 1.0 or node.attr("beta", 1.0) != 1.0 or node.attr("transA", 0):
            raise UnsupportedNode("Gemm '%s': only alpha=1, beta=1, transA=0 is supported" % node.name)
        tb = bool(node.attr("transB", 0))
        has_c = len(ins) > 2 and bool(ins[2])

        def run(env):
            y = ops.matmul(env[ins[0]], env[ins[1]], out=env[out], trans_b=tb, math_mode=mm)
            if has_c:
                ops._binary(ops.ADD, y, env[ins[2]], y)

        return run

    def _conv_step(self, node):
        ins, out, mm, ir = node.inputs, node.outputs[0], self.math_mode, self.ir
        pads = tuple(node.attr("pads", [0, 0, 0, 0]))
        strides = tuple(node.attr("strides", [1, 1]))
        dil = tuple(node.attr("dilations", [1, 1]))
        group = node.attr("group", 1)
        relu = bool(node.attr("relu", 0))
        has_b = len(ins) > 2 and bool(ins[2])
        x_nhwc, y_nhwc = bool(node.attr("x_nhwc", 0)), bool(node.attr("y_nhwc", 0))
        const_filter = ins[1] in ir.consts and (not has_b or ins[2] in ir.consts)
        if const_filter and (self.fusion_stats or x_nhwc or y_nhwc):
            # constant filter: repacked (and split) once, when the plan is built -- what the reference's cuDNN
            # expansion does with its descriptors in the SDFG init hook (cudnn_implementations.py:281-301)
            conv = ops.PreparedConv(self.const(ins[1]), self.const(ins[2]) if has_b else None, pads=pads,
                                    strides=strides, dilations=dil, group=group, relu=relu, math_mode=mm)
            n = ir.shapes[ins[0]][0]
            need = 0 if x_nhwc else int(np.prod(ir.shapes[ins[0]], dtype=np.int64)) + 64
            ws = self.scratch("conv_ws", need).view(torch.uint8) if need else None

            def run_prepared(env):
                conv(env[ins[0]], out=env[out], x_nhwc=x_nhwc, y_nhwc=y_nhwc, workspace=ws)

            return run_prepared
        need = ops.conv2d_workspace_bytes(ir.shapes[ins[0]], tuple(ir.consts[ins[1]].shape) if ins[1] in ir.consts
                                          else ir.shapes[ins[1]], pads, strides, mm)
        ws = self.scratch("conv_ws", (need + 3) // 4) if need else None

        def run(env):
            ops.conv2d(env[ins[0]], env[ins[1]], env[ins[2]] if has_b else None, out=env[out], pads=pads,
                       strides=strides, dilations=dil, group=group, relu=relu, workspace=ws, math_mode=mm)

        return run

    def _attention_step(self, node):
        ins, out, mm, ir = node.inputs, node.outputs[0], self.math_mode, self.ir
        heads, scale = node.attr("heads"), float(node.attr("scale"))
        b, s, hidden = ir.shapes[out]
        d = hidden // heads
        merged = node.op_type == "B200SelfAttention"
        if merged:
            # [K, 3H] weight and [3H] bias of the single projection GEMM, assembled once on the device
            w = torch.cat([self.const(ins[1]), self.const(ins[3]), self.const(ins[5])], dim=1).contiguous()
            bias = torch.cat([self.const(ins[2]), self.const(ins[4]), self.const(ins[6])]).contiguous()
            qkv = self.scratch("qkv", b * s * 3 * hidden)[:b * s * 3 * hidden].view(b, s, 3 * heads, d)
            k_in = ir.shapes[ins[0]][-1]

        def run(env):
            if merged:
                ops.matmul(env[ins[0]].view(b * s, k_in), w, out=qkv.view(b * s, 3 * hidden), trans_b=False,
                           epilogue=ops.EPI_BIAS, bias=bias, math_mode=mm)
                q, k, v = qkv[:, :, :heads], qkv[:, :, heads:2 * heads], qkv[:, :, 2 * heads:]
            else:
                q, k, v = (env[n].view(b, s, heads, d) for n in ins[:3])
            o = env[out].view(b, s, heads, d)
            if ops.attention_views(q, k, v, o, scale, math_mode=mm):
                return
            # MatMul -> Mul -> Softmax -> MatMul on strided head views: no head transposes are materialised
            n_sc = b * heads * s * s
            scores = self.scratch("scores", n_sc)[:n_sc].view(b, heads, s, s)
            probs = self.scratch("probs", n_sc)[:n_sc].view(b, heads, s, s)
            ops.gemm_raw(q, k, scores, batch_outer=b, batch_inner=heads, M=s, N=s, K=d, lda=q.stride(1),
                         ldb=k.stride(1), ldy=s, a_strides=(q.stride(0), q.stride(2)),
                         b_strides=(k.stride(0), k.stride(2)), y_strides=(heads * s * s, s * s), trans_b=True,
                         epilogue=ops.EPI_SCALE, scale=scale, math_mode=mm)
            ops.softmax(scores, 3, out=probs)
            ops.gemm_raw(probs, v, o, batch_outer=b, batch_inner=heads, M=s, N=d, K=s, lda=s, ldb=v.stride(1),
                         ldy=o.stride(1), a_strides=(heads * s * s, s * s), b_strides=(v.stride(0), v.stride(2)),
                         y_strides=(o.stride(0), o.stride(2)), trans_b=False, math_mode=mm)

        return run

    # -- execution -------------------------------------------------------------------------------------
    def run(self, inputs: Sequence[torch.Tensor]):
        env: Dict[str, torch.Tensor] = dict(self._consts)
        env.update(self.prealloc)
        for name, t in zip(self.ir.inputs, inputs):
            env[name] = t
        for name, shape in self.per_call.items():
            env[name] = torch.empty(shape, device=self.device, dtype=torch.float32)
        for step in self.steps:
            step(env)
        outs = []
        for o in self.ir.outputs:
            if o in env:
                outs.append(env[o])
            elif o in self.ir.consts:
                outs.append(self.const(o).clone())
            else:
                r = self._root(o)
                outs.append(env[r].view(self.ir.shapes[o]))
        return outs


class _GraphReplay:
    """A plan captured into a CUDA graph: one launch per call instead of one per node. The captured kernels
    read input buffers owned by the replay and write output buffers that were current at capture time: inputs are
    first copied into those buffers (unless the caller passes the buffers themselves, see
    ONNXModelB200.static_inputs), and the returned tensors are overwritten by the next call."""

    def __init__(self, plan: _Plan, inputs: Sequence[torch.Tensor]):
        self.plan = plan
        self.inputs = [t.to(plan.device, copy=True) for t in inputs]
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream(device=plan.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):  # every lazily created scratch buffer and per-device table exists before the capture
                plan.run(self.inputs)
        cur.wait_stream(side)
        torch.cuda.synchronize(plan.device)
        _lib.device_status()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.outputs = plan.run(self.inputs)

    def __call__(self, inputs: Sequence[torch.Tensor]):
        for mine, given in zip(self.inputs, inputs):
            if mine.data_ptr() != given.data_ptr():
                mine.copy_(given, non_blocking=True)
        self.graph.replay()
        return self.outputs


class ONNXModelB200:
    """Loads an ONNX model and executes it on one B200.

    :param name: a label for messages.
    :param model: serialized ModelProto (bytes), a path to one, or an `onnx_wire.Model`.
    :param cuda: must be True; kept so that call sites of the reference (`ONNXModel(name, model, cuda=True)`)
                 read the same. There is no CPU execution.
    :param fuse: apply the chain fusions (LayerNorm, Gelu, attention, GEMM epilogues, weight transposes).
                 With False every exported node runs as its own kernel, the way the reference's per-node
                 expansion does.
    :param math_mode: "fp32x3" (fp32-accurate, default), "tf32" or "fp32" for the contractions.
    :param cuda_graph: capture each plan into a CUDA graph on its first call and replay it afterwards (for
                 graphs of many small kernels, where launch latency dominates). The returned tensors are then
                 owned by the model and overwritten by its next call with the same input shapes.
    """

    def __init__(self, name, model, cuda=True, fuse=True, math_mode=None, device=None, cuda_graph=False):
        if not cuda:
            raise ValueError("ONNXModelB200 runs on a CUDA device only (cuda=False is not available)")
        if isinstance(model, onnx_wire.Model):
            self.model = model
        elif isinstance(model, (bytes, bytearray, memoryview)):
            self.model = onnx_wire.parse_model(model)
        else:
            self.model = onnx_wire.load_model(model)
        self.name = name
        self.fuse = fuse
        self.math_mode = math_mode
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        # Models of other opsets are accepted: onnx_graph.specialize rewrites the nodes whose definition changed
        # after opset 12 (Softmax / LogSoftmax default axis, `axes` as an input) or refuses them at plan time.
        _lib.load()  # fail now, not at the first call, when the CUDA library is missing
        self._plans: Dict[tuple, _Plan] = {}
        self.cuda_graph = bool(cuda_graph)
        self._replays: Dict[tuple, _GraphReplay] = {}

    @property
    def input_names(self):
        return [vi.name for vi in self.model.graph.inputs]

    @property
    def output_names(self):
        return [vi.name for vi in self.model.graph.outputs]

    def plan(self, *shapes) -> _Plan:
        """The execution plan for one set of input shapes (built on first use, then cached)."""
        key = tuple(tuple(int(d) for d in s) for s in shapes)
        p = self._plans.get(key)
        if p is None:
            with torch.cuda.device(self.device):
                p = _Plan(self.model, key, self.device, self.fuse, self.math_mode)
            self._plans[key] = p
        return p

    def static_inputs(self, *shapes):
        """With cuda_graph=True: the input buffers the captured graph of these shapes reads (after its first call).
        Filling them in place and passing them to the call avoids the copy of the inputs."""
        key = tuple(tuple(int(d) for d in s) for s in shapes)
        if key not in self._replays:
            raise KeyError("no captured graph for input shapes %s yet" % (key,))
        return list(self._replays[key].inputs)

    def _bind(self, args, kwargs):
        names = self.input_names
        if len(args) > len(names):
            raise TypeError("%s takes %d inputs, got %d" % (self.name, len(names), len(args)))
        given = dict(zip(names, args))
        lookup = {clean_name(n): n for n in names}
        for k, v in kwargs.items():
            n = k if k in names else lookup.get(k)
            if n is None:
                raise TypeError("%s has no input named '%s' (inputs: %s)" % (self.name, k, names))
            if n in given:
                raise TypeError("input '%s' given twice" % n)
            given[n] = v
        missing = [n for n in names if n not in given]
        if missing:
            raise TypeError("%s: missing inputs %s" % (self.name, missing))
        out = []
        for n in names:
            t = given[n]
            if isinstance(t, np.ndarray):
                t = torch.from_numpy(t)
            if not isinstance(t, torch.Tensor):
                raise TypeError("input '%s' must be a torch.Tensor or numpy array" % n)
            if t.dtype != torch.float32:
                raise TypeError("input '%s' must be float32, got %s" % (n, t.dtype))
            out.append(t.to(self.device).contiguous())
        return out

    def __call__(self, *args, **kwargs):
        """Execute the model. Positional arguments bind to the graph inputs in order, keyword arguments by
        (cleaned) name. Returns the output as a CUDA tensor, or a tuple when there are several."""
        inputs = self._bind(args, kwargs)
        with torch.cuda.device(self.device):
            plan = self.plan(*[t.shape for t in inputs])
            if self.cuda_graph:
                key = tuple(tuple(t.shape) for t in inputs)
                replay = self._replays.get(key)
                if replay is None:
                    replay = self._replays[key] = _GraphReplay(plan, inputs)
                outs = replay(inputs)
            else:
                outs = plan.run(inputs)
        return outs[0] if len(outs) == 1 else tuple(outs)
