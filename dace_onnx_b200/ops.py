"""Tensor-level host API over the C ABI: one function per ONNX node on the hot path.

Inputs are contiguous fp32 CUDA tensors (torch is used only for device memory and streams);
every function launches on torch's current stream and returns without synchronising. There is no
CPU path: a tensor that is not on a CUDA device is an error.
"""
import ctypes

import torch

from . import _lib
from ._lib import (ADD, DIV, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RELU, EPI_BIAS_RESIDUAL, EPI_NONE, EPI_SCALE, ERF,
                   GELU, MATH_MODES, MUL, POW, RELU, SQRT, SUB, AttentionDesc, ConvDesc, GemmDesc, check)  # noqa: F401

default_math_mode = "fp32x3"  # "fp32x3" | "tf32" | "bf16" | "fp32"; overridable per call


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _chk(t, name):
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s must be a torch.Tensor" % name)
    if not t.is_cuda:
        raise ValueError("%s must live on a CUDA device (this library has no CPU path)" % name)
    if t.dtype != torch.float32:
        raise TypeError("%s must be float32, got %s" % (name, t.dtype))
    return t


def _contig(t, name):
    _chk(t, name)
    return t if t.is_contiguous() else t.contiguous()


def _math(mode):
    mode = default_math_mode if mode is None else mode
    if mode not in MATH_MODES:
        raise ValueError("math mode must be one of %s" % sorted(MATH_MODES))
    return MATH_MODES[mode]


# ------------------------------------------------------------------------------------------------
# contractions
# ------------------------------------------------------------------------------------------------
def gemm_raw(A, B, Y, *, batch_outer=1, batch_inner=1, M, N, K, lda, ldb, ldy, a_strides=(0, 0), b_strides=(0, 0),
             y_strides=(0, 0), trans_b=False, epilogue=EPI_NONE, bias=None, residual=None, scale=1.0,
             math_mode=None):
    """Direct call of b200_gemm_f32 with explicit strides (A, B, Y are base tensors of the views)."""
    d = GemmDesc(batch_outer, batch_inner, M, N, K, lda, ldb, ldy, a_strides[0], a_strides[1], b_strides[0],
                 b_strides[1], y_strides[0], y_strides[1], int(trans_b), epilogue, float(scale), _math(math_mode))
    lib = _lib.load()
    need = lib.b200_gemm_workspace_bytes(ctypes.byref(d))
    if need:
        ws = _gemm_workspace(Y.device, need)
        check(lib.b200_gemm_ws_f32(_stream(), ctypes.byref(d), _ptr(A), _ptr(B), _ptr(bias), _ptr(residual), _ptr(Y),
                                   _ptr(ws), ws.numel()))
    else:
        check(lib.b200_gemm_f32(_stream(), ctypes.byref(d), _ptr(A), _ptr(B), _ptr(bias), _ptr(residual), _ptr(Y)))
    return Y


_GEMM_WS = {}


def _gemm_workspace(device, nbytes):
    """Scratch for b200_gemm_ws_f32, one buffer per (device, stream), grown on demand: calls on one stream are
    ordered, so they can share it; calls on different streams must not."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _GEMM_WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = _GEMM_WS[key] = torch.empty(max(nbytes, 1 << 20), device=device, dtype=torch.uint8)
    return ws


def _batch_view(shape, mat_elems):
    """Collapse leading batch dims of a contiguous tensor into (outer, inner) extents and strides."""
    n = 1
    for s in shape:
        n *= s
    return n, mat_elems


def matmul(A, B, out=None, *, trans_b=False, epilogue=EPI_NONE, bias=None, residual=None, scale=1.0,
           math_mode=None):
    """ONNXMatMul: numpy matmul semantics with batch broadcasting (1-D operands are rejected, as
    PureMatMul.forward_can_be_applied does). With trans_b the last two axes of B are [N, K]."""
    A = _contig(A, "A")
    B = _contig(B, "B")
    if A.dim() < 2 or B.dim() < 2:
        raise ValueError("matmul: 1-D operands are not supported")
    M, K = A.shape[-2], A.shape[-1]
    if trans_b:
        N, Kb = B.shape[-2], B.shape[-1]
    else:
        Kb, N = B.shape[-2], B.shape[-1]
    if K != Kb:
        raise ValueError("matmul: inner dimensions differ (%d vs %d)" % (K, Kb))
    batch_shape = torch.broadcast_shapes(A.shape[:-2], B.shape[:-2])
    out_shape = tuple(batch_shape) + (M, N)
    if out is None:
        out = torch.empty(out_shape, device=A.device, dtype=torch.float32)
    else:
        _chk(out, "out")
        if tuple(out.shape) != out_shape or not out.is_contiguous():
            raise ValueError("matmul: out must be contiguous with shape %s" % (out_shape,))
    if bias is not None:
        bias = _contig(bias, "bias")
        if bias.numel() != N:
            raise ValueError("matmul: bias must have N=%d entries" % N)
    if residual is not None:
        residual = _contig(residual, "residual")
        if tuple(residual.shape) != out_shape:
            raise ValueError("matmul: residual must have the output shape")
    # Express the broadcast batch as at most two strided levels.
    nb = len(batch_shape)
    Ae = A.expand(tuple(batch_shape) + (M, K)) if nb else A
    Be = B.expand(tuple(batch_shape) + tuple(B.shape[-2:])) if nb else B
    levels = _two_level(batch_shape, Ae.stride()[:nb], Be.stride()[:nb], out.stride()[:nb])
    if levels is None:
        # irregular broadcast: materialise (rare; keeps the kernel interface at two batch levels)
        Ae = Ae.contiguous()
        Be = Be.contiguous()
        levels = _two_level(batch_shape, Ae.stride()[:nb], Be.stride()[:nb], out.stride()[:nb])
    (bo, bi), sa, sb, sy = levels
    return gemm_raw(Ae, Be, out, batch_outer=bo, batch_inner=bi, M=M, N=N, K=K, lda=K, ldb=B.shape[-1], ldy=N,
                    a_strides=sa, b_strides=sb, y_strides=sy, trans_b=trans_b, epilogue=epilogue, bias=bias,
                    residual=residual, scale=scale, math_mode=math_mode)


def _two_level(batch_shape, sa, sb, sy):
    """Merge batch axes into <= 2 levels (outer, inner) for all three tensors, or None."""
    dims = [(n, a, b, y) for n, a, b, y in zip(batch_shape, sa, sb, sy) if n != 1]
    merged = []
    for n, a, b, y in dims:
        if merged:
            pn, pa, pb, py = merged[-1]
            if pa == a * n and pb == b * n and py == y * n:
                merged[-1] = (pn * n, a, b, y)
                continue
        merged.append((n, a, b, y))
    if len(merged) > 2:
        return None
    while len(merged) < 2:
        merged.insert(0, (1, 0, 0, 0))
    (no, ao, bo_, yo), (ni, ai, bi_, yi) = merged
    return (no, ni), (ao, ai), (bo_, bi_), (yo, yi)


def gemm(A, B, C=None, out=None, *, alpha=1.0, beta=1.0, transA=0, transB=1, relu=False, math_mode=None):
    """ONNXGemm in the only form the reference expands (alpha=beta=1, transA=0, transB=1):
    Y = A @ B^T + C, C broadcast over rows. `relu` fuses a following Relu node."""
    if not (alpha == 1.0 and beta == 1.0 and transA == 0 and transB == 1):
        raise NotImplementedError("Gemm: only alpha=1, beta=1, transA=0, transB=1 is supported")
    if C is None:
        if relu:
            raise ValueError("Gemm: relu fusion needs a bias operand")
        return matmul(A, B, out, trans_b=True, math_mode=math_mode)
    C = _contig(C, "C")
    # a per-column bias: [N], or [1, ..., 1, N]. Anything else (e.g. a per-row [M, 1] with M == N) broadcasts
    # differently and takes the generic Add.
    if C.numel() == B.shape[0] and C.dim() >= 1 and C.shape[-1] == B.shape[0]:
        return matmul(A, B, out, trans_b=True, epilogue=EPI_BIAS_RELU if relu else EPI_BIAS, bias=C.reshape(-1),
                      math_mode=math_mode)
    Y = matmul(A, B, out, trans_b=True, math_mode=math_mode)
    Y = add(Y, C, out=Y)
    return relu_(Y) if relu else Y


def attention_views(q, k, v, out, scale, math_mode=None):
    """Fused Softmax(q k^T * scale) v. q, k, v, out are 4-D [batch, seq, heads, head_dim] views (any
    strides with head_dim contiguous, e.g. slices of a fused QKV projection). Returns False without
    launching when the fused kernel does not cover the case (the caller then runs the nodes unfused)."""
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (out, "out")):
        _chk(t, n)
        if t.dim() != 4 or t.stride(3) != 1:
            raise ValueError("%s must be a [batch, seq, heads, head_dim] view with contiguous head_dim" % n)
    b, s, h, dh = q.shape
    if tuple(k.shape) != (b, s, h, dh) or tuple(v.shape) != (b, s, h, dh) or tuple(out.shape) != (b, s, h, dh):
        raise ValueError("attention: q, k, v, out must have the same shape")
    d = AttentionDesc(b, h, s, dh, q.stride(1), q.stride(2), q.stride(0), k.stride(1), k.stride(2), k.stride(0),
                      v.stride(1), v.stride(2), v.stride(0), out.stride(1), out.stride(2), out.stride(0),
                      float(scale), _math(math_mode))
    lib = _lib.load()
    if not lib.b200_attention_supported(ctypes.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(out)):
        return False
    check(lib.b200_attention_f32(_stream(), ctypes.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(out)))
    return True


def conv2d_workspace_bytes(x_shape, w_shape, pads=(0, 0, 0, 0), strides=(1, 1), math_mode=None):
    """Device scratch b200_conv2d_f32 wants for this convolution (0 when it runs without any)."""
    N, C, H, Wd = x_shape
    M, _, KH, KW = w_shape
    d = ConvDesc(N, C, H, Wd, M, KH, KW, pads[0], pads[1], strides[0], strides[1], EPI_NONE, _math(math_mode))
    return int(_lib.load().b200_conv2d_workspace_bytes(ctypes.byref(d)))


def conv2d(X, W, B=None, out=None, *, pads=(0, 0, 0, 0), strides=(1, 1), dilations=(1, 1), group=1, relu=False,
           workspace=None, math_mode=None):
    """ONNXConv, NCHW / OIHW, group 1, dilation 1, symmetric pads [top, left, bottom, right]."""
    X = _contig(X, "X")
    W = _contig(W, "W")
    if X.dim() != 4 or W.dim() != 4:
        raise NotImplementedError("Conv: only 2-D convolutions")
    if group != 1 or tuple(dilations) != (1, 1):
        raise NotImplementedError("Conv: group and dilations must be 1")
    if pads[0] != pads[2] or pads[1] != pads[3]:
        raise NotImplementedError("Conv: padding must be symmetric")
    if X.shape[1] != W.shape[1]:
        raise ValueError("Conv: channel mismatch")
    N, C, H, Wd = X.shape
    M, _, KH, KW = W.shape
    OH = (H + 2 * pads[0] - KH) // strides[0] + 1
    OW = (Wd + 2 * pads[1] - KW) // strides[1] + 1
    if out is None:
        out = torch.empty((N, M, OH, OW), device=X.device, dtype=torch.float32)
    epi = EPI_NONE
    if B is not None:
        B = _contig(B, "B")
        epi = EPI_BIAS_RELU if relu else EPI_BIAS
    elif relu:
        raise ValueError("Conv: relu fusion needs a bias operand")
    d = ConvDesc(N, C, H, Wd, M, KH, KW, pads[0], pads[1], strides[0], strides[1], epi, _math(math_mode))
    lib = _lib.load()
    need = lib.b200_conv2d_workspace_bytes(ctypes.byref(d))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=X.device, dtype=torch.uint8)
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    check(lib.b200_conv2d_f32(_stream(), ctypes.byref(d), _ptr(X), _ptr(W), _ptr(B), _ptr(out), _ptr(workspace),
                              ws_bytes))
    return out


class PreparedConv:
    """A convolution whose constant work is done once: the filter repacked (and, in fp32x3 mode, split) into a
    device buffer by b200_conv2d_prepare_filter_f32, the way the reference's cuDNN expansion builds its descriptors
    in the SDFG init hook (cudnn_implementations.py:281-301). Calls then run b200_conv2d_prepared_f32.

    W: [M, C, KH, KW], B: [M] or None (both CUDA fp32). `nhwc_ok` says whether this convolution can take / produce
    [N, H, W, C] tensors, which saves the layout change between the convolutions of a stack."""

    def __init__(self, W, B=None, *, pads=(0, 0, 0, 0), strides=(1, 1), dilations=(1, 1), group=1, relu=False,
                 math_mode=None):
        W = _contig(W, "W")
        if W.dim() != 4:
            raise NotImplementedError("Conv: only 2-D convolutions")
        if group != 1 or tuple(dilations) != (1, 1):
            raise NotImplementedError("Conv: group and dilations must be 1")
        if pads[0] != pads[2] or pads[1] != pads[3]:
            raise NotImplementedError("Conv: padding must be symmetric")
        if B is None and relu:
            raise ValueError("Conv: relu fusion needs a bias operand")
        self.M, self.C, self.KH, self.KW = (int(v) for v in W.shape)
        self.pads, self.strides = (int(pads[0]), int(pads[1])), (int(strides[0]), int(strides[1]))
        self.bias = _contig(B, "B") if B is not None else None
        self.epilogue = EPI_NONE if B is None else (EPI_BIAS_RELU if relu else EPI_BIAS)
        self.mode = _math(math_mode)
        lib = _lib.load()
        d = self.desc(1, 1, 1)
        self.nhwc_ok = bool(lib.b200_conv2d_nhwc_supported(ctypes.byref(d)))
        nbytes = int(lib.b200_conv2d_filter_bytes(ctypes.byref(d)))
        self.filter = torch.empty(max(nbytes, 16), device=W.device, dtype=torch.uint8)
        check(lib.b200_conv2d_prepare_filter_f32(_stream(), ctypes.byref(d), _ptr(W), _ptr(self.filter), nbytes))
        self._ws = None

    def desc(self, n, h, w):
        return ConvDesc(n, self.C, h, w, self.M, self.KH, self.KW, self.pads[0], self.pads[1], self.strides[0],
                        self.strides[1], self.epilogue, self.mode)

    def out_hw(self, h, w):
        return ((h + 2 * self.pads[0] - self.KH) // self.strides[0] + 1,
                (w + 2 * self.pads[1] - self.KW) // self.strides[1] + 1)

    def __call__(self, X, out=None, *, x_nhwc=False, y_nhwc=False, workspace=None):
        """X: [N, C, H, W], or [N, H, W, C] with x_nhwc. Returns [N, M, OH, OW], or [N, OH, OW, M] with y_nhwc."""
        X = _contig(X, "X")
        if X.dim() != 4:
            raise NotImplementedError("Conv: only 2-D convolutions")
        n, c, h, w = (X.shape[0], X.shape[3], X.shape[1], X.shape[2]) if x_nhwc else X.shape
        if c != self.C:
            raise ValueError("Conv: channel mismatch")
        oh, ow = self.out_hw(h, w)
        oshape = (n, oh, ow, self.M) if y_nhwc else (n, self.M, oh, ow)
        if out is None:
            out = torch.empty(oshape, device=X.device, dtype=torch.float32)
        elif tuple(out.shape) != oshape or not out.is_contiguous():
            raise ValueError("Conv: out must be contiguous with shape %s" % (oshape,))
        flags = (_lib.CONV_X_NHWC if x_nhwc else 0) | (_lib.CONV_Y_NHWC if y_nhwc else 0)
        lib = _lib.load()
        d = self.desc(n, h, w)
        need = int(lib.b200_conv2d_prepared_workspace_bytes(ctypes.byref(d), flags))
        if need:
            if workspace is None or workspace.numel() * workspace.element_size() < need:
                if self._ws is None or self._ws.numel() < need or self._ws.device != X.device:
                    self._ws = torch.empty(need, device=X.device, dtype=torch.uint8)
                workspace = self._ws
        else:
            workspace = None
        ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
        check(lib.b200_conv2d_prepared_f32(_stream(), ctypes.byref(d), flags, _ptr(X), _ptr(self.filter),
                                           _ptr(self.bias), _ptr(out), _ptr(workspace), ws_bytes))
        return out


# ------------------------------------------------------------------------------------------------
# row-wise
# ------------------------------------------------------------------------------------------------
def _axis_view(shape, axis):
    nd = len(shape)
    if not -nd <= axis < nd:
        raise ValueError("axis %d out of range for rank %d" % (axis, nd))
    axis %= nd
    outer = 1
    for s in shape[:axis]:
        outer *= s
    inner = 1
    for s in shape[axis + 1:]:
        inner *= s
    return outer, shape[axis], inner


def _rowwise(fn_name, x, axis, out):
    x = _contig(x, "input")
    if out is None:
        out = torch.empty_like(x)
    outer, length, inner = _axis_view(tuple(x.shape), axis)
    check(getattr(_lib.load(), fn_name)(_stream(), _ptr(x), _ptr(out), outer, length, inner))
    return out


def softmax(x, axis=-1, out=None):
    """ONNXSoftmax over one numpy axis."""
    return _rowwise("b200_softmax_f32", x, axis, out)


def logsoftmax(x, axis=-1, out=None):
    """ONNXLogSoftmax over one numpy axis."""
    return _rowwise("b200_logsoftmax_f32", x, axis, out)


def reduce_mean(x, axes, keepdims=1, out=None):
    """ONNXReduceMean over a contiguous block of axes."""
    x = _contig(x, "data")
    nd = x.dim()
    axes = sorted(a % nd for a in axes)
    if axes != list(range(axes[0], axes[-1] + 1)):
        raise NotImplementedError("ReduceMean: axes must be adjacent")
    shape = tuple(x.shape)
    outer = 1
    for s in shape[:axes[0]]:
        outer *= s
    length = 1
    for a in axes:
        length *= shape[a]
    inner = 1
    for s in shape[axes[-1] + 1:]:
        inner *= s
    if keepdims:
        oshape = tuple(1 if i in axes else s for i, s in enumerate(shape))
    else:
        oshape = tuple(s for i, s in enumerate(shape) if i not in axes)
    if out is None:
        out = torch.empty(oshape, device=x.device, dtype=torch.float32)
    check(_lib.load().b200_reduce_mean_f32(_stream(), _ptr(x), _ptr(out), outer, length, inner))
    return out


def layernorm(x, gamma=None, beta=None, eps=1e-12, out=None):
    """The fused LayerNormalization node chain over the last axis."""
    x = _contig(x, "x")
    length = x.shape[-1]
    rows = x.numel() // length if length else 0
    if gamma is not None:
        gamma = _contig(gamma, "gamma")
    if beta is not None:
        beta = _contig(beta, "beta")
    if out is None:
        out = torch.empty_like(x)
    check(_lib.load().b200_layernorm_f32(_stream(), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(out), rows, length,
                                         float(eps)))
    return out


# ------------------------------------------------------------------------------------------------
# elementwise
# ------------------------------------------------------------------------------------------------
def _binary(op, a, b, out):
    if not isinstance(a, torch.Tensor):
        a = torch.tensor(a, dtype=torch.float32, device=b.device)
    if not isinstance(b, torch.Tensor):
        b = torch.tensor(b, dtype=torch.float32, device=a.device)
    a = _contig(a, "A")
    b = _contig(b, "B")
    shape = tuple(torch.broadcast_shapes(a.shape, b.shape))
    if len(shape) > 8:
        raise NotImplementedError("elementwise: rank > 8")
    if out is None:
        out = torch.empty(shape, device=a.device, dtype=torch.float32)
    elif tuple(out.shape) != shape or not out.is_contiguous():
        raise ValueError("elementwise: out must be contiguous with the broadcast shape")
    ae, be = a.expand(shape), b.expand(shape)
    n = len(shape)
    arr = ctypes.c_int64 * max(n, 1)
    check(_lib.load().b200_binary_f32(_stream(), op, _ptr(ae), _ptr(be), _ptr(out), n, arr(*shape),
                                      arr(*ae.stride()), arr(*be.stride())))
    return out


def add(a, b, out=None):
    return _binary(ADD, a, b, out)


def sub(a, b, out=None):
    return _binary(SUB, a, b, out)


def mul(a, b, out=None):
    return _binary(MUL, a, b, out)


def div(a, b, out=None):
    return _binary(DIV, a, b, out)


def pow(a, b, out=None):  # noqa: A001 - mirrors the ONNX node name
    return _binary(POW, a, b, out)


def _unary(op, x, out):
    x = _contig(x, "X")
    if out is None:
        out = torch.empty_like(x)
    check(_lib.load().b200_unary_f32(_stream(), op, _ptr(x), _ptr(out), x.numel()))
    return out


def sqrt(x, out=None):
    return _unary(SQRT, x, out)


def erf(x, out=None):
    return _unary(ERF, x, out)


def relu(x, out=None):
    return _unary(RELU, x, out)


def relu_(x):
    return _unary(RELU, x, x)


def gelu(x, out=None):
    """The fused Div(sqrt 2) -> Erf -> Add 1 -> Mul x -> Mul 0.5 chain."""
    return _unary(GELU, x, out)


def transpose_0213(x, out=None):
    """ONNXTranspose perm [0,2,1,3]."""
    x = _contig(x, "data")
    d0, d1, d2, d3 = x.shape
    if out is None:
        out = torch.empty((d0, d2, d1, d3), device=x.device, dtype=torch.float32)
    check(_lib.load().b200_transpose_0213_f32(_stream(), _ptr(x), _ptr(out), d0, d1, d2, d3))
    return out


def maxpool2d(X, kernel_shape, strides=None, out=None):
    """ONNXMaxPool on NCHW, 2-D windows, no padding (what the pure expansion accepts)."""
    X = _contig(X, "X")
    if X.dim() != 4:
        raise NotImplementedError("MaxPool: only 2-D pooling of NCHW tensors")
    kh, kw = (int(k) for k in kernel_shape)
    sh, sw = (int(s) for s in (strides or (1, 1)))
    n, c, h, w = X.shape
    if kh > h or kw > w:
        raise ValueError("MaxPool: window larger than the image")
    oh, ow = (h - kh) // sh + 1, (w - kw) // sw + 1
    if out is None:
        out = torch.empty((n, c, oh, ow), device=X.device, dtype=torch.float32)
    check(_lib.load().b200_maxpool2d_f32(_stream(), _ptr(X), _ptr(out), n * c, h, w, kh, kw, sh, sw))
    return out


_ONES = {}


def permute(x, perm, out=None):
    """ONNXTranspose with an arbitrary perm (rank <= 8): the strided elementwise kernel reads the input
    through permuted strides and multiplies by a broadcast 1.0, which returns every value unchanged."""
    x = _contig(x, "data")
    n = x.dim()
    perm = [int(p) % n for p in perm]
    if sorted(perm) != list(range(n)):
        raise ValueError("permute: %s is not a permutation of %d axes" % (perm, n))
    if n > 8:
        raise NotImplementedError("permute: rank > 8")
    xv = x.permute(perm)  # a view: no data moves here
    if out is None:
        out = torch.empty(tuple(xv.shape), device=x.device, dtype=torch.float32)
    elif tuple(out.shape) != tuple(xv.shape) or not out.is_contiguous():
        raise ValueError("permute: out must be contiguous with shape %s" % (tuple(xv.shape),))
    one = _ONES.get(x.device)
    if one is None:
        one = _ONES[x.device] = torch.ones((), device=x.device, dtype=torch.float32)
    arr = ctypes.c_int64 * max(n, 1)
    check(_lib.load().b200_binary_f32(_stream(), MUL, _ptr(xv), _ptr(one), _ptr(out), n, arr(*xv.shape),
                                      arr(*xv.stride()), arr(*([0] * n))))
    return out


def transpose_last2(x, out=None):
    """ONNXTranspose swapping the last two axes (perm [1,0] for matrices)."""
    x = _contig(x, "data")
    rows, cols = x.shape[-2], x.shape[-1]
    batch = x.numel() // (rows * cols) if rows * cols else 0
    if out is None:
        out = torch.empty(tuple(x.shape[:-2]) + (cols, rows), device=x.device, dtype=torch.float32)
    check(_lib.load().b200_transpose_2d_f32(_stream(), _ptr(x), _ptr(out), batch, rows, cols))
    return out
