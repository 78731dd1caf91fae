"""Node-level host API with the signatures of DaCeML's generated `donnx.ONNX<Op>` library nodes.

In the reference a node is called from a `@dace.program` with its ONNX connector names as
keywords, outputs included, and attributes beside them
(`donnx.ONNXMatMul(A=X, B=Z, Y=Y)`, tests/test_python_frontend.py:12-22; connector / attribute
names come from the opset-12 schemas, daceml/onnx/nodes/onnx_op.py:418-496). The functions here
take the same keywords and run the `b200` kernels eagerly on CUDA tensors, writing the output
connector in place, so that tests of this library read like the reference's node tests. Checks
mirror `forward_can_be_applied` of the corresponding pure expansion; a node that the reference
would hand to another implementation raises instead (there is no fallback).
"""
import torch

from . import ops
from ._lib import EPI_BIAS

default_implementation = "b200"


def _out(dst, result_fn, shape):
    if dst is None:
        raise TypeError("the output connector must be passed (outputs are written in place)")
    if tuple(dst.shape) != tuple(shape):
        raise ValueError("output connector has shape %s, expected %s" % (tuple(dst.shape), tuple(shape)))
    if dst.is_contiguous():
        result_fn(dst)
    else:
        tmp = torch.empty(shape, device=dst.device, dtype=dst.dtype)
        result_fn(tmp)
        dst.copy_(tmp)
    return dst


def ONNXMatMul(*, A, B, Y, math_mode=None):
    """MatMul (pure_implementations.py:130-235): numpy matmul; 1-D operands are not expandable."""
    if A.dim() == 1 or B.dim() == 1:
        raise NotImplementedError("MatMul: 1-D operands (PureMatMul.forward_can_be_applied is False)")
    shape = tuple(torch.broadcast_shapes(A.shape[:-2], B.shape[:-2])) + (A.shape[-2], B.shape[-1])
    return _out(Y, lambda o: ops.matmul(A, B, out=o, math_mode=math_mode), shape)


def ONNXGemm(*, A, B, Y, C=None, alpha=1.0, beta=1.0, transA=0, transB=0, math_mode=None):
    """Gemm (pure_implementations.py:433-459): only alpha=1, beta=1, transA=0, transB=1."""
    if not (alpha == 1.0 and beta == 1.0 and transA == 0 and transB == 1):
        raise NotImplementedError("Gemm: PureGemm.forward_can_be_applied is False for these attributes")
    return _out(Y, lambda o: ops.gemm(A, B, C, out=o, math_mode=math_mode), (A.shape[0], B.shape[0]))


def ONNXConv(*, X, W, Y, B=None, auto_pad="NOTSET", dilations=None, group=1, kernel_shape=None, pads=None,
             strides=None, math_mode=None):
    """Conv (img_op_implementations.py:164-326), with the symmetric padding the cuDNN expansion
    also accepts (cudnn_implementations.py:164-168)."""
    if auto_pad != "NOTSET":
        raise NotImplementedError("Conv: auto_pad must be NOTSET")
    if X.dim() != 4 or W.dim() != 4:
        raise NotImplementedError("Conv: only 2-D convolutions")
    if kernel_shape is not None and tuple(kernel_shape) != tuple(W.shape[2:]):
        raise ValueError("Conv: kernel_shape does not match W")
    pads = tuple(pads) if pads is not None else (0, 0, 0, 0)
    strides = tuple(strides) if strides is not None else (1, 1)
    dilations = tuple(dilations) if dilations is not None else (1, 1)
    oh = (X.shape[2] + pads[0] + pads[2] - W.shape[2]) // strides[0] + 1
    ow = (X.shape[3] + pads[1] + pads[3] - W.shape[3]) // strides[1] + 1
    return _out(Y, lambda o: ops.conv2d(X, W, B, out=o, pads=pads, strides=strides, dilations=dilations, group=group,
                                        math_mode=math_mode), (X.shape[0], W.shape[0], oh, ow))


def ONNXSoftmax(*, input, output, axis=1):  # noqa: A002 - ONNX connector name
    """Softmax over one numpy axis (pure_implementations.py:346-366)."""
    return _out(output, lambda o: ops.softmax(input, axis, out=o), input.shape)


def ONNXLogSoftmax(*, input, output, axis=1):  # noqa: A002
    """LogSoftmax over one numpy axis (pure_implementations.py:594-616)."""
    return _out(output, lambda o: ops.logsoftmax(input, axis, out=o), input.shape)


def ONNXReduceMean(*, data, reduced, axes, keepdims=1):
    """ReduceMean (pure_implementations.py:97-109)."""
    nd = data.dim()
    ax = sorted(a % nd for a in axes)
    shape = tuple((1 if i in ax else s) for i, s in enumerate(data.shape)) if keepdims else \
        tuple(s for i, s in enumerate(data.shape) if i not in ax)
    return _out(reduced, lambda o: ops.reduce_mean(data, axes, keepdims, out=o), shape)


def _binary(fn, A, B, C):
    shape = torch.broadcast_shapes(A.shape if isinstance(A, torch.Tensor) else (),
                                   B.shape if isinstance(B, torch.Tensor) else ())
    return _out(C, lambda o: fn(A, B, out=o), shape)


def ONNXAdd(*, A, B, C):
    """Add (pure_implementations.py:77-79), numpy broadcasting, scalar operands included."""
    return _binary(ops.add, A, B, C)


def ONNXSub(*, A, B, C):
    """Sub (pure_implementations.py:82-84)."""
    return _binary(ops.sub, A, B, C)


def ONNXMul(*, A, B, C):
    """Mul (pure_implementations.py:87-89)."""
    return _binary(ops.mul, A, B, C)


def ONNXDiv(*, A, B, C):
    """Div (pure_implementations.py:92-94)."""
    return _binary(ops.div, A, B, C)


def ONNXPow(*, X, Y, Z):
    """Pow (pure_implementations.py:59-74): float tensors only."""
    return _binary(ops.pow, X, Y, Z)


def ONNXSqrt(*, X, Y):
    """Sqrt (pure_implementations.py:41-56)."""
    return _out(Y, lambda o: ops.sqrt(X, out=o), X.shape)


def ONNXErf(*, input, output):  # noqa: A002
    """Erf (pure_implementations.py:112-127)."""
    return _out(output, lambda o: ops.erf(input, out=o), input.shape)


def ONNXRelu(*, X, Y):
    """Relu (pure_implementations.py:462-474)."""
    return _out(Y, lambda o: ops.relu(X, out=o), X.shape)


def ONNXTranspose(*, data, transposed, perm):
    """Transpose (pure_implementations.py:369-379) for the two permutations the BERT graph uses."""
    perm = [int(p) for p in perm]
    nd = data.dim()
    if perm == list(range(nd - 2)) + [nd - 1, nd - 2]:
        return _out(transposed, lambda o: ops.transpose_last2(data, out=o), tuple(data.shape[:-2]) +
                    (data.shape[-1], data.shape[-2]))
    if nd == 4 and perm == [0, 2, 1, 3]:
        return _out(transposed, lambda o: ops.transpose_0213(data, out=o),
                    (data.shape[0], data.shape[2], data.shape[1], data.shape[3]))
    raise NotImplementedError("Transpose: perm %s is not on the hot path" % perm)
