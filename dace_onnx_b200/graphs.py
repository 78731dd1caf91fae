"""Runners for the two small BASELINE graphs, node by node through the C ABI.

`mlp_forward`: Gemm(+Relu) x2, Gemm, LogSoftmax(axis=1) -- the exported graph of the MLP in the
reference's autodiff example (Linear 784->120->32->10), as `@dace_module` would run it.
`conv_stack_forward`: [Conv 3x3 pad 1 + bias, Relu] x n -- the README model of the reference
(tests/pytorch/test_conv2d.py:11-37), NCHW.
Relu is folded into the producing contraction's epilogue; every node also exists standalone in `ops`.
"""
from . import ops


def mlp_forward(x, params, math_mode=None):
    """x: [batch, in] CUDA fp32; params: [(W[out, in], b[out]), ...] CUDA fp32. Returns log-probabilities."""
    h = x
    last = len(params) - 1
    for i, (w, b) in enumerate(params):
        h = ops.gemm(h, w, b, relu=i < last, math_mode=math_mode)
    return ops.logsoftmax(h, axis=1)


def prepare_conv_stack(params, math_mode=None):
    """Set-up of conv_stack_forward: each layer's filter repacked once (ops.PreparedConv)."""
    return [ops.PreparedConv(w, b, pads=(1, 1, 1, 1), relu=True, math_mode=math_mode) for w, b in params]


def conv_stack_forward(x, params, math_mode=None, workspace=None):
    """x: [N, C, H, W]; params: [(W[M, C, 3, 3], b[M]), ...] or the result of prepare_conv_stack. Returns NCHW.

    Between two consecutive convolutions the activations stay in the [N, H, W, C] layout the tensor-core kernel
    reads and writes natively; only the stack's input and output pay the NCHW <-> NHWC change."""
    layers = params if params and isinstance(params[0], ops.PreparedConv) else prepare_conv_stack(params, math_mode)
    h, nhwc = x, False
    for i, conv in enumerate(layers):
        keep = i + 1 < len(layers) and conv.nhwc_ok and layers[i + 1].nhwc_ok
        h = conv(h, x_nhwc=nhwc, y_nhwc=keep, workspace=workspace)
        nhwc = keep
    return h
