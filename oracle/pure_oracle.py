"""CPU oracle: a restatement of DaCeML's `pure` expansions for the ONNX nodes on the hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product (`dace_onnx_b200/`) may import this module; it
is used by `tests/`, by `__graft_entry__.smoke()` and by the CPU-baseline legs of `bench.py`, and
only as the checker or as the timed CPU baseline.

What it restates. The reference (spcl/dace-onnx) describes each node's arithmetic as a
numpy-style program that DaCe (an un-vendored dependency, dace@4c6a674, setup.py:40) lowers to
loops / BLAS calls. Each function below follows one such program op for op, in the same order and
with the same full-size intermediates, in fp32 on the CPU (torch CPU tensors, so that every op
uses all host threads the way DaCe's OpenMP maps do). Citations are paths inside the reference.

How it is pinned. The reference holds no golden vectors: its tests compare each expansion with
torch / numpy on unseeded random inputs (tests/pure_expansions/test_expansions.py,
test_conv_expansion.py, tests/pytorch/test_bert_encoder.py), and DaCe cannot be installed where
this repository is developed (dace, onnx missing; Python 3.12 vs the pinned <3.10). Two pins:
  1. `tests/golden/ref_pins.npz` holds vectors computed by the reference's OWN source:
     `tests/golden/make_reference_pins.py` loads pure_implementations.py and
     op_implementations/utils.py unmodified, calls each Pure<Op>.forward() and executes the numpy-style
     program it hands to DaCe with numpy arrays (MatMul: the einsum string it builds, through
     np.einsum). `tests/test_reference_pins.py` holds this module to those vectors -- elementwise
     nodes bit for bit, reductions / contractions within 2e-6 -- for every node on the path and for
     the LayerNorm, Gelu and attention node chains. Not covered by this pin: DaCe's code generation
     (loop order, libm), and Conv, whose expansion is written in DaCe map / tasklet syntax.
  2. `tests/test_oracle_pins.py` repeats the reference tests' shapes, comparators and tolerances
     (torch / numpy as the yardstick) against this module, Conv included.
Against outputs of the DaCe-compiled reference the parity remains unpinned.
"""
import math

import numpy as np
import torch

F32 = torch.float32


def _t(x):
    """fp32 CPU tensor view of a numpy array / tensor / python scalar."""
    if isinstance(x, torch.Tensor):
        return x.detach().to("cpu", F32)
    return torch.as_tensor(np.asarray(x, dtype=np.float32))


# ---------------------------------------------------------------------------------------------
# elementwise nodes
# ---------------------------------------------------------------------------------------------
def Add(A, B):
    """daceml/onnx/op_implementations/pure_implementations.py:77-79  C[:] = A + B"""
    return _t(A) + _t(B)


def Sub(A, B):
    """pure_implementations.py:82-84  C[:] = A - B"""
    return _t(A) - _t(B)


def Mul(A, B):
    """pure_implementations.py:87-89  C[:] = A * B"""
    return _t(A) * _t(B)


def Div(A, B):
    """pure_implementations.py:92-94  C[:] = A / B"""
    return _t(A) / _t(B)


def Pow(X, Y):
    """pure_implementations.py:59-74  Z[:] = X ** Y"""
    return torch.pow(_t(X), _t(Y))


def Sqrt(X):
    """pure_implementations.py:41-56  elementwise sqrt"""
    return torch.sqrt(_t(X))


def Erf(input):
    """pure_implementations.py:112-127  elementwise erf"""
    return torch.erf(_t(input))


def Relu(X):
    """pure_implementations.py:462-474  max(x, 0) in the input dtype"""
    x = _t(X)
    return torch.maximum(x, torch.zeros((), dtype=F32))


# ---------------------------------------------------------------------------------------------
# reductions / row-wise nodes
# ---------------------------------------------------------------------------------------------
def ReduceMean(data, axes, keepdims=1):
    """pure_implementations.py:97-109  reduced[:] = np.mean(data, axis=axes); keepdims only changes
    the output shape."""
    x = _t(data)
    return torch.mean(x, dim=tuple(int(a) for a in axes), keepdim=bool(keepdims))


def Softmax(input, axis):
    """pure_implementations.py:346-366: max, reshape keepdims, exp(input - max), sum, reshape,
    divide -- `axis` is one numpy axis (tests/pure_expansions/test_expansions.py:343-379)."""
    x = _t(input)
    mx = torch.amax(x, dim=axis, keepdim=True)
    exp_arr = torch.exp(x - mx)
    s = torch.sum(exp_arr, dim=axis, keepdim=True)
    return exp_arr / s


def LogSoftmax(input, axis):
    """pure_implementations.py:594-616: max_sub = input - max; log_sum = log(sum(exp(max_sub)));
    output = max_sub - log_sum."""
    x = _t(input)
    mx = torch.amax(x, dim=axis, keepdim=True)
    max_sub = x - mx
    exp_arr = torch.exp(max_sub)
    s = torch.sum(exp_arr, dim=axis, keepdim=True)
    return max_sub - torch.log(s)


# ---------------------------------------------------------------------------------------------
# contractions
# ---------------------------------------------------------------------------------------------
def MatMul(A, B):
    """pure_implementations.py:130-235: numpy matmul semantics; the expansion builds the einsum
    'ik,kj->ij' with broadcast batch letters (:151-210) and lowers it through ONNXEinsum to DaCe's
    einsum (:238-267), i.e. a (batched) fp32 GEMM. 1-D operands are rejected (:135-140)."""
    a, b = _t(A), _t(B)
    if a.dim() < 2 or b.dim() < 2:
        raise ValueError("PureMatMul cannot be applied to 1-D operands")
    return torch.matmul(a, b)


def Gemm(A, B, C=None, alpha=1.0, beta=1.0, transA=0, transB=1):
    """pure_implementations.py:433-459: only alpha=beta=1, transA=0, transB=1 (:438);
    Y = A @ np.transpose(B) + C (:450-455)."""
    if not (alpha == 1.0 and beta == 1.0 and transA == 0 and transB == 1):
        raise ValueError("PureGemm cannot be applied")
    y = torch.matmul(_t(A), torch.transpose(_t(B), 0, 1).contiguous())
    if C is not None:
        y = y + _t(C)
    return y


def Conv(X, W, B=None, pads=(0, 0, 0, 0), strides=(1, 1)):
    """daceml/onnx/op_implementations/img_op_implementations.py:164-326. The pure expansion accepts
    pads == 0 only (:201-203); a padded Conv is the explicit zero Pad followed by it, which is what
    PadConvFusion treats as equivalent (daceml/transformation/pad_conv_fusion.py:77-95). Y starts
    as the broadcast bias, or zero (:246-266), and the 7-D map accumulates
    W[m,cin,hx,hy] * X[b,cin,hx+out_x,hy+out_y] into it (:268-293). The reference's index has no
    stride factor (:278,:291), so it is only meaningful for stride 1; other strides follow the
    ONNX definition here and are outside the parity claim."""
    x, w = _t(X), _t(W)
    n, c, h, wd = x.shape
    m, c2, kh, kw = w.shape
    if c != c2:
        raise ValueError("PureConv2D cannot be applied: channel mismatch")
    if pads[0] != pads[2] or pads[1] != pads[3]:
        raise ValueError("asymmetric padding")
    ph, pw = int(pads[0]), int(pads[1])
    if ph or pw:
        xp = torch.zeros((n, c, h + 2 * ph, wd + 2 * pw), dtype=F32)
        xp[:, :, ph:ph + h, pw:pw + wd] = x
        x = xp
    sh, sw = int(strides[0]), int(strides[1])
    oh = (x.shape[2] - kh) // sh + 1
    ow = (x.shape[3] - kw) // sw + 1
    if B is not None:
        y = _t(B).reshape(1, m, 1, 1).expand(n, m, oh, ow).clone()
    else:
        y = torch.zeros((n, m, oh, ow), dtype=F32)
    for hx in range(kh):
        for hy in range(kw):
            patch = x[:, :, hx:hx + (oh - 1) * sh + 1:sh, hy:hy + (ow - 1) * sw + 1:sw]
            # sum over cin of W[m,cin,hx,hy] * X[b,cin,...]
            y += torch.einsum("mc,bchw->bmhw", w[:, :, hx, hy], patch)
    return y


def MaxPool(X, kernel_shape, strides=(1, 1)):
    """daceml/onnx/op_implementations/img_op_implementations.py:29-140 (PureMaxPool2D): pads 0, ceil_mode 0,
    dilations 1; Y starts at the lowest value of the dtype (:90-104) and a map over (b, c, out_x, out_y, hx, hy)
    takes the maximum of X[b, c, stride_x*out_x + hx, stride_y*out_y + hy] into it."""
    x = _t(X)
    kh, kw = int(kernel_shape[0]), int(kernel_shape[1])
    sh, sw = int(strides[0]), int(strides[1])
    n, c, h, w = x.shape
    oh, ow = (h - kh) // sh + 1, (w - kw) // sw + 1
    y = torch.full((n, c, oh, ow), torch.finfo(F32).min, dtype=F32)
    for hx in range(kh):
        for hy in range(kw):
            y = torch.maximum(y, x[:, :, hx:hx + (oh - 1) * sh + 1:sh, hy:hy + (ow - 1) * sw + 1:sw])
    return y


# ---------------------------------------------------------------------------------------------
# node chains that opset-12 export produces for LayerNorm and Gelu
# ---------------------------------------------------------------------------------------------
def LayerNormChain(x, gamma, beta, eps):
    """The nine nodes torch.onnx.export(opset 12) emits for nn.LayerNorm, each as its pure
    expansion: ReduceMean[-1] -> Sub -> Pow(., 2) -> ReduceMean[-1] -> Add(., eps) -> Sqrt -> Div
    -> Mul(., weight) -> Add(., bias)."""
    mean = ReduceMean(x, axes=[-1], keepdims=1)
    d = Sub(x, mean)
    sq = Pow(d, 2.0)
    var = ReduceMean(sq, axes=[-1], keepdims=1)
    sd = Sqrt(Add(var, eps))
    y = Div(d, sd)
    if gamma is not None:
        y = Mul(y, gamma)
    if beta is not None:
        y = Add(y, beta)
    return y


SQRT2 = np.float32(math.sqrt(2.0))


def GeluChain(x):
    """F.gelu at opset 12: Div(x, sqrt 2) -> Erf -> Add(., 1) -> Mul(x, .) -> Mul(., 0.5)."""
    t = Erf(Div(x, SQRT2))
    return Mul(Mul(x, Add(t, 1.0)), 0.5)


# ---------------------------------------------------------------------------------------------
# the BASELINE configurations, node by node
# ---------------------------------------------------------------------------------------------
def mlp_forward(x, params):
    """Config 1: Gemm+Relu, Gemm+Relu, Gemm, LogSoftmax(axis=1). params = [(W[N,K], b[N])] * 3."""
    h = _t(x)
    for i, (w, b) in enumerate(params):
        h = Gemm(h, w, b)
        if i + 1 < len(params):
            h = Relu(h)
    return LogSoftmax(h, axis=1)


def conv_stack_forward(x, params):
    """Config 2: [Conv 3x3 pad 1 + bias -> Relu] per (W, b) in params."""
    h = _t(x)
    for w, b in params:
        h = Relu(Conv(h, w, b, pads=(1, 1, 1, 1), strides=(1, 1)))
    return h


def bert_layer_forward(x, p, heads, eps=1e-12):
    """Configs 3 and 5: one BERT encoder layer as the exported ONNX subgraph, node by node.

    p holds wq,bq,wk,bk,wv,bv,wo,bo,ln1_g,ln1_b,wi,bi,wo2,bo2,ln2_g,ln2_b with Linear weights in
    torch layout [out, in]; every Linear is MatMul(x, Transpose(W)) then Add(bias, .); the score
    scale is Mul(., 1/sqrt(d)); the mask is all ones and contributes nothing.
    """
    x = _t(x)
    bsz, seq, hid = x.shape
    dh = hid // heads

    def linear(t, w, b):
        return Add(_t(b), MatMul(t, torch.transpose(_t(w), 0, 1).contiguous()))

    def split_heads(t):  # Reshape [B,S,h,d] -> Transpose [0,2,1,3]
        return t.reshape(bsz, seq, heads, dh).permute(0, 2, 1, 3).contiguous()

    q = split_heads(linear(x, p["wq"], p["bq"]))
    k = linear(x, p["wk"], p["bk"]).reshape(bsz, seq, heads, dh).permute(0, 2, 3, 1).contiguous()
    v = split_heads(linear(x, p["wv"], p["bv"]))
    scores = Mul(MatMul(q, k), np.float32(1.0 / math.sqrt(dh)))
    probs = Softmax(scores, axis=3)
    ctx = MatMul(probs, v).permute(0, 2, 1, 3).contiguous().reshape(bsz, seq, hid)
    attn = Add(linear(ctx, p["wo"], p["bo"]), x)
    h1 = LayerNormChain(attn, p["ln1_g"], p["ln1_b"], eps)
    inter = GeluChain(linear(h1, p["wi"], p["bi"]))
    out = Add(linear(inter, p["wo2"], p["bo2"]), h1)
    return LayerNormChain(out, p["ln2_g"], p["ln2_b"], eps)


def bert_encoder_forward(x, layers, heads, eps=1e-12):
    h = _t(x)
    for p in layers:
        h = bert_layer_forward(h, p, heads, eps)
    return h


# ---------------------------------------------------------------------------------------------
# seeded synthetic inputs of the BASELINE configurations (no dataset is involved anywhere)
# ---------------------------------------------------------------------------------------------
def make_bert_layer_params(hidden, ffn, seed, std=0.02):
    """Weights ~ N(0, std^2), biases 0, LayerNorm gamma 1 / beta 0, from a torch CPU generator."""
    g = torch.Generator().manual_seed(seed)

    def w(o, i):
        return torch.randn(o, i, generator=g, dtype=F32) * std

    z = lambda n: torch.zeros(n, dtype=F32)  # noqa: E731
    one = lambda n: torch.ones(n, dtype=F32)  # noqa: E731
    return dict(wq=w(hidden, hidden), bq=z(hidden), wk=w(hidden, hidden), bk=z(hidden), wv=w(hidden, hidden),
                bv=z(hidden), wo=w(hidden, hidden), bo=z(hidden), ln1_g=one(hidden), ln1_b=z(hidden),
                wi=w(ffn, hidden), bi=z(ffn), wo2=w(hidden, ffn), bo2=z(hidden), ln2_g=one(hidden), ln2_b=z(hidden))


def make_mlp_params(seed=0, sizes=(784, 120, 32, 10)):
    """nn.Linear default (Kaiming-uniform) initialisation under a fixed seed."""
    torch.manual_seed(seed)
    params = []
    for i, o in zip(sizes[:-1], sizes[1:]):
        lin = torch.nn.Linear(i, o)
        params.append((lin.weight.detach().clone(), lin.bias.detach().clone()))
    return params


def make_conv_params(seed=0, channels=64, layers=2, k=3):
    g = torch.Generator().manual_seed(seed)
    bound = 1.0 / math.sqrt(channels * k * k)
    out = []
    for _ in range(layers):
        w = (torch.rand(channels, channels, k, k, generator=g, dtype=F32) * 2 - 1) * bound
        b = (torch.rand(channels, generator=g, dtype=F32) * 2 - 1) * bound
        out.append((w, b))
    return out
