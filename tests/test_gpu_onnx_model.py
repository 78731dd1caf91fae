"""The ONNX front door on the GPU: exported graphs executed by ONNXModelB200 (fused and node by node)
against the unfused CPU graph oracle and against the exporting torch module's own output."""
import os

import numpy as np
import pytest
import torch

from dace_onnx_b200 import ops
from dace_onnx_b200.onnx_graph import UnsupportedNode
from dace_onnx_b200.onnx_model import ONNXModelB200
from dace_onnx_b200.torch_module import B200Module, export_onnx
from oracle import graph_oracle
from tests._util import ATOL, GOLDEN, REF_ATOL, REF_RTOL, RTOL, TF32_ATOL, TF32_RTOL, close, golden

pytestmark = pytest.mark.gpu

CASES = ["mlp", "conv_stack", "norm_acts", "bert_layer", "bert_layer_nofold"]


def _path(name):
    return os.path.join(GOLDEN, name + ".onnx")


@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("mode", ["fp32x3", "fp32"])
@pytest.mark.parametrize("name", CASES)
def test_exported_graph_matches_oracle(name, mode, fuse, cuda):
    g = golden("onnx_" + name)
    model = ONNXModelB200(name, _path(name), cuda=True, fuse=fuse, math_mode=mode)
    y = model(torch.from_numpy(g["x"]))
    assert y.is_cuda and y.dtype == torch.float32
    ref = graph_oracle.run(_path(name), [g["x"]])[0]
    close(y, ref, RTOL, ATOL)
    close(y, g["y"], REF_RTOL, REF_ATOL)   # the reference's own criterion against the torch module


@pytest.mark.parametrize("name", ["mlp", "conv_stack", "bert_layer"])
def test_exported_graph_tf32(name, cuda):
    g = golden("onnx_" + name)
    y = ONNXModelB200(name, _path(name), math_mode="tf32")(torch.from_numpy(g["x"]).cuda())
    close(y, graph_oracle.run(_path(name), [g["x"]])[0], TF32_RTOL, TF32_ATOL)


def test_fused_and_unfused_plans(cuda):
    fused = ONNXModelB200("bert", _path("bert_layer"), fuse=True).plan((2, 32, 128))
    plain = ONNXModelB200("bert", _path("bert_layer"), fuse=False).plan((2, 32, 128))
    assert len(fused.steps) == 6 and len(plain.steps) == 49
    assert fused.fusion_stats["attention"] == 1 and plain.fusion_stats == {}
    # liveness-based reuse: far fewer distinct buffers than values
    assert plain.buffer_bytes < 4 * sum(int(np.prod(s)) for s in plain.ir.shapes.values()) / 2


def test_conv_chain_stays_nhwc_between_convolutions(cuda):
    g = golden("onnx_conv_stack")
    fused = ONNXModelB200("conv_stack", _path("conv_stack"), fuse=True)
    x = torch.from_numpy(g["x"])
    plan = fused.plan(tuple(x.shape))
    assert plan.fusion_stats["conv_relu"] == 2 and plan.fusion_stats["conv_nhwc_links"] == 1
    convs = [n for n in plan.ir.nodes if n.op_type == "Conv"]
    assert convs[0].attr("y_nhwc") == 1 and convs[1].attr("x_nhwc") == 1 and not convs[1].attr("y_nhwc", 0)
    close(fused(x), graph_oracle.run(_path("conv_stack"), [g["x"]])[0], RTOL, ATOL)
    plain = ONNXModelB200("conv_stack", _path("conv_stack"), fuse=False).plan(tuple(x.shape))
    assert not any(n.attr("x_nhwc", 0) or n.attr("y_nhwc", 0) for n in plain.ir.nodes)


def test_calling_conventions(cuda):
    g = golden("onnx_mlp")
    model = ONNXModelB200("mlp", open(_path("mlp"), "rb").read())
    x = torch.from_numpy(g["x"])
    name = model.input_names[0]
    y1 = model(x)
    y2 = model(**{name: g["x"]})                       # numpy, by name
    y3 = model(x.cuda())
    assert torch.equal(y1, y2) and torch.equal(y1, y3)
    assert y1.data_ptr() != y3.data_ptr()              # every call returns storage of its own
    keep = y1.clone()
    model(torch.zeros_like(x))
    assert torch.equal(y1, keep)
    with pytest.raises(TypeError):
        model()
    with pytest.raises(TypeError):
        model(x, x)
    with pytest.raises(TypeError):
        model(x.double())
    with pytest.raises(ValueError):
        model(x[:16])                                  # the graph was exported for batch 32
    with pytest.raises(ValueError):
        ONNXModelB200("mlp", _path("mlp"), cuda=False)


def test_unsupported_operator_is_refused(cuda):
    class M(torch.nn.Module):
        def forward(self, x):
            return torch.tanh(x) + 1.0

    model = ONNXModelB200("tanh", export_onnx(M(), (torch.zeros(2, 3),)))
    with pytest.raises(UnsupportedNode):
        model(torch.zeros(2, 3))


def test_general_permute(cuda):
    x = torch.randn(3, 5, 4, 7, generator=torch.Generator().manual_seed(5))
    for perm in ([3, 0, 2, 1], [1, 0, 3, 2], [2, 3, 0, 1], [0, 1, 2, 3]):
        assert torch.equal(ops.permute(x.cuda(), perm).cpu(), x.permute(perm).contiguous())
    x = torch.tensor([[-0.0, float("inf")], [1.5, -2.0]])
    y = ops.permute(x.cuda(), [1, 0]).cpu()
    assert torch.equal(y, x.t().contiguous()) and torch.signbit(y[0, 0])


def test_b200_module_live_export_with_fused_attention(cuda):
    """transformers.BertLayer wrapped like the reference's DaceModule (tests/pytorch/test_bert_encoder.py:10-34),
    at a size the fused TF32 attention kernel covers (head_dim 64, sequence a multiple of 32)."""
    from transformers import BertConfig, BertLayer
    torch.manual_seed(7)
    cfg = BertConfig(hidden_size=256, num_attention_heads=4, intermediate_size=512, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    cfg._attn_implementation = "eager"
    layer = BertLayer(cfg).eval()
    x = torch.randn(4, 128, 256)
    with torch.no_grad():
        ref = layer(x)
    ref = ref[0] if isinstance(ref, (tuple, list)) else ref
    for mode, rtol, atol in (("tf32", TF32_RTOL, TF32_ATOL), ("fp32x3", REF_RTOL, REF_ATOL)):
        mod = B200Module(layer, math_mode=mode, sdfg_name="bert_layer")
        out = mod(x.cuda())
        close(out, ref, rtol, atol)
        plan = mod.onnx_model.plan((4, 128, 256))
        assert plan.ir.op_histogram() == {"B200SelfAttention": 1, "B200Gemm": 3, "B200LayerNorm": 2}
        close(mod(x.cuda()), out, 0, 0)              # same plan, same buffers, same result


@pytest.mark.parametrize("name", ["mlp", "bert_layer", "conv_stack"])
def test_cuda_graph_replay_equals_eager(name, cuda):
    g = golden("onnx_" + name)
    x = torch.from_numpy(g["x"]).cuda()
    eager = ONNXModelB200(name, _path(name))(x)
    model = ONNXModelB200(name, _path(name), cuda_graph=True)
    y1 = model(x).clone()                      # first call captures
    y2 = model(x).clone()                      # replay, same input address
    y3 = model(x.clone()).clone()              # replay after a copy into the captured input buffer
    assert torch.equal(y1, eager) and torch.equal(y2, eager) and torch.equal(y3, eager)
    z = model(torch.zeros_like(x)).clone()
    assert not torch.equal(z, eager)
    assert torch.equal(model(x), eager)
    assert torch.equal(x.cpu(), torch.from_numpy(g["x"]))      # the caller's tensors are never written
    buf = model.static_inputs(x.shape)[0]
    buf.copy_(x)
    assert torch.equal(model(buf), eager)


@pytest.mark.parametrize("kernel,stride,shape", [((2, 2), (2, 2), (8, 6, 30, 30)), ((3, 3), (1, 1), (2, 3, 9, 11)),
                                                 ((2, 3), (3, 2), (1, 4, 17, 13)), ((2, 2), (2, 2), (64, 16, 56, 56))])
def test_maxpool_node(kernel, stride, shape, cuda):
    from oracle import pure_oracle as po
    x = torch.randn(*shape, generator=torch.Generator().manual_seed(41))
    assert torch.equal(ops.maxpool2d(x.cuda(), kernel, stride).cpu(), po.MaxPool(x, kernel, stride))
    assert ops.maxpool2d(torch.empty(0, 3, 8, 8, device="cuda"), (2, 2), (2, 2)).shape == (0, 3, 4, 4)
    with pytest.raises(ValueError):
        ops.maxpool2d(x.cuda()[:, :, :1], (2, 2))


def test_lenet_like_the_reference_test(cuda):
    """tests/pytorch/test_lenet.py:14-54 with B200Module in place of DaceModule and the same comparator."""
    import torch.nn as nn
    import torch.nn.functional as F

    class LeNet(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = nn.Conv2d(1, 6, (3, 3))
            self.conv2 = nn.Conv2d(6, 16, (3, 3))
            self.fc1 = nn.Linear(16 * 6 * 6, 120)
            self.fc2 = nn.Linear(120, 84)
            self.fc3 = nn.Linear(84, 10)

        def forward(self, x):
            x = F.max_pool2d(F.relu(self.conv1(x)), 2)
            x = F.max_pool2d(F.relu(self.conv2(x)), 2)
            x = x.view(-1, 16 * 6 * 6)
            x = F.relu(self.fc1(x))
            x = F.relu(self.fc2(x))
            return F.log_softmax(self.fc3(x), dim=1)

    torch.manual_seed(11)
    net = LeNet().eval()
    x = torch.rand(8, 1, 32, 32)
    with torch.no_grad():
        ref = net(x)
    for fuse in (True, False):
        mod = B200Module(net, fuse=fuse, sdfg_name="lenet")
        out = mod(x)
        close(out, ref, REF_RTOL, REF_ATOL)
        close(out, graph_oracle.run(export_onnx(net, (x,)), [x])[0], RTOL, ATOL)
    hist = B200Module(net, dummy_inputs=(x,)).onnx_model.plan((8, 1, 32, 32)).ir.op_histogram()
    assert hist == {"Conv": 2, "MaxPool": 2, "Reshape": 1, "B200Gemm": 3, "LogSoftmax": 1}
