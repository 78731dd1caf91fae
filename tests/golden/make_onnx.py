"""Exports the small torch models whose ONNX graphs the front-door tests load (tests/golden/*.onnx) and
stores each model's input and the exporting torch module's own output beside it (tests/golden/onnx_*.npz).

Run from the repository root:  python tests/golden/make_onnx.py
The graphs are what the reference's DaceModule would import for the same modules (opset 12, TorchScript
exporter, daceml/pytorch/module.py:238-255); the modules follow the reference's tests: an MLP with
LogSoftmax (tests/autodiff/pytorch/test_training.py:68-96 shape family), a Conv-ReLU stack
(tests/pytorch/test_conv2d.py:11-37) and transformers.BertLayer (tests/pytorch/test_bert_encoder.py:10-34),
all shrunk so that the files stay small.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from dace_onnx_b200.torch_module import export_onnx  # noqa: E402


class MLP(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1, self.fc2, self.fc3 = torch.nn.Linear(96, 40), torch.nn.Linear(40, 24), torch.nn.Linear(24, 10)

    def forward(self, x):
        x = torch.relu(self.fc1(x))
        x = torch.relu(self.fc2(x))
        return torch.log_softmax(self.fc3(x), dim=1)


class ConvStack(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.c1 = torch.nn.Conv2d(16, 16, 3, padding=1)
        self.c2 = torch.nn.Conv2d(16, 8, 3, padding=1)

    def forward(self, x):
        return torch.relu(self.c2(torch.relu(self.c1(x))))


class NormActs(torch.nn.Module):
    """LayerNorm without affine parameters, Gelu, a softmax over the last axis and a general transpose."""

    def __init__(self):
        super().__init__()
        self.ln = torch.nn.LayerNorm(48, eps=1e-5, elementwise_affine=False)

    def forward(self, x):
        y = torch.nn.functional.gelu(self.ln(x))
        return torch.softmax(y.permute(2, 0, 1), dim=-1)


def bert_layer():
    from transformers import BertConfig, BertLayer
    cfg = BertConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    cfg._attn_implementation = "eager"
    return BertLayer(cfg)


def main():
    cases = [("mlp", MLP, (32, 96), True), ("conv_stack", ConvStack, (2, 16, 12, 12), True),
             ("norm_acts", NormActs, (3, 20, 48), True), ("bert_layer", bert_layer, (2, 32, 128), True),
             ("bert_layer_nofold", bert_layer, (2, 32, 128), False)]
    for seed, (name, make, shape, fold) in enumerate(cases):
        torch.manual_seed(100 + (3 if name == "bert_layer_nofold" else seed))
        model = make().eval()
        # biases and LayerNorm parameters away from their 0 / 1 defaults so that every operand matters
        with torch.no_grad():
            for pname, p in model.named_parameters():
                if p.dim() == 1:
                    p.add_(0.1 * torch.randn_like(p))
        x = torch.randn(*shape)
        with torch.no_grad():
            y = model(x)
        y = y[0] if isinstance(y, (tuple, list)) else y
        data = export_onnx(model, (x,), fold_constants=fold)
        with open(os.path.join(HERE, name + ".onnx"), "wb") as fh:
            fh.write(data)
        np.savez(os.path.join(HERE, "onnx_" + name + ".npz"), x=x.numpy(), y=y.numpy())
        print(name, len(data), "bytes", tuple(y.shape))


if __name__ == "__main__":
    main()
