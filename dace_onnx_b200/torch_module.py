"""B200Module: wrap a torch.nn.Module so that its forward runs on the b200 kernels.

Mirror of the reference's `daceml.pytorch.DaceModule` (daceml/pytorch/module.py:58-120 constructor,
:238-255 export step): the module is exported to ONNX (opset 12, TorchScript exporter, constant folding on)
with the first call's inputs as example inputs, loaded into `ONNXModelB200`, and every call is then executed
from that graph. Inference only. The weights are the ones the module held when it was exported.
"""
import io
import warnings

import torch

from .onnx_model import ONNXModelB200


def export_onnx(module: torch.nn.Module, dummy_inputs, opset: int = 12, fold_constants: bool = True) -> bytes:
    """Serialized ONNX ModelProto of `module` traced on `dummy_inputs` (CPU tensors)."""
    if isinstance(dummy_inputs, torch.Tensor):
        dummy_inputs = (dummy_inputs,)
    restore = None
    try:
        import onnx  # noqa: F401
    except ImportError:
        # The TorchScript exporter serialises the graph itself; it imports the `onnx` package only to splice
        # onnx-script functions into the result. A plain module has none, so that step is the identity.
        from torch.onnx._internal.torchscript_exporter import onnx_proto_utils
        restore = (onnx_proto_utils, onnx_proto_utils._add_onnxscript_fn)
        onnx_proto_utils._add_onnxscript_fn = lambda model_bytes, custom_opsets: model_bytes
    try:
        buf = io.BytesIO()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            torch.onnx.export(module, tuple(dummy_inputs), buf, dynamo=False, opset_version=opset,
                              do_constant_folding=fold_constants, training=torch.onnx.TrainingMode.EVAL)
        return buf.getvalue()
    finally:
        if restore is not None:
            restore[0]._add_onnxscript_fn = restore[1]


class B200Module(torch.nn.Module):
    """:param module: the model to run (put in eval mode for the export).
    :param dummy_inputs: example inputs to export with now; otherwise the first call's inputs are used.
    :param cuda: must stay True (there is no CPU execution).
    :param fuse, math_mode, cuda_graph: see ONNXModelB200."""

    def __init__(self, module, dummy_inputs=None, cuda=True, training=False, fuse=True, math_mode=None,
                 sdfg_name=None, cuda_graph=False):
        super().__init__()
        if training:
            raise NotImplementedError("B200Module runs inference only")
        if cuda is False:
            raise ValueError("B200Module runs on a CUDA device only")
        self.model = module
        self.sdfg_name = sdfg_name or type(module).__name__
        self.fuse = fuse
        self.math_mode = math_mode
        self.cuda_graph = cuda_graph
        self.onnx_model = None
        if dummy_inputs is not None:
            self._initialize(dummy_inputs if isinstance(dummy_inputs, (tuple, list)) else (dummy_inputs,))

    def _initialize(self, inputs):
        was_training = self.model.training
        self.model.eval()
        cpu_model = self.model.to("cpu")
        data = export_onnx(cpu_model, tuple(t.detach().to("cpu") for t in inputs))
        self.model.train(was_training)
        self.onnx_model = ONNXModelB200(self.sdfg_name, data, cuda=True, fuse=self.fuse, math_mode=self.math_mode,
                                        cuda_graph=self.cuda_graph)

    def forward(self, *inputs):
        if self.onnx_model is None:
            self._initialize(inputs)
        return self.onnx_model(*inputs)
