"""B200-native kernels for the ONNX library-node hot path of DaCeML, behind a C ABI.

`ops` holds the tensor-level host API, `donnx` mirrors the reference's `donnx.ONNX<Op>` node
signatures, `encoder` runs the BERT encoder configurations, and `b200_implementations` is the
`@op_implementation(..., name="b200")` plugin for a DaCeML installation.
"""
from . import _lib  # noqa: F401
from ._lib import B200Error  # noqa: F401

__all__ = ["B200Error", "ops", "donnx", "encoder"]
