"""Reader for the ONNX protobuf wire format, limited to what an exported inference graph holds.

The reference loads models with the `onnx` package (daceml/onnx/onnx_importer.py:95-140 walks
`model.graph.node`, `.initializer`, `.input`, `.output`); that package is not a dependency here, so
the handful of messages involved (ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto,
ValueInfoProto) are decoded directly from their published field numbers. Host-only code: bytes in,
plain Python objects and numpy arrays out.
"""
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

# TensorProto.DataType -> numpy
_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_,
           10: np.float16, 11: np.float64, 12: np.uint32, 13: np.uint64}


class OnnxFormatError(ValueError):
    pass


@dataclass
class Node:
    op_type: str
    name: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, object] = field(default_factory=dict)
    domain: str = ""

    def attr(self, key, default=None):
        return self.attrs.get(key, default)


@dataclass
class ValueInfo:
    name: str
    dtype: Optional[type]
    shape: Optional[Tuple[object, ...]]  # ints, or str for symbolic dimensions


@dataclass
class Graph:
    name: str
    nodes: List[Node]
    initializers: Dict[str, np.ndarray]
    inputs: List[ValueInfo]   # graph inputs that are not initializers
    outputs: List[ValueInfo]


@dataclass
class Model:
    graph: Graph
    opset: int
    producer: str = ""


def _varint(buf, pos):
    result = 0
    shift = 0
    while True:
        if pos >= len(buf):
            raise OnnxFormatError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise OnnxFormatError("varint too long")


def _fields(buf):
    """Yield (field number, wire type, value) for one message; length-delimited values are memoryviews."""
    pos = 0
    n = len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        fno, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _varint(buf, pos)
        elif wt == 1:
            v = bytes(buf[pos:pos + 8])
            pos += 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            if pos + ln > n:
                raise OnnxFormatError("length-delimited field runs past the end of its message")
            v = buf[pos:pos + ln]
            pos += ln
        elif wt == 5:
            v = bytes(buf[pos:pos + 4])
            pos += 4
        else:
            raise OnnxFormatError("unsupported wire type %d" % wt)
        yield fno, wt, v


def _sint64(v):
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(wt, v):
    if wt == 0:
        return [_sint64(v)]
    out = []
    pos = 0
    while pos < len(v):
        x, pos = _varint(v, pos)
        out.append(_sint64(x))
    return out


def _packed_fixed(wt, v, fmt, size):
    if wt in (1, 5):
        return [struct.unpack("<" + fmt, v)[0]]
    return list(struct.unpack("<%d%s" % (len(v) // size, fmt), bytes(v)))


def _text(v):
    return bytes(v).decode("utf-8")


def _tensor(buf):
    dims, dtype, name, raw = [], 1, "", None
    floats, int32s, int64s, doubles, uint64s = [], [], [], [], []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            dims += _packed_varints(wt, v)
        elif fno == 2:
            dtype = v
        elif fno == 4:
            floats += _packed_fixed(wt, v, "f", 4)
        elif fno == 5:
            int32s += _packed_varints(wt, v)
        elif fno == 7:
            int64s += _packed_varints(wt, v)
        elif fno == 8:
            name = _text(v)
        elif fno == 9:
            raw = bytes(v)
        elif fno == 10:
            doubles += _packed_fixed(wt, v, "d", 8)
        elif fno == 11:
            uint64s += _packed_varints(wt, v)
        elif fno in (13, 14) and (fno == 13 or v != 0):
            raise OnnxFormatError("tensor '%s' keeps its data in an external file" % name)
    if dtype not in _DTYPES:
        raise OnnxFormatError("tensor '%s': unsupported data type %d" % (name, dtype))
    np_dtype = _DTYPES[dtype]
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(np_dtype).newbyteorder("<")).astype(np_dtype, copy=True)
    elif dtype == 1:
        arr = np.asarray(floats, dtype=np.float32)
    elif dtype == 11:
        arr = np.asarray(doubles, dtype=np.float64)
    elif dtype == 7:
        arr = np.asarray(int64s, dtype=np.int64)
    elif dtype in (12, 13):
        arr = np.asarray(uint64s, dtype=np_dtype)
    elif dtype == 10:
        arr = np.asarray(int32s, dtype=np.uint16).view(np.float16)
    else:
        arr = np.asarray(int32s).astype(np_dtype)
    count = int(np.prod(dims)) if dims else 1
    if arr.size != count:
        raise OnnxFormatError("tensor '%s': %d values for shape %s" % (name, arr.size, dims))
    return name, arr.reshape(dims)


def _attribute(buf):
    name, kind = "", 0
    f = i = s = t = None
    floats, ints, strings = [], [], []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            name = _text(v)
        elif fno == 20:
            kind = v
        elif fno == 2:
            f = struct.unpack("<f", v)[0]
        elif fno == 3:
            i = _sint64(v)
        elif fno == 4:
            s = bytes(v)
        elif fno == 5:
            t = _tensor(v)[1]
        elif fno == 7:
            floats += _packed_fixed(wt, v, "f", 4)
        elif fno == 8:
            ints += _packed_varints(wt, v)
        elif fno == 9:
            strings.append(bytes(v))
        elif fno in (6, 11):
            raise OnnxFormatError("attribute '%s': subgraphs (control flow) are not supported" % name)
    if kind == 0:  # writers older than IR 3 leave the type out
        kind = 1 if f is not None else 2 if i is not None else 3 if s is not None else 4 if t is not None else \
            6 if floats else 7 if ints else 8 if strings else 0
    value = {1: f, 2: i, 3: s.decode("utf-8", "replace") if s is not None else None, 4: t, 6: floats, 7: ints,
             8: [x.decode("utf-8", "replace") for x in strings]}.get(kind)
    if kind in (1, 2) and value is None:
        value = 0.0 if kind == 1 else 0  # proto3 leaves zero scalars out
    if kind not in (1, 2, 3, 4, 6, 7, 8):
        raise OnnxFormatError("attribute '%s': unsupported attribute type %d" % (name, kind))
    return name, value


def _node(buf):
    n = Node("", "", [], [])
    for fno, _wt, v in _fields(buf):
        if fno == 1:
            n.inputs.append(_text(v))
        elif fno == 2:
            n.outputs.append(_text(v))
        elif fno == 3:
            n.name = _text(v)
        elif fno == 4:
            n.op_type = _text(v)
        elif fno == 5:
            k, val = _attribute(v)
            n.attrs[k] = val
        elif fno == 7:
            n.domain = _text(v)
    return n


def _value_info(buf):
    name, dtype, shape = "", None, None
    for fno, _wt, v in _fields(buf):
        if fno == 1:
            name = _text(v)
        elif fno == 2:  # TypeProto
            for f2, _w2, v2 in _fields(v):
                if f2 != 1:  # only tensor_type
                    continue
                for f3, _w3, v3 in _fields(v2):
                    if f3 == 1:
                        dtype = _DTYPES.get(v3)
                    elif f3 == 2:  # TensorShapeProto
                        dims = []
                        for f4, _w4, v4 in _fields(v3):
                            if f4 != 1:
                                continue
                            d = None
                            for f5, _w5, v5 in _fields(v4):
                                if f5 == 1:
                                    d = _sint64(v5)
                                elif f5 == 2:
                                    d = _text(v5)
                            dims.append(d)
                        shape = tuple(dims)
    return ValueInfo(name, dtype, shape)


def _graph(buf):
    g = Graph("", [], {}, [], [])
    inputs = []
    for fno, _wt, v in _fields(buf):
        if fno == 1:
            g.nodes.append(_node(v))
        elif fno == 2:
            g.name = _text(v)
        elif fno == 5:
            name, arr = _tensor(v)
            g.initializers[name] = arr
        elif fno == 11:
            inputs.append(_value_info(v))
        elif fno == 12:
            g.outputs.append(_value_info(v))
        elif fno == 15:
            raise OnnxFormatError("sparse initializers are not supported")
    g.inputs = [vi for vi in inputs if vi.name not in g.initializers]
    return g


def parse_model(data) -> Model:
    """Decode a serialized ONNX ModelProto (bytes, bytearray or memoryview)."""
    buf = memoryview(bytes(data))
    graph, opset, producer = None, 0, ""
    for fno, _wt, v in _fields(buf):
        if fno == 7:
            graph = _graph(v)
        elif fno == 2:
            producer = _text(v)
        elif fno == 8:  # OperatorSetIdProto
            domain, version = "", 0
            for f2, _w2, v2 in _fields(v):
                if f2 == 1:
                    domain = _text(v2)
                elif f2 == 2:
                    version = v2
            if domain in ("", "ai.onnx"):
                opset = version
    if graph is None:
        raise OnnxFormatError("no graph in the model")
    return Model(graph, opset, producer)


def load_model(path) -> Model:
    with open(path, "rb") as fh:
        return parse_model(fh.read())
