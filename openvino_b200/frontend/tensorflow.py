"""TensorFlow frontend: frozen ``GraphDef`` (``.pb``) -> ``Model``.

The protobuf wire format is decoded here (no ``tensorflow`` / ``protobuf`` package needed). Placeholders become
Parameters, Const nodes Constants, every other node goes through a table of translators. TensorFlow graphs are NHWC:
spatial operations are wrapped in Transposes to the NCHW operations of the opset, which the layout passes of the device
pipelines sink and merge. Role of src/frontends/tensorflow/src/frontend.cpp (GraphDef iterator, `input_model.cpp`) and
the shared translators of src/frontends/tensorflow_common/src/op/*.cpp.
"""
from __future__ import annotations

import struct
from typing import Callable, Dict, List, Optional

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output, as_output, constant, parameter, result
from .._types import PartialShape
from . import common_translators as CT
from .onnx import _fields, _packed_ints, _sint


class TensorFlowError(RuntimeError):
    pass


_NP = {1: np.float32, 2: np.float64, 3: np.int32, 4: np.uint8, 5: np.int16, 6: np.int8, 9: np.int64, 10: np.bool_, 19: np.float16}
_OV = {1: "f32", 2: "f64", 3: "i32", 4: "u8", 5: "i16", 6: "i8", 9: "i64", 10: "boolean", 19: "f16", 14: "bf16"}


def _shape_proto(b) -> Optional[List[int]]:
    dims, unknown = [], False
    for f, w, v in _fields(b):
        if f == 2:
            size = 0
            for f2, _, v2 in _fields(v):
                if f2 == 1:
                    size = _sint(v2)
            dims.append(size)
        elif f == 3:
            unknown = bool(v)
    return None if unknown else dims


def _tensor_proto(b) -> np.ndarray:
    dtype, shape, content = 1, [], None
    floats, ints, int64s, halfs, bools, doubles = [], [], [], [], [], []
    for f, w, v in _fields(b):
        if f == 1:
            dtype = v
        elif f == 2:
            shape = _shape_proto(v) or []
        elif f == 4:
            content = bytes(v)
        elif f == 5:
            floats += list(np.frombuffer(v, "<f4")) if w == 2 else [struct.unpack("<f", v)[0]]
        elif f == 6:
            doubles += list(np.frombuffer(v, "<f8")) if w == 2 else [struct.unpack("<d", v)[0]]
        elif f == 7:
            ints += _packed_ints(v) if w == 2 else [_sint(v)]
        elif f == 10:
            int64s += _packed_ints(v) if w == 2 else [_sint(v)]
        elif f == 11:
            bools += _packed_ints(v) if w == 2 else [v]
        elif f == 13:
            halfs += _packed_ints(v) if w == 2 else [v]
    if dtype == 14:
        raw = np.frombuffer(content, "<u2") if content is not None else np.array(halfs, np.uint16)
        return (raw.astype(np.uint32) << 16).view(np.float32).reshape(shape)
    if dtype not in _NP:
        raise TensorFlowError("unsupported tensor dtype %d" % dtype)
    np_t = _NP[dtype]
    n = int(np.prod(shape)) if shape else 1
    if content is not None:
        return np.frombuffer(content, dtype=np.dtype(np_t).newbyteorder("<")).astype(np_t).reshape(shape)
    vals = {1: floats, 2: doubles, 3: ints, 4: ints, 5: ints, 6: ints, 9: int64s, 10: bools}.get(dtype)
    if dtype == 19:
        arr = np.array(halfs, np.uint16).view(np.float16)
    else:
        arr = np.array(vals, dtype=np_t)
    if arr.size == 1 and n != 1:
        arr = np.full(n, arr.reshape(-1)[0], dtype=np_t)      # a splat constant stores one value
    if arr.size == 0 and n:
        arr = np.zeros(n, dtype=np_t)
    return arr.reshape(shape)


def _attr_value(b):
    for f, w, v in _fields(b):
        if f == 2:
            return bytes(v)
        if f == 3:
            return _sint(v)
        if f == 4:
            return struct.unpack("<f", v)[0]
        if f == 5:
            return bool(v)
        if f == 6:
            return ("type", v)
        if f == 7:
            return ("shape", _shape_proto(v))
        if f == 8:
            return _tensor_proto(v)
        if f == 1:
            out = []
            for f2, w2, v2 in _fields(v):
                if f2 == 2:
                    out.append(bytes(v2))
                elif f2 == 3:
                    out += _packed_ints(v2) if w2 == 2 else [_sint(v2)]
                elif f2 == 4:
                    out += list(np.frombuffer(v2, "<f4")) if w2 == 2 else [struct.unpack("<f", v2)[0]]
                elif f2 == 5:
                    out += [bool(x) for x in (_packed_ints(v2) if w2 == 2 else [v2])]
                elif f2 == 6:
                    out += [("type", x) for x in (_packed_ints(v2) if w2 == 2 else [v2])]
                elif f2 == 7:
                    out.append(("shape", _shape_proto(v2)))
            return out
    return None


class _NodeDef:
    def __init__(self, b):
        self.name, self.op, self.inputs, self.attrs = "", "", [], {}
        for f, w, v in _fields(b):
            if f == 1:
                self.name = bytes(v).decode()
            elif f == 2:
                self.op = bytes(v).decode()
            elif f == 3:
                self.inputs.append(bytes(v).decode())
            elif f == 5:
                key, val = "", None
                for f2, _, v2 in _fields(v):
                    if f2 == 1:
                        key = bytes(v2).decode()
                    elif f2 == 2:
                        val = _attr_value(v2)
                self.attrs[key] = val


# ------------------------------------------------------------------------------------------------ translators
_T: Dict[str, Callable] = {}


def _op(*names):
    def deco(fn):
        for n in names:
            _T[n] = fn
        return fn
    return deco


def _i64(v) -> Output:
    return constant(np.array(v, dtype=np.int64)).output(0)


def _ints_of(o: Output) -> List[int]:
    from .onnx import _const_ints
    return _const_ints(o)


def _nchw(x):
    return ops.transpose(x, _i64([0, 3, 1, 2])).output(0)


def _nhwc(x):
    return ops.transpose(x, _i64([0, 2, 3, 1])).output(0)


def _is_nhwc(n) -> bool:
    return n.attrs.get("data_format", b"NHWC") == b"NHWC"


def _spatial(v, nhwc):
    return [int(v[1]), int(v[2])] if nhwc else [int(v[2]), int(v[3])]


def _auto_pad(n):
    return {b"SAME": "same_upper", b"VALID": "valid"}.get(n.attrs.get("padding", b"VALID"), "explicit")


for _name, _f in (("Add", ops.add), ("AddV2", ops.add), ("Sub", ops.subtract), ("Mul", ops.multiply), ("RealDiv", ops.divide), ("Maximum", ops.maximum),
                  ("Minimum", ops.minimum), ("Pow", ops.power), ("Equal", ops.equal), ("Greater", ops.greater), ("Less", ops.less), ("BiasAddNCHW", ops.add)):
    _T[_name] = (lambda f: lambda n, i: f(i[0], i[1]).output(0))(_f)
for _name, _f in (("Relu", ops.relu), ("Sigmoid", ops.sigmoid), ("Tanh", ops.tanh), ("Exp", ops.exp), ("Sqrt", ops.sqrt), ("Neg", ops.negative),
                  ("Erf", ops.erf), ("Abs", ops.abs), ("Log", ops.log), ("Floor", ops.floor), ("Softplus", ops.softplus)):
    _T[_name] = (lambda f: lambda n, i: f(i[0]).output(0))(_f)


@_op("Identity", "StopGradient", "PlaceholderWithDefault", "Snapshot")
def _identity(n, i):
    return i[0]


@_op("Relu6")
def _relu6(n, i):
    return ops.clamp(i[0], 0.0, 6.0).output(0)


@_op("LeakyRelu")
def _leaky(n, i):
    return ops.prelu(i[0], constant(np.array(n.attrs.get("alpha", 0.2), np.float32), i[0].get_element_type())).output(0)


@_op("Rsqrt")
def _rsqrt(n, i):
    return ops.divide(constant(np.array(1.0, np.float32), i[0].get_element_type()), ops.sqrt(i[0])).output(0)


@_op("Square")
def _square(n, i):
    return ops.multiply(i[0], i[0]).output(0)


@_op("BiasAdd")
def _bias_add(n, i):
    if _is_nhwc(n):
        return ops.add(i[0], i[1]).output(0)
    r = len(i[0].get_partial_shape())
    return ops.add(i[0], ops.reshape(i[1], _i64([1, -1] + [1] * (r - 2)), False)).output(0)


@_op("Conv2D")
def _conv2d(n, i):
    nhwc = _is_nhwc(n)
    w = ops.transpose(i[1], _i64([3, 2, 0, 1])).output(0)          # HWIO -> OIHW
    strides, dil = _spatial(n.attrs.get("strides", [1, 1, 1, 1]), nhwc), _spatial(n.attrs.get("dilations", [1, 1, 1, 1]), nhwc)
    pad = _auto_pad(n)
    pb = pe = [0, 0]
    if pad == "explicit":
        ep = n.attrs.get("explicit_paddings", [0] * 8)
        hw = (ep[2:6] if nhwc else ep[4:8])
        pb, pe = [int(hw[0]), int(hw[2])], [int(hw[1]), int(hw[3])]
    return CT.conv2d(i[0], w, strides, dil, pad, pb, pe, nhwc=nhwc)


@_op("DepthwiseConv2dNative")
def _depthwise(n, i):
    nhwc = _is_nhwc(n)
    kh, kw, cin, mult = i[1].get_shape()
    w = ops.transpose(i[1], _i64([2, 3, 0, 1]))                       # HWIM -> IMHW
    w = ops.reshape(w, _i64([cin, mult, 1, kh, kw]), False).output(0)  # groups = I, out per group = M, in per group = 1
    strides, dil = _spatial(n.attrs.get("strides", [1, 1, 1, 1]), nhwc), _spatial(n.attrs.get("dilations", [1, 1, 1, 1]), nhwc)
    return CT.depthwise_conv2d(i[0], w, strides, dil, _auto_pad(n), nhwc=nhwc)


@_op("MaxPool", "AvgPool")
def _pool(n, i):
    nhwc = _is_nhwc(n)
    return CT.pool2d(i[0], _spatial(n.attrs["ksize"], nhwc), _spatial(n.attrs["strides"], nhwc), _auto_pad(n), n.op == "MaxPool", nhwc=nhwc)


@_op("FusedBatchNorm", "FusedBatchNormV2", "FusedBatchNormV3")
def _fused_bn(n, i):
    return CT.batch_norm(i[0], i[1], i[2], i[3], i[4], float(n.attrs.get("epsilon", 1e-3)), nhwc=_is_nhwc(n))


@_op("MatMul")
def _matmul(n, i):
    return ops.matmul(i[0], i[1], bool(n.attrs.get("transpose_a", False)), bool(n.attrs.get("transpose_b", False))).output(0)


@_op("BatchMatMul", "BatchMatMulV2")
def _batch_matmul(n, i):
    return ops.matmul(i[0], i[1], bool(n.attrs.get("adj_x", False)), bool(n.attrs.get("adj_y", False))).output(0)


@_op("Softmax")
def _softmax(n, i):
    return ops.softmax(i[0], -1).output(0)


@_op("Reshape")
def _reshape(n, i):
    return ops.reshape(i[0], i[1], False).output(0)


@_op("Squeeze")
def _squeeze(n, i):
    dims = n.attrs.get("squeeze_dims") or []
    return (ops.squeeze(i[0], _i64([int(d) for d in dims])) if dims else ops.squeeze(i[0])).output(0)


@_op("ExpandDims")
def _expand_dims(n, i):
    return ops.unsqueeze(i[0], i[1]).output(0)


def _reduce(f):
    def fn(n, i):
        return f(i[0], i[1], bool(n.attrs.get("keep_dims", False))).output(0)
    return fn


for _name, _f in (("Mean", ops.reduce_mean), ("Sum", ops.reduce_sum), ("Max", ops.reduce_max), ("Min", ops.reduce_min), ("Prod", ops.reduce_prod)):
    _T[_name] = _reduce(_f)


@_op("Pad", "PadV2")
def _pad(n, i):
    p = np.array(_ints_of(i[1])).reshape(-1, 2)
    value = i[2] if len(i) > 2 else constant(np.array(0, np.float32), i[0].get_element_type()).output(0)
    return ops.pad(i[0], _i64(p[:, 0].tolist()), _i64(p[:, 1].tolist()), value, "constant").output(0)


@_op("ConcatV2")
def _concat(n, i):
    return ops.concat(i[:-1], _ints_of(i[-1])[0]).output(0)


@_op("Pack")
def _pack(n, i):
    axis = int(n.attrs.get("axis", 0))
    return ops.concat([ops.unsqueeze(x, _i64([axis])).output(0) for x in i], axis).output(0)


@_op("Transpose")
def _transpose(n, i):
    return ops.transpose(i[0], i[1]).output(0)


@_op("Shape")
def _shape(n, i):
    out = n.attrs.get("out_type")
    return ops.shape_of(i[0], "i64" if out == ("type", 9) else "i32").output(0)


@_op("Cast")
def _cast(n, i):
    return ops.convert(i[0], _OV[n.attrs["DstT"][1]]).output(0)


@_op("GatherV2")
def _gather(n, i):
    return ops.gather(i[0], i[1], i[2]).output(0)


@_op("StridedSlice")
def _strided_slice(n, i):
    def bits(name, rank):
        m = int(n.attrs.get(name, 0))
        return [(m >> k) & 1 for k in range(rank)]
    rank = len(_ints_of(i[1]))
    return ops.strided_slice(i[0], i[1], i[2], i[3], bits("begin_mask", rank), bits("end_mask", rank), bits("new_axis_mask", rank),
                             bits("shrink_axis_mask", rank), bits("ellipsis_mask", rank)).output(0)


def supported_ops() -> List[str]:
    return sorted(_T) + ["Const", "Placeholder", "NoOp"]


def convert(path_or_bytes) -> Model:
    data = path_or_bytes
    if not isinstance(data, (bytes, bytearray, memoryview)):
        with open(str(path_or_bytes), "rb") as f:
            data = f.read()
    nodes = [_NodeDef(v) for f, w, v in _fields(memoryview(data)) if f == 1]
    if not nodes:
        raise TensorFlowError("no nodes in the GraphDef (is this a frozen graph .pb?)")
    values: Dict[str, List[Output]] = {}
    params, consumed = [], set()
    for n in nodes:
        ins = []
        for ref in n.inputs:
            if ref.startswith("^"):
                continue                                  # control dependency
            name, _, idx = ref.partition(":")
            if name not in values:
                raise TensorFlowError("node '%s' reads '%s' before it is defined" % (n.name, ref))
            ins.append(values[name][int(idx or 0)])
            consumed.add(name)
        if n.op == "Placeholder":
            shape = n.attrs.get("shape")
            dims = shape[1] if isinstance(shape, tuple) else None
            p = parameter(PartialShape(dims) if dims is not None else PartialShape.dynamic(), _OV[n.attrs["dtype"][1]], n.name)
            p.output(0).set_names({n.name, n.name + ":0"})
            params.append(p)
            values[n.name] = [p.output(0)]
            continue
        if n.op == "Const":
            values[n.name] = [constant(n.attrs["value"], name=n.name).output(0)]
            continue
        if n.op == "NoOp":
            values[n.name] = []
            continue
        fn = _T.get(n.op)
        if fn is None:
            raise TensorFlowError("no translator for TensorFlow operation %s (node '%s')" % (n.op, n.name))
        out = fn(n, ins)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        outs = [as_output(o) for o in outs]
        for k, o in enumerate(outs):
            o.add_names({"%s:%d" % (n.name, k)} | ({n.name} if k == 0 else set()))
        if outs and outs[0].get_node().get_type_name() not in ("Parameter", "Constant"):
            outs[0].get_node().set_friendly_name(n.name)
        values[n.name] = outs
    # graph outputs: nodes nobody reads (Const / Placeholder / NoOp excluded)
    results = [result(values[n.name][0], n.name) for n in nodes
               if n.name not in consumed and n.op not in ("Const", "Placeholder", "NoOp") and values[n.name]]
    if not results:
        raise TensorFlowError("the graph has no output node")
    return Model(results, params, "tf_model")


from . import tensorflow_more   # noqa: E402,F401  (second part of the translator table)
