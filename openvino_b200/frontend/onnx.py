"""ONNX frontend: ``.onnx`` file -> ``Model``.

Self-contained: the protobuf wire format of ``ModelProto`` is decoded here (no ``onnx`` / ``protobuf`` package needed),
initializers become Constants, and every node is translated by a table of per-operator functions (opset 13-21
semantics for the covered operators). Role of the reference ONNX frontend (src/frontends/onnx/frontend/src: core/graph.cpp
builds the graph, op/*.cpp hold one translator per operator).
"""
from __future__ import annotations

import struct
from typing import Any, Callable, Dict, List, Optional

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output, as_output, constant, make_op, parameter, result
from .._types import PartialShape, Type


class OnnxError(RuntimeError):
    pass


# ------------------------------------------------------------------------------------------------ protobuf wire format
def _varint(b: memoryview, i: int):
    v, s = 0, 0
    while True:
        c = b[i]
        i += 1
        v |= (c & 0x7F) << s
        if c < 0x80:
            return v, i
        s += 7


def _fields(b: memoryview):
    """Yield (field number, wire type, value) of one message; length-delimited values are memoryviews."""
    i, n = 0, len(b)
    while i < n:
        key, i = _varint(b, i)
        f, w = key >> 3, key & 7
        if w == 0:
            v, i = _varint(b, i)
        elif w == 1:
            v = bytes(b[i:i + 8]); i += 8
        elif w == 2:
            ln, i = _varint(b, i)
            v = b[i:i + ln]; i += ln
        elif w == 5:
            v = bytes(b[i:i + 4]); i += 4
        else:
            raise OnnxError("unsupported protobuf wire type %d" % w)
        yield f, w, v


def _sint(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_ints(v) -> List[int]:
    out, i = [], 0
    while i < len(v):
        x, i = _varint(v, i)
        out.append(_sint(x))
    return out


_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_, 10: np.float16,
           11: np.float64, 12: np.uint32, 13: np.uint64}
_OV_TYPES = {1: "f32", 2: "u8", 3: "i8", 4: "u16", 5: "i16", 6: "i32", 7: "i64", 9: "boolean", 10: "f16", 11: "f64", 12: "u32", 13: "u64", 16: "bf16"}


def _tensor(b: memoryview):
    dims, dt, raw, name = [], 1, None, ""
    f32, i32, i64, f64 = [], [], [], []
    for f, w, v in _fields(b):
        if f == 1:
            dims += _packed_ints(v) if w == 2 else [_sint(v)]
        elif f == 2:
            dt = v
        elif f == 4:
            f32 += list(np.frombuffer(v, dtype="<f4")) if w == 2 else [struct.unpack("<f", v)[0]]
        elif f == 5:
            i32 += _packed_ints(v) if w == 2 else [_sint(v)]
        elif f == 7:
            i64 += _packed_ints(v) if w == 2 else [_sint(v)]
        elif f == 8:
            name = bytes(v).decode()
        elif f == 9:
            raw = bytes(v)
        elif f == 10:
            f64 += list(np.frombuffer(v, dtype="<f8")) if w == 2 else [struct.unpack("<d", v)[0]]
    if dt == 16:   # bfloat16: widen to float32
        src = np.frombuffer(raw, dtype="<u2") if raw is not None else np.array(i32, dtype=np.uint16)
        arr = (src.astype(np.uint32) << 16).view(np.float32)
    elif dt not in _DTYPES:
        raise OnnxError("tensor '%s' has unsupported data type %d" % (name, dt))
    elif raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(_DTYPES[dt]).newbyteorder("<")).astype(_DTYPES[dt])
    elif dt == 1:
        arr = np.array(f32, dtype=np.float32)
    elif dt == 7:
        arr = np.array(i64, dtype=np.int64)
    elif dt == 11:
        arr = np.array(f64, dtype=np.float64)
    elif dt == 10:
        arr = np.array(i32, dtype=np.uint16).view(np.float16)
    else:
        arr = np.array(i32).astype(_DTYPES[dt])
    return name, arr.reshape(dims)


def _attribute(b: memoryview):
    name, val, ints, floats, strings = "", None, [], [], []
    atype = 0
    for f, w, v in _fields(b):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:
            val = struct.unpack("<f", v)[0]
        elif f == 3:
            val = _sint(v)
        elif f == 4:
            val = bytes(v)
        elif f == 5:
            val = _tensor(v)[1]
        elif f == 6:
            val = ("graph", v)
        elif f == 7:
            floats += list(np.frombuffer(v, dtype="<f4")) if w == 2 else [struct.unpack("<f", v)[0]]
        elif f == 8:
            ints += _packed_ints(v) if w == 2 else [_sint(v)]
        elif f == 9:
            strings.append(bytes(v))
        elif f == 20:
            atype = v
    if atype == 7 or (val is None and ints):
        val = ints
    elif atype == 6 or (val is None and floats):
        val = [float(x) for x in floats]
    elif atype == 8 or (val is None and strings):
        val = strings
    if val is None and atype in (7, 6, 8):
        val = []
    return name, val


def _value_info(b: memoryview):
    name, elem, dims = "", 1, None
    for f, w, v in _fields(b):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:
            for f2, _, v2 in _fields(v):
                if f2 == 1:   # tensor_type
                    for f3, _, v3 in _fields(v2):
                        if f3 == 1:
                            elem = v3
                        elif f3 == 2:
                            dims = []
                            for f4, _, v4 in _fields(v3):
                                if f4 == 1:
                                    d = -1
                                    for f5, _, v5 in _fields(v4):
                                        if f5 == 1:
                                            d = _sint(v5)
                                    dims.append(d)
    return name, elem, dims


class _NodeProto:
    def __init__(self, b: memoryview):
        self.inputs, self.outputs, self.name, self.op_type, self.domain, self.attrs = [], [], "", "", "", {}
        for f, w, v in _fields(b):
            if f == 1:
                self.inputs.append(bytes(v).decode())
            elif f == 2:
                self.outputs.append(bytes(v).decode())
            elif f == 3:
                self.name = bytes(v).decode()
            elif f == 4:
                self.op_type = bytes(v).decode()
            elif f == 5:
                k, val = _attribute(v)
                self.attrs[k] = val
            elif f == 7:
                self.domain = bytes(v).decode()


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


def _const_ints(o: Output) -> List[int]:
    from .. import _ovcore as _c
    from .._tensor import Tensor
    packed = _c.constant_value(o._core())
    if packed is None:
        raise OnnxError("a shape-like input must be constant")
    return [int(x) for x in Tensor._from_core(packed).data.reshape(-1)]


for _name, _f in (("Add", ops.add), ("Sub", ops.subtract), ("Mul", ops.multiply), ("Div", ops.divide), ("Pow", ops.power), ("Equal", ops.equal),
                  ("Less", ops.less), ("Greater", ops.greater), ("LessOrEqual", ops.less_equal), ("GreaterOrEqual", ops.greater_equal),
                  ("And", ops.logical_and), ("Or", ops.logical_or), ("Xor", ops.logical_xor)):
    _T[_name] = (lambda f: lambda n, i: f(i[0], i[1]).output(0))(_f)
for _name, _f in (("Relu", ops.relu), ("Sigmoid", ops.sigmoid), ("Tanh", ops.tanh), ("Exp", ops.exp), ("Log", ops.log), ("Sqrt", ops.sqrt),
                  ("Neg", ops.negative), ("Abs", ops.abs), ("Erf", ops.erf), ("Floor", ops.floor), ("Ceil", ops.ceiling), ("Not", ops.logical_not),
                  ("Sin", ops.sin), ("Cos", ops.cos), ("Sign", ops.sign), ("Softplus", ops.softplus), ("HardSwish", ops.hswish), ("Mish", ops.mish)):
    _T[_name] = (lambda f: lambda n, i: f(i[0]).output(0))(_f)


@_op("Identity", "Dropout")
def _identity(n, i):
    return i[0]


@_op("Max", "Min", "Sum", "Mean")
def _variadic(n, i):
    f = {"Max": ops.maximum, "Min": ops.minimum, "Sum": ops.add, "Mean": ops.add}[n.op_type]
    acc = i[0]
    for x in i[1:]:
        acc = f(acc, x).output(0)
    if n.op_type == "Mean":
        acc = ops.divide(acc, constant(np.array(len(i), dtype=np.float32), acc.get_element_type())).output(0)
    return acc


@_op("LeakyRelu")
def _leaky(n, i):
    return ops.prelu(i[0], constant(np.array(n.attrs.get("alpha", 0.01), dtype=np.float32), i[0].get_element_type())).output(0)


@_op("PRelu")
def _prelu(n, i):
    return ops.prelu(i[0], i[1]).output(0)


@_op("Elu")
def _elu(n, i):
    return ops.elu(i[0], float(n.attrs.get("alpha", 1.0))).output(0)


@_op("Gelu")
def _gelu(n, i):
    return ops.gelu(i[0], "tanh" if n.attrs.get("approximate", b"none") == b"tanh" else "erf").output(0)


@_op("Clip")
def _clip(n, i):
    x = i[0]
    lo = i[1] if len(i) > 1 and i[1] is not None else (constant(np.array(n.attrs["min"], dtype=np.float32)).output(0) if "min" in n.attrs else None)
    hi = i[2] if len(i) > 2 and i[2] is not None else (constant(np.array(n.attrs["max"], dtype=np.float32)).output(0) if "max" in n.attrs else None)
    if lo is not None:
        x = ops.maximum(x, lo).output(0)
    if hi is not None:
        x = ops.minimum(x, hi).output(0)
    return x


def _conv_pads(n, nd):
    pads = n.attrs.get("pads", [0] * (2 * nd))
    auto = {b"NOTSET": "explicit", b"SAME_UPPER": "same_upper", b"SAME_LOWER": "same_lower", b"VALID": "valid"}[n.attrs.get("auto_pad", b"NOTSET")]
    return list(pads[:nd]), list(pads[nd:]), auto


@_op("Conv")
def _conv(n, i):
    x, w = i[0], i[1]
    nd = len(w.get_partial_shape()) - 2
    pb, pe, auto = _conv_pads(n, nd)
    strides, dil, group = n.attrs.get("strides", [1] * nd), n.attrs.get("dilations", [1] * nd), n.attrs.get("group", 1)
    if group == 1:
        y = ops.convolution(x, w, strides, pb, pe, dil, auto)
    else:
        ws = w.get_shape()
        wg = ops.reshape(w, _i64([group, ws[0] // group] + list(ws[1:])), False)
        y = ops.group_convolution(x, wg, strides, pb, pe, dil, auto)
    y = y.output(0)
    if len(i) > 2 and i[2] is not None:
        y = ops.add(y, ops.reshape(i[2], _i64([1, -1] + [1] * nd), False)).output(0)
    return y


@_op("MaxPool", "AveragePool")
def _pool(n, i):
    k = n.attrs["kernel_shape"]
    nd = len(k)
    pb, pe, auto = _conv_pads(n, nd)
    strides = n.attrs.get("strides", [1] * nd)
    rounding = "ceil" if n.attrs.get("ceil_mode", 0) else "floor"
    if n.op_type == "MaxPool":
        return ops.max_pool(i[0], strides, n.attrs.get("dilations", [1] * nd), pb, pe, k, rounding, auto).output(0)
    return ops.avg_pool(i[0], strides, pb, pe, k, not n.attrs.get("count_include_pad", 0), rounding, auto).output(0)


@_op("GlobalAveragePool", "GlobalMaxPool")
def _global_pool(n, i):
    r = len(i[0].get_partial_shape())
    f = ops.reduce_mean if n.op_type == "GlobalAveragePool" else ops.reduce_max
    return f(i[0], _i64(list(range(2, r))), True).output(0)


@_op("BatchNormalization")
def _bn(n, i):
    return ops.batch_norm_inference(i[0], i[1], i[2], i[3], i[4], float(n.attrs.get("epsilon", 1e-5))).output(0)


@_op("LayerNormalization")
def _ln(n, i):
    x = i[0]
    axis = n.attrs.get("axis", -1)
    r = len(x.get_partial_shape())
    axes = list(range(axis if axis >= 0 else r + axis, r))
    y = ops.mvn(x, _i64(axes), True, float(n.attrs.get("epsilon", 1e-5)), "inside_sqrt").output(0)
    if len(i) > 1 and i[1] is not None:
        y = ops.multiply(y, i[1]).output(0)
    if len(i) > 2 and i[2] is not None:
        y = ops.add(y, i[2]).output(0)
    return y


@_op("InstanceNormalization")
def _in(n, i):
    x = i[0]
    r = len(x.get_partial_shape())
    y = ops.mvn(x, _i64(list(range(2, r))), True, float(n.attrs.get("epsilon", 1e-5)), "inside_sqrt")
    shape = _i64([1, -1] + [1] * (r - 2))
    return ops.add(ops.multiply(y, ops.reshape(i[1], shape, False)), ops.reshape(i[2], shape, False)).output(0)


@_op("MatMul")
def _matmul(n, i):
    return ops.matmul(i[0], i[1], False, False).output(0)


@_op("Gemm")
def _gemm(n, i):
    a, b = i[0], i[1]
    y = ops.matmul(a, b, bool(n.attrs.get("transA", 0)), bool(n.attrs.get("transB", 0))).output(0)
    alpha, beta = n.attrs.get("alpha", 1.0), n.attrs.get("beta", 1.0)
    if alpha != 1.0:
        y = ops.multiply(y, constant(np.array(alpha, dtype=np.float32), y.get_element_type())).output(0)
    if len(i) > 2 and i[2] is not None:
        c = i[2]
        if beta != 1.0:
            c = ops.multiply(c, constant(np.array(beta, dtype=np.float32), c.get_element_type())).output(0)
        y = ops.add(y, c).output(0)
    return y


@_op("Softmax", "LogSoftmax")
def _softmax(n, i):
    f = ops.softmax if n.op_type == "Softmax" else ops.log_softmax
    return f(i[0], int(n.attrs.get("axis", -1))).output(0)


@_op("Flatten")
def _flatten(n, i):
    axis = n.attrs.get("axis", 1)
    if axis == 0:
        return ops.reshape(i[0], _i64([1, -1]), False).output(0)
    shp = ops.shape_of(i[0])
    head = ops.reduce_prod(ops.slice(shp, _i64([0]), _i64([axis]), _i64([1])), _i64([0]), True)
    return ops.reshape(i[0], ops.concat([head.output(0), _i64([-1])], 0), False).output(0)


@_op("Reshape")
def _reshape(n, i):
    return ops.reshape(i[0], i[1], not n.attrs.get("allowzero", 0)).output(0)


@_op("Transpose")
def _transpose(n, i):
    r = len(i[0].get_partial_shape())
    return ops.transpose(i[0], _i64(n.attrs.get("perm", list(range(r - 1, -1, -1))))).output(0)


@_op("Concat")
def _concat(n, i):
    return ops.concat(i, int(n.attrs["axis"])).output(0)


@_op("Unsqueeze")
def _unsqueeze(n, i):
    axes = i[1] if len(i) > 1 else _i64(n.attrs["axes"])
    return ops.unsqueeze(i[0], axes).output(0)


@_op("Squeeze")
def _squeeze(n, i):
    if len(i) > 1 and i[1] is not None:
        return ops.squeeze(i[0], i[1]).output(0)
    if "axes" in n.attrs:
        return ops.squeeze(i[0], _i64(n.attrs["axes"])).output(0)
    return ops.squeeze(i[0]).output(0)


@_op("Shape")
def _shape(n, i):
    s = ops.shape_of(i[0]).output(0)
    if "start" in n.attrs or "end" in n.attrs:
        s = ops.slice(s, _i64([n.attrs.get("start", 0)]), _i64([n.attrs.get("end", 2 ** 31)]), _i64([1])).output(0)
    return s


@_op("Gather")
def _gather(n, i):
    return ops.gather(i[0], i[1], _i64(n.attrs.get("axis", 0))).output(0)


@_op("GatherElements")
def _gather_elements(n, i):
    return ops.gather_elements(i[0], i[1], int(n.attrs.get("axis", 0))).output(0)


@_op("Slice")
def _slice(n, i):
    if len(i) == 1:   # opset < 10: attributes
        starts, ends = n.attrs["starts"], n.attrs["ends"]
        axes = n.attrs.get("axes", list(range(len(starts))))
        return ops.slice(i[0], _i64(starts), _i64(ends), _i64([1] * len(starts)), _i64(axes)).output(0)
    steps = i[4] if len(i) > 4 and i[4] is not None else ops.broadcast(_i64(1), ops.shape_of(i[1])).output(0)
    if len(i) > 3 and i[3] is not None:
        return ops.slice(i[0], i[1], i[2], steps, i[3]).output(0)
    return ops.slice(i[0], i[1], i[2], steps).output(0)


@_op("Split")
def _split(n, i):
    axis = n.attrs.get("axis", 0)
    if len(i) > 1 and i[1] is not None:
        lens = i[1]
        count = len(_const_ints(lens))
    elif "split" in n.attrs:
        lens, count = _i64(n.attrs["split"]), len(n.attrs["split"])
    else:
        node = ops.split(i[0], _i64(axis), len(n.outputs))
        return tuple(node.output(k) for k in range(len(n.outputs)))
    node = ops.variadic_split(i[0], _i64(axis), lens)
    return tuple(node.output(k) for k in range(count))


@_op("Cast")
def _cast(n, i):
    return ops.convert(i[0], _OV_TYPES[n.attrs["to"]]).output(0)


def _reduce(f):
    def fn(n, i):
        keep = bool(n.attrs.get("keepdims", 1))
        if len(i) > 1 and i[1] is not None:
            axes = i[1]
        elif "axes" in n.attrs:
            axes = _i64(n.attrs["axes"])
        else:
            axes = _i64(list(range(len(i[0].get_partial_shape()))))
        return f(i[0], axes, keep).output(0)
    return fn


for _name, _f in (("ReduceMean", ops.reduce_mean), ("ReduceSum", ops.reduce_sum), ("ReduceMax", ops.reduce_max), ("ReduceMin", ops.reduce_min),
                  ("ReduceProd", ops.reduce_prod), ("ReduceL2", ops.reduce_l2), ("ReduceL1", ops.reduce_l1)):
    _T[_name] = _reduce(_f)


@_op("Where")
def _where(n, i):
    return ops.select(i[0], i[1], i[2]).output(0)


@_op("Expand")
def _expand(n, i):
    return ops.broadcast(i[0], i[1], "bidirectional").output(0)


@_op("Tile")
def _tile(n, i):
    return ops.tile(i[0], i[1]).output(0)


@_op("Constant")
def _constant(n, i):
    for k in ("value", "value_float", "value_int", "value_floats", "value_ints"):
        if k in n.attrs:
            v = n.attrs[k]
            if k == "value_float":
                v = np.array(v, dtype=np.float32)
            elif k == "value_int":
                v = np.array(v, dtype=np.int64)
            elif k == "value_floats":
                v = np.array(v, dtype=np.float32)
            elif k == "value_ints":
                v = np.array(v, dtype=np.int64)
            return constant(v).output(0)
    raise OnnxError("Constant node without a value")


@_op("ConstantOfShape")
def _constant_of_shape(n, i):
    v = n.attrs.get("value", np.zeros(1, dtype=np.float32))
    return ops.broadcast(constant(np.asarray(v).reshape(())), i[0]).output(0)


@_op("Range")
def _range(n, i):
    return ops.range(i[0], i[1], i[2], i[0].get_element_type()).output(0)


@_op("Pad")
def _pad(n, i):
    mode = {b"constant": "constant", b"reflect": "reflect", b"edge": "edge"}[n.attrs.get("mode", b"constant")]
    pads = _const_ints(i[1]) if len(i) > 1 else n.attrs["pads"]
    r = len(pads) // 2
    value = i[2] if len(i) > 2 and i[2] is not None else constant(np.array(n.attrs.get("value", 0.0), dtype=np.float32), i[0].get_element_type()).output(0)
    return ops.pad(i[0], _i64(pads[:r]), _i64(pads[r:]), value, mode).output(0)


@_op("Resize", "Upsample")
def _resize(n, i):
    x = i[0]
    mode = n.attrs.get("mode", b"nearest").decode()
    ct = n.attrs.get("coordinate_transformation_mode", b"half_pixel").decode()
    nearest = n.attrs.get("nearest_mode", b"round_prefer_floor").decode()
    r = len(x.get_partial_shape())
    scales = i[2] if n.op_type == "Resize" and len(i) > 2 and i[2] is not None else (i[1] if n.op_type == "Upsample" else None)
    sizes = i[3] if len(i) > 3 and i[3] is not None else None
    ov_mode = {"nearest": "nearest", "linear": "linear_onnx", "cubic": "cubic"}[mode]
    axes = _i64(list(range(r)))
    if sizes is not None:
        return ops.interpolate(x, sizes, axes, ov_mode, "sizes", [0] * r, [0] * r, ct, nearest, False, float(n.attrs.get("cubic_coeff_a", -0.75))).output(0)
    return ops.interpolate(x, scales, axes, ov_mode, "scales", [0] * r, [0] * r, ct, nearest, False, float(n.attrs.get("cubic_coeff_a", -0.75))).output(0)


@_op("ArgMax", "ArgMin")
def _argmax(n, i):
    axis, keep = n.attrs.get("axis", 0), bool(n.attrs.get("keepdims", 1))
    node = ops.topk(i[0], constant(np.array(1, dtype=np.int64)), axis, "max" if n.op_type == "ArgMax" else "min", "none", "i64")
    return node.output(1) if keep else ops.squeeze(node.output(1), _i64([axis])).output(0)


@_op("TopK")
def _topk(n, i):
    k = ops.squeeze(i[1]).output(0)
    node = ops.topk(i[0], k, n.attrs.get("axis", -1), "max" if n.attrs.get("largest", 1) else "min", "value" if n.attrs.get("sorted", 1) else "none", "i64")
    return (node.output(0), node.output(1))


@_op("CumSum")
def _cumsum(n, i):
    return ops.cumsum(i[0], i[1], bool(n.attrs.get("exclusive", 0)), bool(n.attrs.get("reverse", 0))).output(0)


@_op("Einsum")
def _einsum(n, i):
    return ops.einsum(i, n.attrs["equation"].decode()).output(0)


@_op("DepthToSpace")
def _d2s(n, i):
    mode = "blocks_first" if n.attrs.get("mode", b"DCR") == b"DCR" else "depth_first"
    return ops.depth_to_space(i[0], mode, int(n.attrs["blocksize"])).output(0)


def supported_ops() -> List[str]:
    return sorted(_T)


# ------------------------------------------------------------------------------------------------ driver
def convert(path_or_bytes) -> Model:
    data = path_or_bytes
    if not isinstance(data, (bytes, bytearray, memoryview)):
        with open(str(path_or_bytes), "rb") as f:
            data = f.read()
    graph = None
    for f, w, v in _fields(memoryview(data)):
        if f == 7:
            graph = v
    if graph is None:
        raise OnnxError("no graph in the model")
    nodes, inits, inputs, outputs, gname = [], {}, [], [], "onnx_model"
    for f, w, v in _fields(graph):
        if f == 1:
            nodes.append(_NodeProto(v))
        elif f == 2:
            gname = bytes(v).decode() or gname
        elif f == 5:
            name, arr = _tensor(v)
            inits[name] = arr
        elif f == 11:
            inputs.append(_value_info(v))
        elif f == 12:
            outputs.append(_value_info(v))
    values: Dict[str, Output] = {}
    params = []
    for name, arr in inits.items():
        values[name] = constant(arr, name=name).output(0)
    for name, elem, dims in inputs:
        if name in inits:
            continue
        if elem not in _OV_TYPES:
            raise OnnxError("input '%s' has unsupported element type %d" % (name, elem))
        p = parameter(PartialShape(dims) if dims is not None else PartialShape.dynamic(), _OV_TYPES[elem], name)
        p.output(0).set_names({name})
        params.append(p)
        values[name] = p.output(0)
    for n in nodes:
        if n.domain not in ("", "ai.onnx", "com.microsoft"):
            raise OnnxError("operator %s of domain '%s' is not supported" % (n.op_type, n.domain))
        fn = _T.get(n.op_type)
        if fn is None:
            raise OnnxError("no translator for ONNX operator %s (node '%s')" % (n.op_type, n.name))
        ins = [values[x] if x else None for x in n.inputs]
        while ins and ins[-1] is None:
            ins.pop()
        out = fn(n, ins)
        outs = tuple(out) if isinstance(out, (tuple, list)) else (out,)
        for k, (oname, o) in enumerate(zip(n.outputs, outs)):
            if not oname or o is None:        # an optional output nobody reads, or one the translator does not produce
                continue
            o = as_output(o)
            values[oname] = o
            o.add_names({oname})
            if n.name and o.get_node().get_type_name() not in ("Parameter", "Constant") and k == 0:
                o.get_node().set_friendly_name(n.name)
    results = []
    for name, _, _ in outputs:
        if name not in values:
            raise OnnxError("graph output '%s' is not produced by any node" % name)
        results.append(result(values[name], name))
    return Model(results, params, gname)


from . import onnx_more   # noqa: E402,F401  (second part of the translator table)
