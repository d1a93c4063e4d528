"""TensorFlow Lite frontend: a ``.tflite`` flatbuffer -> ``Model``.

The flatbuffer is read directly (no ``flatbuffers`` / ``tflite`` package needed): tables, vtables, vectors and strings of
the TFLite schema (``Model`` -> ``SubGraph`` -> ``Tensor`` / ``Operator`` -> builtin option tables). Sub-graph inputs
become Parameters, tensors with a data buffer Constants, operators go through a table of translators keyed by builtin
operator code. TFLite graphs are NHWC: spatial operations are wrapped in Transposes to the NCHW operations of the opset,
like the TensorFlow frontend does. Quantised constants (int8 / uint8 / int16 with scale and zero point, per tensor or
per channel) and fp16 constants behind DEQUANTIZE are turned into float Constants; fully quantised activations are not
modelled (a ``TFLiteError`` names the tensor).

Role in the reference: src/frontends/tensorflow_lite/src (graph_iterator_flatbuffer.cpp, decoder_flatbuffer.cpp,
op_table.cpp, op/*.cpp, quantization_info.cpp).
"""
from __future__ import annotations

import struct
from typing import Callable, Dict, List, Optional

import numpy as np

from .. import opset as ops
from .._graph import Model, Output, constant, parameter, result
from .._types import PartialShape
from . import common_translators as CT


class TFLiteError(RuntimeError):
    pass


# ---------------------------------------------------------------------------------------------- flatbuffer reader
class _Table:
    """One flatbuffer table: field i sits at ``pos + vtable[i]`` when its vtable entry is non-zero."""

    def __init__(self, buf: bytes, pos: int):
        self.buf, self.pos = buf, pos
        vt = pos - struct.unpack_from("<i", buf, pos)[0]
        self.vt = vt
        self.vt_size = struct.unpack_from("<H", buf, vt)[0]

    def _off(self, field: int) -> int:
        at = 4 + 2 * field
        if at + 2 > self.vt_size:
            return 0
        return struct.unpack_from("<H", self.buf, self.vt + at)[0]

    def scalar(self, field: int, fmt: str, default=0):
        o = self._off(field)
        return struct.unpack_from("<" + fmt, self.buf, self.pos + o)[0] if o else default

    def _indirect(self, field: int) -> Optional[int]:
        o = self._off(field)
        if not o:
            return None
        p = self.pos + o
        return p + struct.unpack_from("<I", self.buf, p)[0]

    def table(self, field: int) -> Optional["_Table"]:
        p = self._indirect(field)
        return _Table(self.buf, p) if p is not None else None

    def string(self, field: int) -> str:
        p = self._indirect(field)
        if p is None:
            return ""
        n = struct.unpack_from("<I", self.buf, p)[0]
        return self.buf[p + 4:p + 4 + n].decode("utf-8", "replace")

    def vector(self, field: int, dtype) -> np.ndarray:
        p = self._indirect(field)
        if p is None:
            return np.zeros(0, dtype=dtype)
        n = struct.unpack_from("<I", self.buf, p)[0]
        return np.frombuffer(self.buf, dtype=np.dtype(dtype).newbyteorder("<"), count=n, offset=p + 4)

    def tables(self, field: int) -> List["_Table"]:
        p = self._indirect(field)
        if p is None:
            return []
        n = struct.unpack_from("<I", self.buf, p)[0]
        out = []
        for i in range(n):
            e = p + 4 + 4 * i
            out.append(_Table(self.buf, e + struct.unpack_from("<I", self.buf, e)[0]))
        return out


def _root(buf: bytes) -> _Table:
    if len(buf) < 8:
        raise TFLiteError("not a flatbuffer")
    if buf[4:8] != b"TFL3":
        raise TFLiteError("missing the TFL3 file identifier")
    return _Table(buf, struct.unpack_from("<I", buf, 0)[0])


# ---------------------------------------------------------------------------------------------- schema constants
_NP = {0: np.float32, 1: np.float16, 2: np.int32, 3: np.uint8, 4: np.int64, 6: np.bool_, 7: np.int16, 9: np.int8, 10: np.float64, 12: np.uint64,
       15: np.uint32, 16: np.uint16}
_OV = {0: "f32", 1: "f16", 2: "i32", 3: "u8", 4: "i64", 6: "boolean", 7: "i16", 9: "i8", 10: "f64", 12: "u64", 15: "u32", 16: "u16", 18: "bf16"}

_OPS = {0: "ADD", 1: "AVERAGE_POOL_2D", 2: "CONCATENATION", 3: "CONV_2D", 4: "DEPTHWISE_CONV_2D", 6: "DEQUANTIZE", 9: "FULLY_CONNECTED", 14: "LOGISTIC",
        17: "MAX_POOL_2D", 18: "MUL", 19: "RELU", 21: "RELU6", 22: "RESHAPE", 25: "SOFTMAX", 28: "TANH", 34: "PAD", 39: "TRANSPOSE", 40: "MEAN", 41: "SUB",
        42: "DIV", 43: "SQUEEZE", 47: "EXP", 53: "CAST", 54: "PRELU", 55: "MAXIMUM", 57: "MINIMUM", 59: "NEG", 75: "SQRT", 76: "RSQRT", 98: "LEAKY_RELU",
        101: "ABS", 117: "HARD_SWISH", 126: "BATCH_MATMUL", 150: "GELU"}


class _Op:
    def __init__(self, name: str, inputs: List[int], outputs: List[int], options: Optional[_Table]):
        self.name, self.inputs, self.outputs, self.options = name, inputs, outputs, options

    def opt(self, field: int, fmt: str = "i", default=0):
        return self.options.scalar(field, fmt, default) if self.options is not None else default


# ---------------------------------------------------------------------------------------------- translators
_T: Dict[str, Callable] = {}


def _op(*names):
    def deco(fn):
        for n in names:
            _T[n] = fn
        return fn
    return deco


def _i64(v):
    return CT.i64(v)


_ACT = {0: "none", 1: "relu", 2: "relu_n1_to_1", 3: "relu6", 4: "tanh"}


def _act(y: Output, code: int) -> Output:
    """Fused activation of the option tables: NONE, RELU, RELU_N1_TO_1, RELU6, TANH."""
    if code not in _ACT:
        raise TFLiteError("fused activation %d is not supported" % code)
    return CT.fused_activation(y, _ACT[code])


def _pad_mode(code: int) -> str:
    return "same_upper" if code == 0 else "valid"


@_op("CONV_2D")
def _conv(op: _Op, ins, g):
    x, w = ins[0], ins[1]                                    # NHWC, filters [O, kh, kw, I]
    pad, sw, sh, act = op.opt(0, "b"), op.opt(1), op.opt(2), op.opt(3, "b")
    dw, dh = op.opt(4, "i", 1), op.opt(5, "i", 1)
    wt = ops.transpose(w, _i64([0, 3, 1, 2])).output(0)
    y = CT.conv2d(x, wt, [sh, sw], [dh, dw], _pad_mode(pad), bias=ins[2] if len(ins) > 2 else None)
    return [_act(y, act)]


@_op("DEPTHWISE_CONV_2D")
def _dwconv(op: _Op, ins, g):
    x, w = ins[0], ins[1]                                    # filters [1, kh, kw, C * multiplier]
    pad, sw, sh, mult, act = op.opt(0, "b"), op.opt(1), op.opt(2), op.opt(3), op.opt(4, "b")
    dw, dh = op.opt(5, "i", 1), op.opt(6, "i", 1)
    ws = w.get_partial_shape()
    kh, kw, cm = (int(ws[i].get_length()) for i in (1, 2, 3))
    mult = max(mult, 1)
    # [1, kh, kw, C * m] -> [C, m, 1, kh, kw]
    wt = ops.reshape(ops.transpose(w, _i64([3, 0, 1, 2])), _i64([cm // mult, mult, 1, kh, kw]), False).output(0)
    y = CT.depthwise_conv2d(x, wt, [sh, sw], [dh, dw], _pad_mode(pad), bias=ins[2] if len(ins) > 2 else None)
    return [_act(y, act)]


def _pool(op: _Op, ins, is_max: bool):
    pad, sw, sh, fw, fh, act = op.opt(0, "b"), op.opt(1), op.opt(2), op.opt(3), op.opt(4), op.opt(5, "b")
    return [_act(CT.pool2d(ins[0], [fh, fw], [sh, sw], _pad_mode(pad), is_max), act)]


@_op("MAX_POOL_2D")
def _max_pool(op, ins, g):
    return _pool(op, ins, True)


@_op("AVERAGE_POOL_2D")
def _avg_pool(op, ins, g):
    return _pool(op, ins, False)


@_op("FULLY_CONNECTED")
def _fc(op: _Op, ins, g):
    x, w = ins[0], ins[1]                                    # weights [out, in]
    act, keep = op.opt(0, "b"), bool(op.opt(2, "b"))
    ws = w.get_partial_shape()
    if not keep:
        x = ops.reshape(x, _i64([-1, int(ws[1].get_length())]), False).output(0)
    y = ops.matmul(x, w, False, True).output(0)
    if len(ins) > 2 and ins[2] is not None:
        y = ops.add(y, ins[2]).output(0)
    return [_act(y, act)]


def _binary(factory):
    def fn(op: _Op, ins, g):
        return [_act(factory(ins[0], ins[1]).output(0), op.opt(0, "b"))]
    return fn


for _n, _f in (("ADD", ops.add), ("SUB", ops.subtract), ("MUL", ops.multiply), ("DIV", ops.divide)):
    _T[_n] = _binary(_f)
_T["MAXIMUM"] = lambda op, ins, g: [ops.maximum(ins[0], ins[1]).output(0)]
_T["MINIMUM"] = lambda op, ins, g: [ops.minimum(ins[0], ins[1]).output(0)]
for _n, _f in (("LOGISTIC", ops.sigmoid), ("TANH", ops.tanh), ("RELU", ops.relu), ("EXP", ops.exp), ("NEG", ops.negative), ("SQRT", ops.sqrt),
               ("ABS", ops.abs), ("HARD_SWISH", ops.hswish)):
    _T[_n] = (lambda f: (lambda op, ins, g: [f(ins[0]).output(0)]))(_f)
_T["RELU6"] = lambda op, ins, g: [ops.clamp(ins[0], 0.0, 6.0).output(0)]
_T["RSQRT"] = lambda op, ins, g: [ops.divide(np.float32(1.0), ops.sqrt(ins[0])).output(0)]
_T["PRELU"] = lambda op, ins, g: [ops.prelu(ins[0], ins[1]).output(0)]
_T["LEAKY_RELU"] = lambda op, ins, g: [ops.prelu(ins[0], np.float32(op.opt(0, "f", 0.0))).output(0)]
_T["GELU"] = lambda op, ins, g: [ops.gelu(ins[0], "tanh" if op.opt(0, "b") else "erf").output(0)]


@_op("SOFTMAX")
def _softmax(op: _Op, ins, g):
    beta = op.opt(0, "f", 1.0)
    x = ins[0] if beta == 1.0 else ops.multiply(ins[0], np.float32(beta)).output(0)
    return [ops.softmax(x, -1).output(0)]


@_op("CONCATENATION")
def _concat(op: _Op, ins, g):
    return [_act(ops.concat(list(ins), op.opt(0)).output(0), op.opt(1, "b"))]


@_op("RESHAPE")
def _reshape(op: _Op, ins, g):
    if len(ins) > 1 and ins[1] is not None:
        return [ops.reshape(ins[0], ins[1], False).output(0)]
    shape = op.options.vector(0, np.int32) if op.options is not None else np.zeros(0, np.int32)
    return [ops.reshape(ins[0], _i64(shape.astype(np.int64)), False).output(0)]


@_op("SQUEEZE")
def _squeeze(op: _Op, ins, g):
    dims = op.options.vector(0, np.int32) if op.options is not None else np.zeros(0, np.int32)
    return [(ops.squeeze(ins[0], _i64(dims.astype(np.int64))) if len(dims) else ops.squeeze(ins[0])).output(0)]


@_op("TRANSPOSE")
def _transpose(op: _Op, ins, g):
    return [ops.transpose(ins[0], ins[1]).output(0)]


@_op("MEAN")
def _mean(op: _Op, ins, g):
    return [ops.reduce_mean(ins[0], ins[1], bool(op.opt(0, "b"))).output(0)]


@_op("PAD")
def _pad(op: _Op, ins, g):
    pads = g.const_value(op.inputs[1])                       # [rank, 2]
    if pads is None:
        raise TFLiteError("PAD with run-time paddings is not supported")
    pads = np.asarray(pads).reshape(-1, 2).astype(np.int64)
    return [ops.pad(ins[0], _i64(pads[:, 0]), _i64(pads[:, 1]), "constant").output(0)]


@_op("CAST")
def _cast(op: _Op, ins, g):
    return [ops.convert(ins[0], _OV[g.tensor_type(op.outputs[0])]).output(0)]


@_op("DEQUANTIZE")
def _dequantize(op: _Op, ins, g):
    # constants were dequantised when they were read; what is left is a change of float type
    x = ins[0]
    return [x if x.get_element_type().name == "f32" else ops.convert(x, "f32").output(0)]


@_op("BATCH_MATMUL")
def _batch_matmul(op: _Op, ins, g):
    return [ops.matmul(ins[0], ins[1], bool(op.opt(0, "b")), bool(op.opt(1, "b"))).output(0)]


def supported_ops() -> List[str]:
    return sorted(_T)


# ---------------------------------------------------------------------------------------------- graph walk
class _Graph:
    def __init__(self, model: _Table, sub: _Table):
        self.buffers = model.tables(4)
        self.tensors = sub.tables(0)
        self.values: Dict[int, Output] = {}

    def tensor_type(self, i: int) -> int:
        return self.tensors[i].scalar(1, "b", 0)

    def tensor_name(self, i: int) -> str:
        return self.tensors[i].string(3) or "tensor_%d" % i

    def _raw(self, i: int) -> Optional[np.ndarray]:
        t = self.tensors[i]
        b = t.scalar(2, "I", 0)
        if b == 0 or b >= len(self.buffers):
            return None
        data = self.buffers[b].vector(0, np.uint8)
        if data.size == 0:
            return None
        tt = self.tensor_type(i)
        if tt not in _NP:
            raise TFLiteError("tensor %s has element type %d, which is not supported" % (self.tensor_name(i), tt))
        shape = [int(d) for d in t.vector(0, np.int32)]
        return np.frombuffer(data.tobytes(), dtype=np.dtype(_NP[tt]).newbyteorder("<")).reshape(shape)

    def const_value(self, i: int) -> Optional[np.ndarray]:
        """Host value of a constant tensor (dequantised when it carries quantisation parameters)."""
        raw = self._raw(i)
        if raw is None:
            return None
        q = self.tensors[i].table(4)
        if q is not None and raw.dtype.kind in "iu" and raw.dtype.itemsize <= 2:
            scale = q.vector(2, np.float32)
            if scale.size:
                zp = q.vector(3, np.int64)
                axis = q.scalar(6, "i", 0)                 # (the details union before it takes two vtable slots)
                shape = [1] * raw.ndim
                if scale.size > 1:
                    shape[axis] = scale.size
                z = zp.astype(np.float32).reshape(shape) if zp.size == scale.size else np.float32(zp[0] if zp.size else 0)
                return ((raw.astype(np.float32) - z) * scale.reshape(shape)).astype(np.float32)
        return raw

    def get(self, i: int) -> Optional[Output]:
        if i < 0:
            return None
        if i not in self.values:
            v = self.const_value(i)
            if v is None:
                raise TFLiteError("tensor %s is used before it is produced" % self.tensor_name(i))
            c = constant(np.ascontiguousarray(v), name=self.tensor_name(i))
            self.values[i] = c.output(0)
        return self.values[i]


def load(path_or_bytes) -> Model:
    """``.tflite`` file (path or bytes) -> ``Model`` (the first sub-graph)."""
    buf = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray, memoryview)) else open(str(path_or_bytes), "rb").read()
    buf = bytes(buf)
    model = _root(buf)
    codes = []
    for oc in model.tables(1):
        code = oc.scalar(3, "i", 0)
        if code == 0:
            code = oc.scalar(0, "b", 0)                      # models written before the 32-bit operator code
        codes.append((code, oc.string(1)))
    subs = model.tables(2)
    if not subs:
        raise TFLiteError("the model has no sub-graph")
    sub = subs[0]
    g = _Graph(model, sub)
    params = []
    for i in sub.vector(1, np.int32):
        i = int(i)
        t = g.tensors[i]
        sig = t.vector(7, np.int32)
        shape = [int(d) for d in (sig if sig.size else t.vector(0, np.int32))]
        q = t.table(4)
        if q is not None and q.vector(2, np.float32).size and g.tensor_type(i) in (3, 9, 7):
            raise TFLiteError("input %s is quantised: fully quantised models are not supported" % g.tensor_name(i))
        p = parameter(PartialShape(shape), _OV[g.tensor_type(i)], g.tensor_name(i))
        p.output(0).set_names({g.tensor_name(i)})
        params.append(p)
        g.values[i] = p.output(0)
    for o in sub.tables(3):
        code, custom = codes[o.scalar(0, "I", 0)]
        name = _OPS.get(code)
        if name is None or name not in _T:
            raise TFLiteError("operator %s is not supported" % (custom or name or "builtin code %d" % code))
        op = _Op(name, [int(i) for i in o.vector(1, np.int32)], [int(i) for i in o.vector(2, np.int32)], o.table(4))
        outs = _T[name](op, [g.get(i) for i in op.inputs], g)
        for idx, out in zip(op.outputs, outs):
            out.get_node().set_friendly_name(g.tensor_name(idx))
            g.values[idx] = out
    results = []
    for i in sub.vector(2, np.int32):
        o = g.get(int(i))
        o.set_names({g.tensor_name(int(i))})
        results.append(result(o))
    return Model(results, params, sub.string(4) or "tflite_model")


from . import tflite_more   # noqa: E402,F401  (second part of the translator table)
