"""PaddlePaddle frontend: an inference model (``.pdmodel`` program + ``.pdiparams`` parameters) -> ``Model``.

The ``ProgramDesc`` protobuf is decoded here (no ``paddle`` / ``protobuf`` package needed), as is the combined
parameter file (per persistable variable, in name order: LoD header, ``TensorDesc``, raw data). ``feed`` operators
become Parameters, ``fetch`` operators Results, persistable variables Constants; every other operator of block 0 goes
through a table of translators. Paddle graphs are NCHW, like the opset.

Role in the reference: src/frontends/paddle/src (input_model.cpp for the program / parameter files, decoder_proto.cpp,
op_table.cpp, op/*.cpp).
"""
from __future__ import annotations

import os
import struct
from typing import Callable, Dict, List, Optional

import numpy as np

from .. import opset as ops
from .._graph import Model, Output, constant, parameter, result
from .._types import PartialShape
from .onnx import _fields, _packed_ints, _sint


class PaddleError(RuntimeError):
    pass


_NP = {0: np.bool_, 1: np.int16, 2: np.int32, 3: np.int64, 4: np.float16, 5: np.float32, 6: np.float64, 20: np.uint8, 21: np.int8}
_OV = {0: "boolean", 1: "i16", 2: "i32", 3: "i64", 4: "f16", 5: "f32", 6: "f64", 20: "u8", 21: "i8", 22: "bf16"}


# ---------------------------------------------------------------------------------------------- program decoding
def _tensor_desc(b):
    dt, dims = 5, []
    for f, w, v in _fields(b):
        if f == 1:
            dt = v
        elif f == 2:
            dims += _packed_ints(v) if w == 2 else [_sint(v)]
    return dt, dims


class _Var:
    def __init__(self, b):
        self.name, self.persistable, self.dtype, self.dims = "", False, 5, None
        for f, w, v in _fields(b):
            if f == 1:
                self.name = bytes(v).decode()
            elif f == 3:
                self.persistable = bool(v)
            elif f == 2:
                for f2, _, v2 in _fields(v):
                    if f2 == 3:                                     # lod_tensor -> tensor
                        for f3, _, v3 in _fields(v2):
                            if f3 == 1:
                                self.dtype, self.dims = _tensor_desc(v3)


class _Op:
    def __init__(self, b):
        self.type, self.inputs, self.outputs, self.attrs = "", {}, {}, {}
        for f, w, v in _fields(b):
            if f == 3:
                self.type = bytes(v).decode()
            elif f in (1, 2):
                name, args = "", []
                for f2, _, v2 in _fields(v):
                    if f2 == 1:
                        name = bytes(v2).decode()
                    elif f2 == 2:
                        args.append(bytes(v2).decode())
                (self.inputs if f == 1 else self.outputs)[name] = args
            elif f == 4:
                self._attr(v)

    def _attr(self, b):
        name, kind = "", 0
        vals: Dict[int, list] = {}
        for f, w, v in _fields(b):
            if f == 1:
                name = bytes(v).decode()
            elif f == 2:
                kind = v
            else:
                vals.setdefault(f, []).append((w, v))

        def ints(field):
            out = []
            for w, v in vals.get(field, []):
                out += _packed_ints(v) if w == 2 else [_sint(v)]
            return [x - (1 << 32) if x >= (1 << 31) and field in (3, 6) else x for x in out]

        def floats(field, fmt="<f", size=4):
            out = []
            for w, v in vals.get(field, []):
                out += list(np.frombuffer(bytes(v), dtype=fmt)) if w == 2 else [struct.unpack(fmt, bytes(v))[0]]
            return [float(x) for x in out]
        if kind == 0:
            self.attrs[name] = (ints(3) or [0])[0]
        elif kind == 1:
            self.attrs[name] = (floats(4) or [0.0])[0]
        elif kind == 2:
            self.attrs[name] = bytes(vals[5][0][1]).decode() if 5 in vals else ""
        elif kind == 3:
            self.attrs[name] = ints(6)
        elif kind == 4:
            self.attrs[name] = floats(7)
        elif kind == 5:
            self.attrs[name] = [bytes(v).decode() for _, v in vals.get(8, [])]
        elif kind == 6:
            self.attrs[name] = bool((ints(10) or [0])[0])
        elif kind == 7:
            self.attrs[name] = [bool(x) for x in ints(11)]
        elif kind == 9:
            self.attrs[name] = (ints(13) or [0])[0]
        elif kind == 11:
            self.attrs[name] = ints(15)
        elif kind == 12:
            self.attrs[name] = floats(16, "<f8", 8)
        elif kind == 15:
            self.attrs[name] = (floats(19, "<f8", 8) or [0.0])[0]

    def inp(self, name: str) -> List[str]:
        return self.inputs.get(name, [])

    def out(self, name: str) -> List[str]:
        return self.outputs.get(name, [])


def _program(data: bytes):
    vars_, ops_ = {}, []
    block0 = None
    for f, w, v in _fields(memoryview(data)):
        if f == 1 and block0 is None:
            block0 = v
    if block0 is None:
        raise PaddleError("the program has no block")
    for f, w, v in _fields(block0):
        if f == 3:
            var = _Var(v)
            vars_[var.name] = var
        elif f == 4:
            ops_.append(_Op(v))
    return vars_, ops_


def _read_params(path: str, names: List[str], vars_: Dict[str, _Var]) -> Dict[str, np.ndarray]:
    """Combined parameter file: the persistable variables in name order, each as
    u32 version, u64 LoD size (+ LoD data), u32 tensor version, i32 desc size, TensorDesc, raw data."""
    out = {}
    data = open(path, "rb").read()
    pos = 0
    for name in sorted(names):
        if pos + 16 > len(data):
            raise PaddleError("the parameter file ends before variable %s" % name)
        pos += 4
        lod = struct.unpack_from("<Q", data, pos)[0]
        pos += 8
        for _ in range(lod):
            n = struct.unpack_from("<Q", data, pos)[0]
            pos += 8 + n
        pos += 4
        size = struct.unpack_from("<i", data, pos)[0]
        pos += 4
        dt, dims = _tensor_desc(memoryview(data)[pos:pos + size])
        pos += size
        if dt not in _NP:
            raise PaddleError("variable %s has element type %d, which is not supported" % (name, dt))
        count = int(np.prod(dims)) if dims else 1
        arr = np.frombuffer(data, dtype=np.dtype(_NP[dt]).newbyteorder("<"), count=count, offset=pos).reshape(dims)
        pos += arr.nbytes
        out[name] = arr
    return out


# ---------------------------------------------------------------------------------------------- translators
_T: Dict[str, Callable] = {}


def _op(*names):
    def deco(fn):
        for n in names:
            _T[n] = fn
        return fn
    return deco


def _i64(v):
    return constant(np.asarray(v, dtype=np.int64))


def _auto_pad(op: _Op) -> str:
    return {"SAME": "same_upper", "VALID": "valid"}.get(str(op.attrs.get("padding_algorithm", "EXPLICIT")).upper(), "explicit")


def _pads(p, nd=2):
    p = [int(x) for x in p] or [0] * nd
    if len(p) == nd:
        return p, p
    return p[0::2], p[1::2]


@_op("conv2d", "depthwise_conv2d")
def _conv(op, g):
    x, w = g.get(op.inp("Input")[0]), g.get(op.inp("Filter")[0])
    groups = int(op.attrs.get("groups", 1))
    pb, pe = _pads(op.attrs.get("paddings", [0, 0]))
    strides, dil = [int(s) for s in op.attrs.get("strides", [1, 1])], [int(d) for d in op.attrs.get("dilations", [1, 1])]
    if groups > 1:
        ws = [int(d.get_length()) for d in w.get_partial_shape()]
        w = ops.reshape(w, _i64([groups, ws[0] // groups] + ws[1:]), False).output(0)
        y = ops.group_convolution(x, w, strides, pb, pe, dil, _auto_pad(op)).output(0)
    else:
        y = ops.convolution(x, w, strides, pb, pe, dil, _auto_pad(op)).output(0)
    return {"Output": [y]}


@_op("pool2d")
def _pool(op, g):
    x = g.get(op.inp("X")[0])
    k = [int(v) for v in op.attrs.get("ksize", [1, 1])]
    is_max = op.attrs.get("pooling_type", "max") == "max"
    if op.attrs.get("global_pooling", False) or (op.attrs.get("adaptive", False) and k == [1, 1]):
        y = (ops.reduce_max if is_max else ops.reduce_mean)(x, _i64([2, 3]), True).output(0)
        return {"Out": [y]}
    if op.attrs.get("adaptive", False):
        raise PaddleError("adaptive pool2d with an output size other than 1 x 1 is not supported")
    pb, pe = _pads(op.attrs.get("paddings", [0, 0]))
    s = [int(v) for v in op.attrs.get("strides", [1, 1])]
    rounding = "ceil" if op.attrs.get("ceil_mode", False) else "floor"
    if is_max:
        y = ops.max_pool(x, s, [1, 1], pb, pe, k, rounding, _auto_pad(op)).output(0)
    else:
        y = ops.avg_pool(x, s, pb, pe, k, bool(op.attrs.get("exclusive", True)), rounding, _auto_pad(op)).output(0)
    return {"Out": [y]}


@_op("batch_norm")
def _bn(op, g):
    x = g.get(op.inp("X")[0])
    y = ops.batch_norm_inference(x, g.get(op.inp("Scale")[0]), g.get(op.inp("Bias")[0]), g.get(op.inp("Mean")[0]), g.get(op.inp("Variance")[0]),
                                 float(op.attrs.get("epsilon", 1e-5))).output(0)
    return {"Y": [y]}


def _unary(factory):
    return lambda op, g: {"Out": [factory(g.get(op.inp("X")[0])).output(0)]}


for _n, _f in (("relu", ops.relu), ("sigmoid", ops.sigmoid), ("tanh", ops.tanh), ("exp", ops.exp), ("sqrt", ops.sqrt), ("abs", ops.abs),
               ("hard_swish", ops.hswish), ("log", ops.log), ("floor", ops.floor), ("silu", ops.swish)):
    _T[_n] = _unary(_f)
_T["relu6"] = lambda op, g: {"Out": [ops.clamp(g.get(op.inp("X")[0]), 0.0, float(op.attrs.get("threshold", 6.0))).output(0)]}
_T["leaky_relu"] = lambda op, g: {"Out": [ops.prelu(g.get(op.inp("X")[0]), np.float32(op.attrs.get("alpha", 0.02))).output(0)]}
_T["gelu"] = lambda op, g: {"Out": [ops.gelu(g.get(op.inp("X")[0]), "tanh" if op.attrs.get("approximate", False) else "erf").output(0)]}
_T["dropout"] = lambda op, g: {"Out": [g.get(op.inp("X")[0]) if op.attrs.get("dropout_implementation", "downgrade_in_infer") == "upscale_in_train"
                                       else ops.multiply(g.get(op.inp("X")[0]), np.float32(1.0 - float(op.attrs.get("dropout_prob", 0.5)))).output(0)]}


def _elementwise(factory):
    def fn(op, g):
        x, y = g.get(op.inp("X")[0]), g.get(op.inp("Y")[0])
        axis = int(op.attrs.get("axis", -1))
        rx, ry = len(x.get_partial_shape()), len(y.get_partial_shape())
        if axis != -1 and ry < rx and axis + ry < rx:
            # Y's axes line up with X's axes [axis, axis + rank(Y)): append the missing trailing axes
            y = ops.unsqueeze(y, _i64(list(range(ry, ry + rx - axis - ry)))).output(0)
        return {"Out": [factory(x, y).output(0)]}
    return fn


for _n, _f in (("elementwise_add", ops.add), ("elementwise_sub", ops.subtract), ("elementwise_mul", ops.multiply), ("elementwise_div", ops.divide),
               ("elementwise_max", ops.maximum), ("elementwise_min", ops.minimum), ("elementwise_pow", ops.power)):
    _T[_n] = _elementwise(_f)


@_op("matmul_v2")
def _matmul_v2(op, g):
    return {"Out": [ops.matmul(g.get(op.inp("X")[0]), g.get(op.inp("Y")[0]), bool(op.attrs.get("trans_x", False)), bool(op.attrs.get("trans_y", False))).output(0)]}


@_op("matmul")
def _matmul(op, g):
    y = ops.matmul(g.get(op.inp("X")[0]), g.get(op.inp("Y")[0]), bool(op.attrs.get("transpose_X", False)), bool(op.attrs.get("transpose_Y", False))).output(0)
    alpha = float(op.attrs.get("alpha", 1.0))
    return {"Out": [y if alpha == 1.0 else ops.multiply(y, np.float32(alpha)).output(0)]}


@_op("mul")
def _mul(op, g):
    x, y = g.get(op.inp("X")[0]), g.get(op.inp("Y")[0])
    xd = int(op.attrs.get("x_num_col_dims", 1))
    xs = x.get_partial_shape()
    if len(xs) != 2:
        keep = ops.slice(ops.shape_of(x), _i64([0]), _i64([xd]), _i64([1]), _i64([0])).output(0)
        x2 = ops.reshape(x, ops.concat([keep, _i64([-1]).output(0)], 0), False).output(0) if xd > 1 else ops.reshape(x, _i64([0, -1]), True).output(0)
    else:
        x2 = x
    return {"Out": [ops.matmul(x2, y, False, False).output(0)]}


@_op("softmax")
def _softmax(op, g):
    return {"Out": [ops.softmax(g.get(op.inp("X")[0]), int(op.attrs.get("axis", -1))).output(0)]}


@_op("scale")
def _scale(op, g):
    x = g.get(op.inp("X")[0])
    s, b = np.float32(op.attrs.get("scale", 1.0)), np.float32(op.attrs.get("bias", 0.0))
    if op.attrs.get("bias_after_scale", True):
        y = ops.add(ops.multiply(x, s), b)
    else:
        y = ops.multiply(ops.add(x, b), s)
    return {"Out": [y.output(0)]}


@_op("reshape2")
def _reshape(op, g):
    x = g.get(op.inp("X")[0])
    if op.inp("Shape"):
        return {"Out": [ops.reshape(x, g.get(op.inp("Shape")[0]), True).output(0)]}
    return {"Out": [ops.reshape(x, _i64([int(v) for v in op.attrs.get("shape", [])]), True).output(0)]}


@_op("transpose2")
def _transpose(op, g):
    return {"Out": [ops.transpose(g.get(op.inp("X")[0]), _i64([int(v) for v in op.attrs.get("axis", [])])).output(0)]}


@_op("flatten_contiguous_range")
def _flatten(op, g):
    x = g.get(op.inp("X")[0])
    r = len(x.get_partial_shape())
    a, b = int(op.attrs.get("start_axis", 1)) % r, int(op.attrs.get("stop_axis", -1)) % r
    shape = [0] * a + [-1] + [0] * (r - 1 - b)
    # "0" copies the input dimension at the same POSITION: valid for the leading axes only, the trailing ones are read from the shape
    if r - 1 - b:
        dims = ops.shape_of(x)
        tail = ops.slice(dims, _i64([b + 1]), _i64([r]), _i64([1]), _i64([0])).output(0)
        head = ops.slice(dims, _i64([0]), _i64([a]), _i64([1]), _i64([0])).output(0)
        return {"Out": [ops.reshape(x, ops.concat([head, _i64([-1]).output(0), tail], 0), False).output(0)]}
    return {"Out": [ops.reshape(x, _i64(shape), True).output(0)]}


@_op("concat")
def _concat(op, g):
    return {"Out": [ops.concat([g.get(n) for n in op.inp("X")], int(op.attrs.get("axis", 0))).output(0)]}


@_op("squeeze2")
def _squeeze(op, g):
    axes = [int(v) for v in op.attrs.get("axes", [])]
    x = g.get(op.inp("X")[0])
    return {"Out": [(ops.squeeze(x, _i64(axes)) if axes else ops.squeeze(x)).output(0)]}


@_op("unsqueeze2")
def _unsqueeze(op, g):
    return {"Out": [ops.unsqueeze(g.get(op.inp("X")[0]), _i64([int(v) for v in op.attrs.get("axes", [])])).output(0)]}


@_op("reduce_mean", "reduce_sum", "reduce_max", "reduce_min")
def _reduce(op, g):
    x = g.get(op.inp("X")[0])
    f = {"reduce_mean": ops.reduce_mean, "reduce_sum": ops.reduce_sum, "reduce_max": ops.reduce_max, "reduce_min": ops.reduce_min}[op.type]
    axes = [int(v) for v in op.attrs.get("dim", [0])]
    if op.attrs.get("reduce_all", False):
        axes = list(range(len(x.get_partial_shape())))
    return {"Out": [f(x, _i64(axes), bool(op.attrs.get("keep_dim", False))).output(0)]}


@_op("layer_norm")
def _layer_norm(op, g):
    x = g.get(op.inp("X")[0])
    r = len(x.get_partial_shape())
    axes = list(range(int(op.attrs.get("begin_norm_axis", 1)), r))
    y = ops.mvn(x, _i64(axes), True, float(op.attrs.get("epsilon", 1e-5)), "inside_sqrt").output(0)
    tail = [int(d.get_length()) for d in list(x.get_partial_shape())[axes[0]:]]
    if op.inp("Scale"):
        y = ops.multiply(y, ops.reshape(g.get(op.inp("Scale")[0]), _i64(tail), False)).output(0)
    if op.inp("Bias"):
        y = ops.add(y, ops.reshape(g.get(op.inp("Bias")[0]), _i64(tail), False)).output(0)
    return {"Y": [y]}


@_op("lookup_table_v2")
def _lookup(op, g):
    return {"Out": [ops.gather(g.get(op.inp("W")[0]), g.get(op.inp("Ids")[0]), _i64(0)).output(0)]}


@_op("cast")
def _cast(op, g):
    return {"Out": [ops.convert(g.get(op.inp("X")[0]), _OV[int(op.attrs.get("out_dtype", 5))]).output(0)]}


@_op("slice")
def _slice(op, g):
    x = g.get(op.inp("Input")[0])
    axes = [int(v) for v in op.attrs.get("axes", [])]
    y = ops.slice(x, _i64([int(v) for v in op.attrs.get("starts", [])]), _i64([int(v) for v in op.attrs.get("ends", [])]), _i64([1] * len(axes)), _i64(axes)).output(0)
    dec = [int(v) for v in op.attrs.get("decrease_axis", [])]
    if dec:
        y = ops.squeeze(y, _i64(dec)).output(0)
    return {"Out": [y]}


def supported_ops() -> List[str]:
    return sorted(_T)


# ---------------------------------------------------------------------------------------------- graph walk
class _Graph:
    def __init__(self, vars_: Dict[str, _Var], consts: Dict[str, np.ndarray]):
        self.vars, self.consts = vars_, consts
        self.values: Dict[str, Output] = {}

    def get(self, name: str) -> Output:
        if name not in self.values:
            if name not in self.consts:
                raise PaddleError("variable %s is used before it is produced" % name)
            self.values[name] = constant(np.ascontiguousarray(self.consts[name]), name=name).output(0)
        return self.values[name]


def load(model_path: str, params_path: Optional[str] = None) -> Model:
    """``<name>.pdmodel`` (+ ``<name>.pdiparams`` beside it, or ``params_path``) -> ``Model``."""
    model_path = str(model_path)
    vars_, ops_ = _program(open(model_path, "rb").read())
    persist = [n for n, v in vars_.items() if v.persistable and n not in ("feed", "fetch")]
    if params_path is None:
        params_path = os.path.splitext(model_path)[0] + ".pdiparams"
    consts = _read_params(params_path, persist, vars_) if persist else {}
    g = _Graph(vars_, consts)
    params, results = {}, {}
    for op in ops_:
        if op.type == "feed":
            name = op.out("Out")[0]
            v = vars_.get(name)
            dims = [int(d) for d in (v.dims if v is not None and v.dims is not None else [])]
            p = parameter(PartialShape(dims), _OV.get(v.dtype if v is not None else 5, "f32"), name)
            p.output(0).set_names({name})
            params[int(op.attrs.get("col", len(params)))] = p
            g.values[name] = p.output(0)
        elif op.type == "fetch":
            name = op.inp("X")[0]
            o = g.get(name)
            o.set_names(set(o.get_names()) | {name})
            results[int(op.attrs.get("col", len(results)))] = result(o)
        else:
            fn = _T.get(op.type)
            if fn is None:
                raise PaddleError("operator %s is not supported" % op.type)
            outs = fn(op, g)
            for slot, vals in outs.items():
                for name, o in zip(op.out(slot), vals):
                    o.get_node().set_friendly_name(name)
                    g.values[name] = o
    if not results:
        raise PaddleError("the program has no fetch operator")
    return Model([results[k] for k in sorted(results)], [params[k] for k in sorted(params)], os.path.splitext(os.path.basename(model_path))[0])


from . import paddle_more   # noqa: E402,F401  (second part of the translator table)
