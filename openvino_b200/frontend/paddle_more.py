"""More PaddlePaddle translators (second part of the table of paddle.py): activations, comparisons and logic,
fill / range / shape helpers, stack / split / gather / expand / tile, arg-max, top-k, cumulative sum, normalisations,
interpolation and transposed convolution. Operator and attribute names as in Paddle's ProgramDesc.

Reference: src/frontends/paddle/src/op/*.cpp and op_table.cpp."""
from __future__ import annotations

import numpy as np

from .. import opset as ops
from .._graph import constant
from .paddle import _OV, _T, _auto_pad, _elementwise, _i64, _op, _pads, _unary

for _n, _f in (("sin", ops.sin), ("cos", ops.cos), ("tan", ops.tan), ("asin", ops.asin), ("acos", ops.acos), ("atan", ops.atan), ("sinh", ops.sinh),
               ("cosh", ops.cosh), ("ceil", ops.ceiling), ("sign", ops.sign), ("erf", ops.erf), ("mish", ops.mish), ("softsign", ops.softsign),
               ("logical_not", ops.logical_not), ("isnan_v2", ops.is_nan), ("isfinite_v2", ops.is_finite), ("swish", ops.swish)):
    _T[_n] = _unary(_f)
for _n, _f in (("equal", ops.equal), ("not_equal", ops.not_equal), ("greater_than", ops.greater), ("greater_equal", ops.greater_equal),
               ("less_than", ops.less), ("less_equal", ops.less_equal), ("logical_and", ops.logical_and), ("logical_or", ops.logical_or),
               ("logical_xor", ops.logical_xor), ("elementwise_mod", ops.floor_mod), ("elementwise_floordiv", None)):
    if _f is not None:
        _T[_n] = _elementwise(_f)


def _x(op, g, name="X"):
    return g.get(op.inp(name)[0])


_T["rsqrt"] = lambda op, g: {"Out": [ops.divide(np.float32(1.0), ops.sqrt(_x(op, g))).output(0)]}
_T["square"] = lambda op, g: {"Out": [ops.multiply(_x(op, g), _x(op, g)).output(0)]}
_T["reciprocal"] = lambda op, g: {"Out": [ops.divide(np.float32(1.0), _x(op, g)).output(0)]}
_T["log1p"] = lambda op, g: {"Out": [ops.log(ops.add(_x(op, g), np.float32(1.0))).output(0)]}
_T["round"] = lambda op, g: {"Out": [ops.round(_x(op, g), "half_away_from_zero").output(0)]}
_T["softplus"] = lambda op, g: {"Out": [ops.softplus(_x(op, g)).output(0)]}
_T["elu"] = lambda op, g: {"Out": [ops.elu(_x(op, g), float(op.attrs.get("alpha", 1.0))).output(0)]}
_T["selu"] = lambda op, g: {"Out": [ops.selu(_x(op, g), np.float32(op.attrs.get("alpha", 1.6732632423543772)), np.float32(op.attrs.get("scale", 1.0507009873554805))).output(0)]}
_T["hard_sigmoid"] = lambda op, g: {"Out": [ops.hard_sigmoid(_x(op, g), np.float32(op.attrs.get("slope", 0.2)), np.float32(op.attrs.get("offset", 0.5))).output(0)]}
_T["prelu"] = lambda op, g: {"Out": [ops.prelu(_x(op, g), g.get(op.inp("Alpha")[0])).output(0)]}
_T["pow"] = lambda op, g: {"Out": [ops.power(_x(op, g), np.float32(op.attrs.get("factor", 1.0))).output(0)]}
_T["clip"] = lambda op, g: {"Out": [ops.clamp(_x(op, g), float(op.attrs.get("min", -3.4e38)), float(op.attrs.get("max", 3.4e38))).output(0)]}
_T["log_softmax"] = lambda op, g: {"Out": [ops.log_softmax(_x(op, g), int(op.attrs.get("axis", -1))).output(0)]}
_T["shape"] = lambda op, g: {"Out": [ops.shape_of(_x(op, g, "Input"), "i32").output(0)]}
_T["assign"] = lambda op, g: {"Out": [_x(op, g)]}
_T["where"] = lambda op, g: {"Out": [ops.select(g.get(op.inp("Condition")[0]), _x(op, g), g.get(op.inp("Y")[0])).output(0)]}
_T["stack"] = lambda op, g: {"Y": [ops.concat([ops.unsqueeze(g.get(n), _i64([int(op.attrs.get("axis", 0))])).output(0) for n in op.inp("X")], int(op.attrs.get("axis", 0))).output(0)]}
_T["tile"] = lambda op, g: {"Out": [ops.tile(_x(op, g), _i64([int(v) for v in op.attrs.get("repeat_times", [])])).output(0)]}
_T["cumsum"] = lambda op, g: {"Out": [ops.cumsum(_x(op, g), _i64(int(op.attrs.get("axis", -1))), bool(op.attrs.get("exclusive", False)), bool(op.attrs.get("reverse", False))).output(0)]}
_T["gather"] = lambda op, g: {"Out": [ops.gather(_x(op, g), g.get(op.inp("Index")[0]), _i64(int(op.attrs.get("axis", 0)))).output(0)]}
_T["gather_nd"] = lambda op, g: {"Out": [ops.gather_nd(_x(op, g), g.get(op.inp("Index")[0]), 0).output(0)]}
_T["index_select"] = lambda op, g: {"Out": [ops.gather(_x(op, g), g.get(op.inp("Index")[0]), _i64(int(op.attrs.get("dim", 0)))).output(0)]}
_T["one_hot_v2"] = lambda op, g: {"Out": [ops.one_hot(_x(op, g), constant(np.array(int(op.attrs["depth"]), np.int64)), np.float32(1), np.float32(0), -1).output(0)]}
_T["p_norm"] = lambda op, g: {"Out": [(ops.reduce_l2 if float(op.attrs.get("porder", 2.0)) == 2.0 else ops.reduce_l1)(
    _x(op, g), _i64([int(op.attrs.get("axis", -1))]), bool(op.attrs.get("keepdim", False))).output(0)]}


@_op("elementwise_floordiv")
def _floordiv(op, g):
    x, y = _x(op, g), g.get(op.inp("Y")[0])
    q = ops.divide(x, y)
    return {"Out": [(ops.floor(q) if x.get_element_type().is_real() else q).output(0)]}


@_op("fill_constant")
def _fill_constant(op, g):
    et = _OV[int(op.attrs.get("dtype", 5))]
    value = constant(np.array(float(op.attrs.get("value", 0.0))), et)
    if op.inp("ShapeTensor"):
        shape = g.get(op.inp("ShapeTensor")[0])
    else:
        shape = _i64([int(v) for v in op.attrs.get("shape", [])])
    return {"Out": [ops.broadcast(value, shape).output(0)]}


@_op("fill_any_like", "fill_zeros_like")
def _fill_like(op, g):
    x = _x(op, g)
    v = float(op.attrs.get("value", 0.0))
    return {"Out": [ops.broadcast(constant(np.array(v), x.get_element_type()), ops.shape_of(x)).output(0)]}


@_op("range")
def _range(op, g):
    s, e, st = (g.get(op.inp(k)[0]) for k in ("Start", "End", "Step"))
    sq = lambda t: ops.squeeze(t).output(0) if len(t.get_partial_shape()) else t   # noqa: E731
    return {"Out": [ops.range(sq(s), sq(e), sq(st), str(s.get_element_type())).output(0)]}


@_op("expand_v2")
def _expand(op, g):
    x = _x(op, g)
    if op.inp("Shape"):
        shape = g.get(op.inp("Shape")[0])
    else:
        shape = _i64([int(v) for v in op.attrs.get("shape", [])])
    # -1 keeps the input extent: take the maximum with the input shape aligned from the right
    r_out = int(shape.get_partial_shape()[0].get_length()) if hasattr(shape, "get_partial_shape") else len(op.attrs.get("shape", []))
    r_in = len(x.get_partial_shape())
    xs = ops.concat([_i64([1] * (r_out - r_in)).output(0), ops.shape_of(x).output(0)], 0) if r_out > r_in else ops.shape_of(x)
    target = ops.maximum(ops.convert(shape, "i64"), xs)
    return {"Out": [ops.broadcast(x, target).output(0)]}


@_op("split")
def _split(op, g):
    x = _x(op, g)
    axis = int(op.attrs.get("axis", 0))
    sections = [int(v) for v in op.attrs.get("sections", [])]
    if sections:
        parts = ops.variadic_split(x, _i64(axis), _i64(sections))
    else:
        parts = ops.split(x, _i64(axis), int(op.attrs.get("num", len(op.out("Out")))))
    return {"Out": [parts.output(k) for k in range(parts.get_output_size())]}


@_op("unstack")
def _unstack(op, g):
    x = _x(op, g)
    axis, num = int(op.attrs.get("axis", 0)), int(op.attrs.get("num", len(op.out("Y"))))
    parts = ops.split(x, _i64(axis), num)
    return {"Y": [ops.squeeze(parts.output(k), _i64([axis])).output(0) for k in range(num)]}


@_op("arg_max", "arg_min")
def _arg(op, g):
    x = _x(op, g)
    axis = int(op.attrs.get("axis", -1))
    keep = bool(op.attrs.get("keepdims", False))
    if op.attrs.get("flatten", False):
        x, axis = ops.reshape(x, _i64([-1]), False).output(0), 0
    et = _OV[int(op.attrs.get("dtype", 3))]
    t = ops.topk(x, constant(np.array(1, np.int64)), axis, "max" if op.type == "arg_max" else "min", "none", et)
    out = t.output(1)
    return {"Out": [out if keep else ops.squeeze(out, _i64([axis])).output(0)]}


@_op("top_k_v2")
def _top_k(op, g):
    x = _x(op, g)
    k = g.get(op.inp("K")[0]) if op.inp("K") else constant(np.array(int(op.attrs.get("k", 1)), np.int64))
    if hasattr(k, "get_partial_shape") and len(k.get_partial_shape()):
        k = ops.squeeze(k)
    t = ops.topk(x, k, int(op.attrs.get("axis", -1)), "max" if op.attrs.get("largest", True) else "min", "value" if op.attrs.get("sorted", True) else "none", "i64")
    return {"Out": [t.output(0)], "Indices": [t.output(1)]}


@_op("strided_slice")
def _strided_slice(op, g):
    x = _x(op, g, "Input")
    axes = [int(v) for v in op.attrs.get("axes", [])]
    r = len(x.get_partial_shape())
    big = np.iinfo(np.int64).max
    b, e, s = [0] * r, [big] * r, [1] * r
    for a, st, en, sd in zip(axes, op.attrs.get("starts", []), op.attrs.get("ends", []), op.attrs.get("strides", [])):
        b[a], e[a], s[a] = int(st), int(en), int(sd)
    return {"Out": [ops.slice(x, _i64(b), _i64(e), _i64(s)).output(0)]}


@_op("instance_norm")
def _instance_norm(op, g):
    x = _x(op, g)
    r = len(x.get_partial_shape())
    y = ops.mvn(x, _i64(list(range(2, r))), True, float(op.attrs.get("epsilon", 1e-5)), "inside_sqrt").output(0)
    shape = _i64([1, -1] + [1] * (r - 2))
    if op.inp("Scale"):
        y = ops.multiply(y, ops.reshape(g.get(op.inp("Scale")[0]), shape, False)).output(0)
    if op.inp("Bias"):
        y = ops.add(y, ops.reshape(g.get(op.inp("Bias")[0]), shape, False)).output(0)
    return {"Y": [y]}


@_op("group_norm")
def _group_norm(op, g):
    from .._graph import make_op
    x = _x(op, g)
    c = int(x.get_partial_shape()[1].get_length())
    scale = g.get(op.inp("Scale")[0]) if op.inp("Scale") else constant(np.ones(c, np.float32), x.get_element_type()).output(0)
    bias = g.get(op.inp("Bias")[0]) if op.inp("Bias") else constant(np.zeros(c, np.float32), x.get_element_type()).output(0)
    return {"Y": [make_op("GroupNormalization", [x, scale, bias], {"num_groups": int(op.attrs["groups"]), "epsilon": float(op.attrs.get("epsilon", 1e-5))}).output(0)]}


@_op("nearest_interp_v2", "bilinear_interp_v2", "bicubic_interp_v2")
def _interp(op, g):
    x = _x(op, g)
    mode = {"nearest_interp_v2": "nearest", "bilinear_interp_v2": "linear", "bicubic_interp_v2": "cubic"}[op.type]
    align = bool(op.attrs.get("align_corners", False))
    if mode == "nearest":
        coord = "align_corners" if align else "asymmetric"
    else:
        coord = "align_corners" if align else ("half_pixel" if int(op.attrs.get("align_mode", 1)) == 0 else "asymmetric")
    if op.inp("OutSize"):
        sizes = ops.convert(g.get(op.inp("OutSize")[0]), "i64")
        return {"Out": [ops.interpolate(x, sizes, mode=mode, shape_calculation_mode="sizes", coordinate_transformation_mode=coord, nearest_mode="floor" if not align else "round_prefer_ceil", axes=_i64([2, 3])).output(0)]}
    oh, ow = int(op.attrs.get("out_h", -1)), int(op.attrs.get("out_w", -1))
    if oh > 0 and ow > 0:
        return {"Out": [ops.interpolate(x, _i64([oh, ow]), mode=mode, shape_calculation_mode="sizes", coordinate_transformation_mode=coord, nearest_mode="floor" if not align else "round_prefer_ceil", axes=_i64([2, 3])).output(0)]}
    scale = [float(v) for v in op.attrs.get("scale", [])] or [1.0, 1.0]
    return {"Out": [ops.interpolate(x, constant(np.array(scale, np.float32)), mode=mode, shape_calculation_mode="scales", coordinate_transformation_mode=coord, nearest_mode="floor" if not align else "round_prefer_ceil", axes=_i64([2, 3])).output(0)]}


@_op("conv2d_transpose")
def _conv2d_transpose(op, g):
    x, w = g.get(op.inp("Input")[0]), g.get(op.inp("Filter")[0])
    groups = int(op.attrs.get("groups", 1))
    strides = [int(v) for v in op.attrs.get("strides", [1, 1])]
    dil = [int(v) for v in op.attrs.get("dilations", [1, 1])]
    pb, pe = _pads(op.attrs.get("paddings", [0, 0]))
    out_pad = [int(v) for v in op.attrs.get("output_padding", [])] or [0, 0]
    auto = _auto_pad(op)
    if groups == 1:
        y = ops.convolution_backprop_data(x, w, strides=strides, pads_begin=pb, pads_end=pe, dilations=dil, auto_pad=auto, output_padding=out_pad)
    else:
        ws = w.get_shape()
        wg = ops.reshape(w, _i64([groups, ws[0] // groups] + list(ws[1:])), False)
        y = ops.group_convolution_backprop_data(x, wg, strides=strides, pads_begin=pb, pads_end=pe, dilations=dil, auto_pad=auto, output_padding=out_pad)
    return {"Output": [y.output(0)]}
