"""More TensorFlow Lite translators (second part of the table of tflite.py): builtin operator codes and option-table
fields as in the TensorFlow Lite schema (``BuiltinOperator`` and the ``*Options`` tables of schema.fbs).

Reference: src/frontends/tensorflow_lite/src/op/*.cpp and op_table.cpp."""
from __future__ import annotations

import numpy as np

from .. import opset as ops
from .._graph import Output, constant
from . import common_translators as CT
from .tflite import TFLiteError, _OPS, _OV, _T, _act, _i64, _op

_OPS.update({5: "DEPTH_TO_SPACE", 7: "EMBEDDING_LOOKUP", 8: "FLOOR", 11: "L2_NORMALIZATION", 23: "RESIZE_BILINEAR", 26: "SPACE_TO_DEPTH", 36: "GATHER",
             45: "STRIDED_SLICE", 48: "TOPK_V2", 49: "SPLIT", 50: "LOG_SOFTMAX", 56: "ARG_MAX", 58: "LESS", 60: "PADV2", 61: "GREATER", 62: "GREATER_EQUAL",
             63: "LESS_EQUAL", 64: "SELECT", 65: "SLICE", 66: "SIN", 67: "TRANSPOSE_CONV", 69: "TILE", 70: "EXPAND_DIMS", 71: "EQUAL", 72: "NOT_EQUAL", 73: "LOG",
             74: "SUM", 77: "SHAPE", 78: "POW", 79: "ARG_MIN", 81: "REDUCE_PROD", 82: "REDUCE_MAX", 83: "PACK", 84: "LOGICAL_OR", 85: "ONE_HOT", 86: "LOGICAL_AND",
             87: "LOGICAL_NOT", 88: "UNPACK", 89: "REDUCE_MIN", 90: "FLOOR_DIV", 91: "REDUCE_ANY", 92: "SQUARE", 93: "ZEROS_LIKE", 94: "FILL", 95: "FLOOR_MOD",
             96: "RANGE", 97: "RESIZE_NEAREST_NEIGHBOR", 99: "SQUARED_DIFFERENCE", 100: "MIRROR_PAD", 102: "SPLIT_V", 104: "CEIL", 105: "REVERSE_V2", 106: "ADD_N",
             107: "GATHER_ND", 108: "COS", 109: "WHERE", 110: "RANK", 111: "ELU", 116: "ROUND", 122: "SCATTER_ND", 123: "SELECT_V2", 128: "CUMSUM",
             130: "BROADCAST_TO", 20: "RELU_N1_TO_1", 135: "SIGN"})

for _n, _f in (("FLOOR", ops.floor), ("SIN", ops.sin), ("COS", ops.cos), ("LOG", ops.log), ("CEIL", ops.ceiling), ("LOGICAL_NOT", ops.logical_not), ("SIGN", ops.sign)):
    _T[_n] = (lambda f: (lambda op, ins, g: [f(ins[0]).output(0)]))(_f)
for _n, _f in (("LESS", ops.less), ("GREATER", ops.greater), ("GREATER_EQUAL", ops.greater_equal), ("LESS_EQUAL", ops.less_equal), ("EQUAL", ops.equal),
               ("NOT_EQUAL", ops.not_equal), ("POW", ops.power), ("LOGICAL_OR", ops.logical_or), ("LOGICAL_AND", ops.logical_and), ("FLOOR_MOD", ops.floor_mod),
               ("SQUARED_DIFFERENCE", ops.squared_difference)):
    _T[_n] = (lambda f: (lambda op, ins, g: [f(ins[0], ins[1]).output(0)]))(_f)
_T["SQUARE"] = lambda op, ins, g: [ops.multiply(ins[0], ins[0]).output(0)]
_T["ROUND"] = lambda op, ins, g: [ops.round(ins[0], "half_to_even").output(0)]
_T["ELU"] = lambda op, ins, g: [ops.elu(ins[0], 1.0).output(0)]
_T["RELU_N1_TO_1"] = lambda op, ins, g: [ops.clamp(ins[0], -1.0, 1.0).output(0)]
_T["LOG_SOFTMAX"] = lambda op, ins, g: [ops.log_softmax(ins[0], -1).output(0)]
_T["ZEROS_LIKE"] = lambda op, ins, g: [ops.multiply(ins[0], constant(np.array(0, np.float32), ins[0].get_element_type())).output(0)]
_T["SELECT"] = _T["SELECT_V2"] = lambda op, ins, g: [ops.select(ins[0], ins[1], ins[2]).output(0)]
_T["WHERE"] = lambda op, ins, g: [ops.transpose(ops.non_zero(ins[0], "i64"), _i64([1, 0])).output(0)]
_T["TILE"] = lambda op, ins, g: [ops.tile(ins[0], ins[1]).output(0)]
_T["EXPAND_DIMS"] = lambda op, ins, g: [ops.unsqueeze(ins[0], ins[1]).output(0)]
_T["FILL"] = lambda op, ins, g: [ops.broadcast(ins[1], ins[0]).output(0)]
_T["BROADCAST_TO"] = lambda op, ins, g: [ops.broadcast(ins[0], ins[1]).output(0)]
_T["RANGE"] = lambda op, ins, g: [ops.range(ins[0], ins[1], ins[2], str(ins[0].get_element_type())).output(0)]
_T["GATHER_ND"] = lambda op, ins, g: [ops.gather_nd(ins[0], ins[1], 0).output(0)]
_T["EMBEDDING_LOOKUP"] = lambda op, ins, g: [ops.gather(ins[1], ins[0], _i64(0)).output(0)]
_T["REVERSE_V2"] = lambda op, ins, g: [ops.reverse(ins[0], ins[1], "index").output(0)]
_T["RANK"] = lambda op, ins, g: [ops.squeeze(ops.shape_of(ops.shape_of(ins[0], "i32"), "i32")).output(0)]


@_op("FLOOR_DIV")
def _floor_div(op, ins, g):
    q = ops.divide(ins[0], ins[1])
    return [(ops.floor(q) if ins[0].get_element_type().is_real() else q).output(0)]


@_op("ADD_N")
def _add_n(op, ins, g):
    acc = ins[0]
    for x in ins[1:]:
        acc = ops.add(acc, x).output(0)
    return [acc]


@_op("L2_NORMALIZATION")
def _l2_norm(op, ins, g):
    return [_act(ops.normalize_l2(ins[0], _i64([-1]), 1e-12, "max").output(0), op.opt(0, "b"))]


@_op("SHAPE")
def _shape(op, ins, g):
    return [ops.shape_of(ins[0], _OV.get(op.opt(0, "b", 2), "i32")).output(0)]


@_op("GATHER")
def _gather(op, ins, g):
    return [ops.gather(ins[0], ins[1], _i64(op.opt(0)), op.opt(1)).output(0)]


def _reducer(factory):
    return lambda op, ins, g: [factory(ins[0], ins[1], bool(op.opt(0, "b"))).output(0)]


for _n, _f in (("SUM", ops.reduce_sum), ("REDUCE_PROD", ops.reduce_prod), ("REDUCE_MAX", ops.reduce_max), ("REDUCE_MIN", ops.reduce_min),
               ("REDUCE_ANY", ops.reduce_logical_or)):
    _T[_n] = _reducer(_f)


@_op("ARG_MAX", "ARG_MIN")
def _arg(op, ins, g):
    axis = g.const_value(op.inputs[1])
    if axis is None:
        raise TFLiteError("%s with a run-time axis is not supported" % op.name)
    axis = int(np.asarray(axis).reshape(-1)[0])
    et = _OV.get(g.tensor_type(op.outputs[0]), "i64")
    t = ops.topk(ins[0], constant(np.array(1, np.int64)), axis, "max" if op.name == "ARG_MAX" else "min", "none", et)
    return [ops.squeeze(t.output(1), _i64([axis])).output(0)]


@_op("TOPK_V2")
def _topk(op, ins, g):
    t = ops.topk(ins[0], ops.squeeze(ops.convert(ins[1], "i64")) if len(ins[1].get_partial_shape()) else ops.convert(ins[1], "i64"), -1, "max", "value", "i32")
    return [t.output(0), t.output(1)]


@_op("PACK")
def _pack(op, ins, g):
    axis = op.opt(1)
    return [ops.concat([ops.unsqueeze(x, _i64([axis])).output(0) for x in ins], axis).output(0)]


@_op("UNPACK")
def _unpack(op, ins, g):
    num, axis = op.opt(0), op.opt(1)
    parts = ops.split(ins[0], _i64(axis), num)
    return [ops.squeeze(parts.output(k), _i64([axis])).output(0) for k in range(num)]


@_op("SPLIT")
def _split(op, ins, g):
    parts = ops.split(ins[1], ins[0], op.opt(0))
    return [parts.output(k) for k in range(parts.get_output_size())]


@_op("SPLIT_V")
def _split_v(op, ins, g):
    parts = ops.variadic_split(ins[0], ins[2], ins[1])
    return [parts.output(k) for k in range(parts.get_output_size())]


@_op("SLICE")
def _slice(op, ins, g):
    begin, size = ins[1], ins[2]
    shp = ops.shape_of(ins[0], str(begin.get_element_type()))
    end = ops.select(ops.less(size, constant(np.array(0, np.int64), size.get_element_type())), shp, ops.add(begin, size))
    rank = len(ins[0].get_partial_shape())
    return [ops.slice(ins[0], begin, end, constant(np.ones(rank, np.int64), begin.get_element_type())).output(0)]


@_op("STRIDED_SLICE")
def _strided_slice(op, ins, g):
    rank = int(np.asarray(g.const_value(op.inputs[1])).size) if g.const_value(op.inputs[1]) is not None else len(ins[0].get_partial_shape())

    def bits(field):
        m = op.opt(field)
        return [(m >> k) & 1 for k in range(rank)]
    return [ops.strided_slice(ins[0], ins[1], ins[2], ins[3], bits(0), bits(1), bits(3), bits(4), bits(2)).output(0)]


@_op("ONE_HOT")
def _one_hot(op, ins, g):
    depth = ops.squeeze(ins[1]) if len(ins[1].get_partial_shape()) else ins[1]
    on = ops.squeeze(ins[2]) if len(ins[2].get_partial_shape()) else ins[2]
    off = ops.squeeze(ins[3]) if len(ins[3].get_partial_shape()) else ins[3]
    return [ops.one_hot(ins[0], depth, on, off, op.opt(0, "i", -1)).output(0)]


@_op("PADV2")
def _pad_v2(op, ins, g):
    pads = g.const_value(op.inputs[1])
    if pads is None:
        raise TFLiteError("PADV2 with run-time paddings is not supported")
    pads = np.asarray(pads).reshape(-1, 2).astype(np.int64)
    value = ops.squeeze(ins[2]) if len(ins[2].get_partial_shape()) else ins[2]
    return [ops.pad(ins[0], _i64(pads[:, 0]), _i64(pads[:, 1]), value, "constant").output(0)]


@_op("MIRROR_PAD")
def _mirror_pad(op, ins, g):
    pads = g.const_value(op.inputs[1])
    if pads is None:
        raise TFLiteError("MIRROR_PAD with run-time paddings is not supported")
    pads = np.asarray(pads).reshape(-1, 2).astype(np.int64)
    return [ops.pad(ins[0], _i64(pads[:, 0]), _i64(pads[:, 1]), "symmetric" if op.opt(0, "b") == 1 else "reflect").output(0)]


@_op("CUMSUM")
def _cumsum(op, ins, g):
    return [ops.cumsum(ins[0], ins[1], bool(op.opt(0, "b")), bool(op.opt(1, "b"))).output(0)]


@_op("SCATTER_ND")
def _scatter_nd(op, ins, g):
    zeros = ops.broadcast(constant(np.array(0, np.float32), ins[1].get_element_type()), ins[2])
    return [ops.scatter_nd_update(zeros, ins[0], ins[1]).output(0)]


def _nchw(x: Output) -> Output:
    return ops.transpose(x, _i64([0, 3, 1, 2])).output(0)


def _nhwc(x: Output) -> Output:
    return ops.transpose(x, _i64([0, 2, 3, 1])).output(0)


@_op("DEPTH_TO_SPACE", "SPACE_TO_DEPTH")
def _space_depth(op, ins, g):
    bs = op.opt(0)
    x = _nchw(ins[0])
    y = (ops.depth_to_space(x, "blocks_first", bs) if op.name == "DEPTH_TO_SPACE" else ops.space_to_depth(x, "blocks_first", bs)).output(0)
    return [_nhwc(y)]


@_op("RESIZE_BILINEAR", "RESIZE_NEAREST_NEIGHBOR")
def _resize(op, ins, g):
    linear = op.name == "RESIZE_BILINEAR"
    align, half = (bool(op.opt(2, "b")), bool(op.opt(3, "b"))) if linear else (bool(op.opt(0, "b")), bool(op.opt(1, "b")))
    if half:
        coord = "half_pixel" if linear else "tf_half_pixel_for_nn"
    else:
        coord = "align_corners" if align else "asymmetric"
    y = ops.interpolate(_nchw(ins[0]), ops.convert(ins[1], "i64"), mode="linear" if linear else "nearest", shape_calculation_mode="sizes",
                        coordinate_transformation_mode=coord, nearest_mode="round_prefer_floor" if half else "floor", axes=_i64([2, 3])).output(0)
    return [_nhwc(y)]


@_op("TRANSPOSE_CONV")
def _transpose_conv(op, ins, g):
    # inputs: output shape [4], weights [O, kh, kw, I], data NHWC, optional bias
    out_shape = g.const_value(op.inputs[0])
    if out_shape is None:
        raise TFLiteError("TRANSPOSE_CONV with a run-time output shape is not supported")
    out_shape = [int(v) for v in np.asarray(out_shape).reshape(-1)]
    w = ops.transpose(ins[1], _i64([3, 0, 1, 2])).output(0)                     # [I, O, kh, kw]
    auto = "same_upper" if op.opt(0, "b") == 0 else "valid"
    y = ops.convolution_backprop_data(_nchw(ins[2]), w, _i64(out_shape[1:3]), strides=[op.opt(2), op.opt(1)], pads_begin=[0, 0], pads_end=[0, 0],
                                      dilations=[1, 1], auto_pad=auto).output(0)
    if len(ins) > 3 and ins[3] is not None:
        y = ops.add(y, ops.reshape(ins[3], _i64([1, -1, 1, 1]), False)).output(0)
    return [_act(_nhwc(y), op.opt(3, "b"))]
