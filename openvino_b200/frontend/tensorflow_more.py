"""More TensorFlow translators (second part of the table of tensorflow.py): element-wise arithmetic and logic,
comparisons, selections, shape and indexing operations, reductions, activations, einsum, top-k, one-hot, ranges and
fills, space / depth rearrangements, resize, cumulative sums, splits and the 3-D / transposed convolutions.

Reference: src/frontends/tensorflow_common/src/op/*.cpp (one file per operation there)."""
from __future__ import annotations

import numpy as np

from .. import opset as ops
from .._graph import Output, constant
from .tensorflow import _OV, _T, _auto_pad, _i64, _ints_of, _is_nhwc, _nchw, _nhwc, _op, _spatial


def _like(v, x: Output) -> Output:
    return constant(np.array(v, dtype=np.float32), x.get_element_type()).output(0)


for _name, _fn in (("Sin", ops.sin), ("Cos", ops.cos), ("Tan", ops.tan), ("Asin", ops.asin), ("Acos", ops.acos), ("Atan", ops.atan), ("Sinh", ops.sinh),
                   ("Cosh", ops.cosh), ("Asinh", ops.asinh), ("Acosh", ops.acosh), ("Atanh", ops.atanh), ("Ceil", ops.ceiling), ("Sign", ops.sign),
                   ("LogicalNot", ops.logical_not), ("IsNan", ops.is_nan), ("IsFinite", ops.is_finite), ("Softsign", ops.softsign), ("Mish", ops.mish),
                   ("Selu", None), ("Elu", None), ("Swish", ops.swish), ("Gelu", None), ("Relu", ops.relu)):
    if _fn is not None and _name not in _T:
        _T[_name] = (lambda f: lambda n, i: f(i[0]).output(0))(_fn)
for _name, _fn in (("NotEqual", ops.not_equal), ("GreaterEqual", ops.greater_equal), ("LessEqual", ops.less_equal), ("LogicalAnd", ops.logical_and),
                   ("LogicalOr", ops.logical_or), ("FloorMod", ops.floor_mod), ("Mod", ops.mod), ("SquaredDifference", ops.squared_difference),
                   ("BitwiseAnd", ops.bitwise_and), ("BitwiseOr", ops.bitwise_or), ("BitwiseXor", ops.bitwise_xor), ("Div", ops.divide),
                   ("TruncateDiv", None), ("FloorDiv", None), ("Xdivy", None)):
    if _fn is not None:
        _T[_name] = (lambda f: lambda n, i: f(i[0], i[1]).output(0))(_fn)


@_op("Selu")
def _selu(n, i):
    return ops.selu(i[0], _like(1.6732632423543772, i[0]), _like(1.0507009873554805, i[0])).output(0)


@_op("Elu")
def _elu(n, i):
    return ops.elu(i[0], 1.0).output(0)


@_op("Gelu")
def _gelu(n, i):
    return ops.gelu(i[0], "tanh" if n.attrs.get("approximate", False) else "erf").output(0)


@_op("FloorDiv")
def _floor_div(n, i):
    q = ops.divide(i[0], i[1])
    return (ops.floor(q) if i[0].get_element_type().is_real() else q).output(0)


@_op("TruncateDiv")
def _truncate_div(n, i):
    q = ops.divide(i[0], i[1])
    if not i[0].get_element_type().is_real():
        return q.output(0)
    return ops.multiply(ops.sign(q), ops.floor(ops.abs(q))).output(0)


@_op("Reciprocal", "Inv")
def _reciprocal(n, i):
    return ops.divide(_like(1.0, i[0]), i[0]).output(0)


@_op("Log1p")
def _log1p(n, i):
    return ops.log(ops.add(i[0], _like(1.0, i[0]))).output(0)


@_op("Expm1")
def _expm1(n, i):
    return ops.subtract(ops.exp(i[0]), _like(1.0, i[0])).output(0)


@_op("Round", "Rint")
def _round(n, i):
    return ops.round(i[0], "half_to_even").output(0)


@_op("AddN")
def _add_n(n, i):
    acc = i[0]
    for x in i[1:]:
        acc = ops.add(acc, x).output(0)
    return acc


@_op("ClipByValue")
def _clip(n, i):
    return ops.minimum(ops.maximum(i[0], i[1]), i[2]).output(0)


@_op("Select", "SelectV2", "Where3")
def _select(n, i):
    return ops.select(i[0], i[1], i[2]).output(0)


@_op("Where")
def _where(n, i):
    return ops.transpose(ops.non_zero(i[0], "i64"), _i64([1, 0])).output(0)


@_op("LogSoftmax")
def _log_softmax(n, i):
    return ops.log_softmax(i[0], -1).output(0)


@_op("ZerosLike")
def _zeros_like(n, i):
    return ops.multiply(i[0], constant(np.array(0, np.float32), i[0].get_element_type())).output(0)


@_op("OnesLike")
def _ones_like(n, i):
    return ops.add(ops.multiply(i[0], constant(np.array(0, np.float32), i[0].get_element_type())), constant(np.array(1, np.float32), i[0].get_element_type())).output(0)


@_op("Fill")
def _fill(n, i):
    return ops.broadcast(i[1], i[0]).output(0)


@_op("BroadcastTo")
def _broadcast_to(n, i):
    return ops.broadcast(i[0], i[1]).output(0)


@_op("Range")
def _range(n, i):
    return ops.range(i[0], i[1], i[2], str(i[0].get_element_type())).output(0)


@_op("Tile")
def _tile(n, i):
    return ops.tile(i[0], i[1]).output(0)


@_op("Size")
def _size(n, i):
    out = n.attrs.get("out_type")
    return ops.reduce_prod(ops.shape_of(i[0], "i64" if out == ("type", 9) else "i32"), _i64([0]), False).output(0)


@_op("Rank")
def _rank(n, i):
    return ops.squeeze(ops.shape_of(ops.shape_of(i[0], "i32"), "i32")).output(0)


@_op("Slice")
def _slice(n, i):
    begin, size = i[1], i[2]
    shp = ops.shape_of(i[0], str(begin.get_element_type()))
    # size -1 means "to the end"
    end = ops.select(ops.less(size, constant(np.array(0, np.int64), size.get_element_type())), shp, ops.add(begin, size))
    rank = len(i[0].get_partial_shape())
    return ops.slice(i[0], begin, end, constant(np.ones(rank, np.int64), begin.get_element_type())).output(0)


@_op("Split")
def _split(n, i):
    parts = ops.split(i[1], i[0], int(n.attrs["num_split"]))
    return tuple(parts.output(k) for k in range(parts.get_output_size()))


@_op("SplitV")
def _split_v(n, i):
    parts = ops.variadic_split(i[0], i[2], i[1])
    return tuple(parts.output(k) for k in range(parts.get_output_size()))


@_op("Unpack")
def _unpack(n, i):
    axis, num = int(n.attrs.get("axis", 0)), int(n.attrs["num"])
    parts = ops.split(i[0], _i64(axis), num)
    return tuple(ops.squeeze(parts.output(k), _i64([axis])).output(0) for k in range(num))


@_op("GatherNd")
def _gather_nd(n, i):
    return ops.gather_nd(i[0], i[1], 0).output(0)


@_op("Gather")
def _gather_v1(n, i):
    return ops.gather(i[0], i[1], _i64(0)).output(0)


@_op("ScatterNd")
def _scatter_nd(n, i):
    zeros = ops.broadcast(constant(np.array(0, np.float32), i[1].get_element_type()), i[2])
    return ops.scatter_nd_update(zeros, i[0], i[1]).output(0)


@_op("TensorScatterUpdate")
def _tensor_scatter_update(n, i):
    return ops.scatter_nd_update(i[0], i[1], i[2]).output(0)


@_op("OneHot")
def _one_hot(n, i):
    return ops.one_hot(i[0], i[1], i[2], i[3], int(n.attrs.get("axis", -1))).output(0)


@_op("TopKV2", "TopK")
def _topk(n, i):
    k = i[1] if len(i) > 1 else constant(np.array(int(n.attrs["k"]), np.int64))
    t = ops.topk(i[0], k, -1, "max", "value" if n.attrs.get("sorted", True) else "none", "i32")
    return t.output(0), t.output(1)


@_op("ArgMax", "ArgMin")
def _arg(n, i):
    axis = _ints_of(i[1])[0]
    out = n.attrs.get("output_type")
    t = ops.topk(i[0], constant(np.array(1, np.int64)), axis, "max" if n.op == "ArgMax" else "min", "none", "i32" if out == ("type", 3) else "i64")
    return ops.squeeze(t.output(1), _i64([axis])).output(0)


@_op("All", "Any")
def _all_any(n, i):
    f = ops.reduce_logical_and if n.op == "All" else ops.reduce_logical_or
    return f(i[0], i[1], bool(n.attrs.get("keep_dims", False))).output(0)


@_op("EuclideanNorm")
def _euclidean_norm(n, i):
    return ops.reduce_l2(i[0], i[1], bool(n.attrs.get("keep_dims", False))).output(0)


@_op("L2Loss")
def _l2_loss(n, i):
    rank = len(i[0].get_partial_shape())
    return ops.multiply(ops.reduce_sum(ops.multiply(i[0], i[0]), _i64(list(range(rank))), False), _like(0.5, i[0])).output(0)


@_op("Cumsum")
def _cumsum(n, i):
    return ops.cumsum(i[0], i[1], bool(n.attrs.get("exclusive", False)), bool(n.attrs.get("reverse", False))).output(0)


@_op("Einsum")
def _einsum(n, i):
    return ops.einsum(list(i), n.attrs["equation"].decode()).output(0)


@_op("ReverseV2")
def _reverse(n, i):
    return ops.reverse(i[0], i[1], "index").output(0)


@_op("ReverseSequence")
def _reverse_sequence(n, i):
    return ops.reverse_sequence(i[0], i[1], int(n.attrs.get("batch_dim", 0)), int(n.attrs["seq_dim"])).output(0)


@_op("MirrorPad")
def _mirror_pad(n, i):
    p = np.array(_ints_of(i[1])).reshape(-1, 2)
    mode = {b"REFLECT": "reflect", b"SYMMETRIC": "symmetric"}[n.attrs.get("mode", b"REFLECT")]
    return ops.pad(i[0], _i64(p[:, 0].tolist()), _i64(p[:, 1].tolist()), constant(np.array(0, np.float32), i[0].get_element_type()), mode).output(0)


@_op("SpaceToDepth", "DepthToSpace")
def _space_depth(n, i):
    nhwc = _is_nhwc(n)
    x = _nchw(i[0]) if nhwc else i[0]
    bs = int(n.attrs["block_size"])
    y = (ops.space_to_depth(x, "blocks_first", bs) if n.op == "SpaceToDepth" else ops.depth_to_space(x, "blocks_first", bs)).output(0)
    return _nhwc(y) if nhwc else y


@_op("ResizeBilinear", "ResizeNearestNeighbor")
def _resize(n, i):
    x = _nchw(i[0])
    mode = "linear" if n.op == "ResizeBilinear" else "nearest"
    if n.attrs.get("half_pixel_centers", False):
        coord = "half_pixel" if mode == "linear" else "tf_half_pixel_for_nn"
    else:
        coord = "align_corners" if n.attrs.get("align_corners", False) else "asymmetric"
    y = ops.interpolate(x, ops.convert(i[1], "i64"), mode=mode, shape_calculation_mode="sizes", coordinate_transformation_mode=coord,
                        nearest_mode="floor" if not n.attrs.get("half_pixel_centers", False) else "round_prefer_floor", axes=_i64([2, 3])).output(0)
    return _nhwc(y)


@_op("Conv3D")
def _conv3d(n, i):
    ndhwc = n.attrs.get("data_format", b"NDHWC") == b"NDHWC"
    x = ops.transpose(i[0], _i64([0, 4, 1, 2, 3])).output(0) if ndhwc else i[0]
    w = ops.transpose(i[1], _i64([4, 3, 0, 1, 2])).output(0)                          # DHWIO -> OIDHW
    pick = (lambda v: list(v[1:4])) if ndhwc else (lambda v: list(v[2:5]))
    y = ops.convolution(x, w, pick(n.attrs.get("strides", [1] * 5)), [0, 0, 0], [0, 0, 0], pick(n.attrs.get("dilations", [1] * 5)), _auto_pad(n)).output(0)
    return ops.transpose(y, _i64([0, 2, 3, 4, 1])).output(0) if ndhwc else y


@_op("Conv2DBackpropInput")
def _conv2d_backprop_input(n, i):
    nhwc = _is_nhwc(n)
    x = _nchw(i[2]) if nhwc else i[2]
    w = ops.transpose(i[1], _i64([3, 2, 0, 1])).output(0)                             # HWOI (O = output of the transposed conv) -> [I, O, H, W]
    out_shape = _ints_of(i[0])
    spatial = out_shape[1:3] if nhwc else out_shape[2:4]
    y = ops.convolution_backprop_data(x, w, _i64(spatial), strides=_spatial(n.attrs.get("strides", [1, 1, 1, 1]), nhwc), pads_begin=[0, 0], pads_end=[0, 0],
                                      dilations=_spatial(n.attrs.get("dilations", [1, 1, 1, 1]), nhwc), auto_pad=_auto_pad(n)).output(0)
    return _nhwc(y) if nhwc else y


@_op("MaxPool3D", "AvgPool3D")
def _pool3d(n, i):
    ndhwc = n.attrs.get("data_format", b"NDHWC") == b"NDHWC"
    x = ops.transpose(i[0], _i64([0, 4, 1, 2, 3])).output(0) if ndhwc else i[0]
    pick = (lambda v: list(v[1:4])) if ndhwc else (lambda v: list(v[2:5]))
    k, s = pick(n.attrs["ksize"]), pick(n.attrs["strides"])
    if n.op == "MaxPool3D":
        y = ops.max_pool(x, s, [1, 1, 1], [0, 0, 0], [0, 0, 0], k, "floor", _auto_pad(n)).output(0)
    else:
        y = ops.avg_pool(x, s, [0, 0, 0], [0, 0, 0], k, True, "floor", _auto_pad(n)).output(0)
    return ops.transpose(y, _i64([0, 2, 3, 4, 1])).output(0) if ndhwc else y


@_op("LRN")
def _lrn(n, i):
    size = 2 * int(n.attrs.get("depth_radius", 5)) + 1
    y = ops.lrn(_nchw(i[0]), _i64([1]), float(n.attrs.get("alpha", 1.0)) * size, float(n.attrs.get("beta", 0.5)), float(n.attrs.get("bias", 1.0)), size).output(0)
    return _nhwc(y)


@_op("Bucketize")
def _bucketize(n, i):
    b = constant(np.array(n.attrs["boundaries"], np.float32), i[0].get_element_type())
    return ops.bucketize(i[0], b, "i32", False).output(0)


@_op("Bitcast", "CheckNumerics", "EnsureShape", "PreventGradient")
def _pass_through(n, i):
    if n.op == "Bitcast" and "type" in n.attrs and _OV.get(n.attrs["type"][1]) not in (None, str(i[0].get_element_type())):
        raise RuntimeError("Bitcast between element types of different meaning is not converted")
    return i[0]
