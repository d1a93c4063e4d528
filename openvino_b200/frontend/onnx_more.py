"""More ONNX translators (second part of the table of onnx.py): trigonometry and rounding, activations with parameters,
bit and modulo arithmetic, indexing (GatherND / Scatter* / OneHot / NonZero / Compress / Trilu), normalisations, reductions
written through other reductions, transposed convolution, quantisation (Q/DQ, MatMulInteger, DynamicQuantizeLinear),
detection (NonMaxSuppression, RoiAlign), signal (DFT, STFT), random generators, recurrent layers and the
``com.microsoft`` contrib operations that exported transformers use (FusedMatMul, BiasGelu, FastGelu,
SkipLayerNormalization, EmbedLayerNormalization, MatMulNBits, RotaryEmbedding, SimplifiedLayerNormalization).

Reference: src/frontends/onnx/frontend/src/op/*.cpp and op/com.microsoft/*.cpp (one file per operation there).
"""
from __future__ import annotations

from typing import List

import numpy as np

from .. import opset as ops
from .._graph import Output, constant, make_op
from .onnx import OnnxError, _T, _const_ints, _conv_pads, _i64, _op


def _f(v, like: Output) -> Output:
    return constant(np.array(v, dtype=np.float32), like.get_element_type()).output(0)


def _rank(o: Output) -> int:
    return len(o.get_partial_shape())


def _axis(a: int, r: int) -> int:
    return a if a >= 0 else a + r


for _name, _fn in (("Tan", ops.tan), ("Asin", ops.asin), ("Acos", ops.acos), ("Atan", ops.atan), ("Sinh", ops.sinh), ("Cosh", ops.cosh),
                   ("Asinh", ops.asinh), ("Acosh", ops.acosh), ("Atanh", ops.atanh), ("Softsign", ops.softsign), ("IsNaN", ops.is_nan),
                   ("BitwiseNot", ops.bitwise_not)):
    _T[_name] = (lambda f: lambda n, i: f(i[0]).output(0))(_fn)
for _name, _fn in (("BitwiseAnd", ops.bitwise_and), ("BitwiseOr", ops.bitwise_or), ("BitwiseXor", ops.bitwise_xor)):
    _T[_name] = (lambda f: lambda n, i: f(i[0], i[1]).output(0))(_fn)


@_op("Round")
def _round(n, i):
    return ops.round(i[0], "half_to_even").output(0)


@_op("Reciprocal")
def _reciprocal(n, i):
    return ops.divide(_f(1.0, i[0]), i[0]).output(0)


@_op("IsInf")
def _is_inf(n, i):
    return ops.is_inf(i[0], bool(n.attrs.get("detect_negative", 1)), bool(n.attrs.get("detect_positive", 1))).output(0)


@_op("Selu")
def _selu(n, i):
    return ops.selu(i[0], _f(n.attrs.get("alpha", 1.6732632423543772), i[0]), _f(n.attrs.get("gamma", 1.0507009873554805), i[0])).output(0)


@_op("HardSigmoid")
def _hard_sigmoid(n, i):
    return ops.hard_sigmoid(i[0], _f(n.attrs.get("alpha", 0.2), i[0]), _f(n.attrs.get("beta", 0.5), i[0])).output(0)


@_op("ThresholdedRelu")
def _thresholded_relu(n, i):
    a = _f(n.attrs.get("alpha", 1.0), i[0])
    return ops.multiply(i[0], ops.convert(ops.greater(i[0], a), i[0].get_element_type())).output(0)


@_op("Celu")
def _celu(n, i):
    a = float(n.attrs.get("alpha", 1.0))
    neg = ops.multiply(_f(a, i[0]), ops.subtract(ops.exp(ops.divide(i[0], _f(a, i[0]))), _f(1.0, i[0])))
    return ops.add(ops.maximum(i[0], _f(0.0, i[0])), ops.minimum(neg, _f(0.0, i[0]))).output(0)


@_op("Shrink")
def _shrink(n, i):
    lambd, bias = float(n.attrs.get("lambd", 0.5)), float(n.attrs.get("bias", 0.0))
    x = i[0]
    et = x.get_element_type()
    hi = ops.multiply(ops.convert(ops.greater(x, _f(lambd, x)), et), ops.subtract(x, _f(bias, x)))
    lo = ops.multiply(ops.convert(ops.less(x, _f(-lambd, x)), et), ops.add(x, _f(bias, x)))
    return ops.add(hi, lo).output(0)


@_op("Swish")
def _swish(n, i):
    return ops.swish(i[0]).output(0)


@_op("Hardmax")
def _hardmax(n, i):
    r = _rank(i[0])
    axis = _axis(n.attrs.get("axis", -1), r)
    idx = ops.topk(i[0], constant(np.array(1, np.int64)), axis, "max", "value", "i64")
    depth = ops.gather(ops.shape_of(i[0]), _i64([axis]), _i64(0))
    oh = ops.one_hot(ops.squeeze(idx.output(1), _i64([axis])), ops.squeeze(depth), _f(1.0, i[0]), _f(0.0, i[0]), axis)
    return oh.output(0)


@_op("Mod")
def _mod(n, i):
    return (ops.mod(i[0], i[1]) if n.attrs.get("fmod", 0) else ops.floor_mod(i[0], i[1])).output(0)


@_op("BitShift")
def _bit_shift(n, i):
    left = n.attrs.get("direction", b"LEFT") == b"LEFT"
    return (ops.bitwise_left_shift(i[0], i[1]) if left else ops.bitwise_right_shift(i[0], i[1])).output(0)


@_op("Size")
def _size(n, i):
    return ops.reduce_prod(ops.shape_of(i[0]), _i64([0]), False).output(0)


@_op("NonZero")
def _non_zero(n, i):
    return ops.non_zero(i[0], "i64").output(0)


@_op("GatherND")
def _gather_nd(n, i):
    return ops.gather_nd(i[0], i[1], int(n.attrs.get("batch_dims", 0))).output(0)


@_op("ScatterND")
def _scatter_nd(n, i):
    red = n.attrs.get("reduction", b"none").decode()
    return make_op("ScatterNDUpdate", [i[0], i[1], i[2]], {"reduction": {"add": "sum", "mul": "prod"}.get(red, red)}).output(0)


@_op("ScatterElements", "Scatter")
def _scatter_elements(n, i):
    red = n.attrs.get("reduction", b"none").decode()
    return make_op("ScatterElementsUpdate", [i[0], i[1], i[2], _i64(n.attrs.get("axis", 0))],
                   {"reduction": {"add": "sum", "mul": "prod"}.get(red, red), "use_init_val": True}).output(0)


@_op("OneHot")
def _one_hot(n, i):
    values = i[2]
    off = ops.gather(values, _i64(0), _i64(0))
    on = ops.gather(values, _i64(1), _i64(0))
    depth = ops.squeeze(ops.convert(i[1], "i64")) if _rank(i[1]) else ops.convert(i[1], "i64")
    return ops.one_hot(ops.convert(i[0], "i64"), depth, on, off, int(n.attrs.get("axis", -1))).output(0)


@_op("ReverseSequence")
def _reverse_sequence(n, i):
    return ops.reverse_sequence(i[0], i[1], int(n.attrs.get("batch_axis", 1)), int(n.attrs.get("time_axis", 0))).output(0)


@_op("SpaceToDepth")
def _space_to_depth(n, i):
    return ops.space_to_depth(i[0], "blocks_first", int(n.attrs["blocksize"])).output(0)


@_op("Trilu")
def _trilu(n, i):
    x = i[0]
    upper = bool(n.attrs.get("upper", 1))
    shp = ops.shape_of(x)
    rows = ops.squeeze(ops.gather(shp, _i64([-2]), _i64(0)))
    cols = ops.squeeze(ops.gather(shp, _i64([-1]), _i64(0)))
    r = ops.unsqueeze(ops.range(constant(np.array(0, np.int64)), rows, constant(np.array(1, np.int64)), "i64"), _i64([1]))
    c = ops.unsqueeze(ops.range(constant(np.array(0, np.int64)), cols, constant(np.array(1, np.int64)), "i64"), _i64([0]))
    k = ops.convert(i[1], "i64") if len(i) > 1 and i[1] is not None else constant(np.array(0, np.int64))
    keep = ops.greater_equal(ops.subtract(c, r), k) if upper else ops.less_equal(ops.subtract(c, r), k)
    zero = constant(np.array(0, dtype=np.float32), x.get_element_type())
    return ops.select(keep, x, zero).output(0)


@_op("EyeLike")
def _eye_like(n, i):
    shp = ops.shape_of(i[0])
    rows = ops.squeeze(ops.gather(shp, _i64([0]), _i64(0)))
    cols = ops.squeeze(ops.gather(shp, _i64([1]), _i64(0)))
    return ops.eye(rows, cols, constant(np.array(int(n.attrs.get("k", 0)), np.int64)), output_type=i[0].get_element_type()).output(0)


@_op("Compress")
def _compress(n, i):
    idx = ops.squeeze(ops.non_zero(ops.convert(i[1], "i32"), "i64"), _i64([0]))
    if "axis" in n.attrs:
        return ops.gather(i[0], idx, _i64(int(n.attrs["axis"]))).output(0)
    return ops.gather(ops.reshape(i[0], _i64([-1]), False), idx, _i64(0)).output(0)


@_op("LRN")
def _lrn(n, i):
    return ops.lrn(i[0], _i64([1]), float(n.attrs.get("alpha", 1e-4)), float(n.attrs.get("beta", 0.75)), float(n.attrs.get("bias", 1.0)), int(n.attrs["size"])).output(0)


@_op("LpNormalization")
def _lp_norm(n, i):
    axis, p = int(n.attrs.get("axis", -1)), int(n.attrs.get("p", 2))
    if p == 2:
        return ops.normalize_l2(i[0], _i64([axis]), 0.0, "add").output(0)
    return ops.divide(i[0], ops.reduce_l1(i[0], _i64([axis]), True)).output(0)


@_op("MeanVarianceNormalization")
def _mvn(n, i):
    return ops.mvn(i[0], _i64(list(n.attrs.get("axes", [0, 2, 3]))), True, 1e-9, "outside_sqrt").output(0)


@_op("GroupNormalization")
def _group_norm(n, i):
    return make_op("GroupNormalization", [i[0], i[1], i[2]], {"num_groups": int(n.attrs["num_groups"]), "epsilon": float(n.attrs.get("epsilon", 1e-5))}).output(0)


def _reduce_axes(n, i):
    if len(i) > 1 and i[1] is not None:
        return i[1]
    if "axes" in n.attrs:
        return _i64(list(n.attrs["axes"]))
    return _i64(list(range(_rank(i[0]))))


@_op("ReduceLogSum")
def _reduce_log_sum(n, i):
    return ops.log(ops.reduce_sum(i[0], _reduce_axes(n, i), bool(n.attrs.get("keepdims", 1)))).output(0)


@_op("ReduceLogSumExp")
def _reduce_log_sum_exp(n, i):
    return ops.log(ops.reduce_sum(ops.exp(i[0]), _reduce_axes(n, i), bool(n.attrs.get("keepdims", 1)))).output(0)


@_op("ReduceSumSquare")
def _reduce_sum_square(n, i):
    return ops.reduce_sum(ops.multiply(i[0], i[0]), _reduce_axes(n, i), bool(n.attrs.get("keepdims", 1))).output(0)


@_op("ConvTranspose")
def _conv_transpose(n, i):
    x, w = i[0], i[1]
    nd = _rank(w) - 2
    pb, pe, auto = _conv_pads(n, nd)
    strides, dil, group = n.attrs.get("strides", [1] * nd), n.attrs.get("dilations", [1] * nd), n.attrs.get("group", 1)
    out_pad = list(n.attrs.get("output_padding", [0] * nd))
    extra = [_i64(list(n.attrs["output_shape"]))] if "output_shape" in n.attrs else []
    if group == 1:
        y = ops.convolution_backprop_data(x, w, *extra, strides=strides, pads_begin=pb, pads_end=pe, dilations=dil, auto_pad=auto, output_padding=out_pad)
    else:
        ws = w.get_shape()
        wg = ops.reshape(w, _i64([group, ws[0] // group] + list(ws[1:])), False)
        y = ops.group_convolution_backprop_data(x, wg, *extra, strides=strides, pads_begin=pb, pads_end=pe, dilations=dil, auto_pad=auto, output_padding=out_pad)
    y = y.output(0)
    if len(i) > 2 and i[2] is not None:
        y = ops.add(y, ops.reshape(i[2], _i64([1, -1] + [1] * nd), False)).output(0)
    return y


# ------------------------------------------------------------------------------------------------ quantisation
def _per_axis(t: Output, like: Output, axis: int) -> Output:
    """A 1-D scale / zero point laid along ``axis`` of ``like``."""
    if _rank(t) != 1:
        return t
    r = _rank(like)
    shape = [1] * r
    shape[_axis(axis, r)] = -1
    return ops.reshape(t, _i64(shape), False).output(0)


@_op("DequantizeLinear")
def _dequantize(n, i):
    x = ops.convert(i[0], "f32").output(0)
    axis = int(n.attrs.get("axis", 1))
    if len(i) > 2 and i[2] is not None:
        x = ops.subtract(x, _per_axis(ops.convert(i[2], "f32").output(0), i[0], axis)).output(0)
    return ops.multiply(x, _per_axis(ops.convert(i[1], "f32").output(0), i[0], axis)).output(0)


@_op("QuantizeLinear")
def _quantize(n, i):
    axis = int(n.attrs.get("axis", 1))
    zp = i[2] if len(i) > 2 and i[2] is not None else None
    et = zp.get_element_type() if zp is not None else ops.constant(np.zeros((), np.uint8)).output(0).get_element_type()
    lo, hi = (-128.0, 127.0) if str(et) == "i8" else (0.0, 255.0)
    y = ops.divide(ops.convert(i[0], "f32"), _per_axis(ops.convert(i[1], "f32").output(0), i[0], axis))
    y = ops.round(y, "half_to_even")
    if zp is not None:
        y = ops.add(y, _per_axis(ops.convert(zp, "f32").output(0), i[0], axis))
    return ops.convert(ops.clamp(y, lo, hi), et).output(0)


@_op("DynamicQuantizeLinear")
def _dynamic_quantize(n, i):
    x = ops.convert(i[0], "f32")
    axes = _i64(list(range(_rank(i[0]))))
    mx = ops.maximum(ops.reduce_max(x, axes, False), np.float32(0))
    mn = ops.minimum(ops.reduce_min(x, axes, False), np.float32(0))
    scale = ops.divide(ops.subtract(mx, mn), np.float32(255))
    zp = ops.clamp(ops.round(ops.divide(ops.negative(mn), scale), "half_to_even"), 0.0, 255.0)
    y = ops.clamp(ops.add(ops.round(ops.divide(x, scale), "half_to_even"), zp), 0.0, 255.0)
    return [ops.convert(y, "u8").output(0), scale.output(0), ops.convert(zp, "u8").output(0)]


@_op("MatMulInteger")
def _matmul_integer(n, i):
    a, b = ops.convert(i[0], "i32").output(0), ops.convert(i[1], "i32").output(0)
    if len(i) > 2 and i[2] is not None:
        a = ops.subtract(a, ops.convert(i[2], "i32")).output(0)
    if len(i) > 3 and i[3] is not None:
        b = ops.subtract(b, ops.convert(i[3], "i32")).output(0)
    return ops.matmul(a, b, False, False).output(0)


# ------------------------------------------------------------------------------------------------ detection / signal / random
@_op("NonMaxSuppression")
def _nms(n, i):
    args = [x for x in i[:5]]
    while args and args[-1] is None:
        args.pop()
    enc = "center" if n.attrs.get("center_point_box", 0) else "corner"
    return ops.non_max_suppression(*args, box_encoding=enc, sort_result_descending=False, output_type="i64").output(0)


@_op("RoiAlign")
def _roi_align(n, i):
    mode = n.attrs.get("mode", b"avg").decode()
    aligned = n.attrs.get("coordinate_transformation_mode", b"half_pixel").decode()
    return ops.roi_align(i[0], i[1], ops.convert(i[2], "i32"), int(n.attrs.get("output_height", 1)), int(n.attrs.get("output_width", 1)),
                         int(n.attrs.get("sampling_ratio", 0)), float(n.attrs.get("spatial_scale", 1.0)), mode,
                         "half_pixel_for_nn" if aligned == "half_pixel" else "asymmetric").output(0)


@_op("GridSample")
def _grid_sample(n, i):
    mode = n.attrs.get("mode", b"bilinear").decode()
    mode = {"linear": "bilinear", "cubic": "bicubic"}.get(mode, mode)
    return ops.grid_sample(i[0], i[1], bool(n.attrs.get("align_corners", 0)), mode, n.attrs.get("padding_mode", b"zeros").decode()).output(0)


@_op("DFT")
def _dft(n, i):
    x = i[0]
    axis = int(n.attrs.get("axis", 1)) if len(i) < 3 or i[2] is None else _const_ints(i[2])[0]
    inverse, onesided = bool(n.attrs.get("inverse", 0)), bool(n.attrs.get("onesided", 0))
    last = x.get_partial_shape()[-1]
    if last.is_static and last.get_length() == 1:            # real signal: [.., 1] -> complex pairs
        x = ops.concat([x, ops.multiply(x, _f(0.0, x)).output(0)], -1).output(0)
    axes = _i64([_axis(axis, _rank(x) - 1)])
    sig = [ops.reshape(ops.convert(i[1], "i64"), _i64([1]), False).output(0)] if len(i) > 1 and i[1] is not None else []
    y = (ops.idft if inverse else ops.dft)(x, axes, *sig).output(0)
    if onesided and not inverse:
        ln = ops.squeeze(ops.gather(ops.shape_of(y), axes, _i64(0)))
        keep = ops.add(ops.divide(ln, constant(np.array(2, np.int64))), constant(np.array(1, np.int64)))
        idx = ops.range(constant(np.array(0, np.int64)), keep, constant(np.array(1, np.int64)), "i64")
        y = ops.gather(y, idx, _i64(_axis(axis, _rank(x) - 1))).output(0)
    return y


@_op("STFT")
def _stft(n, i):
    sig = i[0]
    if _rank(sig) == 3:                                     # [batch, length, 1]
        sig = ops.squeeze(sig, _i64([2])).output(0)
    step = ops.squeeze(ops.convert(i[1], "i64")) if _rank(i[1]) else ops.convert(i[1], "i64")
    if len(i) > 2 and i[2] is not None:
        window = i[2]
        fs = ops.squeeze(ops.gather(ops.shape_of(window), _i64([0]), _i64(0)))
    else:
        fs_v = _const_ints(i[3])[0]
        window = constant(np.ones(fs_v, np.float32), sig.get_element_type()).output(0)
        fs = constant(np.array(fs_v, np.int64))
    return ops.stft(sig, window, fs, step, False).output(0)


def _onnx_type(code: int) -> str:
    return {1: "f32", 2: "u8", 3: "i8", 5: "i16", 6: "i32", 7: "i64", 9: "boolean", 10: "f16", 11: "f64", 12: "u32", 13: "u64", 16: "bf16"}[int(code)]


@_op("RandomUniform", "RandomUniformLike")
def _random_uniform(n, i):
    shape = ops.shape_of(i[0]).output(0) if n.op_type.endswith("Like") else _i64(list(n.attrs["shape"]))
    et = _onnx_type(n.attrs["dtype"]) if "dtype" in n.attrs else (str(i[0].get_element_type()) if i else "f32")
    lo, hi = np.array(n.attrs.get("low", 0.0), np.float32), np.array(n.attrs.get("high", 1.0), np.float32)
    seed = int(float(n.attrs.get("seed", 0)))
    return ops.random_uniform(shape, constant(lo, et), constant(hi, et), et, seed, seed).output(0)


@_op("Multinomial")
def _multinomial(n, i):
    et = _onnx_type(n.attrs.get("dtype", 6))
    seed = int(float(n.attrs.get("seed", 0)))
    return ops.multinomial(ops.softmax(i[0], -1), constant(np.array([int(n.attrs.get("sample_size", 1))], np.int64)), et, True, False, seed, seed).output(0)


# ------------------------------------------------------------------------------------------------ recurrent layers
def _rnn_common(n, i, gates: int, reorder: List[int]):
    """ONNX weights [dirs, gates*H, I] with its gate order -> the operation set's order; returns X [B, S, I], W, R, B, lens, H0."""
    hs = int(n.attrs["hidden_size"])
    direction = n.attrs.get("direction", b"forward").decode()
    x = ops.transpose(i[0], _i64([1, 0, 2])).output(0) if not n.attrs.get("layout", 0) else i[0]

    def regate(w: Output, width_axis: int = 1) -> Output:
        parts = ops.split(w, _i64(width_axis), gates)
        return ops.concat([parts.output(k) for k in reorder], width_axis).output(0)
    W, R = regate(i[1]), regate(i[2])
    if len(i) > 3 and i[3] is not None:
        wb = ops.split(i[3], _i64(1), 2)
        Bv = regate(ops.add(wb.output(0), wb.output(1)).output(0))
    else:
        dirs = 2 if direction == "bidirectional" else 1
        Bv = constant(np.zeros((dirs, gates * hs), np.float32), x.get_element_type()).output(0)
    shp = ops.shape_of(x)
    batch = ops.gather(shp, _i64([0]), _i64(0))
    if len(i) > 4 and i[4] is not None:
        lens = ops.convert(i[4], "i32").output(0)
    else:
        lens = ops.broadcast(ops.convert(ops.gather(shp, _i64([1]), _i64(0)), "i32"), batch).output(0)
    dirs = 2 if direction == "bidirectional" else 1

    def state(idx: int) -> Output:
        if len(i) > idx and i[idx] is not None:
            return ops.transpose(i[idx], _i64([1, 0, 2])).output(0)            # [dirs, B, H] -> [B, dirs, H]
        return ops.broadcast(constant(np.zeros((), np.float32), x.get_element_type()), ops.concat([batch.output(0), _i64([dirs, hs])], 0)).output(0)
    return x, W, R, Bv, lens, state, hs, direction


def _rnn_outputs(seq, n):
    """[B, dirs, S, H] -> ONNX Y [S, dirs, B, H]; states [B, dirs, H] -> [dirs, B, H]."""
    y = ops.transpose(seq.output(0), _i64([2, 1, 0, 3])).output(0)
    return [y] + [ops.transpose(seq.output(k), _i64([1, 0, 2])).output(0) for k in range(1, seq.get_output_size())]


@_op("LSTM")
def _lstm(n, i):
    x, W, R, Bv, lens, state, hs, direction = _rnn_common(n, i, 4, [2, 0, 3, 1])      # ONNX i o f c -> f i c o
    seq = ops.lstm_sequence(x, state(5), state(6), lens, W, R, Bv, hs, direction)
    return _rnn_outputs(seq, n)


@_op("GRU")
def _gru(n, i):
    x, W, R, Bv, lens, state, hs, direction = _rnn_common(n, i, 3, [0, 1, 2])         # z r h in both
    if n.attrs.get("linear_before_reset", 0):
        raise OnnxError("GRU with linear_before_reset is not converted")
    seq = ops.gru_sequence(x, state(5), lens, W, R, Bv, hs, direction)
    return _rnn_outputs(seq, n)


@_op("RNN")
def _rnn(n, i):
    x, W, R, Bv, lens, state, hs, direction = _rnn_common(n, i, 1, [0])
    acts = [a.decode().lower() for a in n.attrs.get("activations", [b"Tanh"])]
    seq = ops.rnn_sequence(x, state(5), lens, W, R, Bv, hs, direction, acts[:1])
    return _rnn_outputs(seq, n)


# ------------------------------------------------------------------------------------------------ com.microsoft
@_op("FusedMatMul")
def _fused_matmul(n, i):
    y = ops.matmul(i[0], i[1], bool(n.attrs.get("transA", 0)), bool(n.attrs.get("transB", 0))).output(0)
    alpha = float(n.attrs.get("alpha", 1.0))
    return y if alpha == 1.0 else ops.multiply(y, _f(alpha, y)).output(0)


@_op("BiasGelu")
def _bias_gelu(n, i):
    return ops.gelu(ops.add(i[0], i[1]), "erf").output(0)


@_op("FastGelu")
def _fast_gelu(n, i):
    x = ops.add(i[0], i[1]).output(0) if len(i) > 1 and i[1] is not None else i[0]
    return ops.gelu(x, "tanh").output(0)


@_op("QuickGelu")
def _quick_gelu(n, i):
    a = float(n.attrs.get("alpha", 1.702))
    return ops.multiply(i[0], ops.sigmoid(ops.multiply(i[0], _f(a, i[0])))).output(0)


def _layer_norm(x: Output, gamma, beta, eps: float) -> Output:
    y = ops.mvn(x, _i64([-1]), True, eps, "inside_sqrt").output(0)
    if gamma is not None:
        y = ops.multiply(y, gamma).output(0)
    if beta is not None:
        y = ops.add(y, beta).output(0)
    return y


@_op("SkipLayerNormalization")
def _skip_layer_norm(n, i):
    s = ops.add(i[0], i[1]).output(0)
    if len(i) > 4 and i[4] is not None:
        s = ops.add(s, i[4]).output(0)
    y = _layer_norm(s, i[2], i[3] if len(i) > 3 else None, float(n.attrs.get("epsilon", 1e-12)))
    return [y, None, None, s]


@_op("SimplifiedLayerNormalization", "RMSNormalization")
def _rms_norm(n, i):
    x = i[0]
    eps = float(n.attrs.get("epsilon", 1e-5))
    var = ops.reduce_mean(ops.multiply(x, x), _i64([-1]), True)
    y = ops.divide(x, ops.sqrt(ops.add(var, _f(eps, x)))).output(0)
    return ops.multiply(y, i[1]).output(0) if len(i) > 1 and i[1] is not None else y


@_op("SkipSimplifiedLayerNormalization")
def _skip_rms_norm(n, i):
    s = ops.add(i[0], i[1]).output(0)
    if len(i) > 3 and i[3] is not None:
        s = ops.add(s, i[3]).output(0)
    eps = float(n.attrs.get("epsilon", 1e-5))
    var = ops.reduce_mean(ops.multiply(s, s), _i64([-1]), True)
    y = ops.multiply(ops.divide(s, ops.sqrt(ops.add(var, _f(eps, s)))), i[2]).output(0)
    return [y, None, None, s]


@_op("EmbedLayerNormalization")
def _embed_layer_norm(n, i):
    ids, seg = ops.convert(i[0], "i64"), (ops.convert(i[1], "i64") if i[1] is not None else None)
    x = ops.gather(i[2], ids, _i64(0)).output(0)
    shp = ops.shape_of(ids)
    seq = ops.squeeze(ops.gather(shp, _i64([1]), _i64(0)))
    if len(i) > 8 and i[8] is not None:
        pos = ops.convert(i[8], "i64")
    else:
        pos = ops.unsqueeze(ops.range(constant(np.array(0, np.int64)), seq, constant(np.array(1, np.int64)), "i64"), _i64([0]))
    x = ops.add(x, ops.gather(i[3], pos, _i64(0))).output(0)
    if seg is not None and len(i) > 4 and i[4] is not None:
        x = ops.add(x, ops.gather(i[4], seg, _i64(0))).output(0)
    y = _layer_norm(x, i[5], i[6], float(n.attrs.get("epsilon", 1e-12)))
    if len(i) > 7 and i[7] is not None:
        mask_index = ops.reduce_sum(ops.convert(i[7], "i32"), _i64([1]), False).output(0)
    else:
        mask_index = ops.broadcast(constant(np.array(0, np.int32)), ops.gather(shp, _i64([0]), _i64(0))).output(0)
    return [y, mask_index, x]


@_op("MatMulNBits")
def _matmul_nbits(n, i):
    """Weights packed 4 bits per value in blocks along K: B [N, blocks, block_size / 2] u8, scales [N * blocks], optional
    zero points packed the same way. Becomes the decompression pattern the weight-compression passes recognise."""
    K, N, bits, bs = int(n.attrs["K"]), int(n.attrs["N"]), int(n.attrs.get("bits", 4)), int(n.attrs["block_size"])
    if bits != 4:
        raise OnnxError("MatMulNBits with %d bits is not converted" % bits)
    from .._tensor import Tensor
    from .. import _ovcore as _c
    blocks = (K + bs - 1) // bs
    packed = Tensor._from_core(_c.constant_value(i[1]._core())).data.reshape(-1)
    w = constant(Tensor(np.ascontiguousarray(packed), [N, blocks, bs], "u4")).output(0)          # low nibble first, as stored
    scales = ops.reshape(ops.convert(i[2], "f16"), _i64([N, blocks, 1]), False).output(0)
    if len(i) > 3 and i[3] is not None:
        zp_packed = Tensor._from_core(_c.constant_value(i[3]._core())).data.reshape(-1)
        lo, hi = zp_packed & 0xF, zp_packed >> 4
        zp_vals = np.stack([lo, hi], -1).reshape(N, -1)[:, :blocks].astype(np.uint8)
        from ..helpers.packing import pack_data
        zp = constant(Tensor(pack_data(zp_vals, "u4"), [N, blocks, 1], "u4")).output(0)
    else:
        zp = constant(Tensor(np.full((N * blocks + 1) // 2, 0x88, np.uint8), [N, blocks, 1], "u4")).output(0)
    deq = ops.multiply(ops.subtract(ops.convert(w, "f16"), ops.convert(zp, "f16")), scales)
    wf = ops.reshape(deq, _i64([N, blocks * bs]), False).output(0)
    if blocks * bs != K:
        wf = ops.slice(wf, _i64([0]), _i64([K]), _i64([1]), _i64([1])).output(0)
    wf = ops.convert(wf, i[0].get_element_type()).output(0)
    y = ops.matmul(i[0], wf, False, True).output(0)
    if len(i) > 5 and i[5] is not None:
        y = ops.add(y, i[5]).output(0)
    return y


@_op("RotaryEmbedding")
def _rotary_embedding(n, i):
    """x [B, S, H*D] or [B, H, S, D], position ids [B, S] (or [1]), cos / sin caches [max_pos, D/2]."""
    x, pos, cos_c, sin_c = i[0], ops.convert(i[1], "i64").output(0), i[2], i[3]
    interleaved = bool(n.attrs.get("interleaved", 0))
    r = _rank(x)
    heads = int(n.attrs.get("num_heads", 0))
    half = cos_c.get_partial_shape()[1].get_length()
    if r == 3:
        if not heads:
            raise OnnxError("RotaryEmbedding on a 3-D input needs num_heads")
        x4 = ops.reshape(x, _i64([0, 0, heads, 2 * half]), True).output(0)           # [B, S, H, D]
    else:
        x4 = ops.transpose(x, _i64([0, 2, 1, 3])).output(0)
    cos = ops.unsqueeze(ops.gather(cos_c, pos, _i64(0)), _i64([2])).output(0)       # [B, S, 1, D/2]
    sin = ops.unsqueeze(ops.gather(sin_c, pos, _i64(0)), _i64([2])).output(0)
    if interleaved:
        pairs = ops.reshape(x4, _i64([0, 0, 0, half, 2]), True)
        a = ops.squeeze(ops.gather(pairs, _i64([0]), _i64(4)), _i64([4]))
        b = ops.squeeze(ops.gather(pairs, _i64([1]), _i64(4)), _i64([4]))
    else:
        sp = ops.split(x4, _i64(3), 2)
        a, b = sp.output(0), sp.output(1)
    ra = ops.subtract(ops.multiply(a, cos), ops.multiply(b, sin))
    rb = ops.add(ops.multiply(a, sin), ops.multiply(b, cos))
    if interleaved:
        y4 = ops.reshape(ops.concat([ops.unsqueeze(ra, _i64([4])).output(0), ops.unsqueeze(rb, _i64([4])).output(0)], 4), _i64([0, 0, 0, -1]), True).output(0)
    else:
        y4 = ops.concat([ra.output(0), rb.output(0)], 3).output(0)
    if r == 3:
        return ops.reshape(y4, _i64([0, 0, -1]), True).output(0)
    return ops.transpose(y4, _i64([0, 2, 1, 3])).output(0)


@_op("GroupQueryAttention")
def _group_query_attention(n, i):
    """com.microsoft GroupQueryAttention: query / key / value [B, S, heads * width] (or one packed tensor), past key /
    value [B, kv heads, past, width], seqlens_k, total_sequence_length and the optional cos / sin caches, position ids,
    attention bias and head sink -> the GroupQueryAttention operation, which works on [B, heads, S, width].
    Reference: src/frontends/onnx/frontend/src/op/com.microsoft/group_query_attention.cpp."""
    heads, kv_heads = int(n.attrs.get("num_heads", 0)), int(n.attrs.get("kv_num_heads", 0))
    if not heads or not kv_heads:
        raise OnnxError("GroupQueryAttention needs num_heads and kv_num_heads")
    got = lambda k: len(i) > k and i[k] is not None
    q = i[0]
    if got(1) and got(2):
        k, v = i[1], i[2]
    else:                        # packed [B, S, (heads + 2 * kv heads) * width]
        hidden = q.get_partial_shape()[2]
        if not hidden.is_static:
            raise OnnxError("GroupQueryAttention with packed QKV needs a static hidden size")
        width = hidden.get_length() // (heads + 2 * kv_heads)
        parts = ops.variadic_split(q, _i64(2), _i64([heads * width, kv_heads * width, kv_heads * width]))
        q, k, v = parts.output(0), parts.output(1), parts.output(2)

    def split_heads(x, count):
        return ops.transpose(ops.reshape(x, _i64([0, 0, count, -1]), True), _i64([0, 2, 1, 3])).output(0)
    absent = lambda: constant(np.zeros((0,), np.float32)).output(0)
    ins = [split_heads(q, heads), split_heads(k, kv_heads), split_heads(v, kv_heads), i[3], i[4], i[5], i[6]]
    last = max([p for p in range(7, 12) if got(p)], default=6)
    ins += [i[p] if got(p) else absent() for p in range(7, last + 1)]
    node = ops.group_query_attention(ins, num_heads=heads, kv_num_heads=kv_heads, scale=float(n.attrs.get("scale", 0.0)),
                                     do_rotary=bool(n.attrs.get("do_rotary", 0)), rotary_interleaved=bool(n.attrs.get("rotary_interleaved", 0)),
                                     local_window_size=int(n.attrs.get("local_window_size", -1)), smooth_softmax=bool(n.attrs.get("smooth_softmax", 0)))
    return [node.output(0), node.output(1), node.output(2)]


# ------------------------------------------------------------------------------------------------ more com.microsoft
def _activation(name: str, x: Output, n) -> Output:
    name = (name.decode() if isinstance(name, bytes) else str(name))
    params = list(n.attrs.get("activation_params", []))
    if name in ("", "None"):
        return x
    if name == "Relu":
        return ops.relu(x).output(0)
    if name == "Sigmoid":
        return ops.sigmoid(x).output(0)
    if name == "Tanh":
        return ops.tanh(x).output(0)
    if name == "LeakyRelu":
        return ops.prelu(x, _f(params[0] if params else 0.01, x)).output(0)
    if name == "Clip":
        return ops.clamp(x, float(params[0]), float(params[1])).output(0)
    if name == "HardSigmoid":
        a, b = (params + [0.2, 0.5])[:2] if len(params) >= 2 else (0.2, 0.5)
        return ops.clamp(ops.add(ops.multiply(x, _f(a, x)), _f(b, x)), 0.0, 1.0).output(0)
    raise OnnxError("fused activation %s is not supported" % name)


@_op("BiasAdd")
def _bias_add(n, i):
    """x [N, S, C] + bias [C] + skip [N, S, C]."""
    return ops.add(ops.add(i[0], i[1]), i[2]).output(0)


@_op("FusedGemm")
def _fused_gemm(n, i):
    return _activation(n.attrs.get("activation", b"Relu"), _T["Gemm"](n, i), n)


@_op("FusedConv")
def _fused_conv(n, i):
    """Conv(x, w, b) [+ z] followed by the named activation."""
    y = _T["Conv"](n, i[:3])
    y = y[0] if isinstance(y, (list, tuple)) else y
    if len(i) > 3 and i[3] is not None:
        y = ops.add(y, i[3]).output(0)
    return _activation(n.attrs.get("activation", b""), y, n)


@_op("GroupNorm")
def _group_norm_contrib(n, i):
    """Channels-last (or channels-first) group normalisation with an optional Swish: x [N, H, W, C], gamma / beta [C]."""
    x = i[0]
    last = bool(n.attrs.get("channels_last", 1))
    r = _rank(x)
    if last:
        x = ops.transpose(x, _i64([0, r - 1] + list(range(1, r - 1)))).output(0)
    y = make_op("GroupNormalization", [x, i[1], i[2]], {"num_groups": int(n.attrs["groups"]), "epsilon": float(n.attrs.get("epsilon", 1e-5))}).output(0)
    if int(n.attrs.get("activation", 0)) == 1:
        y = ops.swish(y).output(0)
    if last:
        y = ops.transpose(y, _i64([0] + list(range(2, r)) + [1])).output(0)
    return y


def _dq(x: Output, scale: Output, zp) -> Output:
    y = ops.convert(x, "f32").output(0)
    if zp is not None:
        y = ops.subtract(y, ops.convert(zp, "f32")).output(0)
    return ops.multiply(y, ops.convert(scale, "f32")).output(0)


def _q(y: Output, scale: Output, zp, like: Output) -> Output:
    et = zp.get_element_type() if zp is not None else like.get_element_type()
    lo, hi = (-128.0, 127.0) if str(et) == "i8" else (0.0, 255.0)
    v = ops.round(ops.divide(y, ops.convert(scale, "f32")), "half_to_even")
    if zp is not None:
        v = ops.add(v, ops.convert(zp, "f32"))
    return ops.convert(ops.clamp(v, lo, hi), et).output(0)


def _opt(i, k):
    return i[k] if len(i) > k and i[k] is not None else None


@_op("QLinearAdd", "QLinearMul")
def _qlinear_binary(n, i):
    """(A, A_scale, A_zp, B, B_scale, B_zp, C_scale, C_zp): the operation on dequantised values, quantised again."""
    a, b = _dq(i[0], i[1], _opt(i, 2)), _dq(i[3], i[4], _opt(i, 5))
    y = (ops.add if n.op_type == "QLinearAdd" else ops.multiply)(a, b).output(0)
    return _q(y, i[6], _opt(i, 7), i[0])


@_op("QLinearSigmoid", "QLinearLeakyRelu")
def _qlinear_unary(n, i):
    x = _dq(i[0], i[1], _opt(i, 2))
    y = ops.sigmoid(x).output(0) if n.op_type == "QLinearSigmoid" else ops.prelu(x, _f(float(n.attrs.get("alpha", 0.01)), x)).output(0)
    return _q(y, i[3], _opt(i, 4), i[0])


@_op("QLinearConcat")
def _qlinear_concat(n, i):
    """(Y_scale, Y_zp, then x, x_scale, x_zp per input)."""
    parts = [_dq(i[k], i[k + 1], _opt(i, k + 2)) for k in range(2, len(i), 3)]
    return _q(ops.concat(parts, int(n.attrs["axis"])).output(0), i[0], i[1], i[2])


@_op("QLinearWhere")
def _qlinear_where(n, i):
    """(condition, X, x_scale, x_zp, Y, y_scale, y_zp, z_scale, z_zp)."""
    y = ops.select(i[0], _dq(i[1], i[2], _opt(i, 3)), _dq(i[4], i[5], _opt(i, 6))).output(0)
    return _q(y, i[7], _opt(i, 8), i[1])


@_op("MatMulIntegerToFloat")
def _matmul_integer_to_float(n, i):
    """(A, B, a_scale, b_scale, a_zp, b_zp, bias): the product of the dequantised operands, in float."""
    y = ops.matmul(_dq(i[0], i[2], _opt(i, 4)), _dq(i[1], i[3], _opt(i, 5)), False, False).output(0)
    return ops.add(y, i[6]).output(0) if _opt(i, 6) is not None else y


@_op("DynamicQuantizeMatMul")
def _dynamic_quantize_matmul(n, i):
    """(A float, B quantised, b_scale, b_zp, bias): A is quantised to u8 with the range of the whole tensor first."""
    q = _T["DynamicQuantizeLinear"](n, [i[0]])
    a = _dq(q[0], q[1], q[2])
    y = ops.matmul(a, _dq(i[1], i[2], _opt(i, 3)), False, False).output(0)
    return ops.add(y, i[4]).output(0) if _opt(i, 4) is not None else y


def _split_heads(x: Output, heads: int) -> Output:
    return ops.transpose(ops.reshape(x, _i64([0, 0, heads, -1]), True), _i64([0, 2, 1, 3])).output(0)


def _merge_heads(x: Output) -> Output:
    return ops.reshape(ops.transpose(x, _i64([0, 2, 1, 3])), _i64([0, 0, -1]), True).output(0)


def _key_padding_bias(mask: Output, like: Output) -> Output:
    """mask [B, S_kv] of 0 / 1 -> additive [B, 1, 1, S_kv]."""
    keep = ops.convert(ops.unsqueeze(mask, _i64([1, 2])), "f32")
    return ops.multiply(ops.subtract(_f(1.0, like), keep), _f(-10000.0, like)).output(0)


@_op("MultiHeadAttention")
def _multi_head_attention(n, i):
    """query / key / value [B, S, hidden] (+ bias [3 * hidden], key padding mask [B, S_kv], attention bias [B or 1, N or 1, S, S_kv])."""
    heads = int(n.attrs["num_heads"])
    q, k, v = i[0], _opt(i, 1), _opt(i, 2)
    if k is None or v is None or _rank(q) != 3 or _rank(k) != 3:
        raise OnnxError("MultiHeadAttention: packed QKV / KV layouts are not supported")
    bias = _opt(i, 3)
    if bias is not None:
        b3 = ops.split(bias, _i64(0), 3)
        q, k, v = ops.add(q, b3.output(0)).output(0), ops.add(k, b3.output(1)).output(0), ops.add(v, b3.output(2)).output(0)
    qh, kh, vh = _split_heads(q, heads), _split_heads(k, heads), _split_heads(v, heads)
    extra = None
    if _opt(i, 4) is not None:
        if _rank(i[4]) != 2:
            raise OnnxError("MultiHeadAttention: only [batch, kv length] key padding masks are supported")
        extra = _key_padding_bias(i[4], qh)
    if _opt(i, 5) is not None:
        extra = i[5] if extra is None else ops.add(extra, i[5]).output(0)
    args = [qh, kh, vh] + ([extra] if extra is not None else [])
    if "scale" in n.attrs and float(n.attrs["scale"]) != 0.0:
        if extra is None:
            args.append(_f(0.0, qh))
        args.append(_f(float(n.attrs["scale"]), qh))
    y = ops.scaled_dot_product_attention(*args, causal=bool(n.attrs.get("unidirectional", 0)) and extra is None).output(0)
    return [_merge_heads(y), None, None]


@_op("Attention")
def _attention(n, i):
    """input [B, S, hidden_in] x weights [hidden_in, 3 * hidden] + bias [3 * hidden], optional mask [B, S] -> [B, S, hidden]."""
    heads = int(n.attrs["num_heads"])
    if _opt(i, 4) is not None:
        raise OnnxError("Attention: a past state input is not supported")
    qkv = ops.matmul(i[0], i[1], False, False).output(0)
    if _opt(i, 2) is not None:
        qkv = ops.add(qkv, i[2]).output(0)
    sizes = n.attrs.get("qkv_hidden_sizes")
    parts = ops.variadic_split(qkv, _i64(2), _i64(list(sizes))) if sizes else ops.split(qkv, _i64(2), 3)
    qh, kh, vh = (_split_heads(parts.output(k), heads) for k in range(3))
    uni = bool(n.attrs.get("unidirectional", 0))
    args = [qh, kh, vh]
    if _opt(i, 3) is not None:
        if _rank(i[3]) != 2:
            raise OnnxError("Attention: only [batch, length] masks are supported")
        bias = _key_padding_bias(i[3], qh)
        if uni:
            raise OnnxError("Attention: a mask together with unidirectional is not supported")
        args.append(bias)
    if "scale" in n.attrs and float(n.attrs["scale"]) != 0.0:
        if len(args) == 3:
            args.append(_f(0.0, qh))
        args.append(_f(float(n.attrs["scale"]), qh))
    y = ops.scaled_dot_product_attention(*args, causal=uni and len(args) == 3).output(0)
    return [_merge_heads(y), None]
