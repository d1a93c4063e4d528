"""Translators shared by the frontends whose source graphs are NHWC (TensorFlow GraphDef and TensorFlow Lite): layout
wrappers and the spatial operations in terms of the NCHW operations of the opset. Each frontend decodes its own
attributes and calls these with plain Python values.

Role in the reference: src/frontends/common_translators and the shared operation library
src/frontends/tensorflow_common/src/op (conv_2d.cpp, depthwise_conv_2d.cpp, max_pool.cpp, avg_pool.cpp,
fused_batch_norm.cpp, utils.cpp)."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from .. import opset as ops
from .._graph import Output, constant


def i64(v):
    return constant(np.asarray(v, dtype=np.int64))


def to_nchw(x: Output) -> Output:
    return ops.transpose(x, i64([0, 3, 1, 2])).output(0)


def to_nhwc(x: Output) -> Output:
    return ops.transpose(x, i64([0, 2, 3, 1])).output(0)


def conv2d(x: Output, w_oihw: Output, strides: Sequence[int], dilations: Sequence[int], auto_pad: str, pads_begin=(0, 0), pads_end=(0, 0),
           bias: Optional[Output] = None, nhwc: bool = True) -> Output:
    """2-D convolution of an NHWC (or NCHW) tensor with OIHW filters; the result has the layout of the input."""
    y = ops.convolution(to_nchw(x) if nhwc else x, w_oihw, list(strides), list(pads_begin), list(pads_end), list(dilations), auto_pad).output(0)
    if bias is not None:
        y = ops.add(y, ops.reshape(bias, i64([1, -1, 1, 1]), False)).output(0)
    return to_nhwc(y) if nhwc else y


def depthwise_conv2d(x: Output, w_gm1hw: Output, strides: Sequence[int], dilations: Sequence[int], auto_pad: str, bias: Optional[Output] = None,
                     nhwc: bool = True) -> Output:
    """Depth-wise convolution with filters already in the group form [C, multiplier, 1, kh, kw]."""
    y = ops.group_convolution(to_nchw(x) if nhwc else x, w_gm1hw, list(strides), [0, 0], [0, 0], list(dilations), auto_pad).output(0)
    if bias is not None:
        y = ops.add(y, ops.reshape(bias, i64([1, -1, 1, 1]), False)).output(0)
    return to_nhwc(y) if nhwc else y


def pool2d(x: Output, kernel: Sequence[int], strides: Sequence[int], auto_pad: str, is_max: bool, nhwc: bool = True) -> Output:
    """Max / average pooling (the average leaves padded cells out of the divisor, as TensorFlow does)."""
    xin = to_nchw(x) if nhwc else x
    if is_max:
        y = ops.max_pool(xin, list(strides), [1, 1], [0, 0], [0, 0], list(kernel), "floor", auto_pad).output(0)
    else:
        y = ops.avg_pool(xin, list(strides), [0, 0], [0, 0], list(kernel), True, "floor", auto_pad).output(0)
    return to_nhwc(y) if nhwc else y


def batch_norm(x: Output, gamma, beta, mean, var, eps: float, nhwc: bool = True) -> Output:
    y = ops.batch_norm_inference(to_nchw(x) if nhwc else x, gamma, beta, mean, var, float(eps)).output(0)
    return to_nhwc(y) if nhwc else y


def fused_activation(y: Output, kind: str) -> Output:
    """``kind``: "" / "none", "relu", "relu_n1_to_1", "relu6", "tanh" (the activations that TensorFlow Lite fuses into an operator)."""
    kind = (kind or "none").lower()
    if kind == "none":
        return y
    if kind == "relu":
        return ops.relu(y).output(0)
    if kind == "relu_n1_to_1":
        return ops.clamp(y, -1.0, 1.0).output(0)
    if kind == "relu6":
        return ops.clamp(y, 0.0, 6.0).output(0)
    if kind == "tanh":
        return ops.tanh(y).output(0)
    raise ValueError("fused activation %r is not supported" % kind)
