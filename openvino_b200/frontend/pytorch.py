"""PyTorch frontend: ``torch.nn.Module`` / ``ExportedProgram`` -> ``Model``.

The module is captured with ``torch.export`` (ATen-level FX graph, no decomposition) and every ``call_function``
node is translated by a table of small converter functions into graph operations. Weights become Constants
that share the module's memory. Symbolic sizes (``sym_size``) are translated to ShapeOf/Gather sub-graphs, so a
model exported with dynamic dimensions stays dynamic.

Plays the role of the reference PyTorch frontend (src/frontends/pytorch/src/frontend.cpp, op_table.cpp and
src/frontends/pytorch/src/op/*.cpp for the per-op translators; Python-side decoders
src/bindings/python/src/openvino/frontend/pytorch/{ts_decoder,fx_decoder}.py) behind ``convert_model``
(tools/ovc/openvino/tools/ovc/convert.py).
"""
from __future__ import annotations

import math
import operator
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output, as_output, constant, parameter, result
from .._tensor import Tensor
from .._types import PartialShape, Type


class ConversionError(RuntimeError):
    pass


_TORCH_TO_OV = None


def _ov_type(dt) -> Type:
    global _TORCH_TO_OV
    import torch
    if _TORCH_TO_OV is None:
        _TORCH_TO_OV = {torch.float32: Type.f32, torch.float16: Type.f16, torch.bfloat16: Type.bf16, torch.float64: Type.f64,
                        torch.int64: Type.i64, torch.int32: Type.i32, torch.int16: Type.i16, torch.int8: Type.i8, torch.uint8: Type.u8,
                        torch.bool: Type.boolean}
    if dt not in _TORCH_TO_OV:
        raise ConversionError("unsupported torch dtype %s" % dt)
    return _TORCH_TO_OV[dt]


class Ctx:
    """Conversion state: fx node -> Output(s)."""

    def __init__(self):
        self.values: Dict[Any, Any] = {}

    def get(self, a):
        """fx argument -> Output (tensors), python value (scalars / lists of python values)."""
        import torch.fx as fx
        if isinstance(a, fx.Node):
            return self.values[a]
        return a

    def out(self, a, like: Optional[Output] = None) -> Output:
        """fx argument -> Output; python scalars become Constants typed like ``like``."""
        v = self.get(a)
        if isinstance(v, Output):
            return v
        if isinstance(v, Node):
            return v.output(0)
        if like is not None and isinstance(v, (int, float, bool)):
            et = like.get_element_type()
            if isinstance(v, float) and not et.is_real():
                et = Type.f32
            return constant(np.array(v), et).output(0)
        if isinstance(v, bool):
            return constant(np.array(v)).output(0)
        if isinstance(v, int):
            return constant(np.array(v, dtype=np.int64)).output(0)
        if isinstance(v, float):
            return constant(np.array(v, dtype=np.float32)).output(0)
        raise ConversionError("cannot make a graph value from %r" % (v,))

    def ints(self, a) -> Output:
        """List of ints and/or symbolic sizes -> 1-D i64 Output."""
        v = self.get(a)
        if isinstance(v, (list, tuple)):
            vals = [self.get(x) for x in v]
            if all(isinstance(x, int) for x in vals):
                return constant(np.array(vals, dtype=np.int64)).output(0)
            parts = []
            for x in vals:
                if isinstance(x, int):
                    parts.append(constant(np.array([x], dtype=np.int64)).output(0))
                else:
                    o = as_output(x)
                    if o.get_element_type() != Type.i64:
                        o = ops.convert(o, Type.i64).output(0)
                    parts.append(ops.reshape(o, np.array([1], dtype=np.int64), False).output(0))
            return ops.concat(parts, 0).output(0)
        if isinstance(v, int):
            return constant(np.array([v], dtype=np.int64)).output(0)
        return as_output(v)


def _i64(vals) -> Output:
    return constant(np.array(vals, dtype=np.int64)).output(0)


def _pair(v, n=2) -> List[int]:
    if isinstance(v, (list, tuple)):
        return [int(x) for x in v] if len(v) == n else [int(v[0])] * n
    return [int(v)] * n


def _rank(o: Output) -> int:
    r = o.get_partial_shape().rank
    if r.is_dynamic:
        raise ConversionError("operation needs a static rank")
    return r.get_length()


def _norm_axis(axis: int, rank: int) -> int:
    return axis + rank if axis < 0 else axis


def _promote(ctx: Ctx, a, b):
    """Binary-op operands as Outputs with PyTorch type promotion between tensor and scalar / tensors."""
    va, vb = ctx.get(a), ctx.get(b)
    ta, tb = isinstance(va, (Output, Node)), isinstance(vb, (Output, Node))
    if ta and tb:
        oa, ob = as_output(va), as_output(vb)
        ea, eb = oa.get_element_type(), ob.get_element_type()
        if ea != eb and ea.is_static() and eb.is_static():
            if ea.is_real() and not eb.is_real():
                ob = ops.convert(ob, ea).output(0)
            elif eb.is_real() and not ea.is_real():
                oa = ops.convert(oa, eb).output(0)
            elif ea.bitwidth >= eb.bitwidth:
                ob = ops.convert(ob, ea).output(0)
            else:
                oa = ops.convert(oa, eb).output(0)
        return oa, ob
    if ta:
        oa = as_output(va)
        if isinstance(vb, float) and not oa.get_element_type().is_real():
            oa = ops.convert(oa, Type.f32).output(0)
        return oa, ctx.out(vb, like=oa)
    if tb:
        ob = as_output(vb)
        if isinstance(va, float) and not ob.get_element_type().is_real():
            ob = ops.convert(ob, Type.f32).output(0)
        return ctx.out(va, like=ob), ob
    return ctx.out(va), ctx.out(vb)


# ------------------------------------------------------------------------------------------------ translators
_TABLE: Dict[str, Callable] = {}


def _op(*names):
    def deco(fn):
        for n in names:
            _TABLE[n] = fn
        return fn
    return deco


def _binary(factory):
    def fn(ctx, n):
        a, b = _promote(ctx, n.args[0], n.args[1])
        return factory(a, b).output(0)
    return fn


for _names, _f in ((("aten.mul.Tensor", "aten.mul.Scalar", "mul"), ops.multiply), (("aten.maximum.default",), ops.maximum),
                   (("aten.minimum.default",), ops.minimum), (("aten.pow.Tensor_Scalar", "aten.pow.Tensor_Tensor", "aten.pow.Scalar"), ops.power),
                   (("aten.eq.Scalar", "aten.eq.Tensor", "eq"), ops.equal), (("aten.ne.Scalar", "aten.ne.Tensor", "ne"), ops.not_equal),
                   (("aten.lt.Scalar", "aten.lt.Tensor", "lt"), ops.less), (("aten.le.Scalar", "aten.le.Tensor", "le"), ops.less_equal),
                   (("aten.gt.Scalar", "aten.gt.Tensor", "gt"), ops.greater), (("aten.ge.Scalar", "aten.ge.Tensor", "ge"), ops.greater_equal),
                   (("aten.logical_and.default", "aten.bitwise_and.Tensor"), ops.logical_and), (("aten.logical_or.default", "aten.bitwise_or.Tensor"), ops.logical_or),
                   (("aten.logical_xor.default",), ops.logical_xor), (("aten.fmod.Tensor", "aten.fmod.Scalar"), ops.mod),
                   (("aten.remainder.Tensor", "aten.remainder.Scalar", "mod"), ops.floor_mod)):
    for _n in _names:
        _TABLE[_n] = _binary(_f)


@_op("aten.add.Tensor", "aten.add.Scalar", "add")
def _add(ctx, n):
    a, b = _promote(ctx, n.args[0], n.args[1])
    alpha = n.kwargs.get("alpha", 1) if hasattr(n, "kwargs") else 1
    if alpha != 1:
        b = ops.multiply(b, ctx.out(alpha, like=b)).output(0)
    return ops.add(a, b).output(0)


@_op("aten.sub.Tensor", "aten.sub.Scalar", "sub")
def _sub(ctx, n):
    a, b = _promote(ctx, n.args[0], n.args[1])
    alpha = n.kwargs.get("alpha", 1)
    if alpha != 1:
        b = ops.multiply(b, ctx.out(alpha, like=b)).output(0)
    return ops.subtract(a, b).output(0)


@_op("aten.rsub.Scalar", "aten.rsub.Tensor")
def _rsub(ctx, n):
    a, b = _promote(ctx, n.args[0], n.args[1])
    return ops.subtract(b, a).output(0)


@_op("aten.div.Tensor", "aten.div.Scalar", "aten.div.Tensor_mode", "aten.div.Scalar_mode", "truediv")
def _div(ctx, n):
    a, b = _promote(ctx, n.args[0], n.args[1])
    mode = n.kwargs.get("rounding_mode")
    if mode is None and not a.get_element_type().is_real():
        a, b = ops.convert(a, Type.f32).output(0), ops.convert(b, Type.f32).output(0)
    r = ops.divide(a, b)
    r.set_attribute("m_pythondiv", mode == "floor")
    if mode == "floor" and a.get_element_type().is_real():
        return ops.floor(r).output(0)
    if mode == "trunc" and a.get_element_type().is_real():
        return ops.multiply(ops.sign(r), ops.floor(ops.abs(r))).output(0)
    return r.output(0)


@_op("floordiv", "aten.floor_divide.default")
def _floordiv(ctx, n):
    a, b = _promote(ctx, n.args[0], n.args[1])
    r = ops.divide(a, b)
    r.set_attribute("m_pythondiv", True)
    return ops.floor(r).output(0) if a.get_element_type().is_real() else r.output(0)


def _unary(factory):
    return lambda ctx, n: factory(ctx.out(n.args[0])).output(0)


for _name, _f in (("relu", ops.relu), ("sigmoid", ops.sigmoid), ("tanh", ops.tanh), ("exp", ops.exp), ("log", ops.log), ("sqrt", ops.sqrt),
                  ("abs", ops.abs), ("neg", ops.negative), ("sin", ops.sin), ("cos", ops.cos), ("tan", ops.tan), ("erf", ops.erf),
                  ("floor", ops.floor), ("ceil", ops.ceiling), ("sign", ops.sign), ("logical_not", ops.logical_not),
                  ("bitwise_not", ops.logical_not), ("hardswish", ops.hswish), ("hardsigmoid", ops.hsigmoid), ("mish", ops.mish),
                  ("asin", ops.asin), ("acos", ops.acos), ("atan", ops.atan), ("sinh", ops.sinh), ("cosh", ops.cosh), ("isnan", ops.is_nan),
                  ("isfinite", ops.is_finite), ("softplus", ops.softplus)):
    _TABLE["aten.%s.default" % _name] = _unary(_f)
    _TABLE["aten.%s_.default" % _name] = _unary(_f)


@_op("aten.silu.default", "aten.silu_.default")
def _silu(ctx, n):
    return ops.swish(ctx.out(n.args[0])).output(0)


@_op("aten.gelu.default")
def _gelu(ctx, n):
    return ops.gelu(ctx.out(n.args[0]), "tanh" if n.kwargs.get("approximate", "none") == "tanh" else "erf").output(0)


@_op("aten.rsqrt.default")
def _rsqrt(ctx, n):
    x = ctx.out(n.args[0])
    return ops.power(x, ctx.out(-0.5, like=x)).output(0)


@_op("aten.reciprocal.default")
def _recip(ctx, n):
    x = ctx.out(n.args[0])
    return ops.power(x, ctx.out(-1.0, like=x)).output(0)


@_op("aten.leaky_relu.default", "aten.leaky_relu_.default")
def _leaky(ctx, n):
    x = ctx.out(n.args[0])
    slope = n.args[1] if len(n.args) > 1 else 0.01
    return ops.prelu(x, ctx.out(float(slope), like=x)).output(0)


@_op("aten.elu.default")
def _elu(ctx, n):
    return ops.elu(ctx.out(n.args[0]), float(n.args[1]) if len(n.args) > 1 else 1.0).output(0)


@_op("aten.hardtanh.default", "aten.hardtanh_.default")
def _hardtanh(ctx, n):
    lo = n.args[1] if len(n.args) > 1 else -1.0
    hi = n.args[2] if len(n.args) > 2 else 1.0
    return ops.clamp(ctx.out(n.args[0]), float(lo), float(hi)).output(0)


@_op("aten.clamp.default", "aten.clamp_min.default", "aten.clamp_max.default", "aten.clip.default")
def _clamp(ctx, n):
    x = ctx.out(n.args[0])
    name = str(n.target)
    lo = n.args[1] if len(n.args) > 1 and "clamp_max" not in name else n.kwargs.get("min")
    hi = (n.args[1] if "clamp_max" in name else (n.args[2] if len(n.args) > 2 else n.kwargs.get("max")))
    if lo is not None:
        x = ops.maximum(x, ctx.out(lo, like=x)).output(0)
    if hi is not None:
        x = ops.minimum(x, ctx.out(hi, like=x)).output(0)
    return x


@_op("aten.conv2d.default", "aten.conv1d.default", "aten.conv3d.default")
def _conv(ctx, n):
    a = list(n.args) + [None] * 7
    x, w, b = ctx.out(a[0]), ctx.out(a[1]), a[2]
    nd = _rank(x) - 2
    stride = _pair(a[3] if a[3] is not None else 1, nd)
    pad = a[4] if a[4] is not None else 0
    dil = _pair(a[5] if a[5] is not None else 1, nd)
    groups = a[6] if a[6] is not None else 1
    auto_pad = "explicit"
    if isinstance(pad, str):
        auto_pad, pad = ("same_upper" if pad == "same" else "valid"), 0
    pad = _pair(pad, nd)
    if groups == 1:
        y = ops.convolution(x, w, stride, pad, pad, dil, auto_pad)
    else:
        ws = w.get_shape()
        wg = ops.reshape(w, _i64([groups, ws[0] // groups] + list(ws[1:])), False)
        y = ops.group_convolution(x, wg, stride, pad, pad, dil, auto_pad)
    y = y.output(0)
    if b is not None:
        bias = ops.reshape(ctx.out(b), _i64([1, -1] + [1] * nd), False)
        y = ops.add(y, bias).output(0)
    return y


@_op("aten.convolution.default")
def _convolution(ctx, n):
    x, w, b, stride, pad, dil, transposed, out_pad, groups = n.args
    if transposed:
        raise ConversionError("transposed convolution is not supported")
    class _N:   # re-dispatch with conv2d argument order
        args = (x, w, b, stride, pad, dil, groups)
        kwargs = {}
    return _conv(ctx, _N)


@_op("aten.batch_norm.default", "aten._native_batch_norm_legit_no_training.default")
def _bn(ctx, n):
    x, w, b, mean, var = (ctx.get(a) for a in n.args[:5])
    eps = n.args[7] if "aten.batch_norm" in str(n.target) else n.args[6]
    x = as_output(x)
    c = x.get_partial_shape()[1].get_length()
    et = x.get_element_type()
    w = as_output(w) if w is not None else constant(np.ones(c, np.float32), et).output(0)
    b = as_output(b) if b is not None else constant(np.zeros(c, np.float32), et).output(0)
    y = ops.batch_norm_inference(x, w, b, as_output(mean), as_output(var), float(eps)).output(0)
    return y if "aten.batch_norm" in str(n.target) else (y, None, None)


@_op("aten.layer_norm.default", "aten.native_layer_norm.default")
def _ln(ctx, n):
    x = ctx.out(n.args[0])
    shape = n.args[1]
    w = ctx.get(n.args[2]) if len(n.args) > 2 else None
    b = ctx.get(n.args[3]) if len(n.args) > 3 else None
    eps = n.args[4] if len(n.args) > 4 else 1e-5
    axes = _i64(list(range(-len(shape), 0)))
    y = ops.mvn(x, axes, True, float(eps), "inside_sqrt").output(0)
    if w is not None:
        y = ops.multiply(y, as_output(w)).output(0)
    if b is not None:
        y = ops.add(y, as_output(b)).output(0)
    return y if "native" not in str(n.target) else (y, None, None)


@_op("aten.rms_norm.default")
def _rms(ctx, n):
    x = ctx.out(n.args[0])
    w = ctx.get(n.args[2]) if len(n.args) > 2 else None
    eps = n.args[3] if len(n.args) > 3 and n.args[3] is not None else 1e-6
    sq = ops.multiply(x, x)
    mean = ops.reduce_mean(sq, _i64([-1]), True)
    inv = ops.power(ops.add(mean, ctx.out(float(eps), like=x)), ctx.out(-0.5, like=x))
    y = ops.multiply(x, inv).output(0)
    if w is not None:
        y = ops.multiply(y, as_output(w)).output(0)
    return y


@_op("aten.group_norm.default")
def _gn(ctx, n):
    x = ctx.out(n.args[0])
    groups = int(n.args[1])
    c = x.get_partial_shape()[1].get_length()
    w = ctx.get(n.args[2]) if len(n.args) > 2 and n.args[2] is not None else None
    b = ctx.get(n.args[3]) if len(n.args) > 3 and n.args[3] is not None else None
    eps = n.args[4] if len(n.args) > 4 else 1e-5
    et = x.get_element_type()
    w = as_output(w) if w is not None else constant(np.ones(c, np.float32), et).output(0)
    b = as_output(b) if b is not None else constant(np.zeros(c, np.float32), et).output(0)
    return ops.group_normalization(x, w, b, groups, float(eps)).output(0)


@_op("aten.linear.default")
def _linear(ctx, n):
    x, w = ctx.out(n.args[0]), ctx.out(n.args[1])
    y = ops.matmul(x, w, False, True).output(0)
    if len(n.args) > 2 and n.args[2] is not None:
        y = ops.add(y, ctx.out(n.args[2])).output(0)
    return y


@_op("aten.matmul.default", "aten.mm.default", "aten.bmm.default")
def _matmul(ctx, n):
    return ops.matmul(ctx.out(n.args[0]), ctx.out(n.args[1]), False, False).output(0)


@_op("aten.addmm.default")
def _addmm(ctx, n):
    b, x, w = ctx.out(n.args[0]), ctx.out(n.args[1]), ctx.out(n.args[2])
    return ops.add(ops.matmul(x, w, False, False), b).output(0)


@_op("aten.t.default")
def _t(ctx, n):
    x = ctx.out(n.args[0])
    return ops.transpose(x, _i64([1, 0])).output(0) if _rank(x) == 2 else x


@_op("aten.transpose.int")
def _transpose(ctx, n):
    x = ctx.out(n.args[0])
    r = _rank(x)
    a, b = _norm_axis(n.args[1], r), _norm_axis(n.args[2], r)
    order = list(range(r))
    order[a], order[b] = order[b], order[a]
    return ops.transpose(x, _i64(order)).output(0)


@_op("aten.permute.default")
def _permute(ctx, n):
    x = ctx.out(n.args[0])
    r = _rank(x)
    return ops.transpose(x, _i64([_norm_axis(a, r) for a in n.args[1]])).output(0)


@_op("aten.view.default", "aten.reshape.default", "aten._unsafe_view.default")
def _view(ctx, n):
    return ops.reshape(ctx.out(n.args[0]), ctx.ints(n.args[1]), False).output(0)


@_op("aten.flatten.using_ints")
def _flatten(ctx, n):
    x = ctx.out(n.args[0])
    r = _rank(x)
    s = _norm_axis(n.args[1] if len(n.args) > 1 else 0, r)
    e = _norm_axis(n.args[2] if len(n.args) > 2 else -1, r)
    if r == 0:
        return ops.reshape(x, _i64([1]), False).output(0)
    # 0 copies a dimension (special_zero), -1 folds the flattened range
    pattern = [0] * s + [-1] + [0] * (r - 1 - e)
    if r - 1 - e > 0:
        # trailing zeros would refer to the wrong input dims after the fold: build the shape from ShapeOf
        shp = ops.shape_of(x)
        head = ops.slice(shp, _i64([0]), _i64([s]), _i64([1]))
        tail = ops.slice(shp, _i64([e + 1]), _i64([r]), _i64([1]))
        return ops.reshape(x, ops.concat([head, _i64([-1]), tail], 0), False).output(0)
    return ops.reshape(x, _i64(pattern), True).output(0)


@_op("aten.unsqueeze.default")
def _unsqueeze(ctx, n):
    return ops.unsqueeze(ctx.out(n.args[0]), _i64([n.args[1]])).output(0)


@_op("aten.squeeze.dim", "aten.squeeze.dims", "aten.squeeze.default")
def _squeeze(ctx, n):
    x = ctx.out(n.args[0])
    if len(n.args) == 1:
        return ops.squeeze(x).output(0)
    dims = n.args[1] if isinstance(n.args[1], (list, tuple)) else [n.args[1]]
    ps = x.get_partial_shape()
    r = _rank(x)
    keep = [d for d in dims if not (ps[_norm_axis(d, r)].is_static and ps[_norm_axis(d, r)].get_length() != 1)]
    if not keep:
        return x
    return ops.squeeze(x, _i64(keep)).output(0)


@_op("aten.expand.default")
def _expand(ctx, n):
    x = ctx.out(n.args[0])
    sizes = ctx.get(n.args[1])
    if all(isinstance(ctx.get(s), int) for s in sizes):
        vals = [1 if ctx.get(s) == -1 else ctx.get(s) for s in sizes]
        return ops.broadcast(x, _i64(vals), "bidirectional").output(0)
    shape = ctx.ints([1 if (isinstance(ctx.get(s), int) and ctx.get(s) == -1) else s for s in sizes])
    return ops.broadcast(x, shape, "bidirectional").output(0)


@_op("aten.expand_as.default")
def _expand_as(ctx, n):
    return ops.broadcast(ctx.out(n.args[0]), ops.shape_of(ctx.out(n.args[1])), "bidirectional").output(0)


@_op("aten.repeat.default")
def _repeat(ctx, n):
    return ops.tile(ctx.out(n.args[0]), ctx.ints(n.args[1])).output(0)


@_op("aten.cat.default", "aten.concat.default")
def _cat(ctx, n):
    parts = [ctx.out(a) for a in n.args[0]]
    axis = n.args[1] if len(n.args) > 1 else 0
    return ops.concat(parts, int(axis)).output(0)


@_op("aten.stack.default")
def _stack(ctx, n):
    axis = n.args[1] if len(n.args) > 1 else 0
    parts = [ops.unsqueeze(ctx.out(a), _i64([axis])).output(0) for a in n.args[0]]
    return ops.concat(parts, int(axis)).output(0)


@_op("aten.split.Tensor", "aten.split_with_sizes.default")
def _split(ctx, n):
    x = ctx.out(n.args[0])
    size = n.args[1]
    axis = n.args[2] if len(n.args) > 2 else 0
    r = _rank(x)
    ax = _norm_axis(axis, r)
    if isinstance(size, int):
        total = x.get_partial_shape()[ax].get_length()
        sizes = [size] * (total // size) + ([total % size] if total % size else [])
    else:
        sizes = list(size)
    node = ops.variadic_split(x, _i64(ax), _i64(sizes))
    return tuple(node.output(i) for i in range(len(sizes)))


@_op("aten.chunk.default")
def _chunk(ctx, n):
    x = ctx.out(n.args[0])
    chunks = int(n.args[1])
    axis = n.args[2] if len(n.args) > 2 else 0
    ax = _norm_axis(axis, _rank(x))
    total = x.get_partial_shape()[ax].get_length()
    size = -(-total // chunks)
    sizes = [size] * (total // size) + ([total % size] if total % size else [])
    node = ops.variadic_split(x, _i64(ax), _i64(sizes))
    return tuple(node.output(i) for i in range(len(sizes)))


@_op("aten.unbind.int")
def _unbind(ctx, n):
    x = ctx.out(n.args[0])
    axis = n.args[1] if len(n.args) > 1 else 0
    ax = _norm_axis(axis, _rank(x))
    cnt = x.get_partial_shape()[ax].get_length()
    node = ops.split(x, _i64(ax), cnt)
    return tuple(ops.squeeze(node.output(i), _i64([ax])).output(0) for i in range(cnt))


@_op("getitem")
def _getitem(ctx, n):
    seq = ctx.get(n.args[0])
    return seq[n.args[1]]


@_op("aten.slice.Tensor")
def _slice(ctx, n):
    x = ctx.out(n.args[0])
    dim = n.args[1] if len(n.args) > 1 else 0
    start = n.args[2] if len(n.args) > 2 and n.args[2] is not None else 0
    end = n.args[3] if len(n.args) > 3 and n.args[3] is not None else 2 ** 63 - 1
    step = n.args[4] if len(n.args) > 4 else 1
    if isinstance(end, int):
        end = min(end, 2 ** 63 - 1)
    return ops.slice(x, ctx.ints([start]), ctx.ints([end]), _i64([step]), _i64([dim])).output(0)


@_op("aten.select.int")
def _select(ctx, n):
    x = ctx.out(n.args[0])
    idx = ctx.get(n.args[2])
    index = _i64(idx) if isinstance(idx, int) else as_output(idx)
    return ops.gather(x, index, _i64(n.args[1])).output(0)


@_op("aten.index_select.default")
def _index_select(ctx, n):
    return ops.gather(ctx.out(n.args[0]), ctx.out(n.args[2]), _i64(n.args[1])).output(0)


@_op("aten.index.Tensor")
def _index(ctx, n):
    x = ctx.out(n.args[0])
    indices = n.args[1]
    given = [(i, ctx.out(ix)) for i, ix in enumerate(indices) if ix is not None]
    if len(given) == 1:
        axis, ix = given[0]
        if ix.get_element_type() == Type.boolean:
            nz = ops.squeeze(ops.non_zero(ix), _i64([0]))
            return ops.gather(x, nz, _i64(axis)).output(0)
        return ops.gather(x, ix, _i64(axis)).output(0)
    if [i for i, _ in given] == list(range(len(given))):
        stacked = ops.concat([ops.unsqueeze(ix, _i64([-1])).output(0) for _, ix in given], -1)
        return ops.gather_nd(x, stacked).output(0)
    raise ConversionError("advanced indexing with gaps is not supported")


@_op("aten.embedding.default")
def _embedding(ctx, n):
    return ops.gather(ctx.out(n.args[0]), ctx.out(n.args[1]), _i64(0)).output(0)


@_op("aten.gather.default")
def _gather(ctx, n):
    return ops.gather_elements(ctx.out(n.args[0]), ctx.out(n.args[2]), int(n.args[1])).output(0)


@_op("aten.scatter.src", "aten.scatter.value", "aten.scatter_add.default")
def _scatter(ctx, n):
    x = ctx.out(n.args[0])
    idx = ctx.out(n.args[2])
    src = ctx.get(n.args[3])
    if not isinstance(src, (Output, Node)):
        src = ops.broadcast(ctx.out(src, like=x), ops.shape_of(idx)).output(0)
    red = "sum" if "scatter_add" in str(n.target) else "none"
    return ops.scatter_elements_update(x, idx, as_output(src), _i64(n.args[1]), red).output(0)


@_op("aten.index_put.default", "aten.index_put_.default")
def _index_put(ctx, n):
    x = ctx.out(n.args[0])
    indices = [ctx.out(i) for i in n.args[1] if i is not None]
    if len(indices) != len(n.args[1]):
        raise ConversionError("index_put with gaps is not supported")
    values = ctx.out(n.args[2], like=x)
    accumulate = bool(n.args[3]) if len(n.args) > 3 else False
    idx = ops.concat([ops.unsqueeze(i, _i64([-1])).output(0) for i in indices], -1)
    return ops.scatter_nd_update(x, idx, values, "sum" if accumulate else "none").output(0)


@_op("aten.where.self", "aten.where.ScalarSelf", "aten.where.ScalarOther", "aten.where.Scalar")
def _where(ctx, n):
    a, b = _promote(ctx, n.args[1], n.args[2])
    return ops.select(ctx.out(n.args[0]), a, b).output(0)


@_op("aten.masked_fill.Scalar", "aten.masked_fill.Tensor", "aten.masked_fill_.Scalar")
def _masked_fill(ctx, n):
    x = ctx.out(n.args[0])
    v = ctx.out(n.args[2], like=x)
    if v.get_element_type() != x.get_element_type():
        v = ops.convert(v, x.get_element_type()).output(0)
    return ops.select(ctx.out(n.args[1]), v, x).output(0)


@_op("aten.softmax.int", "aten._softmax.default")
def _softmax(ctx, n):
    x = ctx.out(n.args[0])
    dt = n.kwargs.get("dtype") or (n.args[2] if len(n.args) > 2 and not isinstance(n.args[2], bool) else None)
    if dt is not None:
        x = ops.convert(x, _ov_type(dt)).output(0)
    return ops.softmax(x, int(n.args[1])).output(0)


@_op("aten.log_softmax.int", "aten._log_softmax.default")
def _log_softmax(ctx, n):
    return ops.log_softmax(ctx.out(n.args[0]), int(n.args[1])).output(0)


def _reduce(factory):
    def fn(ctx, n):
        x = ctx.out(n.args[0])
        dims = n.args[1] if len(n.args) > 1 else None
        keep = bool(n.args[2]) if len(n.args) > 2 else bool(n.kwargs.get("keepdim", False))
        if dims is None or dims == []:
            dims = list(range(_rank(x)))
        if isinstance(dims, int):
            dims = [dims]
        if x.get_element_type() == Type.boolean and factory in (ops.reduce_sum, ops.reduce_mean):
            x = ops.convert(x, Type.i64).output(0)
        return factory(x, _i64(list(dims)), keep).output(0)
    return fn


for _name, _f in (("aten.mean.dim", ops.reduce_mean), ("aten.mean.default", ops.reduce_mean), ("aten.sum.dim_IntList", ops.reduce_sum),
                  ("aten.sum.default", ops.reduce_sum), ("aten.amax.default", ops.reduce_max), ("aten.amin.default", ops.reduce_min),
                  ("aten.prod.dim_int", ops.reduce_prod), ("aten.any.dim", ops.reduce_logical_or), ("aten.all.dim", ops.reduce_logical_and),
                  ("aten.any.default", ops.reduce_logical_or), ("aten.all.default", ops.reduce_logical_and)):
    _TABLE[_name] = _reduce(_f)


@_op("aten.max.dim", "aten.min.dim")
def _max_dim(ctx, n):
    x = ctx.out(n.args[0])
    axis = int(n.args[1])
    keep = bool(n.args[2]) if len(n.args) > 2 else False
    node = ops.topk(x, constant(np.array(1, dtype=np.int64)), axis, "max" if "max" in str(n.target) else "min", "none", "i64")
    v, i = node.output(0), node.output(1)
    if not keep:
        v, i = ops.squeeze(v, _i64([axis])).output(0), ops.squeeze(i, _i64([axis])).output(0)
    return (v, i)


@_op("aten.argmax.default", "aten.argmin.default")
def _argmax(ctx, n):
    x = ctx.out(n.args[0])
    axis = n.args[1] if len(n.args) > 1 else None
    keep = bool(n.args[2]) if len(n.args) > 2 else False
    if axis is None:
        x, axis, keep = ops.reshape(x, _i64([-1]), False).output(0), 0, False
    node = ops.topk(x, constant(np.array(1, dtype=np.int64)), int(axis), "max" if "argmax" in str(n.target) else "min", "none", "i64")
    i = node.output(1)
    return i if keep else ops.squeeze(i, _i64([axis])).output(0)


@_op("aten.topk.default")
def _topk(ctx, n):
    x = ctx.out(n.args[0])
    k = ctx.get(n.args[1])
    axis = n.args[2] if len(n.args) > 2 else -1
    largest = n.args[3] if len(n.args) > 3 else True
    node = ops.topk(x, constant(np.array(k, dtype=np.int64)), int(axis), "max" if largest else "min", "value", "i64")
    return (node.output(0), node.output(1))


@_op("aten.cumsum.default")
def _cumsum(ctx, n):
    x = ctx.out(n.args[0])
    dt = n.kwargs.get("dtype")
    if dt is not None:
        x = ops.convert(x, _ov_type(dt)).output(0)
    elif x.get_element_type() == Type.boolean:
        x = ops.convert(x, Type.i64).output(0)
    return ops.cumsum(x, _i64(n.args[1])).output(0)


@_op("aten.max_pool2d.default", "aten.max_pool2d_with_indices.default", "aten.max_pool1d.default", "aten.max_pool3d.default")
def _max_pool(ctx, n):
    x = ctx.out(n.args[0])
    nd = _rank(x) - 2
    k = _pair(n.args[1], nd)
    s = _pair(n.args[2], nd) if len(n.args) > 2 and n.args[2] not in (None, []) else k
    p = _pair(n.args[3], nd) if len(n.args) > 3 else [0] * nd
    d = _pair(n.args[4], nd) if len(n.args) > 4 else [1] * nd
    ceil = bool(n.args[5]) if len(n.args) > 5 else False
    node = ops.max_pool(x, s, d, p, p, k, "ceil" if ceil else "floor", "explicit", "i64", 0)
    return (node.output(0), node.output(1)) if "with_indices" in str(n.target) else node.output(0)


@_op("aten.avg_pool2d.default", "aten.avg_pool1d.default", "aten.avg_pool3d.default")
def _avg_pool(ctx, n):
    x = ctx.out(n.args[0])
    nd = _rank(x) - 2
    k = _pair(n.args[1], nd)
    s = _pair(n.args[2], nd) if len(n.args) > 2 and n.args[2] not in (None, []) else k
    p = _pair(n.args[3], nd) if len(n.args) > 3 else [0] * nd
    ceil = bool(n.args[4]) if len(n.args) > 4 else False
    include = bool(n.args[5]) if len(n.args) > 5 else True
    return ops.avg_pool(x, s, p, p, k, not include, "ceil" if ceil else "floor", "explicit").output(0)


@_op("aten.adaptive_avg_pool2d.default", "aten._adaptive_avg_pool2d.default", "aten.adaptive_avg_pool1d.default")
def _adaptive_avg(ctx, n):
    x = ctx.out(n.args[0])
    size = n.args[1] if isinstance(n.args[1], (list, tuple)) else [n.args[1]]
    if all(s == 1 for s in size):
        return ops.reduce_mean(x, _i64(list(range(-len(size), 0))), True).output(0)
    return ops.adaptive_avg_pool(x, _i64(list(size))).output(0)


@_op("aten.upsample_nearest2d.default", "aten.upsample_nearest2d.vec", "aten.upsample_bilinear2d.default", "aten.upsample_bilinear2d.vec")
def _upsample(ctx, n):
    x = ctx.out(n.args[0])
    bilinear = "bilinear" in str(n.target)
    size = n.args[1]
    align = bool(n.args[2]) if bilinear and len(n.args) > 2 else False
    scales = None
    if size is None:
        scales = n.args[3] if bilinear else n.args[2]
    mode = "linear_onnx" if bilinear else "nearest"
    ct = "align_corners" if align else ("pytorch_half_pixel" if bilinear else "asymmetric")
    if size is not None:
        return ops.interpolate(x, ctx.ints(size), _i64([2, 3]), mode, "sizes", [0, 0, 0, 0], [0, 0, 0, 0], ct, "floor").output(0)
    return ops.interpolate(x, constant(np.array(scales, dtype=np.float32)), _i64([2, 3]), mode, "scales", [0, 0, 0, 0], [0, 0, 0, 0], ct, "floor").output(0)


@_op("aten.scaled_dot_product_attention.default")
def _sdpa(ctx, n):
    q, k, v = ctx.out(n.args[0]), ctx.out(n.args[1]), ctx.out(n.args[2])
    mask = n.args[3] if len(n.args) > 3 else n.kwargs.get("attn_mask")
    causal = n.args[5] if len(n.args) > 5 else n.kwargs.get("is_causal", False)
    scale = n.kwargs.get("scale")
    ins = [q, k, v]
    if mask is not None or scale is not None:
        ins.append(ctx.out(mask) if mask is not None else constant(np.array(0, dtype=np.float32), q.get_element_type()).output(0))
    if scale is not None:
        ins.append(ctx.out(float(scale), like=q))
    from .._graph import make_op
    return make_op("ScaledDotProductAttention", ins, {"causal": bool(causal)}).output(0)


@_op("aten.dropout.default", "aten.dropout_.default", "aten.feature_dropout.default", "aten.contiguous.default", "aten.clone.default",
     "aten.detach.default", "aten.detach_.default", "aten.alias.default", "aten.lift_fresh_copy.default", "aten.lift_fresh.default",
     "aten._assert_tensor_metadata.default", "aten.to.device")
def _identity(ctx, n):
    return ctx.get(n.args[0])


@_op("aten.to.dtype", "aten.to.dtype_layout", "aten._to_copy.default", "aten.type_as.default")
def _to(ctx, n):
    x = ctx.out(n.args[0])
    if "type_as" in str(n.target):
        return ops.convert_like(x, ctx.out(n.args[1])).output(0)
    dt = n.kwargs.get("dtype")
    if dt is None and len(n.args) > 1 and not isinstance(n.args[1], (bool, int)):
        dt = n.args[1]
    if dt is None or _ov_type(dt) == x.get_element_type():
        return x
    return ops.convert(x, _ov_type(dt)).output(0)


@_op("aten.arange.default", "aten.arange.start", "aten.arange.start_step")
def _arange(ctx, n):
    a = [ctx.get(x) for x in n.args]
    start, stop, step = (0, a[0], 1) if len(a) == 1 else ((a[0], a[1], 1) if len(a) == 2 else a[:3])
    dt = n.kwargs.get("dtype")
    any_float = any(isinstance(x, float) for x in (start, stop, step))
    et = _ov_type(dt) if dt is not None else (Type.f32 if any_float else Type.i64)
    def sc(v):
        if isinstance(v, (int, float)):
            return constant(np.array(v), et).output(0)
        o = as_output(v)
        o = ops.squeeze(o).output(0) if o.get_partial_shape().rank.get_length() else o
        return o if o.get_element_type() == et else ops.convert(o, et).output(0)
    return ops.range(sc(start), sc(stop), sc(step), et).output(0)


def _fill(ctx, shape_out: Output, value, et: Type) -> Output:
    return ops.broadcast(constant(np.array(value), et), shape_out).output(0)


@_op("aten.full.default", "aten.zeros.default", "aten.ones.default", "aten.empty.memory_format", "aten.new_zeros.default", "aten.new_ones.default",
     "aten.new_full.default", "aten.new_empty.default")
def _full(ctx, n):
    name = str(n.target)
    new = ".new_" in name
    args = n.args[1:] if new else n.args
    value = args[1] if "full" in name else (1 if "ones" in name else 0)
    dt = n.kwargs.get("dtype")
    if dt is not None:
        et = _ov_type(dt)
    elif new:
        et = ctx.out(n.args[0]).get_element_type()
    else:
        et = Type.boolean if isinstance(value, bool) else (Type.i64 if isinstance(value, int) and "full" in name else Type.f32)
    return _fill(ctx, ctx.ints(args[0]), value, et)


@_op("aten.full_like.default", "aten.zeros_like.default", "aten.ones_like.default", "aten.empty_like.default")
def _full_like(ctx, n):
    x = ctx.out(n.args[0])
    name = str(n.target)
    value = n.args[1] if "full_like" in name else (1 if "ones" in name else 0)
    dt = n.kwargs.get("dtype")
    et = _ov_type(dt) if dt is not None else x.get_element_type()
    return _fill(ctx, ops.shape_of(x).output(0), value, et)


@_op("aten.scalar_tensor.default")
def _scalar_tensor(ctx, n):
    dt = n.kwargs.get("dtype")
    return constant(np.array(n.args[0]), _ov_type(dt) if dt is not None else Type.f32).output(0)


@_op("aten.sym_size.int", "aten.size.int")
def _sym_size(ctx, n):
    x = ctx.out(n.args[0])
    d = x.get_partial_shape()[n.args[1]]
    if d.is_static:
        return d.get_length()
    return ops.gather(ops.shape_of(x), _i64(n.args[1]), _i64(0)).output(0)


@_op("aten.tril.default", "aten.triu.default")
def _tri(ctx, n):
    x = ctx.out(n.args[0])
    k = n.args[1] if len(n.args) > 1 else 0
    shp = ops.shape_of(x)
    rows = ops.gather(shp, _i64(-2), _i64(0))
    cols = ops.gather(shp, _i64(-1), _i64(0))
    zero, one = constant(np.array(0, dtype=np.int64)), constant(np.array(1, dtype=np.int64))
    r = ops.unsqueeze(ops.range(zero, rows, one, "i64"), _i64([1]))
    c = ops.unsqueeze(ops.range(zero, cols, one, "i64"), _i64([0]))
    diff = ops.subtract(c, r)
    keep = ops.less_equal(diff, _i64(k)) if "tril" in str(n.target) else ops.greater_equal(diff, _i64(k))
    return ops.select(keep, x, ctx.out(0, like=x)).output(0)


@_op("aten.einsum.default")
def _einsum(ctx, n):
    return ops.einsum([ctx.out(a) for a in n.args[1]], n.args[0]).output(0)


@_op("aten.pad.default", "aten.constant_pad_nd.default")
def _pad(ctx, n):
    x = ctx.out(n.args[0])
    pads = list(n.args[1])
    mode = n.args[2] if "aten.pad" in str(n.target) and len(n.args) > 2 else "constant"
    value = (n.args[3] if "aten.pad" in str(n.target) and len(n.args) > 3 else (n.args[2] if "constant_pad" in str(n.target) and len(n.args) > 2 else 0)) or 0
    r = _rank(x)
    begin, end = [0] * r, [0] * r
    for i in range(len(pads) // 2):
        begin[r - 1 - i], end[r - 1 - i] = pads[2 * i], pads[2 * i + 1]
    mode = {"constant": "constant", "reflect": "reflect", "replicate": "edge", "circular": "constant"}[mode]
    return ops.pad(x, _i64(begin), _i64(end), ctx.out(value, like=x), mode).output(0)


@_op("aten.roll.default")
def _roll(ctx, n):
    return ops.roll(ctx.out(n.args[0]), _i64(list(n.args[1])), _i64(list(n.args[2]))).output(0)


@_op("aten.pixel_shuffle.default")
def _pixel_shuffle(ctx, n):
    return ops.depth_to_space(ctx.out(n.args[0]), "depth_first", int(n.args[1])).output(0)


@_op("aten.sym_constrain_range_for_size.default", "aten._assert_scalar.default", "aten.sym_constrain_range.default")
def _noop(ctx, n):
    return None


# ------------------------------------------------------------------------------------------------ driver
def _target_name(target) -> str:
    if isinstance(target, str):
        return target
    if target in (operator.getitem,):
        return "getitem"
    for op, name in ((operator.add, "add"), (operator.sub, "sub"), (operator.mul, "mul"), (operator.truediv, "truediv"), (operator.floordiv, "floordiv"),
                     (operator.mod, "mod"), (operator.eq, "eq"), (operator.ne, "ne"), (operator.lt, "lt"), (operator.le, "le"), (operator.gt, "gt"),
                     (operator.ge, "ge")):
        if target is op:
            return name
    return str(target)


def supported_ops() -> List[str]:
    return sorted(_TABLE)


def _python_scalar_op(name, args):
    fn = {"add": operator.add, "sub": operator.sub, "mul": operator.mul, "truediv": operator.truediv, "floordiv": operator.floordiv,
          "mod": operator.mod, "eq": operator.eq, "ne": operator.ne, "lt": operator.lt, "le": operator.le, "gt": operator.gt, "ge": operator.ge}[name]
    return fn(*args)


def _untranslated(ep) -> list:
    missing = []
    for node in ep.graph.nodes:
        if node.op != "call_function":
            continue
        name = _target_name(node.target)
        if name.startswith("aten.") is False and not isinstance(node.target, str) and hasattr(node.target, "_schema"):
            name = str(node.target)
        if name not in _TABLE and node.target not in missing:
            missing.append(node.target)
    return missing


def _decompose_untranslated(ep, rounds: int = 3):
    import torch
    try:
        from torch._decomp import decomposition_table
    except ImportError:
        return ep
    for _ in range(rounds):
        missing = [t for t in _untranslated(ep) if hasattr(t, "_schema")]
        table = {t: decomposition_table[t] for t in missing if t in decomposition_table}
        if not table:
            break
        try:
            ep = ep.run_decompositions(table)
        except Exception:   # noqa: BLE001 - one of the decompositions does not apply here: take them one at a time
            progressed = False
            for t, fn in table.items():
                try:
                    ep = ep.run_decompositions({t: fn})
                    progressed = True
                except Exception:   # noqa: BLE001 - the conversion below then names the operation that has no translator
                    pass
            if not progressed:
                break
    left = _untranslated(ep)
    if left:
        # composite operations (var.dim, std.dim, ...) have no table entry of their own: the default decomposition to the
        # core ATen set resolves them
        try:
            full = ep.run_decompositions()
            if len(_untranslated(full)) < len(left):
                ep = full
        except Exception:   # noqa: BLE001
            pass
    return ep


def from_exported_program(ep, share_weights: bool = True, input_names: Optional[Sequence[str]] = None) -> Model:
    """``torch.export.ExportedProgram`` -> ``Model``. Operations without a translator are first rewritten by their ATen
    decompositions (``ExportedProgram.run_decompositions`` with a table of just those operations), so the table above only
    has to cover what the decompositions bottom out in."""
    import torch
    from torch.export.graph_signature import InputKind
    ep = _decompose_untranslated(ep)
    ctx = Ctx()
    sig = ep.graph_signature
    spec_by_name = {s.arg.name: s for s in sig.input_specs if hasattr(s.arg, "name")}
    params: List[Node] = []
    user_idx = 0
    for node in ep.graph.nodes:
        if node.op == "placeholder":
            spec = spec_by_name.get(node.name)
            if spec is not None and spec.kind in (InputKind.PARAMETER, InputKind.BUFFER, InputKind.CONSTANT_TENSOR):
                if spec.kind == InputKind.CONSTANT_TENSOR:
                    t = ep.constants[spec.target]
                else:
                    t = ep.state_dict[spec.target] if spec.target in ep.state_dict else ep.constants[spec.target]
                c = constant(Tensor(t.detach().contiguous(), shared_memory=share_weights), name=spec.target, shared_memory=share_weights)
                ctx.values[node] = c.output(0)
                continue
            val = node.meta.get("val")
            if val is None or not hasattr(val, "shape"):
                raise ConversionError("input %s is not a tensor" % node.name)
            dims = [int(d) if isinstance(d, int) else -1 for d in val.shape]
            name = input_names[user_idx] if input_names and user_idx < len(input_names) else node.name
            p = parameter(PartialShape(dims), _ov_type(val.dtype), name)
            p.output(0).set_names({name})
            params.append(p)
            ctx.values[node] = p.output(0)
            user_idx += 1
        elif node.op == "call_function":
            name = _target_name(node.target)
            if name.startswith("aten.") is False and not isinstance(node.target, str) and hasattr(node.target, "_schema"):
                name = str(node.target)
            plain_args = [ctx.get(a) for a in node.args] if name in ("add", "sub", "mul", "truediv", "floordiv", "mod", "eq", "ne", "lt", "le", "gt", "ge") else None
            if plain_args is not None and all(isinstance(a, (int, float, bool)) for a in plain_args):
                ctx.values[node] = _python_scalar_op(name, plain_args)
                continue
            fn = _TABLE.get(name)
            if fn is None:
                raise ConversionError("no translator for %s (node %s)" % (name, node.name))
            out = fn(ctx, node)
            if isinstance(out, Node):
                out = out.output(0)
            ctx.values[node] = out
            if isinstance(out, Output) and out.get_node().get_type_name() not in ("Parameter", "Constant"):
                out.get_node().set_friendly_name(node.name)
        elif node.op == "get_attr":
            t = getattr(ep.graph_module, node.target)
            ctx.values[node] = constant(Tensor(t.detach().contiguous(), shared_memory=share_weights), name=str(node.target), shared_memory=share_weights).output(0)
        elif node.op == "output":
            flat = []

            def walk(a):
                if isinstance(a, (list, tuple)):
                    for x in a:
                        walk(x)
                elif isinstance(a, dict):
                    for x in a.values():
                        walk(x)
                elif a is not None:
                    flat.append(a)
            walk(node.args[0])
            results = []
            for a in flat:
                o = ctx.out(a)
                r = result(o)
                nm = a.name if hasattr(a, "name") else "output_%d" % len(results)
                if not o.get_names():
                    o.set_names({nm})
                results.append(r)
            return Model(results, params, "Model")
    raise ConversionError("the exported graph has no output node")


def from_fx(gm, example_inputs: Sequence[Any], share_weights: bool = True) -> Model:
    """A ``torch.fx.GraphModule`` whose call_function nodes are aten operators (what ``make_fx`` and the partitioner of the
    ``torch.compile`` backend produce) -> ``Model``. Placeholders become Parameters shaped like ``example_inputs``
    (fake or real tensors; python scalars are inlined), ``get_attr`` tensors become Constants."""
    import torch
    ctx = Ctx()
    params: List[Node] = []
    idx = 0
    for node in gm.graph.nodes:
        if node.op == "placeholder":
            ex = example_inputs[idx] if idx < len(example_inputs) else node.meta.get("val")
            idx += 1
            if isinstance(ex, (int, float, bool)):
                ctx.values[node] = ex
                continue
            if ex is None or not hasattr(ex, "shape"):
                raise ConversionError("input %s is not a tensor" % node.name)
            dims = [int(d) if isinstance(d, int) else -1 for d in ex.shape]
            p = parameter(PartialShape(dims), _ov_type(ex.dtype), node.name)
            p.output(0).set_names({node.name})
            params.append(p)
            ctx.values[node] = p.output(0)
        elif node.op == "get_attr":
            t = gm
            for part in str(node.target).split("."):
                t = getattr(t, part)
            ctx.values[node] = constant(Tensor(t.detach().contiguous(), shared_memory=share_weights), name=str(node.target), shared_memory=share_weights).output(0)
        elif node.op == "call_function":
            name = _target_name(node.target)
            plain_args = [ctx.get(a) for a in node.args] if name in ("add", "sub", "mul", "truediv", "floordiv", "mod", "eq", "ne", "lt", "le", "gt", "ge") else None
            if plain_args is not None and all(isinstance(a, (int, float, bool)) for a in plain_args):
                ctx.values[node] = _python_scalar_op(name, plain_args)
                continue
            fn = _TABLE.get(name)
            if fn is None:
                raise ConversionError("no translator for %s (node %s)" % (name, node.name))
            out = fn(ctx, node)
            if isinstance(out, Node):
                out = out.output(0)
            ctx.values[node] = out
        elif node.op == "output":
            flat = []

            def walk(a):
                if isinstance(a, (list, tuple)):
                    for x in a:
                        walk(x)
                elif a is not None:
                    flat.append(a)
            walk(node.args[0])
            results = []
            for i, a in enumerate(flat):
                o = ctx.out(a)
                if not o.get_names():
                    o.set_names({"output_%d" % i})
                results.append(result(o))
            return Model(results, params, "Model")
        else:
            raise ConversionError("fx node kind %s is not supported" % node.op)
    raise ConversionError("the fx graph has no output node")


def convert(module, example_input=None, input=None, dynamic_shapes=None, share_weights: bool = True, strict: bool = False) -> Model:
    """``torch.nn.Module`` (or ``ExportedProgram``) -> ``Model``.

    ``example_input``: tensor / tuple / dict used for tracing. ``input``: optional shapes (list, or
    ``[(name, shape, type)]`` / ``{name: shape}``): dynamic dimensions (-1) there are exported as symbolic.
    """
    import torch
    if hasattr(module, "graph_signature") and hasattr(module, "graph"):
        return from_exported_program(module, share_weights)
    if isinstance(module, (torch.jit.ScriptModule, torch.jit.ScriptFunction)):
        # traced / scripted models keep their TorchScript graph: decoded by the TorchScript front end
        from .torchscript import from_script
        return from_script(module, example_input=example_input, input=input, share_weights=share_weights)
    if not isinstance(module, torch.nn.Module):
        raise ConversionError("expected a torch.nn.Module, a ScriptModule or an ExportedProgram, got %r" % type(module))
    if example_input is None:
        if input is None:
            raise ConversionError("convert_model of a torch module needs example_input (or static input shapes)")
        shapes = _input_shapes(input)
        example_input = tuple(torch.zeros([d if d > 0 else 2 for d in s]) for s in shapes)
    args, kwargs = (), {}
    if isinstance(example_input, dict):
        kwargs = dict(example_input)
    elif isinstance(example_input, (list, tuple)):
        args = tuple(example_input)
    else:
        args = (example_input,)
    args = tuple(torch.as_tensor(a) if isinstance(a, np.ndarray) else a for a in args)
    was_training = module.training
    module.eval()
    try:
        if dynamic_shapes is None and input is not None:
            dynamic_shapes = _dynamic_spec(input, args, kwargs)
        with torch.no_grad():
            ep = torch.export.export(module, args, kwargs, dynamic_shapes=dynamic_shapes, strict=strict)
    finally:
        module.train(was_training)
    model = from_exported_program(ep, share_weights)
    if input is not None and dynamic_shapes is None:
        shapes = _input_shapes(input)
        if len(shapes) == len(model.inputs):
            model.reshape({i: s for i, s in enumerate(shapes)})
    return model


def _input_shapes(input) -> List[List[int]]:
    if isinstance(input, dict):
        input = list(input.values())
    if isinstance(input, (PartialShape,)) or (isinstance(input, (list, tuple)) and input and all(isinstance(d, int) for d in input)):
        input = [input]
    shapes = []
    for item in input:
        if isinstance(item, tuple) and len(item) >= 2 and isinstance(item[0], str):
            item = item[1]
        ps = item if isinstance(item, PartialShape) else PartialShape(list(item))
        shapes.append([d.get_length() if d.is_static else -1 for d in ps])
    return shapes


def _dynamic_spec(input, args, kwargs):
    import torch
    shapes = _input_shapes(input)
    if not any(d < 0 for s in shapes for d in s) or kwargs or len(shapes) != len(args):
        return None
    spec = []
    for ai, s in enumerate(shapes):
        spec.append({i: torch.export.Dim.AUTO if hasattr(torch.export.Dim, "AUTO") else torch.export.Dim("d%d_%d" % (ai, i)) for i, d in enumerate(s) if d < 0} or None)
    return tuple(spec)


# ---------------------------------------------------------------------------------------------- public decoder objects
class TorchScriptPythonDecoder:
    """What ``FrontEnd.load`` accepts for a PyTorch model: the module (traced or scripted when it is not yet a
    ScriptModule) with its example input. ``FrontEnd.convert`` of the loaded model decodes the TorchScript graph
    (torchscript.py). Reference: src/bindings/python/src/openvino/frontend/pytorch/ts_decoder.py."""

    def __init__(self, pt_module, example_input=None, skip_freeze: bool = False, shared_memory: bool = True, trace_kwargs=None, module_extensions=None):
        import torch
        self.example_input, self.shared_memory = example_input, shared_memory
        self.module_extensions = dict(module_extensions or {})
        if isinstance(pt_module, (torch.jit.ScriptModule, torch.jit.ScriptFunction)):
            self.pt_module = pt_module
        else:
            pt_module.eval()
            if example_input is None:
                self.pt_module = torch.jit.script(pt_module)
            else:
                args = example_input if isinstance(example_input, (tuple, list)) else (example_input,)
                self.pt_module = torch.jit.trace(pt_module, tuple(args), strict=False, **(trace_kwargs or {}))

    def convert(self) -> Model:
        from .torchscript import from_script
        return from_script(self.pt_module, example_input=self.example_input, share_weights=self.shared_memory)


class TorchFXPythonDecoder:
    """An ``fx.GraphModule`` (``torch.export`` / ``make_fx`` output) for ``FrontEnd.load``; ``from_fx`` does the work.
    Reference: src/bindings/python/src/openvino/frontend/pytorch/fx_decoder.py."""

    def __init__(self, pt_module, fx_gm=None, input_shapes=None, input_types=None, dynamic_shapes: bool = False):
        self.pt_module = fx_gm if fx_gm is not None else pt_module
        self.input_shapes, self.input_types = input_shapes, input_types

    @classmethod
    def from_exported_program(cls, exported_program):
        d = cls(exported_program)
        d._exported = True
        return d

    def convert(self) -> Model:
        if getattr(self, "_exported", False) or (hasattr(self.pt_module, "graph_signature") and hasattr(self.pt_module, "graph")):
            return from_exported_program(self.pt_module, True)
        return from_fx(self.pt_module)


class ModuleExtension:
    """Replaces a sub-module during conversion: ``ModuleExtension(MyAttention, "MyAttentionOp", convert=...)``. With
    ``convert(module, target_op, *args, **kwargs)`` the sub-module's forward is swapped for that callable while the model
    is traced, so the traced graph holds what it returns. Reference: frontend/pytorch/module_extension.py."""

    def __init__(self, module, target_op: str = None, evaluate=None, convert=None, condition=None):
        self.module, self.target_op, self.evaluate, self.convert, self.condition = module, target_op, evaluate, convert, condition

    def matches(self, name: str, sub) -> bool:
        if self.condition is not None and not self.condition(sub):
            return False
        if isinstance(self.module, str):
            return name == self.module
        if isinstance(self.module, type):
            return isinstance(sub, self.module)
        return sub is self.module


def apply_module_extensions(model, extensions):
    """Patch the forwards named by ``extensions``; returns the undo list for ``restore_module_extensions``."""
    undo = []
    for name, sub in model.named_modules():
        for ext in extensions:
            if ext.matches(name, sub) and ext.convert is not None:
                orig = sub.forward
                target = ext.target_op

                def patched(*a, _ext=ext, _sub=sub, _orig=orig, _t=target, **kw):
                    return _ext.convert(_sub, (lambda *x, **y: _orig(*x, **y)) if _t is None else _t, *a, **kw)
                sub.forward = patched
                undo.append((sub, orig))
    return undo


def restore_module_extensions(undo) -> None:
    for sub, orig in undo:
        sub.forward = orig


from .input_model import ConversionExtension   # noqa: E402,F401  (the PyTorch table takes (ctx, node) translators)


from . import pytorch_more   # noqa: E402,F401  (second part of the translator table)
