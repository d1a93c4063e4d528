"""JAX frontend: a ``ClosedJaxpr`` (``jax.make_jaxpr(fn)(*example)``) or a jitted function plus example inputs -> ``Model``.

A jaxpr is a flat list of equations ``outvars = primitive(invars, **params)`` over typed variables. The walk needs only
that structure (``jaxpr.invars / constvars / eqns / outvars``, ``eqn.primitive.name``, ``eqn.params``, ``var.aval.shape /
dtype``, literals with ``.val``), so it works on the objects of any JAX version and the ``jax`` package is only imported
when the caller passes a function instead of a jaxpr. Inner jaxprs (``pjit`` / ``closed_call`` / ``custom_jvp_call``
/ ``remat``) are inlined.

Role in the reference: src/frontends/jax/src (jaxpr decoder protocol, op_table.cpp, op/*.cpp) and the Python decoder
src/bindings/python/src/openvino/frontend/jax/jaxpr_decoder.py.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Sequence

import numpy as np

from .. import opset as ops
from .._graph import Model, Output, constant, parameter, result
from .._types import PartialShape


class JaxError(RuntimeError):
    pass


_OV = {"float32": "f32", "float16": "f16", "bfloat16": "bf16", "float64": "f64", "int32": "i32", "int64": "i64", "int8": "i8", "uint8": "u8",
       "int16": "i16", "uint32": "u32", "bool": "boolean"}


def _ov_type(dtype) -> str:
    name = getattr(dtype, "name", None) or str(dtype)
    if name not in _OV:
        raise JaxError("element type %s is not supported" % name)
    return _OV[name]


def _i64(v):
    return constant(np.asarray(v, dtype=np.int64))


_T: Dict[str, Callable] = {}


def _prim(*names):
    def deco(fn):
        for n in names:
            _T[n] = fn
        return fn
    return deco


def _unary(factory):
    return lambda ins, p, eqn: [factory(ins[0]).output(0)]


def _binary(factory):
    return lambda ins, p, eqn: [factory(ins[0], ins[1]).output(0)]


for _n, _f in (("exp", ops.exp), ("log", ops.log), ("tanh", ops.tanh), ("logistic", ops.sigmoid), ("sqrt", ops.sqrt), ("abs", ops.abs),
               ("neg", ops.negative), ("sin", ops.sin), ("cos", ops.cos), ("erf", ops.erf), ("floor", ops.floor), ("ceil", ops.ceiling),
               ("sign", ops.sign), ("not", ops.logical_not)):
    _T[_n] = _unary(_f)
for _n, _f in (("add", ops.add), ("add_any", ops.add), ("sub", ops.subtract), ("mul", ops.multiply), ("div", ops.divide), ("max", ops.maximum),
               ("min", ops.minimum), ("pow", ops.power), ("eq", ops.equal), ("ne", ops.not_equal), ("lt", ops.less), ("le", ops.less_equal),
               ("gt", ops.greater), ("ge", ops.greater_equal), ("and", ops.logical_and), ("or", ops.logical_or), ("rem", ops.mod)):
    _T[_n] = _binary(_f)
_T["rsqrt"] = lambda ins, p, eqn: [ops.divide(constant(np.array(1.0, np.float32), ins[0].get_element_type()), ops.sqrt(ins[0])).output(0)]
_T["stop_gradient"] = _T["copy"] = _T["copy_p"] = lambda ins, p, eqn: [ins[0]]


@_prim("integer_pow")
def _integer_pow(ins, p, eqn):
    return [ops.power(ins[0], constant(np.array(p["y"], np.float32), ins[0].get_element_type())).output(0)]


@_prim("square")
def _square(ins, p, eqn):
    return [ops.multiply(ins[0], ins[0]).output(0)]


@_prim("convert_element_type")
def _convert(ins, p, eqn):
    return [ops.convert(ins[0], _ov_type(p["new_dtype"])).output(0)]


@_prim("reshape")
def _reshape(ins, p, eqn):
    return [ops.reshape(ins[0], _i64(list(p["new_sizes"])), False).output(0)]


@_prim("squeeze")
def _squeeze(ins, p, eqn):
    return [ops.squeeze(ins[0], _i64(list(p["dimensions"]))).output(0)]


@_prim("expand_dims")
def _expand_dims(ins, p, eqn):
    return [ops.unsqueeze(ins[0], _i64(list(p["dimensions"]))).output(0)]


@_prim("transpose")
def _transpose(ins, p, eqn):
    return [ops.transpose(ins[0], _i64(list(p["permutation"]))).output(0)]


@_prim("broadcast_in_dim")
def _broadcast_in_dim(ins, p, eqn):
    shape, dims = list(p["shape"]), list(p["broadcast_dimensions"])
    x = ins[0]
    # place the operand's axes at `dims` of a rank-len(shape) tensor of ones, then broadcast
    in_rank = len(x.get_partial_shape())
    if in_rank != len(shape):
        full = [1] * len(shape)
        xs = x.get_partial_shape()
        for i, d in enumerate(dims):
            full[d] = int(xs[i].get_length())
        x = ops.reshape(x, _i64(full), False).output(0)
    return [ops.broadcast(x, _i64(shape)).output(0)]


@_prim("concatenate")
def _concatenate(ins, p, eqn):
    return [ops.concat(list(ins), int(p["dimension"])).output(0)]


@_prim("slice")
def _slice(ins, p, eqn):
    start, limit = list(p["start_indices"]), list(p["limit_indices"])
    strides = list(p.get("strides") or [1] * len(start))
    return [ops.slice(ins[0], _i64(start), _i64(limit), _i64(strides), _i64(list(range(len(start))))).output(0)]


@_prim("select_n")
def _select_n(ins, p, eqn):
    if len(ins) != 3:
        raise JaxError("select_n with %d cases is not supported" % (len(ins) - 1))
    pred = ins[0]
    if pred.get_element_type().name != "boolean":
        pred = ops.convert(pred, "boolean").output(0)
    return [ops.select(pred, ins[2], ins[1]).output(0)]          # case 0 when the predicate is false


def _reduce(factory):
    return lambda ins, p, eqn: [factory(ins[0], _i64(list(p["axes"])), False).output(0)]


for _n, _f in (("reduce_sum", ops.reduce_sum), ("reduce_max", ops.reduce_max), ("reduce_min", ops.reduce_min), ("reduce_prod", ops.reduce_prod)):
    _T[_n] = _reduce(_f)


@_prim("argmax", "argmin")
def _argmax(ins, p, eqn):
    axis = int(list(p["axes"])[0])
    top = ops.topk(ins[0], _i64(1), axis, "max" if eqn.primitive.name == "argmax" else "min", "value", _ov_type(p["index_dtype"]))
    return [ops.squeeze(top.output(1), _i64([axis])).output(0)]


@_prim("dot_general")
def _dot_general(ins, p, eqn):
    (lc, rc), (lb, rb) = p["dimension_numbers"]
    a, b = ins
    ra, rb_rank = len(a.get_partial_shape()), len(b.get_partial_shape())
    lc, rc, lb, rb = list(lc), list(rc), list(lb), list(rb)
    if len(lc) != 1 or len(rc) != 1:
        raise JaxError("dot_general with %d contracting dimensions is not supported" % len(lc))
    # bring both operands to [batch..., free..., contract] / [batch..., contract, free...]
    a_free = [i for i in range(ra) if i not in lb and i not in lc]
    b_free = [i for i in range(rb_rank) if i not in rb and i not in rc]
    a_perm, b_perm = lb + a_free + lc, rb + rc + b_free
    if a_perm != list(range(ra)):
        a = ops.transpose(a, _i64(a_perm)).output(0)
    if b_perm != list(range(rb_rank)):
        b = ops.transpose(b, _i64(b_perm)).output(0)
    if len(a_free) > 1 or len(b_free) > 1:
        raise JaxError("dot_general with more than one free dimension per operand is not supported")
    y = ops.matmul(a, b, False, False).output(0)
    if not a_free and ra == len(lb) + 1 and b_free:
        pass                                                    # vector x matrix: MatMul already drops the missing axis
    return [y]


@_prim("conv_general_dilated")
def _conv(ins, p, eqn):
    dn = p["dimension_numbers"]
    lhs_spec, rhs_spec, out_spec = tuple(dn.lhs_spec), tuple(dn.rhs_spec), tuple(dn.out_spec)
    x, w = ins
    nd = len(lhs_spec) - 2
    if any(int(d) != 1 for d in (p.get("lhs_dilation") or [1] * nd)):
        raise JaxError("transposed convolution (lhs_dilation) is not supported")
    # lhs_spec = (batch, feature, spatial...) positions; bring to NC+spatial and OI+spatial
    if lhs_spec != tuple(range(nd + 2)):
        x = ops.transpose(x, _i64(list(lhs_spec))).output(0)
    if rhs_spec != tuple(range(nd + 2)):
        w = ops.transpose(w, _i64(list(rhs_spec))).output(0)
    pads = [tuple(int(v) for v in pr) for pr in p["padding"]]
    strides = [int(s) for s in p["window_strides"]]
    dil = [int(d) for d in (p.get("rhs_dilation") or [1] * nd)]
    groups = int(p.get("feature_group_count", 1))
    pb, pe = [a for a, _ in pads], [b for _, b in pads]
    if groups > 1:
        ws = [int(d.get_length()) for d in w.get_partial_shape()]
        w = ops.reshape(w, _i64([groups, ws[0] // groups] + ws[1:]), False).output(0)
        y = ops.group_convolution(x, w, strides, pb, pe, dil, "explicit").output(0)
    else:
        y = ops.convolution(x, w, strides, pb, pe, dil, "explicit").output(0)
    if out_spec != tuple(range(nd + 2)):
        inv = [0] * (nd + 2)
        for i, d in enumerate(out_spec):
            inv[d] = i
        y = ops.transpose(y, _i64(inv)).output(0)
    return [y]


@_prim("iota")
def _iota(ins, p, eqn):
    shape, dim = list(p["shape"]), int(p["dimension"])
    r = np.arange(shape[dim]).reshape([shape[dim] if i == dim else 1 for i in range(len(shape))])
    return [constant(np.broadcast_to(r, shape).astype(np.dtype(getattr(p["dtype"], "name", str(p["dtype"]))))).output(0)]


def supported_primitives() -> List[str]:
    return sorted(_T)


_INLINE = ("pjit", "closed_call", "core_call", "custom_jvp_call", "custom_vjp_call", "remat", "checkpoint", "jit")


def _inner_jaxpr(params: dict):
    for key in ("jaxpr", "call_jaxpr", "fun_jaxpr"):
        if key in params:
            return params[key]
    return None


def _walk(jaxpr, consts: Sequence[Any], inputs: Sequence[Output]) -> List[Output]:
    """``jaxpr``: an open jaxpr (``.invars`` ...); ``consts``: values of its constvars."""
    env: Dict[int, Output] = {}

    def read(v) -> Output:
        if hasattr(v, "val"):                                   # a literal
            val = np.asarray(v.val)
            aval = getattr(v, "aval", None)
            dt = np.dtype(getattr(getattr(aval, "dtype", None), "name", None) or val.dtype)
            return constant(val.astype(dt)).output(0)
        return env[id(v)]

    for v, c in zip(jaxpr.constvars, consts):
        env[id(v)] = constant(np.ascontiguousarray(np.asarray(c))).output(0)
    for v, o in zip(jaxpr.invars, inputs):
        env[id(v)] = o
    for eqn in jaxpr.eqns:
        name = eqn.primitive.name
        ins = [read(v) for v in eqn.invars]
        if name in _INLINE:
            inner = _inner_jaxpr(eqn.params)
            if inner is None:
                raise JaxError("%s without an inner jaxpr" % name)
            open_j = getattr(inner, "jaxpr", inner)
            outs = _walk(open_j, getattr(inner, "consts", ()), ins)
        else:
            fn = _T.get(name)
            if fn is None:
                raise JaxError("primitive %s is not supported" % name)
            outs = fn(ins, eqn.params, eqn)
        for v, o in zip(eqn.outvars, outs):
            env[id(v)] = o
    return [read(v) for v in jaxpr.outvars]


def convert(fn_or_jaxpr, example_input=None) -> Model:
    """A ``ClosedJaxpr`` (or anything with ``.jaxpr`` and ``.consts``), or a function plus ``example_input`` -> ``Model``."""
    closed = fn_or_jaxpr
    if not hasattr(closed, "jaxpr"):
        if example_input is None:
            raise JaxError("tracing a function needs example_input")
        import jax   # only needed on this path
        args = tuple(example_input) if isinstance(example_input, (list, tuple)) else (example_input,)
        closed = jax.make_jaxpr(fn_or_jaxpr)(*args)
    jaxpr = closed.jaxpr
    params = []
    for i, v in enumerate(jaxpr.invars):
        name = "arg_%d" % i
        p = parameter(PartialShape([int(d) for d in v.aval.shape]), _ov_type(v.aval.dtype), name)
        p.output(0).set_names({name})
        params.append(p)
    outs = _walk(jaxpr, closed.consts, [p.output(0) for p in params])
    results = []
    for i, o in enumerate(outs):
        if not o.get_names():
            o.set_names({"output_%d" % i})
        results.append(result(o))
    return Model(results, params, "jax_model")
