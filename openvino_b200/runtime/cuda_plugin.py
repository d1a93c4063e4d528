"""The "CUDA" device: compiles a ``Model`` into a program of device kernels for one B200.

Compilation (``CudaPlugin.compile_model``): clone -> common optimisations -> LLM fusions (RMS, RoPE, FullyConnected,
FullyConnectedCompressed, GLU, SDPA) -> ``GraphProgram``: one step per operation in topological order, constants
uploaded once (converted to the inference precision, weights of FullyConnected packed into the tile layout of the
tcgen05 GEMM). Execution: hot operations run on this framework's sm_100a kernels (GEMM with fused dequantisation /
bias / activation, RMSNorm, LayerNorm, dense attention, paged attention); the long tail of data-movement and
elementwise operations runs as tensor operations on the same stream; an operation without a device implementation is
evaluated by the native reference executor on the host (and reported by ``query_model`` as unsupported, so HETERO can
place it). Shape sub-graphs (ShapeOf -> Gather -> Concat ...) are computed on the host, so dynamic shapes cost no
device synchronisation.

Role in the reference: the intel_gpu plugin (src/plugins/intel_gpu/src/plugin/plugin.cpp:188-246 compile_model,
program_builder.cpp:129-178 one primitive per op, transformations_pipeline.cpp for the pass order, graph/network.cpp
for execution).
"""
from __future__ import annotations

import math
import os
import contextlib
import threading
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F

from .. import _ovcore as _c
from .. import properties as props
from .._graph import Model, Node, Output
from .._tensor import Tensor, torch_dtype
from .._types import Type
from ..ops import generic as G
from .plugin_config import ConfigOption, OptionVisibility, PluginConfig
from .core import CompiledModel, InferRequest, Plugin, ProfilingInfo, VariableState

_FLOAT = ("f32", "f16", "bf16", "f64")


def _tdtype(t: Type, precision: Optional[torch.dtype]) -> torch.dtype:
    if precision is not None and t.name == "f32":
        return precision
    return torch_dtype(t)


class Ctx:
    """What an operation implementation may use: the device, the compute precision, the kernel library."""

    def __init__(self, device: torch.device, precision: Optional[torch.dtype]):
        self.device, self.precision = device, precision
        self.on_gpu = device.type == "cuda"
        self.K = None
        if self.on_gpu:
            from ..ops import cuda as K
            K.lib()
            self.K = K
        self.cache: Dict[int, object] = {}      # per-node prepared state (packed weights)
        self.variables: Dict[str, torch.Tensor] = {}


# ---------------------------------------------------------------------------------------------- op table
_OPS: Dict[str, Callable] = {}


def op(*names):
    def deco(fn):
        for n in names:
            _OPS[n] = fn
        return fn
    return deco


@op("FunctionCall")
def _npuw_function_call(n, ins, ctx):
    """A folded block: the shared body runs as its own graph program (built once per device), with this block's weights."""
    from .npuw import function_of
    f = function_of(n)
    progs = f.__dict__.setdefault("_cuda_programs", {})
    key = (str(ctx.device), ctx.precision)
    prog = progs.get(key)
    if prog is None:
        prog = progs[key] = GraphProgram(f.body, ctx.device, ctx.precision)
        f.compiles += 1
    f.calls += 1
    prog.ctx.variables = ctx.variables
    return prog.run([t if isinstance(t, torch.Tensor) else torch.as_tensor(np.asarray(t)).to(ctx.device) for t in ins], None)


@op("Subgraph")
def _snippet_subgraph(n, ins, ctx):
    from ..snippets.runtime import run_subgraph
    return run_subgraph(n, ins, ctx, _OPS)


def _ints(t) -> List[int]:
    if isinstance(t, torch.Tensor):
        return [int(v) for v in t.reshape(-1).tolist()]
    return [int(v) for v in np.asarray(t).reshape(-1).tolist()]


def _scalar(t) -> float:
    return t.reshape(-1)[0].item()


def _same_device(ctx: Ctx, ins: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    """Host-side (shape) tensors meet device tensors: bring the small host ones over."""
    if not ctx.on_gpu or all(not t.is_cuda for t in ins) or all(t.is_cuda for t in ins):
        return list(ins)
    return [t if t.is_cuda else t.to(ctx.device, non_blocking=True) for t in ins]


def _dense(t: torch.Tensor) -> torch.Tensor:
    """``t`` laid out densely: the package's tile-transpose / strided-copy kernels for device tensors of the types they
    serve, the library's copy otherwise."""
    if t.is_contiguous():
        return t
    if G.enabled() and t.is_cuda and t.numel() > 0 and t.element_size() in (1, 2, 4, 8):
        try:
            return G.contiguous(t)
        except NotImplementedError:
            pass
    return t.contiguous()


def _native(*ts) -> bool:
    """Floating-point device tensors go to the package's own generic kernels (ops/generic.py); integer / boolean tensors
    and host-side values keep the torch expression."""
    return G.enabled() and all(G.supported(t) for t in ts)


_NATIVE_BINARY = {"Add": "add", "Subtract": "sub", "Multiply": "mul", "Maximum": "max", "Minimum": "min", "Power": "pow",
                  "SquaredDifference": "sqdiff"}


def _binary(fn, bool_out=False, name=None):
    native = _NATIVE_BINARY.get(name)

    def impl(n, ins, ctx):
        a, b = _same_device(ctx, ins[:2])
        if a.dtype != b.dtype:
            dt = torch.promote_types(a.dtype, b.dtype)
            a, b = a.to(dt), b.to(dt)
        if native and _native(a, b):
            try:
                return [G.binary(native, a, b)]
            except NotImplementedError:
                pass
        return [fn(a, b)]
    return impl


for _name, _fn in (("Add", torch.add), ("Subtract", torch.sub), ("Multiply", torch.mul), ("Maximum", torch.maximum), ("Minimum", torch.minimum),
                   ("Power", torch.pow), ("Equal", torch.eq), ("NotEqual", torch.ne), ("Less", torch.lt), ("LessEqual", torch.le),
                   ("Greater", torch.gt), ("GreaterEqual", torch.ge), ("LogicalAnd", torch.logical_and), ("LogicalOr", torch.logical_or),
                   ("LogicalXor", torch.logical_xor), ("FloorMod", torch.remainder), ("Mod", torch.fmod),
                   ("SquaredDifference", lambda a, b: (a - b) * (a - b))):
    _OPS[_name] = _binary(_fn, name=_name)


@op("Divide")
def _divide(n, ins, ctx):
    a, b = _same_device(ctx, ins[:2])
    if a.dtype.is_floating_point:
        if a.dtype == b.dtype and _native(a, b):
            try:
                return [G.binary("div", a, b)]
            except NotImplementedError:
                pass
        return [a / b]
    return [torch.div(a, b, rounding_mode="floor" if n.get_attribute("m_pythondiv") else "trunc")]


_NATIVE_UNARY = {"Abs": "abs", "Negative": "neg", "Exp": "exp", "Log": "log", "Sqrt": "sqrt", "Relu": "relu", "Sigmoid": "sigmoid", "Tanh": "tanh",
                 "Floor": "floor", "Ceiling": "ceil", "Sign": "sign", "Sin": "sin", "Cos": "cos", "Erf": "erf", "HSwish": "hswish",
                 "HSigmoid": "hsigmoid", "Mish": "mish", "SoftPlus": "softplus", "SoftSign": "softsign"}


def _unary(fn, name=None):
    native = _NATIVE_UNARY.get(name)

    def impl(n, ins, ctx):
        if native and _native(ins[0]):
            return [G.unary(native, ins[0])]
        return [fn(ins[0])]
    return impl


for _name, _fn in (("Abs", torch.abs), ("Negative", torch.neg), ("Exp", torch.exp), ("Log", torch.log), ("Sqrt", torch.sqrt), ("Relu", torch.relu),
                   ("Sigmoid", torch.sigmoid), ("Tanh", torch.tanh), ("Floor", torch.floor), ("Ceiling", torch.ceil), ("Sign", torch.sign),
                   ("Sin", torch.sin), ("Cos", torch.cos), ("Tan", torch.tan), ("Erf", torch.erf), ("LogicalNot", torch.logical_not),
                   ("HSwish", F.hardswish), ("HSigmoid", F.hardsigmoid), ("Mish", F.mish), ("SoftPlus", F.softplus), ("Asin", torch.asin),
                   ("Acos", torch.acos), ("Atan", torch.atan), ("Sinh", torch.sinh), ("Cosh", torch.cosh), ("Asinh", torch.asinh),
                   ("Acosh", torch.acosh), ("Atanh", torch.atanh), ("IsNaN", torch.isnan), ("IsFinite", torch.isfinite),
                   ("SoftSign", F.softsign), ("BitwiseNot", torch.bitwise_not)):
    _OPS[_name] = _unary(_fn, name=_name)


@op("Parameter", "Constant")
def _never(n, ins, ctx):
    raise RuntimeError("%s is bound before execution" % n.get_type_name())


@op("Result")
def _result(n, ins, ctx):
    return [ins[0]]


@op("Convert")
def _convert(n, ins, ctx):
    t = n.get_attribute("destination_type")
    if t.name == "boolean":
        return [ins[0] != 0]
    return [ins[0].to(_tdtype(t, ctx.precision))]


@op("ConvertLike")
def _convert_like(n, ins, ctx):
    return [ins[0].to(ins[1].dtype)]


@op("Swish")
def _swish(n, ins, ctx):
    b = _scalar(ins[1]) if len(ins) > 1 else 1.0
    if _native(ins[0]):
        return [G.unary("swish", ins[0], b)]
    if len(ins) > 1:
        return [ins[0] * torch.sigmoid(ins[0] * b)]
    return [F.silu(ins[0])]


@op("Gelu")
def _gelu(n, ins, ctx):
    mode = str(n.get_attributes().get("approximation_mode", "ERF")).lower()
    if _native(ins[0]):
        return [G.unary("gelu_tanh" if mode == "tanh" else "gelu_erf", ins[0])]
    return [F.gelu(ins[0], approximate="tanh" if mode == "tanh" else "none")]


@op("Elu")
def _elu(n, ins, ctx):
    if _native(ins[0]):
        return [G.unary("elu", ins[0], float(n.get_attribute("alpha")))]
    return [F.elu(ins[0], n.get_attribute("alpha"))]


@op("Clamp")
def _clamp(n, ins, ctx):
    if _native(ins[0]):
        return [G.unary("clamp", ins[0], float(n.get_attribute("min")), float(n.get_attribute("max")))]
    return [torch.clamp(ins[0], n.get_attribute("min"), n.get_attribute("max"))]


@op("PRelu")
def _prelu(n, ins, ctx):
    x, s = _same_device(ctx, ins)
    if s.dim() == 1 and x.dim() > 1 and s.numel() == x.shape[1] and s.numel() > 1:
        s = s.reshape([1, -1] + [1] * (x.dim() - 2))
    if x.dtype == s.dtype and _native(x, s):
        try:
            return [G.binary("prelu", x, s)]
        except NotImplementedError:
            pass
    return [torch.where(x >= 0, x, x * s)]


@op("Select")
def _select(n, ins, ctx):
    c, a, b = _same_device(ctx, ins)
    if a.dtype != b.dtype:
        dt = torch.promote_types(a.dtype, b.dtype)
        a, b = a.to(dt), b.to(dt)
    return [torch.where(c, a, b)]


@op("Round")
def _round(n, ins, ctx):
    if _native(ins[0]):
        return [G.unary("round_even" if n.get_attribute("mode") == "half_to_even" else "round_away", ins[0])]
    if n.get_attribute("mode") == "half_to_even":
        return [torch.round(ins[0])]
    x = ins[0]
    return [torch.sign(x) * torch.floor(torch.abs(x) + 0.5)]


# ---- shapes and data movement
@op("ShapeOf")
def _shape_of(n, ins, ctx):
    t = n.get_attributes().get("output_type", Type.i64)
    return [torch.tensor(list(ins[0].shape), dtype=torch_dtype(t))]            # host tensor


@op("Reshape")
def _reshape(n, ins, ctx):
    x = ins[0]
    pattern = _ints(ins[1])
    if n.get_attribute("special_zero"):
        pattern = [x.shape[i] if d == 0 else d for i, d in enumerate(pattern)]
    if not x.is_contiguous():
        try:
            return [x.view(pattern)]            # a permuted tensor whose new shape is still a view
        except RuntimeError:
            x = _dense(x)
    return [x.reshape(pattern)]


@op("Squeeze")
def _squeeze(n, ins, ctx):
    x = ins[0]
    if len(ins) == 1:
        return [x.squeeze()]
    axes = sorted({a % max(x.dim(), 1) for a in _ints(ins[1])}, reverse=True)
    for a in axes:
        if x.shape[a] == 1:
            x = x.squeeze(a)
    return [x]


@op("Unsqueeze")
def _unsqueeze(n, ins, ctx):
    x = ins[0]
    axes = _ints(ins[1])
    rank = x.dim() + len(axes)
    for a in sorted(a % rank for a in axes):
        x = x.unsqueeze(a)
    return [x]


@op("Transpose")
def _transpose(n, ins, ctx):
    order = _ints(ins[1])
    if not order:
        order = list(range(ins[0].dim() - 1, -1, -1))
    # a view: the consumer decides whether the permuted order is ever materialised (the attention and FullyConnected
    # operations read strided rows; element-wise, softmax and reduction kernels call _dense)
    return [ins[0].permute(order)]


@op("Concat")
def _concat(n, ins, ctx):
    ins = _same_device(ctx, ins)
    dt = ins[0].dtype
    ts = [t.to(dt) for t in ins]
    if ts[0].is_cuda and G.enabled() and ts[0].dim() > 0 and all(t.dim() == ts[0].dim() for t in ts):
        try:
            return [G.concat(ts, n.get_attribute("axis"))]
        except NotImplementedError:
            pass
    return [torch.cat(ts, dim=n.get_attribute("axis"))]


@op("Split")
def _split(n, ins, ctx):
    axis = _ints(ins[1])[0]
    return list(torch.chunk(ins[0], n.get_attribute("num_splits"), dim=axis))


@op("VariadicSplit")
def _vsplit(n, ins, ctx):
    axis = _ints(ins[1])[0]
    lengths = _ints(ins[2])
    total = ins[0].shape[axis]
    if -1 in lengths:
        lengths[lengths.index(-1)] = total - (sum(lengths) + 1)
    return list(torch.split(ins[0], lengths, dim=axis))


@op("Slice")
def _slice(n, ins, ctx):
    x = ins[0]
    start, stop, step = _ints(ins[1]), _ints(ins[2]), _ints(ins[3])
    axes = _ints(ins[4]) if len(ins) > 4 else list(range(len(start)))
    idx = [slice(None)] * x.dim()
    flips = []
    for s, e, st, a in zip(start, stop, step, axes):
        a %= x.dim()
        dim = x.shape[a]
        if st > 0:
            idx[a] = slice(max(min(s if s >= 0 else s + dim, dim), 0), max(min(e if e >= 0 else e + dim, dim), 0), st)
        else:
            # negative step: take the mirrored range, then flip
            s2 = min(s if s >= 0 else s + dim, dim - 1)
            e2 = max(e if e >= 0 else e + dim, -1)
            sel = list(range(s2, e2, st))
            idx[a] = torch.tensor(sel, dtype=torch.long, device=x.device)
    out = x
    for a, i in enumerate(idx):
        if isinstance(i, torch.Tensor):
            out = out.index_select(a, i)
        elif i != slice(None):
            out = out[(slice(None),) * a + (i,)]
    return [out]


@op("StridedSlice")
def _strided_slice(n, ins, ctx):
    x = ins[0]
    begin, end = _ints(ins[1]), _ints(ins[2])
    stride = _ints(ins[3]) if len(ins) > 3 else [1] * len(begin)
    at = n.get_attributes()
    pad = lambda m: list(m) + [0] * (len(begin) - len(m))
    bm, em, nm, sm, elm = pad(at["begin_mask"]), pad(at["end_mask"]), pad(at["new_axis_mask"]), pad(at["shrink_axis_mask"]), pad(at["ellipsis_mask"])
    idx = []
    for i in range(len(begin)):
        if elm[i]:
            idx.append(Ellipsis)
        elif nm[i]:
            idx.append(None)
        elif sm[i]:
            idx.append(begin[i])
        else:
            b = None if bm[i] else begin[i]
            e = None if em[i] else end[i]
            if stride[i] < 0:
                raise NotImplementedError("negative strides in StridedSlice")
            idx.append(slice(b, e, stride[i]))
    return [x[tuple(idx)]]


@op("Gather")
def _gather(n, ins, ctx):
    data, indices = ins[0], ins[1]
    axis = _ints(ins[2])[0] % max(data.dim(), 1)
    bd = n.get_attributes().get("batch_dims", 0)
    if indices.device != data.device:
        indices = indices.to(data.device)
    indices = indices.long()
    indices = torch.where(indices < 0, indices + data.shape[axis], indices)
    if bd == 0:
        out = data.index_select(axis, indices.reshape(-1))
        return [out.reshape(list(data.shape[:axis]) + list(indices.shape) + list(data.shape[axis + 1:]))]
    # batched gather: move to take_along_dim form
    bd %= indices.dim()
    idx_shape = list(indices.shape)
    view = idx_shape[:bd] + [1] * (axis - bd) + [int(np.prod(idx_shape[bd:]))] + [1] * (data.dim() - axis - 1)
    idx = indices.reshape(view).expand(list(data.shape[:axis]) + [view[axis]] + list(data.shape[axis + 1:]))
    out = torch.take_along_dim(data, idx, dim=axis)
    return [out.reshape(list(data.shape[:axis]) + idx_shape[bd:] + list(data.shape[axis + 1:]))]


@op("GatherElements")
def _gather_elements(n, ins, ctx):
    return [torch.gather(ins[0], n.get_attribute("axis"), ins[1].long().to(ins[0].device))]


@op("GatherND")
def _gather_nd(n, ins, ctx):
    data, idx = ins[0], ins[1].long().to(ins[0].device)
    if n.get_attributes().get("batch_dims", 0) != 0:
        raise NotImplementedError("GatherND with batch_dims")
    k = idx.shape[-1]
    return [data[tuple(idx[..., i] for i in range(k))]]


@op("ScatterNDUpdate")
def _scatter_nd(n, ins, ctx):
    data, idx, upd = ins[0].clone(), ins[1].long().to(ins[0].device), ins[2].to(ins[0].device)
    k = idx.shape[-1]
    key = tuple(idx[..., i] for i in range(k))
    red = n.get_attributes().get("reduction", "none")
    if red == "none":
        data[key] = upd.to(data.dtype)
    elif red == "sum":
        data.index_put_(key, upd.to(data.dtype), accumulate=True)
    else:
        raise NotImplementedError("ScatterNDUpdate reduction %s" % red)
    return [data]


@op("ScatterElementsUpdate")
def _scatter_elements(n, ins, ctx):
    data, idx, upd = ins[0], ins[1].long().to(ins[0].device), ins[2].to(ins[0].device)
    axis = _ints(ins[3])[0]
    red = n.get_attributes().get("reduction", "none")
    if red == "none":
        return [data.scatter(axis, idx, upd.to(data.dtype))]
    mode = {"sum": "sum", "prod": "prod", "min": "amin", "max": "amax", "mean": "mean"}[red]
    return [data.scatter_reduce(axis, idx, upd.to(data.dtype), reduce=mode, include_self=bool(n.get_attributes().get("use_init_val", True)))]


@op("ScatterUpdate")
def _scatter_update(n, ins, ctx):
    data, idx, upd = ins[0].clone(), ins[1].long().to(ins[0].device), ins[2]
    axis = _ints(ins[3])[0] % data.dim()
    flat = idx.reshape(-1)
    upd = upd.reshape(list(data.shape[:axis]) + [flat.numel()] + list(data.shape[axis + 1:]))
    data.index_copy_(axis, flat, upd.to(data.dtype))
    return [data]


@op("Broadcast")
def _broadcast(n, ins, ctx):
    x = ins[0]
    shape = _ints(ins[1])
    mode = n.get_attribute("mode")
    if mode == "bidirectional":
        full = [1] * (max(len(shape), x.dim()))
        xs = [1] * (len(full) - x.dim()) + list(x.shape)
        ss = [1] * (len(full) - len(shape)) + shape
        shape = [max(a, b) for a, b in zip(xs, ss)]
    elif mode == "explicit":
        axes = _ints(ins[2])
        view = [1] * len(shape)
        for a, d in zip(axes, x.shape):
            view[a] = d
        x = x.reshape(view)
    return [x.expand(shape)]


@op("Tile")
def _tile(n, ins, ctx):
    reps = _ints(ins[1])
    x = ins[0]
    if len(reps) < x.dim():
        reps = [1] * (x.dim() - len(reps)) + reps
    return [x.repeat(reps)]


@op("Range")
def _range(n, ins, ctx):
    a, b, s = (_scalar(t) for t in ins[:3])
    dt = torch_dtype(n.get_attributes().get("output_type", Type.i64))
    return [torch.arange(a, b, s, dtype=dt)]                                   # host tensor


@op("Pad")
def _pad(n, ins, ctx):
    x = ins[0]
    pb, pe = _ints(ins[1]), _ints(ins[2])
    mode = n.get_attribute("pad_mode")
    pads = []
    for b, e in zip(reversed(pb), reversed(pe)):
        pads += [b, e]
    if mode == "constant":
        v = _scalar(ins[3]) if len(ins) > 3 else 0
        return [F.pad(x, pads, value=v)]
    tmode = {"reflect": "reflect", "edge": "replicate", "symmetric": "reflect"}[mode]
    # torch pads at most the last 3 dims for non-constant modes: trim leading zero pairs
    while len(pads) > 2 and pads[-1] == 0 and pads[-2] == 0:
        pads = pads[:-2]
    lead = x.dim() - len(pads) // 2
    xx = x.reshape([-1] + list(x.shape[lead:])) if lead != 1 else x
    if lead == 0:
        xx = x.unsqueeze(0)
    out = F.pad(xx, pads, mode=tmode)
    return [out.reshape(list(x.shape[:lead]) + list(out.shape[1:])) if lead != 1 else out]


@op("Roll")
def _roll(n, ins, ctx):
    return [torch.roll(ins[0], _ints(ins[1]), _ints(ins[2]))]


@op("DepthToSpace")
def _d2s(n, ins, ctx):
    x, b = ins[0], n.get_attribute("block_size")
    if n.get_attribute("mode") == "depth_first":
        return [F.pixel_shuffle(x, b)]
    N, C, H, W = x.shape
    x = x.reshape(N, b, b, C // (b * b), H, W).permute(0, 3, 4, 1, 5, 2)
    return [x.reshape(N, C // (b * b), H * b, W * b)]


@op("OneHot")
def _one_hot(n, ins, ctx):
    idx, depth = ins[0].long(), _ints(ins[1])[0]
    on, off = ins[2].reshape(()), ins[3].reshape(())
    oh = F.one_hot(idx.clamp(0, depth - 1), depth).bool() & ((idx >= 0) & (idx < depth)).unsqueeze(-1)
    out = torch.where(oh, on.to(idx.device), off.to(idx.device))
    axis = n.get_attribute("axis")
    if axis != -1 and axis != out.dim() - 1:
        out = out.movedim(-1, axis)
    return [out]


@op("NonZero")
def _non_zero(n, ins, ctx):
    return [torch.nonzero(ins[0]).t().to(torch_dtype(n.get_attributes().get("output_type", Type.i64)))]


@op("CumSum")
def _cumsum(n, ins, ctx):
    x = ins[0]
    axis = _ints(ins[1])[0] if len(ins) > 1 else 0
    at = n.get_attributes()
    if at["reverse"]:
        x = x.flip(axis)
    out = torch.cumsum(x, axis)
    if at["exclusive"]:
        out = out - x
    return [out.flip(axis) if at["reverse"] else out]


@op("TopK")
def _topk(n, ins, ctx):
    at = n.get_attributes()
    k = _ints(ins[1])[0]
    v, i = torch.topk(ins[0], k, dim=at["axis"], largest=at["mode"] == "max", sorted=True)
    if at["sort"] == "index":
        order = torch.argsort(i, dim=at["axis"])
        v, i = torch.gather(v, at["axis"], order), torch.gather(i, at["axis"], order)
    return [v, i.to(torch_dtype(at["index_element_type"]))]


_NATIVE_REDUCE = {"ReduceSum": "sum", "ReduceMean": "mean", "ReduceMax": "max", "ReduceMin": "min", "ReduceProd": "prod", "ReduceL1": "l1",
                  "ReduceL2": "l2"}


def _reduce(fn, name=None):
    native = _NATIVE_REDUCE.get(name)

    def impl(n, ins, ctx):
        axes = sorted({a % max(ins[0].dim(), 1) for a in _ints(ins[1])})
        keep = n.get_attribute("keep_dims")
        x = ins[0]
        if not axes:
            return [x]
        if native and _native(x):
            return [G.reduce(native, x, axes, bool(keep))]
        return [fn(x, axes, keep)]
    return impl


def _prod(x, axes, keep):
    for a in reversed(axes):
        x = torch.prod(x, a, keepdim=keep)
    return x


for _name, _fn in (("ReduceSum", lambda x, a, k: torch.sum(x, a, keepdim=k)), ("ReduceMean", lambda x, a, k: torch.mean(x, a, keepdim=k)),
                   ("ReduceMax", lambda x, a, k: torch.amax(x, a, keepdim=k)), ("ReduceMin", lambda x, a, k: torch.amin(x, a, keepdim=k)),
                   ("ReduceProd", _prod), ("ReduceL1", lambda x, a, k: torch.sum(torch.abs(x), a, keepdim=k)),
                   ("ReduceL2", lambda x, a, k: torch.sqrt(torch.sum(x * x, a, keepdim=k))),
                   ("ReduceLogicalAnd", lambda x, a, k: torch.all(x, a[0], keepdim=k) if len(a) == 1 else torch.amin(x.to(torch.uint8), a, keepdim=k).bool()),
                   ("ReduceLogicalOr", lambda x, a, k: torch.any(x, a[0], keepdim=k) if len(a) == 1 else torch.amax(x.to(torch.uint8), a, keepdim=k).bool())):
    _OPS[_name] = _reduce(_fn, name=_name)


# ---- neural network layers
@op("Softmax")
def _softmax(n, ins, ctx):
    if _native(ins[0]) and ins[0].dim() > 0:
        return [G.softmax(ins[0], n.get_attribute("axis"))]
    return [torch.softmax(ins[0], n.get_attribute("axis"))]


@op("LogSoftmax")
def _log_softmax(n, ins, ctx):
    if _native(ins[0]) and ins[0].dim() > 0:
        return [G.softmax(ins[0], n.get_attribute("axis"), log=True)]
    return [torch.log_softmax(ins[0], n.get_attribute("axis"))]


@op("MatMul")
def _matmul(n, ins, ctx):
    a, b = _same_device(ctx, ins)
    at = n.get_attributes()
    if at["transpose_a"] and a.dim() > 1:
        a = a.transpose(-1, -2)
    if at["transpose_b"] and b.dim() > 1:
        b = b.transpose(-1, -2)
    if a.dtype != b.dtype:
        b = b.to(a.dtype)
    return [torch.matmul(a, b)]


def _auto_pad(x, kernel, strides, dilations, pb, pe, auto_pad):
    if auto_pad in ("explicit", "notset"):
        return pb, pe
    if auto_pad == "valid":
        return [0] * len(kernel), [0] * len(kernel)
    pb2, pe2 = [], []
    for i, k in enumerate(kernel):
        size = x.shape[2 + i]
        out = -(-size // strides[i])
        total = max((out - 1) * strides[i] + (k - 1) * dilations[i] + 1 - size, 0)
        lo, hi = total // 2, total - total // 2
        if auto_pad == "same_lower":
            lo, hi = hi, lo
        pb2.append(lo)
        pe2.append(hi)
    return pb2, pe2


def _conv(x, w, at, groups):
    nd = x.dim() - 2
    kernel = list(w.shape[2:])
    pb, pe = _auto_pad(x, kernel, at["strides"], at["dilations"], at["pads_begin"], at["pads_end"], at["auto_pad"])
    if list(pb) != list(pe):
        pads = []
        for b, e in zip(reversed(pb), reversed(pe)):
            pads += [b, e]
        x = F.pad(x, pads)
        pb = [0] * nd
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
    return fn(x, w.to(x.dtype), None, at["strides"], list(pb), at["dilations"], groups)


@op("Convolution")
def _convolution(n, ins, ctx):
    x, w = _same_device(ctx, ins)
    # 16-bit 2-D convolutions with constant filters run as im2col + the tcgen05 GEMM (filters packed once)
    if ctx.K is not None and ctx.on_gpu and x.is_cuda and x.dim() == 4 and x.dtype in (torch.float16, torch.bfloat16) and x.shape[0] * x.shape[2] * x.shape[3] > 0:
        st = ctx.cache.get(id(n))
        if st is None:
            st = {"packed": None}
            src = n.input_value(1).get_node()
            if src.get_type_name() == "Convert":
                src = src.input_value(0).get_node()
            if src.get_type_name() == "Constant":
                st["packed"] = ctx.K.pack_conv_weight(w.to(x.dtype))
            ctx.cache[id(n)] = st
        if st["packed"] is not None:
            at = n.get_attributes()
            kernel = list(w.shape[2:])
            pb, pe = _auto_pad(x, kernel, at["strides"], at["dilations"], at["pads_begin"], at["pads_end"], at["auto_pad"])
            return [ctx.K.conv2d(x, st["packed"], kernel, at["strides"], pb, pe, at["dilations"])]
    return [_conv(x, w, n.get_attributes(), 1)]


@op("GroupConvolution")
def _group_convolution(n, ins, ctx):
    x, w = _same_device(ctx, ins)
    g = w.shape[0]
    return [_conv(x, w.reshape([g * w.shape[1]] + list(w.shape[2:])), n.get_attributes(), g)]


def _pool_out_hw(x, kernel, strides, dil, pb, pe, ceil):
    """Output extent of a pooling window walk: floor or ceil rounding; with ceil the last window must start inside the
    input or its left padding (the rule of the reference's shape inference, src/core/shape_inference/include/pooling_shape_inference_util.hpp)."""
    out = []
    for i in range(2):
        span = x.shape[2 + i] + pb[i] + pe[i] - (dil[i] * (kernel[i] - 1) + 1)
        o = (-(-span // strides[i]) if ceil else span // strides[i]) + 1
        if ceil and (o - 1) * strides[i] >= x.shape[2 + i] + pb[i]:
            o -= 1
        out.append(max(o, 0))
    return out


@op("MaxPool")
def _max_pool(n, ins, ctx):
    x, at = ins[0], n.get_attributes()
    nd = x.dim() - 2
    dil = at.get("dilations") or [1] * nd
    pb, pe = _auto_pad(x, at["kernel"], at["strides"], dil, at["pads_begin"], at["pads_end"], at["auto_pad"])
    ceil = at["rounding_type"] == "ceil"
    if nd == 2 and n.get_output_size() == 1 and _native(x):
        return [G.pool2d(x, at["kernel"], at["strides"], pb, pe, dil, _pool_out_hw(x, at["kernel"], at["strides"], dil, pb, pe, ceil), True, False)]
    if list(pb) != list(pe):
        pads = []
        for b, e in zip(reversed(pb), reversed(pe)):
            pads += [b, e]
        x = F.pad(x, pads, value=float("-inf"))
        pb = [0] * nd
    fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nd]
    if n.get_output_size() > 1:
        v, i = fn(x, at["kernel"], at["strides"], list(pb), dil, ceil, return_indices=True)
        return [v, i.to(torch_dtype(at.get("index_element_type", Type.i64)))]
    return [fn(x, at["kernel"], at["strides"], list(pb), dil, ceil)]


@op("AvgPool")
def _avg_pool(n, ins, ctx):
    x, at = ins[0], n.get_attributes()
    nd = x.dim() - 2
    pb, pe = _auto_pad(x, at["kernel"], at["strides"], [1] * nd, at["pads_begin"], at["pads_end"], at["auto_pad"])
    ceil = at["rounding_type"] == "ceil"
    if nd == 2 and _native(x):
        return [G.pool2d(x, at["kernel"], at["strides"], pb, pe, [1, 1], _pool_out_hw(x, at["kernel"], at["strides"], [1, 1], pb, pe, ceil), False,
                         bool(at["exclude-pad"]))]
    fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd]
    if list(pb) != list(pe):
        raise NotImplementedError("AvgPool with asymmetric padding")
    return [fn(x, at["kernel"], at["strides"], list(pb), ceil, not at["exclude-pad"])]


@op("AdaptiveAvgPool")
def _adaptive_avg(n, ins, ctx):
    size = _ints(ins[1])
    fn = {1: F.adaptive_avg_pool1d, 2: F.adaptive_avg_pool2d, 3: F.adaptive_avg_pool3d}[len(size)]
    return [fn(ins[0], size)]


@op("BatchNormInference")
def _bn(n, ins, ctx):
    x, g, b, m, v = _same_device(ctx, ins)
    return [F.batch_norm(x, m.to(x.dtype), v.to(x.dtype), g.to(x.dtype), b.to(x.dtype), False, 0.0, n.get_attribute("epsilon"))]


@op("MVN")
def _mvn(n, ins, ctx):
    x = ins[0]
    axes = [a % x.dim() for a in _ints(ins[1])]
    at = n.get_attributes()
    mean = x.mean(axes, keepdim=True)
    xc = x - mean
    if not at["normalize_variance"]:
        return [xc]
    var = (xc * xc).mean(axes, keepdim=True)
    if at["eps_mode"] == "inside_sqrt":
        return [xc * torch.rsqrt(var + at["eps"])]
    return [xc / (torch.sqrt(var) + at["eps"])]


@op("NormalizeL2")
def _l2(n, ins, ctx):
    x = ins[0]
    axes = [a % x.dim() for a in _ints(ins[1])]
    at = n.get_attributes()
    s = (x * x).sum(axes, keepdim=True) if axes else x * x
    s = s + at["eps"] if at["eps_mode"] == "add" else torch.clamp(s, min=at["eps"])
    return [x * torch.rsqrt(s)]


@op("GroupNormalization")
def _gn(n, ins, ctx):
    x, g, b = _same_device(ctx, ins)
    return [F.group_norm(x, n.get_attribute("num_groups"), g.to(x.dtype), b.to(x.dtype), n.get_attribute("epsilon"))]


@op("RMS", "RMSNorm")
def _rms(n, ins, ctx):
    x = ins[0]
    gamma = ins[1].to(x.device) if len(ins) > 1 else None
    eps = n.get_attribute("epsilon")
    if ctx.K is not None and x.dtype == torch.bfloat16 and gamma is not None and gamma.dim() == 1 and x.shape[-1] == gamma.numel() and x.shape[-1] % 8 == 0:
        x2 = _dense(x.reshape(-1, x.shape[-1]))
        return [ctx.K.rmsnorm(x2, gamma.to(torch.bfloat16).contiguous(), eps).reshape(x.shape)]
    xf = x.float()
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    if gamma is not None:
        y = y * gamma.float()
    return [y.to(x.dtype)]


@op("FakeQuantize")
def _fq(n, ins, ctx):
    x, il, ih, ol, oh = _same_device(ctx, ins)
    levels = n.get_attribute("levels")
    xc = torch.minimum(torch.maximum(x, il), ih)
    q = torch.round((xc - il) / (ih - il) * (levels - 1))
    return [q / (levels - 1) * (oh - ol) + ol]


@op("ScaledDotProductAttention")
def _sdpa(n, ins, ctx):
    ins = _same_device(ctx, ins)
    q, k, v = ins[:3]
    causal = n.get_attribute("causal")
    mask = ins[3] if len(ins) > 3 and ins[3].numel() > 0 and not (ins[3].dim() == 0 and not causal and len(ins) > 4) else None
    scale = _scalar(ins[4]) if len(ins) > 4 else None
    if mask is not None and mask.dim() == 0:
        mask = None
    if mask is not None and mask.dtype != torch.bool and mask.dtype != q.dtype:
        mask = mask.to(q.dtype)
    K = ctx.K
    if (K is not None and mask is None and q.dim() == 4 and q.dtype in (torch.float16, torch.bfloat16) and q.shape[-1] in (64, 128)
            and q.shape == k.shape == v.shape and len(ins) <= 5):
        B, H, S, D = q.shape
        # kernel layout: [B*S, H*D] rows with head h at column h*D
        pack = lambda t: _dense(t.transpose(1, 2)).reshape(B * S, H * D)
        out = K.sdpa_dense(pack(q), pack(k), pack(v), B, S, H, D, H * D, scale=scale, causal=bool(causal))
        return [out.reshape(B, S, H, D).transpose(1, 2)]
    return [F.scaled_dot_product_attention(q, k.to(q.dtype), v.to(q.dtype), attn_mask=None if causal else mask, is_causal=bool(causal) and mask is None, scale=scale)]


def _prepare_fc(n: Node, ins, ctx: Ctx):
    """Pack the constant weight of a FullyConnected(-Compressed) once: tile layout for the tcgen05 GEMM."""
    st = ctx.cache.get(id(n))
    if st is not None:
        return st
    K = ctx.K
    t = n.get_type_name()
    st = {"packed": None, "act": n.get_rt_info().get("fused_activation")}
    if st["act"] is not None:
        st["act"] = str(st["act"])
    w_node = n.input_value(1).get_node()
    if K is not None and w_node.get_type_name() == "Constant":
        bias = None
        bn = n.input_value(2).get_node() if n.get_input_size() > 2 else None
        if bn is not None and bn.get_type_name() == "Constant" and bn.get_output_partial_shape(0).is_static and int(np.prod(bn.get_output_shape(0) or [1])) > 0:
            bias = ins[2].reshape(-1)
        if t == "FullyConnected" and ins[1].dtype in (torch.float16, torch.bfloat16) and ins[1].dim() == 2 and ins[1].shape[1] % 64 == 0:
            st["packed"] = K.PackedWeight.from_dense(ins[1].contiguous(), bias.to(ins[1].dtype) if bias is not None and bias.numel() == ins[1].shape[0] else None)
        elif t == "FullyConnectedCompressed":
            wt = w_node.get_tensor_view()
            sc_node = n.input_value(3).get_node()
            zp_node = n.input_value(4).get_node() if n.get_input_size() > 4 else None
            et = wt.element_type.name
            N = wt.shape[0]
            Kd = int(np.prod(wt.shape[1:]))
            scales = torch.from_numpy(np.ascontiguousarray(sc_node.get_tensor_view().to_float32())).reshape(N, -1)
            G = scales.shape[1]
            if et in ("u4", "u8") and Kd % 64 == 0 and (Kd // G) % 64 == 0:
                dev = ctx.device
                wq = torch.from_numpy(np.ascontiguousarray(wt.data).reshape(-1).view(np.uint8).copy()).to(dev)
                zp = None
                if zp_node is not None and zp_node.get_type_name() == "Constant" and zp_node.get_tensor_view().size > 0:
                    zp = torch.from_numpy(np.ascontiguousarray(zp_node.get_tensor_view().to_float32())).reshape(-1)
                    zp = (zp.expand(N * G) if zp.numel() == 1 else zp).reshape(N, G).to(torch.uint8).to(dev)
                b16 = bias.to(torch.bfloat16) if bias is not None and bias.numel() == N else None
                sc16 = scales.to(torch.float16).contiguous().to(dev)
                if et == "u4":
                    st["packed"] = K.PackedWeight.from_ir_u4(wq.reshape(-1), sc16, zp.contiguous() if zp is not None else None, N, Kd, Kd // G,
                                                             zp_is_u8=True, bias=b16)
                else:
                    st["packed"] = K.PackedWeight.from_ir_u8(wq.reshape(N, Kd), sc16, zp, N, Kd, Kd // G, bias=b16)
    ctx.cache[id(n)] = st
    return st


def _dequant_weight(n: Node, ins, ctx: Ctx) -> torch.Tensor:
    st = ctx.cache.setdefault(("deq", id(n)), {})
    if "w" not in st:
        w_node = n.input_value(1).get_node()
        wf = torch.from_numpy(np.ascontiguousarray(w_node.get_tensor_view().to_float32())) if w_node.get_type_name() == "Constant" else ins[1].float().cpu()
        N = wf.shape[0]
        wf = wf.reshape(N, -1)
        s = ins[3].float().cpu().reshape(N, -1)
        G = s.shape[1]
        z = ins[4].float().cpu() if len(ins) > 4 and ins[4].numel() > 0 else torch.zeros(1)
        z = z.reshape(-1)
        z = (z.expand(N * G) if z.numel() == 1 else z).reshape(N, G)
        w = ((wf.reshape(N, G, -1) - z.unsqueeze(-1)) * s.unsqueeze(-1)).reshape(N, -1)
        st["w"] = w.to(ctx.device)
    return st["w"]


@op("FullyConnected", "FullyConnectedCompressed")
def _fc(n, ins, ctx):
    x = ins[0]
    if ctx.on_gpu and not x.is_cuda:
        x = x.to(ctx.device)
    st = _prepare_fc(n, ins, ctx)
    pw = st["packed"]
    has_bias = len(ins) > 2 and ins[2].numel() > 0 and ins[2].dim() > 0
    if pw is not None and x.dtype in (torch.float16, torch.bfloat16) and (pw.mode != ctx.K.W_F16) == (x.dtype == torch.bfloat16):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = _dense(x2)
        act = st.get("act")
        fused = act is not None and not (has_bias and pw.bias is None)      # the epilogue order is bias, then activation
        out = ctx.K.gemm(x2, pw, act=_GEMM_ACTS[act] if fused else 0)
        if has_bias and pw.bias is None:
            out = out + ins[2].to(out.device, out.dtype)
        if act is not None and not fused:
            out = _TORCH_ACTS[act](out)
        return [out.reshape(list(x.shape[:-1]) + [pw.N])]
    w = _dequant_weight(n, ins, ctx) if n.get_type_name() == "FullyConnectedCompressed" else ins[1]
    out = torch.matmul(x, w.to(x.device, x.dtype).t())
    if has_bias:
        out = out + ins[2].to(out.device, out.dtype)
    if st.get("act") is not None:
        out = _TORCH_ACTS[st["act"]](out)
    return [out]


_GEMM_ACTS = {"gelu_erf": 1, "relu": 2, "silu": 3, "gelu_tanh": 5}
_TORCH_ACTS = {"gelu_erf": F.gelu, "relu": F.relu, "silu": F.silu, "gelu_tanh": lambda t: F.gelu(t, approximate="tanh")}


@op("LayerNormFused")
def _layer_norm_fused(n, ins, ctx):
    x, g, b = ins[0], ins[1], ins[2]
    eps = float(n.get_attribute("eps"))
    if ctx.K is not None and x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and x.shape[-1] % 8 == 0:
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = _dense(x2)
        out = ctx.K.layernorm(x2, g.to(x.device, x.dtype).contiguous(), b.to(x.device, x.dtype).contiguous(), eps)
        return [out.reshape(x.shape)]
    return [F.layer_norm(x, [x.shape[-1]], g.to(x.device, x.dtype), b.to(x.device, x.dtype), eps)]


@op("AllReduce")
def _all_reduce(n, ins, ctx):
    x = ins[0]
    dist = torch.distributed
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        if ctx.on_gpu and x.is_cuda and x.dtype in (torch.float32, torch.float16, torch.bfloat16) and os.environ.get("OVB_GRAPH_TP_NCCL", "0") != "1":
            # the package's own peer-memory all-reduce (in-switch reduction when the heap has a multicast mapping)
            return [_graph_comm(ctx).all_reduce_any(x.contiguous())]
        x = x.contiguous().clone() if not ctx.on_gpu else x.contiguous()
        dist.all_reduce(x)
    return [x]


_GRAPH_COMMS: Dict[int, object] = {}


def _graph_comm(ctx: Ctx):
    """One peer-memory communicator per device for the AllReduce nodes of tensor-parallel graphs (created on first use by
    all ranks together; sized by OVB_GRAPH_TP_HEAP_MB, 256 MB by default)."""
    key = ctx.device.index or 0
    c = _GRAPH_COMMS.get(key)
    if c is None:
        from ..parallel.comm import PeerCommunicator
        dist = torch.distributed
        mb = int(os.environ.get("OVB_GRAPH_TP_HEAP_MB", "256"))
        c = PeerCommunicator(dist.get_rank(), dist.get_world_size(), ctx.device)
        c.setup(hidden=1024, max_tokens=1024, num_layers=1, tensor_bytes=mb << 20)
        _GRAPH_COMMS[key] = c
    return c


@op("Einsum")
def _einsum(n, ins, ctx):
    return [torch.einsum(n.get_attribute("equation"), *_same_device(ctx, ins))]


@op("HardSigmoid")
def _hard_sigmoid(n, ins, ctx):
    return [torch.clamp(ins[0] * _scalar(ins[1]) + _scalar(ins[2]), 0.0, 1.0)]


@op("Interpolate")
def _interpolate(n, ins, ctx):
    at = n.get_attributes()
    x = ins[0]
    axes = _ints(ins[2]) if len(ins) > 2 else list(range(x.dim()))
    if sorted(a % x.dim() for a in axes) != list(range(2, x.dim())) or any(at["pads_begin"]) or any(at["pads_end"]):
        raise NotImplementedError("Interpolate over non-spatial axes or with pads")
    order = np.argsort([a % x.dim() for a in axes])
    mode, ct = at["mode"], at["coordinate_transformation_mode"]
    tmode = {"nearest": "nearest", "linear": "bilinear", "linear_onnx": "bilinear", "cubic": "bicubic"}.get(mode)
    supported = (mode == "nearest" and ct == "asymmetric" and at["nearest_mode"] == "floor") or \
                (mode in ("linear", "linear_onnx", "cubic") and ct in ("pytorch_half_pixel", "half_pixel", "align_corners"))
    if tmode is None or not supported or x.dim() != 4:
        raise NotImplementedError("Interpolate mode %s / %s" % (mode, ct))
    kw = {} if mode == "nearest" else {"align_corners": ct == "align_corners"}
    if at["shape_calculation_mode"] == "sizes":
        sizes = _ints(ins[1])
        return [F.interpolate(x, size=[sizes[i] for i in order], mode=tmode, **kw)]
    scales = [float(v) for v in ins[1].reshape(-1).tolist()]
    return [F.interpolate(x, scale_factor=[scales[i] for i in order], mode=tmode, **kw)]


@op("GLU")
def _glu(n, ins, ctx):
    at = n.get_attributes()
    x = ins[0]
    a, b = torch.split(x, [at["split_lengths"], x.shape[at["axis"]] - at["split_lengths"]], dim=at["axis"])
    gate, up = (a, b) if at["split_to_glu_idx"] == 0 else (b, a)
    act = {"Swish": F.silu, "Gelu": F.gelu, "Gelu_Tanh": lambda t: F.gelu(t, approximate="tanh")}[at["glu_type"]]
    return [act(gate) * up]


@op("RoPE")
def _rope(n, ins, ctx):
    """Half-rotate and interleaved forms over [B, H, L, S] (or [B, L, H, S] with the transposition flags), partial rotary
    widths, and the fused-QKV forms of Qwen ([B, L, W], tables [1, positions, 1, S]) and ChatGLM ([L, B, W], cache
    [L, B or 1, 1, rot / 2, 2]). Same arithmetic as the reference evaluation (csrc/core/eval_llm.cpp)."""
    at = n.get_attributes()
    if at.get("support_2d_rope") or at.get("support_3d_rope") or at.get("is_ltx_video") or at.get("use_rope_cache"):
        return NotImplemented
    x, cos, sin = _same_device(ctx, ins[:3])
    pos = ins[3].to(x.device).long() if len(ins) > 3 and ins[3].numel() > 0 else None
    H, S = at.get("head_cnt", 0), at.get("head_size", 0)
    if at.get("is_chatglm"):
        L, B = x.shape[0], x.shape[1]
        rot = at.get("rotary_ndims") or S
        xh = x[..., at.get("slice_start", 0):at.get("slice_start", 0) + H * S].reshape(L, B, H, S)
        pairs = xh[..., :rot].reshape(L, B, H, rot // 2, 2).float()
        cache = cos[:L].float()                                              # [L, B or 1, 1, rot / 2, 2]
        c, s_ = cache[..., 0], cache[..., 1]
        out = torch.stack([pairs[..., 0] * c - pairs[..., 1] * s_, pairs[..., 1] * c + pairs[..., 0] * s_], -1).reshape(L, B, H, rot)
        return [torch.cat([out.to(x.dtype), xh[..., rot:]], -1)]
    if at.get("is_qwen"):
        B, L = x.shape[0], x.shape[1]
        xh = x[..., at.get("slice_start", 0):at.get("slice_start", 0) + H * S].reshape(B, L, H, S).float()
        c2, s2 = cos.reshape(-1, S).float(), sin.reshape(-1, S).float()
        rows = torch.arange(c2.shape[0] - L, c2.shape[0], device=x.device) if c2.shape[0] >= L else torch.arange(L, device=x.device).clamp(max=c2.shape[0] - 1)
        if pos is not None:
            rows = pos.reshape(-1, L) if pos.numel() == B * L else pos.reshape(1, -1)
            c4, s4 = c2[rows].unsqueeze(2), s2[rows].unsqueeze(2)          # [B or 1, L, 1, S]
        else:
            c4, s4 = c2[rows].reshape(1, L, 1, S), s2[rows].reshape(1, L, 1, S)
        half = S // 2
        rotd = torch.cat([-xh[..., half:], xh[..., :half]], -1)
        return [(xh * c4 + rotd * s4).to(x.dtype)]
    if x.dim() != 4 or at.get("slice_stop", 0) > at.get("slice_start", 0):
        return NotImplemented
    it, ot = bool(at.get("input_trans0213")), bool(at.get("output_trans0213"))
    xb = x.transpose(1, 2) if it else x                                      # [B, H, L, S]
    B, Hh, L, D = xb.shape
    nd = at.get("rotary_ndims") or D
    half = nd // 2
    # tables: last axis nd or nd / 2 wide, the axis before it (if any) runs over positions, an optional leading batch
    cw = cos.shape[-1]
    crow = cos.shape[-2] if cos.dim() >= 2 else 1
    c3, s3 = cos.reshape(-1, crow, cw).float(), sin.reshape(-1, crow, cw).float()
    rows = torch.arange(L, device=x.device)
    if pos is not None:
        rows = pos.reshape(1, L) if pos.numel() == L else pos.reshape(-1, L)
    rows = torch.zeros_like(rows) if crow == 1 else rows.clamp(max=crow - 1)
    if rows.dim() == 1:
        ct, st_ = c3[:, rows], s3[:, rows]                                  # [cb, L, cw]
    else:
        bi = torch.arange(rows.shape[0], device=x.device).clamp(max=c3.shape[0] - 1).unsqueeze(1)
        ct, st_ = c3[bi, rows], s3[bi, rows]                                # [B or 1, L, cw]
    ct, st_ = ct.unsqueeze(1), st_.unsqueeze(1)                             # [., 1, L, cw]
    xr = xb[..., :nd].float()
    if at.get("is_interleaved"):
        x0, x1 = xr[..., 0::2], xr[..., 1::2]
        cc, ss = (ct[..., 0::2], st_[..., 0::2]) if cw == nd else (ct, st_)
        out = torch.stack([x0 * cc - x1 * ss, x1 * cc + x0 * ss], -1).reshape(B, Hh, L, nd)
    else:
        x0, x1 = xr[..., :half], xr[..., half:]
        c0, s0 = ct[..., :half], st_[..., :half]
        c1, s1 = (ct[..., half:nd], st_[..., half:nd]) if cw == nd else (c0, s0)
        out = torch.cat([x0 * c0 - x1 * s0, x1 * c1 + x0 * s1], -1)
    out = out.to(x.dtype)
    if nd != D:
        out = torch.cat([out, xb[..., nd:]], -1)
    return [out.transpose(1, 2) if ot else out]


@op("SelectiveSSM")
def _selective_ssm(n, ins, ctx):
    """A [H], dt [B, L, H], B [B, L, G, S], x [B, L, H, P], C [B, L, G, S], state [B, H, P, S] -> y, new state."""
    if ctx.K is None or ins[2].shape[-1] > 256:
        return NotImplemented
    A, dt, Bm, x, Cm, state = _same_device(ctx, ins)
    y, new_state = ctx.K.selective_ssm(A, dt, Bm, x, Cm, state)
    return [y.to(x.dtype), new_state.to(state.dtype)]


@op("GatedDeltaNet")
def _gated_delta_net(n, ins, ctx):
    """query / key [B, L, Hq, Dk], value [B, L, Hv, Dv], state [B, Hv, Dk, Dv], gate / beta [B, L, Hv] -> y, new state."""
    if ctx.K is None or ins[0].shape[-1] > 256:
        return NotImplemented
    q, k, v, state, gate, beta = _same_device(ctx, ins)
    at = n.get_attributes()
    qf, kf = q.float(), k.float()
    scale = float(q.shape[-1]) ** -0.5
    if at.get("fuse_qk_l2norm"):
        qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + float(at.get("q_l2_norm_eps", 1e-6))) * scale
        kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + float(at.get("k_l2_norm_eps", 1e-6)))
    else:
        qf = qf * scale
    y, new_state = ctx.K.gated_delta_rule(qf, kf, v, gate, beta, state)
    return [y.to(v.dtype), new_state.to(state.dtype)]


def _paged_segments(begins, blocks, bbeg, past, interval):
    """Host walk of the paged-state bookkeeping: for every sequence the block to read, then (token begin, token end, block
    to write) per stretch of tokens up to the next multiple of the cache interval."""
    plan = []
    for s in range(len(begins) - 1):
        slots = blocks[bbeg[s]:bbeg[s + 1]]
        tb, te, pst, iv = begins[s], begins[s + 1], past[s], interval[s]
        if len(slots) == 0:
            raise RuntimeError("a sequence needs at least one state block")
        to_boundary = (iv - pst % iv if pst % iv else iv) if iv > 0 else te - tb
        segs, slot, tok = [], 1, tb
        while tok < te:
            end = min(tok + to_boundary, te)
            if slot >= len(slots):
                raise RuntimeError("block slot %d is beyond the %d slots of the sequence" % (slot, len(slots)))
            segs.append((tok, end, int(slots[slot])))
            slot += 1
            tok = end
            to_boundary = iv if iv > 0 else te - tb
        plan.append((int(slots[0]), segs))
    return plan


def _host_ints(t):
    return [int(v) for v in t.detach().to("cpu").reshape(-1).tolist()]


@op("PagedSelectiveSSM")
def _paged_selective_ssm(n, ins, ctx):
    """Token-major inputs (dt [T, H], B / C [T, G, S], x [T, H, P]) and a state table [blocks, H, P, S] updated in place:
    the scan kernel runs once per stretch between cache-interval boundaries."""
    if ctx.K is None or ins[2].shape[-1] > 256 or not ins[5].is_cuda:
        return NotImplemented
    A, dt, Bm, x, Cm, table = _same_device(ctx, ins[:6])
    plan = _paged_segments(*(_host_ints(t) for t in ins[6:11]))
    y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    for first, segs in plan:
        state = table[first:first + 1].float()
        for t0, t1, blk in segs:
            ys, state = ctx.K.selective_ssm(A, dt[None, t0:t1], Bm[None, t0:t1], x[None, t0:t1], Cm[None, t0:t1], state)
            y[t0:t1] = ys[0]
            table[blk].copy_(state[0])
    return [y.to(x.dtype)]


@op("PagedGatedDeltaNet")
def _paged_gated_delta_net(n, ins, ctx):
    """Token-major q / k [T, Hq, Dk], v [T, Hv, Dv], gate / beta [T, Hv]; state table [blocks, Hv, Dv, Dk] updated in place."""
    if ctx.K is None or ins[0].shape[-1] > 256 or not ins[3].is_cuda:
        return NotImplemented
    q, k, v, table, gate, beta = _same_device(ctx, ins[:6])
    at = n.get_attributes()
    qf, kf = q.float(), k.float()
    scale = float(q.shape[-1]) ** -0.5
    if at.get("use_qk_l2norm"):
        qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + float(at.get("q_l2_norm_eps", 1e-6))) * scale
        kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + float(at.get("k_l2_norm_eps", 1e-6)))
    else:
        qf = qf * scale
    plan = _paged_segments(*(_host_ints(t) for t in ins[6:11]))
    y = torch.empty(v.shape, dtype=torch.float32, device=v.device)
    for first, segs in plan:
        state = table[first:first + 1].float().transpose(-1, -2).contiguous()          # the kernel keeps [Dk, Dv]
        for t0, t1, blk in segs:
            ys, state = ctx.K.gated_delta_rule(qf[None, t0:t1], kf[None, t0:t1], v[None, t0:t1], gate[None, t0:t1], beta[None, t0:t1], state)
            y[t0:t1] = ys[0]
            table[blk].copy_(state[0].transpose(-1, -2))
    return [y.to(v.dtype)]


@op("PagedCausalConv1D")
def _paged_causal_conv1d(n, ins, ctx):
    """x [T, hidden], window table [blocks, hidden, kernel] updated in place, weights [hidden, hidden / groups, kernel], bias [hidden] or empty:
    per stretch between cache-interval boundaries one grouped convolution over (window ++ new tokens)."""
    if not ins[1].is_cuda:
        return NotImplemented
    x, table, w, bias = _same_device(ctx, ins[:4])
    Kk, groups = table.shape[2], x.shape[1] // w.shape[1]
    plan = _paged_segments(*(_host_ints(t) for t in ins[4:9]))
    y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    wf, bf = w.float(), (bias.float() if bias.numel() else None)
    for first, segs in plan:
        window = table[first].float()                                              # [hidden, kernel]
        for t0, t1, blk in segs:
            seq = torch.cat([window, x[t0:t1].float().t()], 1)                     # [hidden, kernel + n]
            y[t0:t1] = torch.nn.functional.conv1d(seq[None], wf, bf, groups=groups)[0, :, 1:].t()
            window = seq[:, -Kk:]
            table[blk].copy_(window)
    return [y.to(x.dtype)]


@op("PaKVReorder")
def _pa_kv_reorder(n, ins, ctx):
    """Rows of the key / value caches [blocks, heads, block_size, head_size] move (source token, destination token) pair by pair,
    in the order given, inside the blocks of their sequence."""
    if not (ins[0].is_cuda and ins[1].is_cuda):
        return NotImplemented
    blocks, bbeg, upd, ubeg = (_host_ints(t) for t in ins[2:6])
    BS = ins[0].shape[2]
    for s in range(len(ubeg) - 1):
        mine = blocks[bbeg[s]:bbeg[s + 1]]
        for o in range(ubeg[s], ubeg[s + 1]):
            src, dst = upd[2 * o], upd[2 * o + 1]
            if src < 0 or dst < 0 or src // BS >= len(mine) or dst // BS >= len(mine):
                raise RuntimeError("PaKVReorder: token %d -> %d is outside the blocks of sequence %d" % (src, dst, s))
            for cache in ins[:2]:
                cache[mine[dst // BS], :, dst % BS] = cache[mine[src // BS], :, src % BS].clone()
    return [torch.zeros(1, dtype=torch.uint8)]


@op("GroupQueryAttention")
def _group_query_attention(n, ins, ctx):
    """q [B, N, S, H], k / v [B, Nkv, S, H], past k / v [B, Nkv, P, H], seqlens_k, total length, then optional rotary caches,
    position ids, attention bias, head sink -> (attention [B, S, N * H], present k, present v). The key / value rows are
    laid out on the device, the attention itself runs on the package's dense kernel when its layout is served (no bias,
    no sink, no window, one of its head sizes, 16-bit) and on the library expression otherwise."""
    ins = _same_device(ctx, ins)
    at = n.get_attributes()
    q, k, v, pk, pv = ins[:5]
    have = lambda i: len(ins) > i and ins[i].numel() > 0
    B, N, S, H = q.shape
    Nkv = k.shape[1]
    total = int(_host_ints(ins[5])[0]) + 1
    P = total - S
    if P < 0 or P > pk.shape[2]:
        raise RuntimeError("GroupQueryAttention: seqlens_k names a past of %d rows, the past tensors hold %d" % (P, pk.shape[2]))
    if at.get("do_rotary"):
        cos, sin = ins[7].float(), ins[8].float()
        half = cos.shape[-1]
        rows = ins[9].to(q.device).long().reshape(-1, S) if have(9) else torch.arange(P, P + S, device=q.device).reshape(1, S)
        c, s_ = cos[rows].unsqueeze(1), sin[rows].unsqueeze(1)                 # [B or 1, 1, S, half]

        def rotate(x):
            xf = x.float()
            if at.get("rotary_interleaved"):
                a, b = xf[..., 0:2 * half:2], xf[..., 1:2 * half:2]
                r = torch.stack([a * c - b * s_, a * s_ + b * c], -1).flatten(-2)
            else:
                a, b = xf[..., :half], xf[..., half:2 * half]
                r = torch.cat([a * c - b * s_, a * s_ + b * c], -1)
            return torch.cat([r, xf[..., 2 * half:]], -1).to(x.dtype)
        q, k = rotate(q), rotate(k)
    K_ = torch.cat([pk[:, :, :P].to(k.dtype), k], 2)
    V_ = torch.cat([pv[:, :, :P].to(v.dtype), v], 2)
    scale = float(at.get("scale") or 0.0) or float(H) ** -0.5
    window = int(at.get("local_window_size", -1))
    sink = ins[11].float() if have(11) else None
    smooth = bool(at.get("smooth_softmax")) or sink is not None
    group = N // Nkv
    Kx, Vx = K_.repeat_interleave(group, 1), V_.repeat_interleave(group, 1)
    if (ctx.K is not None and P == 0 and not have(10) and not smooth and window <= 0 and q.dtype in (torch.float16, torch.bfloat16) and H in (64, 128)):
        pack = lambda t: _dense(t.transpose(1, 2)).reshape(B * S, N * H)
        out = ctx.K.sdpa_dense(pack(q), pack(Kx), pack(Vx), B, S, N, H, N * H, scale=scale, causal=True).reshape(B, S, N * H)
        return [out, K_, V_]
    sc = torch.matmul(q.float(), Kx.float().transpose(-1, -2)) * scale
    if have(10):
        sc = sc + ins[10].float()[..., :total]
    i = torch.arange(S, device=q.device).unsqueeze(1) + P
    j = torch.arange(total, device=q.device).unsqueeze(0)
    keep = j <= i
    if window > 0:
        keep = keep & (j > i - window)
    sc = sc.masked_fill(~keep, float("-inf"))
    if smooth:
        col = (sink if sink is not None else torch.zeros(N, device=q.device)).reshape(1, N, 1, 1).expand(B, N, S, 1)
        w = torch.softmax(torch.cat([sc, col], -1), -1)[..., :-1]
    else:
        w = torch.softmax(sc, -1)
    out = torch.matmul(w, Vx.float()).to(q.dtype).transpose(1, 2).reshape(B, S, N * H)
    return [out, K_, V_]


@op("ReadValue")
def _read_value(n, ins, ctx):
    vid = n.get_attribute("variable_id")
    if vid in ctx.variables:
        return [ctx.variables[vid]]
    if ins:
        return [ins[0]]
    shape = n.get_attributes().get("variable_shape")
    dims = [d.get_length() if d.is_static else 0 for d in shape] if shape is not None and shape.rank.is_static else [0]
    return [torch.zeros(dims, dtype=_tdtype(n.get_output_element_type(0), ctx.precision), device=ctx.device)]


@op("Assign")
def _assign(n, ins, ctx):
    ctx.variables[n.get_attribute("variable_id")] = ins[0]
    return [ins[0]]


@op("PagedAttentionExtension")
def _paged_attention(n, ins, ctx):
    """Inputs as in the op definition: q, k, v [T, H*S]; caches [blocks, Hkv, block_size, S] (written in place)."""
    q, k, v, kc, vc, past_lens, sub_begins, block_idx, block_begins, scale = ins[:10]
    sliding = int(_scalar(ins[10])) if ins[10].numel() else 0
    rt = n.rt_info
    Hkv, S = kc.shape[1], kc.shape[3]
    bs = kc.shape[2]
    T = q.shape[0]
    Hq = q.shape[1] // S
    dev = q.device
    to_dev = lambda t: t.to(dev) if t.device != dev else t
    past_lens, sub_begins, block_idx, block_begins = (to_dev(t).to(torch.int32) for t in (past_lens, sub_begins, block_idx, block_begins))
    B = past_lens.numel()
    # slot of every new token: block_indices[block_begins[b] + pos // bs] * bs + pos % bs
    q_lens = (sub_begins[1:] - sub_begins[:-1]).long()
    seq_of_tok = torch.repeat_interleave(torch.arange(B, device=dev), q_lens, output_size=T)
    pos = torch.arange(T, device=dev) - sub_begins[:-1].long()[seq_of_tok] + past_lens.long()[seq_of_tok]
    blk = block_idx.long()[block_begins.long()[seq_of_tok] + pos // bs]
    off = pos % bs
    kc[blk, :, off] = k.reshape(T, Hkv, S).to(kc.dtype)
    vc[blk, :, off] = v.reshape(T, Hkv, S).to(vc.dtype)
    sc = float(_scalar(scale)) if scale.numel() else 1.0 / math.sqrt(S)
    K = ctx.K
    max_ctx = int(_scalar(ins[12])) if ins[12].numel() else int((past_lens.long() + q_lens).max().item())
    if K is not None and q.dtype == torch.bfloat16 and kc.dtype == torch.bfloat16 and S in (64, 128) and bs == 16 and q.is_contiguous():
        max_q = int(q_lens.max().item()) if T != B else 1
        out = K.paged_attention(q, kc, vc, past_lens, sub_begins, block_idx, block_begins, Hq, Hkv, S, scale=sc,
                                max_context_len=max_ctx, max_q_len=max_q, sliding_window=sliding, block_size=bs)
    else:
        outs = []
        G = Hq // Hkv
        for b in range(B):
            t0, t1 = int(sub_begins[b]), int(sub_begins[b + 1])
            ctx_len = int(past_lens[b]) + (t1 - t0)
            nblk = (ctx_len + bs - 1) // bs
            blocks = block_idx.long()[int(block_begins[b]): int(block_begins[b]) + nblk]
            kk = kc[blocks].permute(1, 0, 2, 3).reshape(Hkv, -1, S)[:, :ctx_len].to(q.dtype)
            vv = vc[blocks].permute(1, 0, 2, 3).reshape(Hkv, -1, S)[:, :ctx_len].to(q.dtype)
            qq = q[t0:t1].reshape(t1 - t0, Hq, S).transpose(0, 1)
            kk, vv = kk.repeat_interleave(G, 0), vv.repeat_interleave(G, 0)
            qpos = torch.arange(int(past_lens[b]), ctx_len, device=dev)[:, None]
            kpos = torch.arange(ctx_len, device=dev)[None, :]
            allowed = kpos <= qpos
            if sliding > 0:
                allowed &= kpos > qpos - sliding
            o = F.scaled_dot_product_attention(qq[None], kk[None], vv[None], attn_mask=allowed[None, None], scale=sc)[0]
            outs.append(o.transpose(0, 1).reshape(t1 - t0, Hq * S))
        out = torch.cat(outs, 0)
    empty = torch.zeros(0, dtype=q.dtype, device=dev)
    return [out, empty, empty][: n.get_output_size()]


def supported_op_types() -> List[str]:
    return sorted(_OPS)


# ---------------------------------------------------------------------------------------------- program
class GraphProgram:
    """A compiled graph: operations in execution order with their implementations and input wiring."""

    def __init__(self, model: Model, device, precision: Optional[torch.dtype] = None, host_fallback: bool = True):
        self.model = model
        self.device = torch.device(device)
        self.ctx = Ctx(self.device, precision)
        self.precision = precision
        self.params = model.get_parameters()
        self.results = model.get_results()
        self.steps = []          # (node, impl | None, [(producer index, port)], n_outputs)
        self.consts: Dict[int, torch.Tensor] = {}
        self.fallback_nodes: List[str] = []
        index: Dict[Node, int] = {}
        self.nodes = model.get_ops()
        last_use: Dict[int, int] = {}
        for i, n in enumerate(self.nodes):
            index[n] = i
            t = n.get_type_name()
            srcs = []
            for k in range(n.get_input_size()):
                src = n.input_value(k)
                si = index[src.get_node()]
                srcs.append((si, src.get_index()))
                last_use[si] = i
            impl = _OPS.get(t)
            if impl is None:
                if not host_fallback or not n._n.has_evaluate():
                    raise RuntimeError("[CUDA] operation %s (%s) has no device implementation" % (n.get_friendly_name(), t))
                self.fallback_nodes.append(n.get_friendly_name())
            if t == "Constant":
                self.consts[i] = self._upload_constant(n)
            self.steps.append((n, impl, srcs, n.get_output_size()))
        self.param_index = {index[p]: k for k, p in enumerate(self.params)}
        self.result_index = [index[r] for r in self.results]
        self.sink_index = [index[s] for s in model.get_sinks()]
        keep = set(self.result_index) | set(self.sink_index)
        # values can be dropped right after their last consumer ran
        self.free_after: Dict[int, List[int]] = {}
        for si, li in last_use.items():
            if si not in keep and si not in self.consts:
                self.free_after.setdefault(li, []).append(si)

    def _upload_constant(self, n: Node) -> torch.Tensor:
        t = n.get_tensor_view()
        et = t.element_type
        if et.name == "string":
            raise RuntimeError("string constants are not supported on this device")
        shape = list(t.shape)
        small_int = (not et.is_real()) and t.size <= 64
        if et.bitwidth % 8 != 0 or et.name.startswith("f8") or et.name in ("nf4", "f4e2m1"):
            # packed types are consumed by FullyConnectedCompressed through their raw bytes; keep a float view for the rest
            arr = torch.from_numpy(np.ascontiguousarray(t.to_float32()).reshape(shape))
        elif et.name == "bf16":
            arr = torch.from_numpy(np.ascontiguousarray(t.data).view(np.int16).reshape(shape)).view(torch.bfloat16)
        else:
            arr = torch.from_numpy(np.ascontiguousarray(t.data).reshape(shape))
        if arr.dtype == torch.float32 and self.precision is not None:
            arr = arr.to(self.precision)
        if small_int:
            return arr                       # shape arithmetic stays on the host
        return arr.to(self.device)

    def _host_eval(self, n: Node, ins: List[torch.Tensor]) -> List[torch.Tensor]:
        """Evaluate one operation with the native reference executor (inputs and outputs cross the host)."""
        from .._graph import parameter, result
        ps, feed = [], []
        for t in ins:
            host = t.detach().to("cpu")
            if host.dtype in (torch.bfloat16, torch.float16):
                host = host.float()
            arr = host.contiguous().numpy()
            ps.append(parameter(list(arr.shape), Type.from_numpy(arr.dtype)))
            feed.append(Tensor(arr)._to_core())
        clone = n.clone_with_new_inputs([p.output(0) for p in ps])
        sub = Model([result(clone.output(i)) for i in range(clone.get_output_size())], ps, "host_fallback")
        outs, _ = _c.evaluate(sub._m, feed)
        res = []
        for o in outs:
            t = Tensor._from_core(o)
            arr = torch.from_numpy(np.ascontiguousarray(t.data))
            if arr.dtype == torch.float32 and self.precision is not None:
                arr = arr.to(self.precision)
            res.append(arr.to(self.device))
        return res

    def run(self, inputs: List[torch.Tensor], profile: Optional[list] = None) -> List[torch.Tensor]:
        values: Dict[int, List[torch.Tensor]] = {}
        ctx = self.ctx
        ev = None
        for i, (n, impl, srcs, nout) in enumerate(self.steps):
            t = n.get_type_name()
            if t == "Parameter":
                values[i] = [inputs[self.param_index[i]]]
                continue
            if t == "Constant":
                values[i] = [self.consts[i]]
                continue
            ins = [values[si][port] for si, port in srcs]
            if profile is not None and ctx.on_gpu:
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
            values[i] = impl(n, ins, ctx) if impl is not None else self._host_eval(n, ins)
            if values[i] is NotImplemented:      # a device implementation that does not serve these sizes
                values[i] = self._host_eval(n, ins)
            if profile is not None:
                if ctx.on_gpu:
                    ev[1].record()
                profile.append((n.get_friendly_name(), t, ev))
            for dead in self.free_after.get(i, ()):
                values.pop(dead, None)
        return [values[ri][0] for ri in self.result_index]


# ---------------------------------------------------------------------------------------------- plugin
class RemoteTensor(Tensor):
    """Device-memory tensor (``ov::RemoteTensor``): wraps a CUDA tensor; ``data`` copies to the host."""

    def __init__(self, t: torch.Tensor):
        super().__init__(t)


class RemoteContext:
    """Device context: creates device and pinned host tensors (``ov::RemoteContext``)."""

    def __init__(self, device: torch.device):
        self.device = device

    def get_device_name(self) -> str:
        return "CUDA.%d" % (self.device.index or 0)

    def create_tensor(self, type, shape, properties=None) -> RemoteTensor:
        return RemoteTensor(torch.empty(list(shape), dtype=torch_dtype(Type(type)), device=self.device))

    def create_host_tensor(self, type, shape) -> Tensor:
        t = torch.empty(list(shape), dtype=torch_dtype(Type(type))).pin_memory()
        return Tensor(t, shared_memory=True)

    def get_params(self) -> dict:
        return {"CONTEXT_TYPE": "CUDA", "DEVICE_ID": str(self.device.index or 0)}


_CAPTURE_LOCK = threading.Lock()


class CudaCompiledModel(CompiledModel):
    def __init__(self, plugin, model, config, runtime_model, device: torch.device, precision):
        super().__init__(plugin, model, config, runtime_model)
        self.device, self.precision = device, precision
        self.program = GraphProgram(runtime_model, device, precision)
        self._out_types = [o.get_element_type() for o in model.outputs]
        # one stream per compiled-model stream: requests of different streams overlap on the GPU
        self._streams = [torch.cuda.Stream(device=device) for _ in range(self._n_streams)] if device.type == "cuda" else [None]
        # requests that share a stream take turns on the host as well: one of them may be capturing a graph on that stream,
        # and a launch or a synchronize from another thread on a capturing stream would end the capture with an error
        self._stream_locks = [threading.Lock() for _ in self._streams]
        # the interpreter keeps the running request's variables in its (shared) context: requests of a model with states
        # walk the program one at a time
        self._has_state = any(n.get_type_name() in ("ReadValue", "Assign") for n in runtime_model.get_ops())
        self._state_lock = threading.Lock()
        self._next_stream = 0

    def _make_runner(self, request: InferRequest):
        stream = self._streams[self._next_stream % len(self._streams)]
        stream_lock = self._stream_locks[self._next_stream % len(self._streams)]
        self._next_stream += 1
        program = self.program
        # variables (states) are per request; constants and packed weights are shared by all requests
        ctx_vars: Dict[str, torch.Tensor] = {}
        request._cuda_vars = ctx_vars
        profile_on = bool(self.config.get(props.enable_profiling))
        dev = self.device

        def to_device(t: Tensor) -> torch.Tensor:
            if t.is_remote:
                x = t.torch()
            else:
                arr = t.data
                if t.element_type.name == "bf16":
                    x = torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).view(torch.bfloat16)
                elif t.element_type.name == "string":
                    raise RuntimeError("string tensors are not supported on this device")
                else:
                    x = torch.from_numpy(np.ascontiguousarray(arr))
                x = x.to(dev, non_blocking=True)
            if x.dtype == torch.float32 and self.precision is not None:
                x = x.to(self.precision)
            return x

        # CUDA graphs for static graphs: the second inference of a request with the same input shapes captures the whole
        # program (every kernel launch of the interpreter walk) into one graph; later inferences copy the inputs into the
        # captured buffers and replay it, so the per-node host work (dispatch, tensor-map encoding, allocation) is paid once.
        # Not for models with states or cross-rank collectives, nor while profiling; a program that reads a device value on
        # the host (data-dependent shapes) cannot be captured and stays in eager mode.
        graphs_on = (stream is not None and not profile_on and bool(self.config.get(props.cuda.use_cuda_graphs, True))
                     and not any(n.get_type_name() in ("ReadValue", "Assign", "AllReduce", "PagedAttentionExtension") for n in self.runtime_model.get_ops()))
        graph_cache: Dict[tuple, object] = {}
        request._cuda_graphs = graph_cache

        def run_graphed(xs: List[torch.Tensor]):
            key = tuple((tuple(x.shape), x.dtype) for x in xs)
            entry = graph_cache.get(key)
            if entry is None:                       # first call: eager (warms up workspaces and one-time kernel set-up)
                graph_cache[key] = "warm"
                return program.run(xs, None)
            if entry == "eager":
                return program.run(xs, None)
            if entry == "warm":
                static_in = [torch.empty_like(x) for x in xs]
                for s_, x in zip(static_in, xs):
                    s_.copy_(x)
                g = torch.cuda.CUDAGraph()
                try:
                    stream.synchronize()
                    # one capture at a time in the process; "thread_local" keeps the calls of other requests' threads
                    # (allocations, launches on their own streams) legal while this thread captures
                    with _CAPTURE_LOCK, torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                        static_out = program.run(static_in, None)
                    entry = (g, static_in, static_out)
                except Exception as e:   # noqa: BLE001 - a host read inside the walk: this shape stays eager
                    from ..utils import log
                    log.debug("cuda", "graph capture failed, staying eager: %s" % str(e)[:200])
                    try:
                        stream.synchronize()
                    except Exception:   # noqa: BLE001 - the failed capture may surface once more here
                        pass
                    graph_cache[key] = "eager"
                    return program.run(xs, None)
                graph_cache[key] = entry
                g.replay()
                return list(entry[2])
            g, static_in, static_out = entry
            for s_, x in zip(static_in, xs):
                s_.copy_(x, non_blocking=True)
            g.replay()
            return list(static_out)

        def run(req: InferRequest, ins: List[Tensor]) -> List[Tensor]:
            prof = [] if profile_on else None
            if stream is not None:
                with (self._state_lock if self._has_state else contextlib.nullcontext()), stream_lock:
                    program.ctx.variables = ctx_vars
                    with torch.cuda.stream(stream):
                        xs = [to_device(t) for t in ins]
                        outs = run_graphed(xs) if graphs_on else program.run(xs, prof)
                        res = self._finish(outs, req)
                    stream.synchronize()
            else:
                with self._state_lock:
                    program.ctx.variables = ctx_vars
                    outs = program.run([to_device(t) for t in ins], prof)
                    res = self._finish(outs, req)
                    torch.cuda.current_stream(self.device).synchronize()
            if prof is not None:
                req._profile = [ProfilingInfo(name, typ, "cuda", (ev[0].elapsed_time(ev[1]) * 1e3) if ev else 0.0) for name, typ, ev in prof]
            return res
        return run

    def _finish(self, outs: List[torch.Tensor], req: InferRequest) -> List[Tensor]:
        res = []
        for i, (o, et) in enumerate(zip(outs, self._out_types)):
            want = torch_dtype(et) if et.is_static() else o.dtype
            if o.dtype != want:
                o = o.to(want)
            user = req._user_out.get(i)
            if user is not None and user.is_remote:
                user.torch().copy_(o)
                res.append(user)
                continue
            # results land in pinned host memory owned by the request (re-used by its next inference): the copy runs at
            # full PCIe rate and without a staging pass; the caller synchronises the stream before handing them out
            o = o.detach()
            if o.is_cuda:
                pinned = req.__dict__.setdefault("_pinned_out", {})
                host = pinned.get(i)
                if host is None or host.shape != o.shape or host.dtype != o.dtype:
                    host = torch.empty(o.shape, dtype=o.dtype, pin_memory=True)
                    pinned[i] = host
                host.copy_(o, non_blocking=True)
            else:
                host = _dense(o)
            if host.dtype == torch.bfloat16:
                res.append(Tensor(host))
            else:
                res.append(Tensor(host.numpy(), shared_memory=True))
        return res

    def _variables(self, request: InferRequest) -> List[VariableState]:
        store = request._cuda_vars
        out = []
        for v in self.runtime_model.get_variables():
            info = v.get_info()
            vid = info.variable_id

            def get(vid=vid, info=info):
                if vid in store:
                    return Tensor(store[vid].detach().float().cpu().numpy() if store[vid].dtype in (torch.float16, torch.bfloat16) else store[vid].detach().cpu().numpy())
                shape = [d.get_length() if d.is_static else 0 for d in info.data_shape] if info.data_shape.rank.is_static else [0]
                return Tensor(info.data_type if info.data_type.is_static() else Type.f32, shape)

            def set_(t, vid=vid):
                x = torch.from_numpy(np.ascontiguousarray(t.data)).to(self.device)
                store[vid] = x.to(self.precision) if (x.dtype == torch.float32 and self.precision is not None) else x

            def reset(vid=vid):
                store.pop(vid, None)
            out.append(VariableState(vid, get, set_, reset))
        return out

    def get_property(self, name):
        if str(name) == props.execution_devices:
            return ["CUDA.%d" % (self.device.index or 0)]
        return super().get_property(name)


_PRECISIONS = {"f32": None, "f16": torch.float16, "bf16": torch.bfloat16}


class CudaConfig(PluginConfig):
    """Option table of the CUDA device (validated types, visibility, ``OV_<NAME>`` environment and config-file overrides)."""

    def declare_options(self) -> None:
        R, RI, D = OptionVisibility.RELEASE, OptionVisibility.RELEASE_INTERNAL, OptionVisibility.DEBUG
        self.register(ConfigOption(props.hint.inference_precision, "f32", "compute precision of graph programs", lambda v: str(v).lower() in _PRECISIONS, R))
        self.register(ConfigOption(props.hint.performance_mode, "LATENCY", "LATENCY | THROUGHPUT | CUMULATIVE_THROUGHPUT",
                                   lambda v: v in ("LATENCY", "THROUGHPUT", "CUMULATIVE_THROUGHPUT"), R))
        self.register(ConfigOption(props.num_streams, 1, "streams (infer requests that run concurrently); -1 = automatic", lambda v: v >= -1, R))
        self.register(ConfigOption(props.hint.model_distribution_policy, "", "'' | TENSOR_PARALLEL | PIPELINE_PARALLEL",
                                   lambda v: all(p in ("", "TENSOR_PARALLEL", "PIPELINE_PARALLEL") for p in str(v).replace(" ", "").split(",")), R))
        self.register(ConfigOption(props.hint.kv_cache_precision, "bf16", "element type of the paged KV cache: bf16 | f16 | u8",
                                   lambda v: str(v).lower() in ("bf16", "f16", "u8", "dynamic"), R))
        self.register(ConfigOption(props.cuda.use_cuda_graphs, True, "capture decode steps of the serving program in CUDA graphs", None, R))
        self.register(ConfigOption(props.cuda.serving_program, False, "compile a decoder-only LLM graph into the serving program", None, R))
        self.register(ConfigOption(props.cuda.tensor_parallel_size, 0, "ranks of the tensor-parallel group (0 = the process group's size)", lambda v: 0 <= v <= 8, R))
        self.register(ConfigOption(props.cuda.memory_fraction, 0.9, "share of the free device memory the KV cache may take", lambda v: 0.0 < v <= 1.0, RI))
        self.register(ConfigOption(props.enable_profiling, False, "per-node timing of graph programs (PERF_COUNT)", None, R))
        self.register(ConfigOption("SNIPPETS_MODE", "DISABLE", "ENABLE: groups of element-wise operations run as generated kernels (built with nvcc at compile time)",
                                   lambda v: str(v).upper() in ("ENABLE", "DISABLE"), R, str))
        self.register(ConfigOption("CUDA_PDL", True, "programmatic dependent launch of the serving kernels", None, RI))
        self.register(ConfigOption("CUDA_DUMP_GRAPH_PROGRAM", "", "write the node list of compiled graph programs to this file", None, D, str))

    def finalize_impl(self) -> None:
        # a throughput hint without an explicit stream count asks for two streams
        if self[props.hint.performance_mode] == "THROUGHPUT" and not self.is_set_by_user(props.num_streams):
            self.set_property({props.num_streams: 2})


class CudaServingCompiledModel(CompiledModel):
    """A decoder-only LLM compiled for serving. The graph (stateful SDPA form or PagedAttention form, dense or
    weight-compressed) is analysed by structure (runtime/llm_import.py); the compiled model keeps the architecture and the
    weights found in the graph and builds this rank's executor on request. The partition over the GPUs follows the graph:
    with ``MODEL_DISTRIBUTION_POLICY = TENSOR_PARALLEL`` and ``torch.distributed`` initialised, rank r takes its slice of
    the attention heads (rows of the q / k / v projections, columns of the output projection), of the MLP channels (rows of
    gate / up, columns of down) and of the vocabulary; the row-parallel projections then run with the all-reduce fused into
    their epilogue. Reference flow: the PagedAttention model compiled by the device plugin for openvino.genai's continuous
    batching (src/core/src/pass/sdpa_to_paged_attention.cpp, src/plugins/intel_gpu/src/plugin/transformations_pipeline.cpp)."""

    def __init__(self, plugin, model, config, device: torch.device):
        super().__init__(plugin, model, config, model)
        from . import llm_import
        self.device = device
        self.llm_config, self._parts = llm_import.analyze(model)
        policy = str(config.get(props.hint.model_distribution_policy, "") or "")
        self.tp_rank, self.tp_size = 0, 1
        if "TENSOR_PARALLEL" in policy and torch.distributed.is_available() and torch.distributed.is_initialized():
            self.tp_rank, self.tp_size = torch.distributed.get_rank(), torch.distributed.get_world_size()
        self._weights = None
        self._comm = None

    def weights(self):
        """This rank's shard in the kernels' layouts (built once)."""
        if self._weights is None:
            from . import llm_import
            with torch.cuda.device(self.device):
                self._weights = llm_import.build_weights(self.llm_config, self._parts, self.device, self.tp_rank, self.tp_size)
            self._parts = None      # the host copies of the constants are not needed any more
        return self._weights

    def create_llm_executor(self, max_num_seqs: int = 64, max_num_batched_tokens: int = 8192, max_model_len: int = 4096, block_size: int = 16,
                            kv_cache_blocks: int = 0, comm=None):
        """The executor of this rank plus the scheduler limits that fit it: ``(executor, SchedulerConfig)``."""
        from ..genai.scheduler import SchedulerConfig
        from .cuda_llm import CudaLlmExecutor
        if self.tp_size > 1 and comm is None:
            if self._comm is None:
                from ..parallel.comm import PeerCommunicator
                self._comm = PeerCommunicator(self.tp_rank, self.tp_size, self.device)
            comm = self._comm
        blocks_per_seq = (max_model_len + block_size - 1) // block_size + 1
        num_blocks = kv_cache_blocks or max_num_seqs * blocks_per_seq + 8
        with torch.cuda.device(self.device):
            ex = CudaLlmExecutor(self.llm_config, self.weights(), num_kv_blocks=num_blocks, block_size=block_size,
                                 max_batch_tokens=max_num_batched_tokens, max_seqs=max_num_seqs, max_blocks_per_seq=blocks_per_seq,
                                 device=self.device, comm=comm, use_cuda_graphs=bool(self.config.get(props.cuda.use_cuda_graphs, True)),
                                 kv_cache_precision=str(self.config.get(props.hint.kv_cache_precision, "bf16") or "bf16"))
        sc = SchedulerConfig(max_num_batched_tokens=max_num_batched_tokens, max_num_seqs=max_num_seqs, num_kv_blocks=num_blocks,
                             block_size=block_size, max_blocks_per_seq=blocks_per_seq)
        return ex, sc

    def _make_runner(self, request):
        raise RuntimeError("[CUDA] a model compiled with CUDA_SERVING_PROGRAM is driven by a generation pipeline "
                           "(openvino_b200.genai.LLMPipeline / ContinuousBatchingPipeline), not by infer requests")


class CudaPlugin(Plugin):
    device_name = "CUDA"
    description = "NVIDIA B200 (sm_100a)"

    def __init__(self, core):
        super().__init__(core)
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available")
        self._contexts: Dict[int, RemoteContext] = {}

    def supported_properties(self):
        return super().supported_properties() + [props.cuda.use_cuda_graphs, props.cuda.tensor_parallel_size, props.cuda.serving_program, props.device.uuid,
                                                 props.device.architecture, props.device.type, props.optimal_batch_size,
                                                 props.hint.kv_cache_precision, props.hint.model_distribution_policy]

    def default_config(self):
        d = super().default_config()
        d[props.hint.inference_precision] = "f32"
        return d

    def available_device_ids(self):
        return [str(i) for i in range(torch.cuda.device_count())]

    def full_name(self, device_id=""):
        return torch.cuda.get_device_name(int(device_id or 0))

    def capabilities(self):
        return ["FP32", "FP16", "BF16", "INT8", "INT4", "EXPORT_IMPORT"]

    def get_property(self, name, arguments=None):
        dev = int((arguments or {}).get(props.device.id, "") or 0)
        if name == props.device.architecture:
            cc = torch.cuda.get_device_capability(dev)
            return "sm_%d%d" % cc
        if name == props.device.type:
            return "discrete"
        if name == props.device.uuid:
            return str(torch.cuda.get_device_properties(dev).uuid)
        if name == props.optimal_batch_size:
            return 16
        if name == props.range_for_async_infer_requests:
            return (1, 16, 1)
        if name == props.range_for_streams:
            return (1, 8)
        return super().get_property(name, arguments)

    def _device(self, cfg) -> torch.device:
        return torch.device("cuda", int(cfg.get(props.device.id, "") or 0))

    def transform(self, model: Model) -> Model:
        rm = model.clone()
        _c.run_moc_transformations(rm._m, True)
        _c.run_llm_fusions(rm._m)
        from . import cuda_fusions
        cuda_fusions.run(rm)
        return rm

    def make_config(self, config: dict, model: Optional[Model] = None, device_name: str = "CUDA") -> CudaConfig:
        """The validated option table of one compile call: public properties (RELEASE options only), then the derived
        options, the configuration file and the environment. Unknown names are left to the generic property handling."""
        pc = CudaConfig()
        known = {k: v for k, v in config.items() if k in pc._options}
        pc.set_user_property(known, OptionVisibility.RELEASE)
        return pc.finalize(model, device_name)

    def compile_model(self, model: Model, config: dict) -> CompiledModel:
        cfg = self.merged_config(config)
        try:
            pc = self.make_config(cfg, model, "CUDA")
        except (ValueError, PermissionError) as e:
            raise RuntimeError("[CUDA] %s" % e)
        cfg.update({k: v for k, v in pc.to_dict().items() if k in cfg or pc._options[k].value != pc._options[k].default})
        if not pc["CUDA_PDL"]:
            from ..ops import cuda as K
            K.lib().ovb_set_pdl(0)
        prec = str(cfg.get(props.hint.inference_precision, "f32")).lower()
        if prec not in _PRECISIONS:
            raise RuntimeError("[CUDA] unsupported inference precision %s" % prec)
        dev = self._device(cfg)
        if str(cfg.get(props.cuda.serving_program, "")).upper() in ("TRUE", "YES", "1"):
            return CudaServingCompiledModel(self, model, cfg, dev)
        rm = self.transform(model)
        if str(pc["SNIPPETS_MODE"]).upper() == "ENABLE":
            from ..snippets import tokenize
            tokenize(rm)
        policy = str(cfg.get(props.hint.model_distribution_policy, "") or "")
        if "TENSOR_PARALLEL" in policy and torch.distributed.is_available() and torch.distributed.is_initialized() \
                and torch.distributed.get_world_size() > 1:
            # one process per GPU: this rank compiles its own shard of the model (attention heads and MLP columns)
            from ..parallel.graph_tp import tensor_parallel_partition
            tensor_parallel_partition(rm, torch.distributed.get_rank(), torch.distributed.get_world_size())
        with torch.cuda.device(dev):
            return CudaCompiledModel(self, model, cfg, rm, dev, _PRECISIONS[prec])

    def query_model(self, model: Model, config: dict) -> Dict[str, str]:
        rm = self.transform(model)
        supported_fused = set()
        for n in rm.get_ops():
            if n.get_type_name() in _OPS:
                fused = n.rt_info.get("fused_names_0")
                supported_fused.update(str(fused).split(",") if fused else [n.get_friendly_name()])
        return {n.get_friendly_name(): self.device_name for n in model.get_ops()
                if n.get_type_name() in _OPS or n.get_friendly_name() in supported_fused}

    def create_context(self, params: dict) -> RemoteContext:
        return self.get_default_context(int(params.get("DEVICE_ID", 0)))

    def get_default_context(self, device_id: int = 0) -> RemoteContext:
        if device_id not in self._contexts:
            self._contexts[device_id] = RemoteContext(torch.device("cuda", device_id))
        return self._contexts[device_id]
