"""Generic primitives of the CUDA device's graph executor on the package's own kernels (``csrc/cuda/generic.cu``):
unary / binary element-wise with broadcasting, softmax, reductions, strided copies (transpose, concat) and 2-D pooling.

Tensors are torch CUDA tensors used as plain device buffers; fp32, fp16 and bf16 storage. Everything else (integer and
boolean tensors, CPU tensors) is not handled here: ``supported(t)`` tells the caller, who keeps its fallback for those.
Role in the reference: the eltwise / softmax / reduce / reorder / pooling primitives of
src/plugins/intel_gpu/src/graph/impls/ocl (eltwise.cpp, softmax.cpp, reduce.cpp, reorder.cpp, pooling.cpp)."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

import torch

from . import cuda as K

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

UNARY = {name: i for i, name in enumerate((
    "relu", "sigmoid", "tanh", "gelu_erf", "gelu_tanh", "swish", "exp", "log", "sqrt", "abs", "neg", "hswish", "hsigmoid", "mish",
    "softplus", "erf", "floor", "ceil", "sign", "clamp", "elu", "sin", "cos", "rsqrt", "softsign", "round_even", "round_away",
    "scale_shift"))}
BINARY = {name: i for i, name in enumerate(("add", "sub", "mul", "div", "max", "min", "pow", "sqdiff", "prelu"))}
REDUCE = {name: i for i, name in enumerate(("sum", "mean", "max", "min", "prod", "l2", "l1"))}
MAX_DIMS = 6


class PoolArgs(C.Structure):
    _fields_ = [("NC", C.c_int64)] + [(f, C.c_int) for f in ("H", "W", "OH", "OW", "kh", "kw", "sh", "sw", "ph", "pw", "ph_end", "pw_end",
                                                              "dh", "dw", "is_max", "exclude_pad")]


def enabled() -> bool:
    """The kernels are used whenever the library is there; OVB_GENERIC=0 keeps the caller's fallback (debugging aid)."""
    return os.environ.get("OVB_GENERIC", "1") != "0" and K.available()


def supported(t: torch.Tensor) -> bool:
    return isinstance(t, torch.Tensor) and t.is_cuda and t.dtype in _DT and t.numel() > 0


def _i64(vals: Sequence[int]):
    return (C.c_int64 * len(vals))(*[int(v) for v in vals])


def _p(t: torch.Tensor):
    return C.c_void_p(t.data_ptr())


def unary(name: str, x: torch.Tensor, a: float = 0.0, b: float = 0.0) -> torch.Tensor:
    x = contiguous(x)
    y = torch.empty_like(x)
    K._check(K.lib().ovb_unary(C.c_int(UNARY[name]), _p(x), _p(y), C.c_int64(x.numel()), C.c_int(_DT[x.dtype]), C.c_float(a), C.c_float(b),
                               C.c_void_p(K._stream())), "ovb_unary")
    return y


def _collapse(shape: List[int], strides: List[List[int]]):
    """Merge neighbouring axes that are contiguous in every operand; drops axes of extent 1."""
    keep = [i for i, s in enumerate(shape) if s != 1]
    if not keep:
        return [1], [[0] for _ in strides]
    shape = [shape[i] for i in keep]
    strides = [[st[i] for i in keep] for st in strides]
    out_shape, out_strides = [shape[0]], [[st[0]] for st in strides]
    for i in range(1, len(shape)):
        if all(os_[-1] == st[i] * shape[i] for os_, st in zip(out_strides, strides)):
            out_shape[-1] *= shape[i]
            for os_, st in zip(out_strides, strides):
                os_[-1] = st[i]
        else:
            out_shape.append(shape[i])
            for os_, st in zip(out_strides, strides):
                os_.append(st[i])
    return out_shape, out_strides


def binary(name: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    assert a.dtype == b.dtype
    shape = list(torch.broadcast_shapes(a.shape, b.shape))
    y = torch.empty(shape, dtype=a.dtype, device=a.device)
    if y.numel() == 0:
        return y
    same = list(a.shape) == shape and list(b.shape) == shape and a.is_contiguous() and b.is_contiguous()
    if same:
        cs, (sa, sb) = [y.numel()], ([1], [1])
    else:
        ea, eb = a.expand(shape), b.expand(shape)
        cs, (sa, sb, _) = _collapse(shape or [1], [list(ea.stride()) or [0], list(eb.stride()) or [0], list(y.stride()) or [1]])
        if len(cs) > MAX_DIMS:
            _too_many_dims()
    K._check(K.lib().ovb_binary(C.c_int(BINARY[name]), _p(a), _p(b), _p(y), C.c_int(len(cs)), _i64(cs), _i64(sa), _i64(sb), C.c_int(1 if same else 0),
                                C.c_int(_DT[a.dtype]), C.c_void_p(K._stream())), "ovb_binary")
    return y


def _too_many_dims():
    raise NotImplementedError("more than %d non-mergeable broadcast axes" % MAX_DIMS)


def strided_copy(src: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[...] = src[...] for two views of equal shape (any strides, same element size)."""
    assert list(src.shape) == list(dst.shape) and src.element_size() == dst.element_size()
    if src.numel() == 0:
        return
    shape = list(src.shape) or [1]
    cs, (sx, sy) = _collapse(shape, [list(src.stride()) or [0], list(dst.stride()) or [0]])
    if len(cs) > MAX_DIMS:
        _too_many_dims()
    es = src.element_size()
    # rows that are contiguous on both sides move as 16-byte (or 8- / 4-byte) units: the innermost run is re-expressed in
    # wider elements when its length, the other strides and both base addresses allow it
    if sx[-1] == 1 and sy[-1] == 1:
        for unit in (16, 8, 4):
            k = unit // es
            if k > 1 and cs[-1] % k == 0 and all(v % k == 0 for v in sx[:-1] + sy[:-1]) and src.data_ptr() % unit == 0 and dst.data_ptr() % unit == 0:
                cs = cs[:-1] + [cs[-1] // k]
                sx = [v // k for v in sx[:-1]] + [1]
                sy = [v // k for v in sy[:-1]] + [1]
                es = unit
                break
    K._check(K.lib().ovb_strided_copy(_p(src), _p(dst), C.c_int(len(cs)), _i64(cs), _i64(sx), _i64(sy), C.c_int(es),
                                      C.c_void_p(K._stream())), "ovb_strided_copy")


def contiguous(x: torch.Tensor) -> torch.Tensor:
    """``x`` laid out densely in its logical order (a no-op for contiguous tensors). A swap of the two innermost axes of a
    dense tensor takes the shared-memory tile transpose; every other layout the strided copy."""
    if x.is_contiguous():
        return x
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    if x.numel() == 0:
        return y
    if x.dim() >= 2 and x.element_size() in (2, 4):
        t = x.transpose(-1, -2)
        if t.is_contiguous():
            batch = 1
            for s in x.shape[:-2]:
                batch *= s
            R, Cc = t.shape[-2], t.shape[-1]          # source is [batch, R, C]; result [batch, C, R]
            if 0 < batch < 65536 and (R + 31) // 32 < 65536:
                K._check(K.lib().ovb_transpose2d(_p(t), _p(y), C.c_int64(batch), C.c_int(R), C.c_int(Cc), C.c_int(x.element_size()),
                                                 C.c_void_p(K._stream())), "ovb_transpose2d")
                return y
    strided_copy(x, y)
    return y


def concat(ts: Sequence[torch.Tensor], axis: int) -> torch.Tensor:
    nd = ts[0].dim()
    axis %= nd
    shape = list(ts[0].shape)
    shape[axis] = sum(t.shape[axis] for t in ts)
    y = torch.empty(shape, dtype=ts[0].dtype, device=ts[0].device)
    o = 0
    for t in ts:
        if t.shape[axis]:
            strided_copy(t, y.narrow(axis, o, t.shape[axis]))
        o += t.shape[axis]
    return y


def _outer_dim_inner(shape: Sequence[int], axis: int):
    outer = 1
    for s in shape[:axis]:
        outer *= s
    inner = 1
    for s in shape[axis + 1:]:
        inner *= s
    return outer, shape[axis], inner


def softmax(x: torch.Tensor, axis: int, log: bool = False) -> torch.Tensor:
    x = contiguous(x)
    axis %= x.dim()
    outer, dim, inner = _outer_dim_inner(list(x.shape), axis)
    y = torch.empty_like(x)
    K._check(K.lib().ovb_softmax(_p(x), _p(y), C.c_int64(outer), C.c_int(dim), C.c_int64(inner), C.c_int(_DT[x.dtype]), C.c_int(1 if log else 0),
                                 C.c_void_p(K._stream())), "ovb_softmax")
    return y


def reduce(name: str, x: torch.Tensor, axes: Sequence[int], keepdim: bool) -> torch.Tensor:
    """Reduction over ``axes``. Neighbouring axes are reduced in one pass; separated groups take one pass each (mean, l1 and
    l2 over separated groups are composed from sums so that the result equals a single reduction)."""
    x = contiguous(x)
    nd = x.dim()
    axes = sorted({a % nd for a in axes})
    groups: List[List[int]] = []
    for a in axes:
        if groups and groups[-1][-1] == a - 1:
            groups[-1].append(a)
        else:
            groups.append([a])
    count = 1
    for a in axes:
        count *= x.shape[a]
    cur, op, post = x, name, None
    if len(groups) > 1 and name in ("mean", "l1", "l2"):
        op = "sum"
        if name == "l2":
            cur, post = binary("mul", cur, cur), ("sqrt", 0.0, 0.0)
        elif name == "l1":
            cur = unary("abs", cur)
        else:
            post = ("scale_shift", 1.0 / count, 0.0)
    shape = list(x.shape)
    for g in reversed(groups):
        outer = 1
        for s in shape[:g[0]]:
            outer *= s
        dim = 1
        for a in g:
            dim *= shape[a]
        inner = 1
        for s in shape[g[-1] + 1:]:
            inner *= s
        y = torch.empty(outer * inner, dtype=x.dtype, device=x.device)
        K._check(K.lib().ovb_reduce(C.c_int(REDUCE[op]), _p(cur), _p(y), C.c_int64(outer), C.c_int(dim), C.c_int64(inner), C.c_int(_DT[x.dtype]),
                                    C.c_void_p(K._stream())), "ovb_reduce")
        shape = shape[:g[0]] + [1] * len(g) + shape[g[-1] + 1:]
        cur = y.reshape(shape)
    if post is not None:
        cur = unary(post[0], cur, post[1], post[2])
    if not keepdim:
        cur = cur.reshape([s for i, s in enumerate(x.shape) if i not in axes])
    return cur


def pool2d(x: torch.Tensor, kernel, strides, pads_begin, pads_end, dilations, out_hw, is_max: bool, exclude_pad: bool) -> torch.Tensor:
    x = contiguous(x)
    N, Cc, H, W = x.shape
    a = PoolArgs()
    a.NC, a.H, a.W, a.OH, a.OW = N * Cc, H, W, out_hw[0], out_hw[1]
    a.kh, a.kw, a.sh, a.sw = kernel[0], kernel[1], strides[0], strides[1]
    a.ph, a.pw, a.ph_end, a.pw_end = pads_begin[0], pads_begin[1], pads_end[0], pads_end[1]
    a.dh, a.dw = dilations[0], dilations[1]
    a.is_max, a.exclude_pad = int(is_max), int(exclude_pad)
    y = torch.empty((N, Cc, out_hw[0], out_hw[1]), dtype=x.dtype, device=x.device)
    if y.numel():
        K._check(K.lib().ovb_pool2d(_p(x), _p(y), C.byref(a), C.c_int(_DT[x.dtype]), C.c_void_p(K._stream())), "ovb_pool2d")
    return y
