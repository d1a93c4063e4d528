"""More ATen translators (second part of the table of pytorch.py): the core-ATen operations that the decompositions of
composite operations bottom out in (var / std with a correction, flip, diagonal, vector norms, atan2, hypot, ...), plus
sorting, indexing with reductions, rearrangements, paddings and sampling operations.

Operations that ATen can express through simpler ones are not listed here: ``from_exported_program`` rewrites them with
their ATen decompositions before the walk. Reference: src/frontends/pytorch/src/op/*.cpp."""
from __future__ import annotations

import numpy as np

from .. import opset as ops
from .._graph import Output, constant
from .._types import Type
from .pytorch import ConversionError, _TABLE, _i64, _op, _rank


def _c(v, like: Output) -> Output:
    return constant(np.array(v, dtype=np.float32), like.get_element_type()).output(0)


def _axis(a: int, r: int) -> int:
    return a if a >= 0 else a + r


def _unary(name, fn):
    _TABLE["aten.%s.default" % name] = lambda ctx, n: fn(ctx.out(n.args[0]))


_unary("log1p", lambda x: ops.log(ops.add(x, _c(1.0, x))).output(0))
_unary("expm1", lambda x: ops.subtract(ops.exp(x), _c(1.0, x)).output(0))
_unary("exp2", lambda x: ops.power(_c(2.0, x), x).output(0))
_unary("log2", lambda x: ops.divide(ops.log(x), _c(np.log(2.0), x)).output(0))
_unary("log10", lambda x: ops.divide(ops.log(x), _c(np.log(10.0), x)).output(0))
_unary("erfc", lambda x: ops.subtract(_c(1.0, x), ops.erf(x)).output(0))
_unary("trunc", lambda x: ops.multiply(ops.sign(x), ops.floor(ops.abs(x))).output(0))
_unary("frac", lambda x: ops.subtract(x, ops.multiply(ops.sign(x), ops.floor(ops.abs(x)))).output(0))
_unary("square", lambda x: ops.multiply(x, x).output(0))
_unary("relu6", lambda x: ops.clamp(x, 0.0, 6.0).output(0))
_unary("selu", lambda x: ops.selu(x, _c(1.6732632423543772, x), _c(1.0507009873554805, x)).output(0))
_unary("isinf", lambda x: ops.is_inf(x, True, True).output(0))
_unary("asinh", lambda x: ops.asinh(x).output(0))
_unary("acosh", lambda x: ops.acosh(x).output(0))
_unary("atanh", lambda x: ops.atanh(x).output(0))
_unary("log_sigmoid", lambda x: ops.negative(ops.softplus(ops.negative(x))).output(0))
_unary("logit", lambda x: ops.log(ops.divide(x, ops.subtract(_c(1.0, x), x))).output(0))
_unary("erfinv", lambda x: ops.erfinv(x).output(0))


@_op("aten.round.default", "aten.round.decimals")
def _round(ctx, n):
    x = ctx.out(n.args[0])
    dec = int(n.kwargs.get("decimals", n.args[1] if len(n.args) > 1 else 0))
    if dec == 0:
        return ops.round(x, "half_to_even").output(0)
    s = _c(10.0 ** dec, x)
    return ops.divide(ops.round(ops.multiply(x, s), "half_to_even"), s).output(0)


@_op("aten.atan2.default")
def _atan2(ctx, n):
    y, x = ctx.out(n.args[0]), ctx.out(n.args[1])
    base = ops.atan(ops.divide(y, x))
    pi = _c(np.pi, x)
    zero = _c(0.0, x)
    # quadrant correction for x < 0; x == 0 gives +-pi/2 by the sign of y (0 for y == 0)
    corr = ops.select(ops.less(x, zero), ops.select(ops.greater_equal(y, zero), pi, ops.negative(pi)), zero)
    val = ops.add(base, corr)
    on_axis = ops.multiply(ops.sign(y), _c(np.pi / 2, x))
    return ops.select(ops.equal(x, zero), on_axis, val).output(0)


@_op("aten.hypot.default")
def _hypot(ctx, n):
    a, b = ctx.out(n.args[0]), ctx.out(n.args[1])
    return ops.sqrt(ops.add(ops.multiply(a, a), ops.multiply(b, b))).output(0)


@_op("aten.clamp.Tensor", "aten.clamp_min.Tensor", "aten.clamp_max.Tensor")
def _clamp_tensor(ctx, n):
    x = ctx.out(n.args[0])
    t = str(n.target)
    lo = n.args[1] if len(n.args) > 1 else n.kwargs.get("min")
    hi = n.args[2] if len(n.args) > 2 else n.kwargs.get("max")
    if "clamp_max" in t:
        lo, hi = None, n.args[1]
    if lo is not None:
        x = ops.maximum(x, ctx.out(lo, x)).output(0)
    if hi is not None:
        x = ops.minimum(x, ctx.out(hi, x)).output(0)
    return x


@_op("aten.var.correction", "aten.std.correction", "aten.var.dim", "aten.std.dim")
def _var(ctx, n):
    x = ctx.out(n.args[0])
    dims = n.args[1] if len(n.args) > 1 else n.kwargs.get("dim")
    t = str(n.target)
    if t.endswith(".dim"):
        correction = 1 if (n.args[2] if len(n.args) > 2 else n.kwargs.get("unbiased", True)) else 0
        keep = bool(n.args[3]) if len(n.args) > 3 else bool(n.kwargs.get("keepdim", False))
    else:
        correction = n.kwargs.get("correction", 1)
        correction = 1 if correction is None else correction
        keep = bool(n.kwargs.get("keepdim", False))
    r = _rank(x)
    dims = list(range(r)) if dims is None or dims == [] else ([dims] if isinstance(dims, int) else list(dims))
    axes = _i64(dims)
    mean = ops.reduce_mean(x, axes, True)
    d = ops.subtract(x, mean)
    ssq = ops.reduce_sum(ops.multiply(d, d), axes, keep)
    count = ops.reduce_prod(ops.gather(ops.shape_of(x), _i64([_axis(a, r) for a in dims]), _i64(0)), _i64([0]), False)
    denom = ops.subtract(ops.convert(count, x.get_element_type()), _c(float(correction), x))
    v = ops.divide(ssq, denom)
    return (ops.sqrt(v) if "std" in t else v).output(0)


@_op("aten.var_mean.correction")
def _var_mean(ctx, n):
    x = ctx.out(n.args[0])
    dims = n.args[1] if len(n.args) > 1 else n.kwargs.get("dim")
    keep = bool(n.kwargs.get("keepdim", False))
    r = _rank(x)
    dims = list(range(r)) if dims is None or dims == [] else ([dims] if isinstance(dims, int) else list(dims))
    return (_var(ctx, n), ops.reduce_mean(x, _i64(dims), keep).output(0))


@_op("aten.linalg_vector_norm.default")
def _vector_norm(ctx, n):
    x = ctx.out(n.args[0])
    p = n.args[1] if len(n.args) > 1 else n.kwargs.get("ord", 2)
    dims = n.args[2] if len(n.args) > 2 else n.kwargs.get("dim")
    keep = bool(n.args[3]) if len(n.args) > 3 else bool(n.kwargs.get("keepdim", False))
    r = _rank(x)
    axes = _i64(list(range(r)) if dims is None or dims == [] else ([dims] if isinstance(dims, int) else list(dims)))
    p = float(p)
    if p == 2.0:
        return ops.reduce_l2(x, axes, keep).output(0)
    if p == 1.0:
        return ops.reduce_l1(x, axes, keep).output(0)
    if p == float("inf"):
        return ops.reduce_max(ops.abs(x), axes, keep).output(0)
    if p == float("-inf"):
        return ops.reduce_min(ops.abs(x), axes, keep).output(0)
    if p == 0.0:
        return ops.reduce_sum(ops.convert(ops.not_equal(x, _c(0.0, x)), x.get_element_type()), axes, keep).output(0)
    return ops.power(ops.reduce_sum(ops.power(ops.abs(x), _c(p, x)), axes, keep), _c(1.0 / p, x)).output(0)


@_op("aten.flip.default")
def _flip(ctx, n):
    x = ctx.out(n.args[0])
    return ops.reverse(x, _i64([int(d) for d in n.args[1]]), "index").output(0)


@_op("aten.diagonal.default")
def _diagonal(ctx, n):
    x = ctx.out(n.args[0])
    offset = int(n.args[1]) if len(n.args) > 1 else int(n.kwargs.get("offset", 0))
    d1 = int(n.args[2]) if len(n.args) > 2 else int(n.kwargs.get("dim1", 0))
    d2 = int(n.args[3]) if len(n.args) > 3 else int(n.kwargs.get("dim2", 1))
    r = _rank(x)
    d1, d2 = _axis(d1, r), _axis(d2, r)
    shp = x.get_partial_shape()
    if not (shp[d1].is_static and shp[d2].is_static):
        raise ConversionError("diagonal over axes of unknown extent is not converted")
    n1, n2 = shp[d1].get_length(), shp[d2].get_length()
    length = max(0, min(n1 + min(offset, 0), n2 - max(offset, 0)))
    rows = np.arange(length, dtype=np.int64) + max(-offset, 0)
    cols = np.arange(length, dtype=np.int64) + max(offset, 0)
    # move the two axes to the end, flatten them and gather the diagonal positions
    rest = [a for a in range(r) if a not in (d1, d2)]
    xt = ops.transpose(x, _i64(rest + [d1, d2]))
    flat = ops.reshape(xt, _i64([0] * len(rest) + [-1]), True)
    return ops.gather(flat, _i64((rows * n2 + cols).tolist()), _i64(len(rest))).output(0)


@_op("aten.narrow.default")
def _narrow(ctx, n):
    x = ctx.out(n.args[0])
    dim, start, length = int(n.args[1]), n.args[2], n.args[3]
    s = ctx.ints(start)
    e = ops.add(s, ctx.ints(length)).output(0)
    return ops.slice(x, s, e, _i64([1]), _i64([dim])).output(0)


@_op("aten.movedim.int", "aten.movedim.intlist")
def _movedim(ctx, n):
    x = ctx.out(n.args[0])
    r = _rank(x)
    src = [n.args[1]] if isinstance(n.args[1], int) else list(n.args[1])
    dst = [n.args[2]] if isinstance(n.args[2], int) else list(n.args[2])
    src, dst = [_axis(a, r) for a in src], [_axis(a, r) for a in dst]
    order = [None] * r
    for s_, d_ in zip(src, dst):
        order[d_] = s_
    rest = [a for a in range(r) if a not in src]
    for k in range(r):
        if order[k] is None:
            order[k] = rest.pop(0)
    return ops.transpose(x, _i64(order)).output(0)


@_op("aten.tile.default")
def _tile(ctx, n):
    x = ctx.out(n.args[0])
    reps = [int(v) for v in n.args[1]]
    r = _rank(x)
    if len(reps) < r:
        reps = [1] * (r - len(reps)) + reps
    return ops.tile(x, _i64(reps)).output(0)


@_op("aten.sort.default", "aten.sort.stable")
def _sort(ctx, n):
    x = ctx.out(n.args[0])
    args = [a for a in n.args[1:] if not isinstance(a, bool) or True]
    dim = int(n.kwargs.get("dim", -1))
    desc = bool(n.kwargs.get("descending", False))
    ints = [a for a in n.args[1:] if isinstance(a, int) and not isinstance(a, bool)]
    bools = [a for a in n.args[1:] if isinstance(a, bool)]
    if ints:
        dim = int(ints[0])
    if str(n.target).endswith(".stable"):
        if len(bools) > 1:
            desc = bools[1]
    elif bools:
        desc = bools[0]
    r = _rank(x)
    k = ops.squeeze(ops.gather(ops.shape_of(x), _i64([_axis(dim, r)]), _i64(0)))
    t = ops.topk(x, k, _axis(dim, r), "max" if desc else "min", "value", "i64", stable=True)
    return (t.output(0), t.output(1))


@_op("aten.argsort.default", "aten.argsort.stable")
def _argsort(ctx, n):
    return _sort(ctx, n)[1]


@_op("aten.nonzero.default")
def _nonzero(ctx, n):
    return ops.transpose(ops.non_zero(ctx.out(n.args[0]), "i64"), _i64([1, 0])).output(0)


@_op("aten.cumprod.default")
def _cumprod(ctx, n):
    x = ctx.out(n.args[0])
    dim = int(n.args[1])
    # exp(cumsum(log|x|)) with the sign from the parity of the negative count; zeros handled through a mask
    zero = ops.equal(x, _c(0.0, x))
    safe = ops.select(zero, _c(1.0, x), ops.abs(x))
    mag = ops.exp(ops.cumsum(ops.log(safe), _i64(dim), False, False))
    negs = ops.cumsum(ops.convert(ops.less(x, _c(0.0, x)), x.get_element_type()), _i64(dim), False, False)
    sign = ops.subtract(_c(1.0, x), ops.multiply(_c(2.0, x), ops.floor_mod(negs, _c(2.0, x))))
    any_zero = ops.greater(ops.cumsum(ops.convert(zero, x.get_element_type()), _i64(dim), False, False), _c(0.0, x))
    return ops.select(any_zero, _c(0.0, x), ops.multiply(mag, sign)).output(0)


@_op("aten.prelu.default", "aten._prelu_kernel.default")
def _prelu(ctx, n):
    x, w = ctx.out(n.args[0]), ctx.out(n.args[1])
    r = _rank(x)
    if _rank(w) == 1 and r > 2:
        w = ops.reshape(w, _i64([1, -1] + [1] * (r - 2)), False).output(0)
    return ops.prelu(x, w).output(0)


@_op("aten.eye.default", "aten.eye.m")
def _eye(ctx, n):
    rows = int(n.args[0])
    cols = int(n.args[1]) if len(n.args) > 1 and isinstance(n.args[1], int) else rows
    dt = n.kwargs.get("dtype")
    from .pytorch import _ov_type
    return ops.eye(constant(np.array(rows, np.int64)), constant(np.array(cols, np.int64)), constant(np.array(0, np.int64)),
                   output_type=_ov_type(dt) if dt is not None else Type.f32).output(0)


@_op("aten.one_hot.default")
def _one_hot(ctx, n):
    x = ctx.out(n.args[0])
    classes = int(n.args[1]) if len(n.args) > 1 else int(n.kwargs.get("num_classes", -1))
    if classes < 0:
        raise ConversionError("one_hot needs num_classes")
    return ops.one_hot(x, constant(np.array(classes, np.int64)), constant(np.array(1, np.int64)), constant(np.array(0, np.int64)), -1).output(0)


@_op("aten.searchsorted.Tensor")
def _searchsorted(ctx, n):
    seq, vals = ctx.out(n.args[0]), ctx.out(n.args[1])
    right = bool(n.kwargs.get("right", False))
    out_i32 = bool(n.kwargs.get("out_int32", False))
    return ops.search_sorted(seq, vals, right, "i32" if out_i32 else "i64").output(0)


@_op("aten.bucketize.Tensor")
def _bucketize(ctx, n):
    x, b = ctx.out(n.args[0]), ctx.out(n.args[1])
    right = bool(n.kwargs.get("right", False))
    return ops.bucketize(x, b, "i32" if n.kwargs.get("out_int32", False) else "i64", not right).output(0)


@_op("aten.pixel_unshuffle.default")
def _pixel_unshuffle(ctx, n):
    return ops.space_to_depth(ctx.out(n.args[0]), "depth_first", int(n.args[1])).output(0)


@_op("aten.channel_shuffle.default")
def _channel_shuffle(ctx, n):
    return ops.shuffle_channels(ctx.out(n.args[0]), 1, int(n.args[1])).output(0)


def _pad_mode(mode):
    def fn(ctx, n):
        x = ctx.out(n.args[0])
        p = [int(v) for v in n.args[1]]
        r = _rank(x)
        pb, pe = [0] * r, [0] * r
        for k in range(len(p) // 2):
            pb[r - 1 - k], pe[r - 1 - k] = p[2 * k], p[2 * k + 1]
        return ops.pad(x, _i64(pb), _i64(pe), _c(0.0, x), mode).output(0)
    return fn


for _nm in ("reflection_pad1d", "reflection_pad2d", "reflection_pad3d"):
    _TABLE["aten.%s.default" % _nm] = _pad_mode("reflect")
for _nm in ("replication_pad1d", "replication_pad2d", "replication_pad3d"):
    _TABLE["aten.%s.default" % _nm] = _pad_mode("edge")


@_op("aten.grid_sampler_2d.default", "aten.grid_sampler.default")
def _grid_sampler(ctx, n):
    x, g = ctx.out(n.args[0]), ctx.out(n.args[1])
    mode = {0: "bilinear", 1: "nearest", 2: "bicubic"}[int(n.args[2])]
    pad = {0: "zeros", 1: "border", 2: "reflection"}[int(n.args[3])]
    return ops.grid_sample(x, g, bool(n.args[4]), mode, pad).output(0)


@_op("aten.index_add.default")
def _index_add(ctx, n):
    x, dim, idx, src = ctx.out(n.args[0]), int(n.args[1]), ctx.out(n.args[2]), ctx.out(n.args[3])
    alpha = n.kwargs.get("alpha", 1)
    if alpha != 1:
        src = ops.multiply(src, ctx.out(alpha, src)).output(0)
    r = _rank(x)
    dim = _axis(dim, r)
    # indices broadcast to the shape of the source along `dim`
    shape = [1] * r
    shape[dim] = -1
    idx_b = ops.broadcast(ops.reshape(idx, _i64(shape), False), ops.shape_of(src), "bidirectional")
    from .._graph import make_op
    return make_op("ScatterElementsUpdate", [x, idx_b.output(0), src, _i64(dim)], {"reduction": "sum", "use_init_val": True}).output(0)


@_op("aten.scatter_reduce.two")
def _scatter_reduce(ctx, n):
    x, dim, idx, src = ctx.out(n.args[0]), int(n.args[1]), ctx.out(n.args[2]), ctx.out(n.args[3])
    red = {"sum": "sum", "prod": "prod", "mean": "mean", "amax": "max", "amin": "min"}[n.args[4]]
    include_self = bool(n.kwargs.get("include_self", True))
    from .._graph import make_op
    return make_op("ScatterElementsUpdate", [x, idx, src, _i64(dim)], {"reduction": red, "use_init_val": include_self}).output(0)


@_op("aten.repeat_interleave.self_int")
def _repeat_interleave(ctx, n):
    x = ctx.out(n.args[0])
    reps = int(n.args[1])
    dim = n.args[2] if len(n.args) > 2 else n.kwargs.get("dim")
    if dim is None:
        x = ops.reshape(x, _i64([-1]), False).output(0)
        dim = 0
    r = _rank(x)
    dim = _axis(int(dim), r)
    u = ops.unsqueeze(x, _i64([dim + 1]))
    tiles = [1] * (r + 1)
    tiles[dim + 1] = reps
    t = ops.tile(u, _i64(tiles))
    shape = [0] * r
    shape[dim] = -1
    return ops.reshape(t, _i64(shape), True).output(0)


@_op("aten.upsample_bicubic2d.default", "aten.upsample_bicubic2d.vec")
def _upsample_bicubic(ctx, n):
    x = ctx.out(n.args[0])
    size = n.args[1]
    align = bool(n.args[2]) if len(n.args) > 2 else False
    if size is None:
        raise ConversionError("upsample_bicubic2d by scale factors is not converted")
    return ops.interpolate(x, ctx.ints(size), mode="cubic", shape_calculation_mode="sizes",
                           coordinate_transformation_mode="align_corners" if align else "pytorch_half_pixel", cube_coeff=-0.75, axes=_i64([2, 3])).output(0)


@_op("aten.multinomial.default")
def _multinomial(ctx, n):
    x = ctx.out(n.args[0])
    samples = int(n.args[1])
    repl = bool(n.args[2]) if len(n.args) > 2 else bool(n.kwargs.get("replacement", False))
    return ops.multinomial(x, constant(np.array([samples], np.int64)), "i64", repl, False, 0, 0).output(0)


@_op("aten.numel.default")
def _numel(ctx, n):
    return ops.reduce_prod(ops.shape_of(ctx.out(n.args[0])), _i64([0]), False).output(0)


@_op("aten.fill.Scalar", "aten.fill.Tensor", "aten.fill_.Scalar", "aten.fill_.Tensor")
def _fill(ctx, n):
    x = ctx.out(n.args[0])
    v = ctx.out(n.args[1], x)
    if v.get_element_type() != x.get_element_type():
        v = ops.convert(v, x.get_element_type()).output(0)
    return ops.broadcast(v, ops.shape_of(x)).output(0)


@_op("aten.dot.default", "aten.vdot.default")
def _dot(ctx, n):
    a, b = ctx.out(n.args[0]), ctx.out(n.args[1])
    return ops.reduce_sum(ops.multiply(a, b), _i64([0]), False).output(0)


@_op("aten.mv.default")
def _mv(ctx, n):
    a, v = ctx.out(n.args[0]), ctx.out(n.args[1])
    return ops.squeeze(ops.matmul(a, ops.unsqueeze(v, _i64([1])), False, False), _i64([1])).output(0)


@_op("aten.cross.default", "aten.linalg_cross.default")
def _cross(ctx, n):
    a, b = ctx.out(n.args[0]), ctx.out(n.args[1])
    dim = n.kwargs.get("dim", n.args[2] if len(n.args) > 2 else -1)
    dim = -1 if dim is None else int(dim)
    r = _rank(a)
    dim = _axis(dim, r)

    def roll(x, k):
        parts = ops.split(x, _i64(dim), 3)
        order = [(j + k) % 3 for j in range(3)]
        return ops.concat([parts.output(j) for j in order], dim).output(0)
    return ops.subtract(ops.multiply(roll(a, 1), roll(b, 2)), ops.multiply(roll(a, 2), roll(b, 1))).output(0)
