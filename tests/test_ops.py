"""Operation set: shape/type inference (static, dynamic, interval) and reference evaluation against numpy / torch.

Follows the per-op pattern of the reference's type_prop and eval suites (src/core/tests/type_prop/*.cpp,
src/core/tests/eval.cpp): build one op, check inferred types and shapes, then evaluate and compare.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import openvino_b200 as ov
from openvino_b200 import Model, PartialShape, Tensor, Type
from openvino_b200 import opset as ops
from openvino_b200 import _ovcore as _c


def run(outputs, params, *arrays):
    outs = outputs if isinstance(outputs, (list, tuple)) else [outputs]
    m = Model([o if isinstance(o, ov.Output) else o.output(0) for o in outs], list(params), "t")
    res, _ = _c.evaluate(m._m, [Tensor(a)._to_core() for a in arrays])
    return [Tensor._from_core(r).data for r in res]


def P(shape, t="f32", name=None):
    return ops.parameter(shape, t, name)


rng = np.random.default_rng(0)


# ---------------------------------------------------------------------------------------- inference
def test_binary_broadcast_inference():
    a, b = P([2, 1, 4]), P([3, 1])
    assert ops.add(a, b).get_output_partial_shape(0) == [2, 3, 4]
    d = ops.add(P([-1, 3]), P([2, -1, 1]))
    assert d.get_output_partial_shape(0).to_string() == "[2,?,3]"
    with pytest.raises(RuntimeError):
        ops.add(P([2, 3]), P([4, 3]))
    with pytest.raises(RuntimeError):
        ops.add(P([2]), P([2], "i32"))
    assert ops.less(a, b).get_output_element_type(0) == Type.boolean


def test_interval_dims_propagate():
    a = P(PartialShape([(1, 4), 8]))
    assert ops.relu(a).get_output_partial_shape(0).to_string() == "[1..4,8]"
    c = ops.concat([a, P(PartialShape([(2, 3), 8]))], 0)
    assert c.get_output_partial_shape(0).to_string() == "[3..7,8]"


def test_matmul_inference():
    assert ops.matmul(P([2, 3, 4]), P([4, 5])).get_output_partial_shape(0) == [2, 3, 5]
    assert ops.matmul(P([2, 3, 4]), P([5, 4]), False, True).get_output_partial_shape(0) == [2, 3, 5]
    assert ops.matmul(P([-1, 3, 4]), P([7, 1, 4, 5])).get_output_partial_shape(0).to_string() == "[7,?,3,5]"
    with pytest.raises(RuntimeError):
        ops.matmul(P([2, 3]), P([4, 5]))


def test_convolution_and_pool_inference():
    y = ops.convolution(P([1, 3, 224, 224]), P([64, 3, 7, 7]), [2, 2], [3, 3], [3, 3], [1, 1])
    assert y.get_output_partial_shape(0) == [1, 64, 112, 112]
    y = ops.convolution(P([-1, 3, -1, 20]), P([8, 3, 3, 3]), [1, 1], [0, 0], [0, 0], [1, 1], "same_upper")
    assert y.get_output_partial_shape(0).to_string() == "[?,8,?,20]"
    g = ops.group_convolution(P([1, 8, 10, 10]), P([4, 3, 2, 3, 3]), [1, 1], [1, 1], [1, 1], [1, 1])
    assert g.get_output_partial_shape(0) == [1, 12, 10, 10]
    p = ops.max_pool(P([1, 4, 9, 9]), [2, 2], [1, 1], [0, 0], [0, 0], [3, 3], "ceil")
    assert p.get_output_partial_shape(0) == [1, 4, 4, 4] and p.get_output_size() == 2
    assert p.get_output_element_type(1) == Type.i64


def test_reshape_special_values_and_value_propagation():
    x = P([2, 3, 4])
    assert ops.reshape(x, [0, -1], True).get_output_partial_shape(0) == [2, 12]
    assert ops.reshape(x, [-1, 6], False).get_output_partial_shape(0) == [4, 6]
    d = P([-1, 3, 4])
    # ShapeOf -> Gather -> Concat keeps the symbolic batch
    batch = ops.gather(ops.shape_of(d), [0], 0)
    r = ops.reshape(d, ops.concat([batch, np.array([12], dtype=np.int64)], 0), False)
    assert r.get_output_partial_shape(0).to_string() == "[?,12]"
    s = P([5, 3, 4])
    batch = ops.gather(ops.shape_of(s), [0], 0)
    r = ops.reshape(s, ops.concat([batch, np.array([-1], dtype=np.int64)], 0), False)
    assert r.get_output_partial_shape(0) == [5, 12]


def test_misc_inference():
    x = P([2, 3, 4])
    assert ops.transpose(x, [2, 0, 1]).get_output_partial_shape(0) == [4, 2, 3]
    assert ops.unsqueeze(x, [0, 4]).get_output_partial_shape(0) == [1, 2, 3, 4, 1]
    assert ops.squeeze(P([1, 3, 1]), [0, 2]).get_output_partial_shape(0) == [3]
    assert ops.reduce_sum(x, [1], True).get_output_partial_shape(0) == [2, 1, 4]
    assert ops.reduce_mean(x, [0, 2]).get_output_partial_shape(0) == [3]
    sp = ops.split(x, 2, 2)
    assert sp.get_output_size() == 2 and sp.get_output_partial_shape(1) == [2, 3, 2]
    vs = ops.variadic_split(x, 1, [1, -1])
    assert vs.get_output_partial_shape(1) == [2, 2, 4]
    assert ops.gather(x, P([5], "i32"), 1).get_output_partial_shape(0) == [2, 5, 4]
    assert ops.slice(x, [1], [3], [1], [2]).get_output_partial_shape(0) == [2, 3, 2]
    assert ops.broadcast(P([3, 1]), [2, 3, 4]).get_output_partial_shape(0) == [2, 3, 4]
    assert ops.shape_of(x, "i32").get_output_element_type(0) == Type.i32
    assert ops.convert(x, "f16").get_output_element_type(0) == Type.f16
    assert ops.topk(x, 2, 2, "max", "value").get_output_partial_shape(1) == [2, 3, 2]
    assert ops.tile(x, [2, 1, 1]).get_output_partial_shape(0) == [4, 3, 4]
    assert ops.one_hot(P([3], "i64"), 5, 1.0, 0.0, -1).get_output_partial_shape(0) == [3, 5]
    assert ops.strided_slice(x, [0, 1], [0, 3], [1, 1], [1, 0], [1, 0]).get_output_partial_shape(0) == [2, 2, 4]
    assert ops.range(0, 10, 2, "i32").get_output_partial_shape(0) == [5]
    assert ops.select(P([2, 3, 4], "boolean"), x, x).get_output_partial_shape(0) == [2, 3, 4]
    assert ops.non_zero(x).get_output_partial_shape(0).to_string() == "[3,..24]"


def test_attributes_visible_and_settable():
    c = ops.convolution(P([1, 3, 8, 8]), P([4, 3, 3, 3]), [2, 2], [1, 1], [1, 1], [1, 1])
    a = c.get_attributes()
    assert a["strides"] == [2, 2] and a["auto_pad"] == "explicit" and list(a) == ["strides", "dilations", "pads_begin", "pads_end", "auto_pad"]
    c.set_attribute("strides", [1, 1])
    c.validate()
    assert c.get_output_partial_shape(0) == [1, 4, 8, 8]
    assert c.get_type_name() == "Convolution" and c.get_version() == "opset1"
    assert ops.convert(c, "i32").get_attributes()["destination_type"] == Type.i32


def test_clone_with_new_inputs_and_names():
    x = P([2, 2], name="x")
    r = ops.relu(x, name="act")
    assert r.get_friendly_name() == "act"
    r2 = r.clone_with_new_inputs([P([4, 4])])
    assert r2.get_output_partial_shape(0) == [4, 4] and r2 != r
    r.output(0).set_names({"t1", "t0"})
    assert r.output(0).get_any_name() == "t0"
    assert x.output(0).get_target_inputs()[0].get_node() == r


# ---------------------------------------------------------------------------------------- evaluation
UNARY = [("abs", np.abs), ("exp", np.exp), ("negative", np.negative), ("relu", lambda v: np.maximum(v, 0)), ("sigmoid", lambda v: 1 / (1 + np.exp(-v))),
         ("tanh", np.tanh), ("floor", np.floor), ("ceiling", np.ceil), ("sign", np.sign), ("sin", np.sin), ("cos", np.cos), ("erf", lambda v: torch.erf(torch.tensor(v)).numpy()),
         ("hswish", lambda v: F.hardswish(torch.tensor(v)).numpy()), ("hsigmoid", lambda v: F.hardsigmoid(torch.tensor(v)).numpy()),
         ("mish", lambda v: F.mish(torch.tensor(v)).numpy()), ("softplus", lambda v: F.softplus(torch.tensor(v)).numpy()),
         ("swish", lambda v: F.silu(torch.tensor(v)).numpy()), ("gelu", lambda v: F.gelu(torch.tensor(v)).numpy()),
         ("softsign", lambda v: v / (1 + np.abs(v))), ("asinh", np.arcsinh), ("atan", np.arctan), ("sinh", np.sinh), ("cosh", np.cosh)]


@pytest.mark.parametrize("name,fn", UNARY, ids=[u[0] for u in UNARY])
def test_unary_eval(name, fn):
    x = rng.standard_normal((3, 5)).astype(np.float32)
    p = P([3, 5])
    (y,) = run(getattr(ops, name)(p), [p], x)
    np.testing.assert_allclose(y, fn(x), rtol=1e-5, atol=1e-6)


def test_sqrt_log_eval():
    x = rng.uniform(0.1, 4, (4, 4)).astype(np.float32)
    p = P([4, 4])
    np.testing.assert_allclose(run(ops.sqrt(p), [p], x)[0], np.sqrt(x), rtol=1e-6)
    np.testing.assert_allclose(run(ops.log(p), [p], x)[0], np.log(x), rtol=1e-5, atol=1e-6)


BINARY = [("add", np.add), ("subtract", np.subtract), ("multiply", np.multiply), ("divide", np.divide), ("maximum", np.maximum),
          ("minimum", np.minimum), ("squared_difference", lambda a, b: (a - b) ** 2), ("less", np.less), ("greater_equal", np.greater_equal),
          ("equal", np.equal)]


@pytest.mark.parametrize("name,fn", BINARY, ids=[b[0] for b in BINARY])
def test_binary_eval_broadcast(name, fn):
    a = rng.standard_normal((2, 1, 4)).astype(np.float32)
    b = rng.standard_normal((3, 1)).astype(np.float32) + 2.0
    pa, pb = P([2, 1, 4]), P([3, 1])
    (y,) = run(getattr(ops, name)(pa, pb), [pa, pb], a, b)
    np.testing.assert_allclose(y, fn(a, b), rtol=1e-6)


def test_integer_divide_and_mod():
    a = np.array([7, -7, 9, -9], dtype=np.int32)
    b = np.array([2, 2, -4, -4], dtype=np.int32)
    pa, pb = P([4], "i32"), P([4], "i32")
    np.testing.assert_array_equal(run(ops.divide(pa, pb), [pa, pb], a, b)[0], a // b)       # python (floor) division
    np.testing.assert_array_equal(run(ops.floor_mod(pa, pb), [pa, pb], a, b)[0], np.mod(a, b))
    np.testing.assert_array_equal(run(ops.mod(pa, pb), [pa, pb], a, b)[0], np.fmod(a, b))


def test_matmul_eval():
    a = rng.standard_normal((2, 3, 4)).astype(np.float32)
    b = rng.standard_normal((5, 4)).astype(np.float32)
    pa, pb = P([2, 3, 4]), P([5, 4])
    np.testing.assert_allclose(run(ops.matmul(pa, pb, False, True), [pa, pb], a, b)[0], a @ b.T, rtol=1e-5, atol=1e-5)
    c = rng.standard_normal((2, 4, 3)).astype(np.float32)
    pc = P([2, 4, 3])
    np.testing.assert_allclose(run(ops.matmul(pc, pb, True, True), [pc, pb], c, b)[0], c.transpose(0, 2, 1) @ b.T, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("stride,pad,dil,groups", [(1, 1, 1, 1), (2, 3, 1, 1), (1, 2, 2, 1), (1, 1, 1, 4), (2, 0, 1, 2)])
def test_convolution_eval(stride, pad, dil, groups):
    x = rng.standard_normal((2, 8, 13, 11)).astype(np.float32)
    k = 7 if pad == 3 else 3
    w = rng.standard_normal((12, 8 // groups, k, k)).astype(np.float32)
    ref = F.conv2d(torch.tensor(x), torch.tensor(w), None, stride, pad, dil, groups).numpy()
    px = P(list(x.shape))
    if groups == 1:
        node = ops.convolution(px, w, [stride] * 2, [pad] * 2, [pad] * 2, [dil] * 2)
    else:
        node = ops.group_convolution(px, w.reshape(groups, 12 // groups, 8 // groups, k, k), [stride] * 2, [pad] * 2, [pad] * 2, [dil] * 2)
    np.testing.assert_allclose(run(node, [px], x)[0], ref, rtol=1e-4, atol=1e-4)


def test_pooling_eval():
    x = rng.standard_normal((1, 3, 9, 10)).astype(np.float32)
    px = P(list(x.shape))
    mp = ops.max_pool(px, [2, 2], [1, 1], [1, 1], [1, 1], [3, 3], "floor")
    vals, idx = F.max_pool2d(torch.tensor(x), 3, 2, 1, return_indices=True)
    got = run([mp.output(0), mp.output(1)], [px], x)
    np.testing.assert_allclose(got[0], vals.numpy())
    np.testing.assert_array_equal(got[1], idx.numpy())
    ap = ops.avg_pool(px, [2, 2], [1, 1], [1, 1], [3, 3], True, "ceil")
    ref = F.avg_pool2d(torch.tensor(x), 3, 2, 1, ceil_mode=True, count_include_pad=False).numpy()
    np.testing.assert_allclose(run(ap, [px], x)[0], ref, rtol=1e-5, atol=1e-6)
    aa = ops.adaptive_avg_pool(px, np.array([4, 3], dtype=np.int64))
    np.testing.assert_allclose(run(aa, [px], x)[0], F.adaptive_avg_pool2d(torch.tensor(x), (4, 3)).numpy(), rtol=1e-5, atol=1e-6)


def test_norms_eval():
    x = rng.standard_normal((2, 6, 5, 5)).astype(np.float32)
    g, b, m, v = (rng.standard_normal(6).astype(np.float32) for _ in range(4))
    v = np.abs(v) + 0.5
    px = P(list(x.shape))
    bn = ops.batch_norm_inference(px, g, b, m, v, 1e-5)
    ref = F.batch_norm(torch.tensor(x), torch.tensor(m), torch.tensor(v), torch.tensor(g), torch.tensor(b), False, 0.0, 1e-5).numpy()
    np.testing.assert_allclose(run(bn, [px], x)[0], ref, rtol=1e-4, atol=1e-5)
    mvn = ops.mvn(px, [-1, -2], True, 1e-6, "inside_sqrt")
    ref = F.layer_norm(torch.tensor(x), [5, 5], eps=1e-6).numpy()
    np.testing.assert_allclose(run(mvn, [px], x)[0], ref, rtol=1e-4, atol=1e-5)
    gn = ops.group_normalization(px, g, b, 3, 1e-5)
    ref = F.group_norm(torch.tensor(x), 3, torch.tensor(g), torch.tensor(b), 1e-5).numpy()
    np.testing.assert_allclose(run(gn, [px], x)[0], ref, rtol=1e-4, atol=1e-5)
    l2 = ops.normalize_l2(px, [1], 1e-12, "add")
    np.testing.assert_allclose(run(l2, [px], x)[0], F.normalize(torch.tensor(x), dim=1).numpy(), rtol=1e-4, atol=1e-5)
    rms = ops.rms_norm(px, np.ones(5, np.float32), 1e-6)
    ref = x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6)
    np.testing.assert_allclose(run(rms, [px], x)[0], ref, rtol=1e-4, atol=1e-5)


def test_softmax_and_reductions_eval():
    x = rng.standard_normal((3, 4, 5)).astype(np.float32)
    px = P([3, 4, 5])
    np.testing.assert_allclose(run(ops.softmax(px, 1), [px], x)[0], F.softmax(torch.tensor(x), 1).numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run(ops.log_softmax(px, -1), [px], x)[0], F.log_softmax(torch.tensor(x), -1).numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(run(ops.reduce_sum(px, [0, 2], True), [px], x)[0], x.sum((0, 2), keepdims=True), rtol=1e-5)
    np.testing.assert_allclose(run(ops.reduce_mean(px, [1]), [px], x)[0], x.mean(1), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run(ops.reduce_max(px, [-1]), [px], x)[0], x.max(-1))
    np.testing.assert_allclose(run(ops.reduce_l2(px, [2]), [px], x)[0], np.sqrt((x * x).sum(2)), rtol=1e-5)
    np.testing.assert_allclose(run(ops.reduce_prod(px, [0]), [px], x)[0], x.prod(0), rtol=1e-5)
    np.testing.assert_allclose(run(ops.cumsum(px, 1), [px], x)[0], x.cumsum(1), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run(ops.cumsum(px, 2, True, True), [px], x)[0],
                               np.flip(np.cumsum(np.flip(x, 2), 2), 2) - x, rtol=1e-4, atol=1e-5)


def test_data_movement_eval():
    x = rng.standard_normal((2, 3, 4)).astype(np.float32)
    px = P([2, 3, 4])
    np.testing.assert_array_equal(run(ops.transpose(px, [2, 0, 1]), [px], x)[0], x.transpose(2, 0, 1))
    np.testing.assert_array_equal(run(ops.reshape(px, [0, -1], True), [px], x)[0], x.reshape(2, 12))
    np.testing.assert_array_equal(run(ops.concat([px, px], 1), [px], x)[0], np.concatenate([x, x], 1))
    sp = ops.split(px, 2, 2)
    got = run([sp.output(0), sp.output(1)], [px], x)
    np.testing.assert_array_equal(got[1], x[:, :, 2:])
    np.testing.assert_array_equal(run(ops.slice(px, [3, 0], [0, 3], [-1, 2], [2, 1]), [px], x)[0], x[:, 0:3:2, 3:0:-1])
    np.testing.assert_array_equal(run(ops.strided_slice(px, [0, 1, 0], [0, 3, 0], [1, 1, 2], [1, 0, 1], [1, 0, 1]), [px], x)[0], x[:, 1:3, ::2])
    np.testing.assert_array_equal(run(ops.strided_slice(px, [0, 1], [0, 0], [1, 1], [1, 0], [1, 0], [], [0, 1]), [px], x)[0], x[:, 1])
    idx = np.array([[2, 0], [1, 1]], dtype=np.int64)
    np.testing.assert_array_equal(run(ops.gather(px, idx, 1), [px], x)[0], np.take(x, idx, 1))
    np.testing.assert_array_equal(run(ops.gather(px, np.array([-1], dtype=np.int64), 2), [px], x)[0], x[:, :, [-1]])
    np.testing.assert_array_equal(run(ops.tile(px, [1, 2, 1]), [px], x)[0], np.tile(x, (1, 2, 1)))
    np.testing.assert_array_equal(run(ops.broadcast(ops.reduce_max(px, [2], True), [2, 3, 4]), [px], x)[0], np.broadcast_to(x.max(2, keepdims=True), x.shape))
    np.testing.assert_array_equal(run(ops.pad(px, [0, 1, 0], [0, 0, 2], np.float32(9), "constant"), [px], x)[0], np.pad(x, ((0, 0), (1, 0), (0, 2)), constant_values=9))
    np.testing.assert_array_equal(run(ops.pad(px, [0, 1, 1], [0, 1, 1], pad_mode="reflect"), [px], x)[0], np.pad(x, ((0, 0), (1, 1), (1, 1)), mode="reflect"))
    np.testing.assert_array_equal(run(ops.roll(px, [1, -1], [1, 2]), [px], x)[0], np.roll(x, (1, -1), (1, 2)))
    np.testing.assert_array_equal(run(ops.shape_of(px), [px], x)[0], [2, 3, 4])
    np.testing.assert_array_equal(run(ops.select(ops.greater(px, 0.0), px, ops.negative(px)), [px], x)[0], np.abs(x))


def test_scatter_gather_family_eval():
    x = np.zeros((3, 4), dtype=np.float32)
    px = P([3, 4])
    idx = np.array([[0, 1], [2, 3]], dtype=np.int64)
    upd = np.array([5.0, 7.0], dtype=np.float32)
    got = run(ops.scatter_nd_update(px, idx, upd), [px], x)[0]
    ref = x.copy(); ref[0, 1] = 5; ref[2, 3] = 7
    np.testing.assert_array_equal(got, ref)
    t = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    gi = torch.tensor([[0, 3], [1, 1], [2, 0]])
    pt = P([3, 4])
    np.testing.assert_array_equal(run(ops.gather_elements(pt, gi.numpy(), 1), [pt], t.numpy())[0], torch.gather(t, 1, gi).numpy())
    src = torch.ones(3, 2)
    got = run(ops.scatter_elements_update(pt, gi.numpy(), src.numpy(), 1, "sum"), [pt], t.numpy())[0]
    np.testing.assert_array_equal(got, t.clone().scatter_add(1, gi, src).numpy())
    nd = np.array([[0, 1], [2, 2]], dtype=np.int64)
    np.testing.assert_array_equal(run(ops.gather_nd(pt, nd), [pt], t.numpy())[0], [1.0, 10.0])
    nz = run(ops.non_zero(pt), [pt], np.eye(3, 4, dtype=np.float32))[0]
    np.testing.assert_array_equal(nz, np.stack(np.nonzero(np.eye(3, 4))))


def test_topk_onehot_range_eval():
    x = rng.standard_normal((3, 7)).astype(np.float32)
    px = P([3, 7])
    tk = ops.topk(px, 3, 1, "max", "value", "i64")
    v, i = torch.topk(torch.tensor(x), 3, 1)
    got = run([tk.output(0), tk.output(1)], [px], x)
    np.testing.assert_array_equal(got[0], v.numpy())
    np.testing.assert_array_equal(got[1], i.numpy())
    oh = ops.one_hot(np.array([1, 0, 3], dtype=np.int64), 4, np.float32(1), np.float32(0), -1)
    np.testing.assert_array_equal(run(oh, [])[0], np.eye(4, dtype=np.float32)[[1, 0, 3]])
    np.testing.assert_array_equal(run(ops.range(np.float32(1), np.float32(2), np.float32(0.25), "f32"), [])[0], np.arange(1, 2, 0.25, dtype=np.float32))


def test_convert_and_fake_quantize_eval():
    x = np.array([-1.7, 0.4, 2.6, 300.0], dtype=np.float32)
    px = P([4])
    np.testing.assert_array_equal(run(ops.convert(px, "i32"), [px], x)[0], x.astype(np.int32))
    np.testing.assert_array_equal(run(ops.convert(px, "boolean"), [px], x)[0], x != 0)
    fq = ops.fake_quantize(px, np.float32(-2), np.float32(2), np.float32(-2), np.float32(2), 5)
    np.testing.assert_allclose(run(fq, [px], x)[0], [-2.0, 0.0, 2.0, 2.0])
    h = ops.convert(ops.convert(px, "f16"), "f32")
    np.testing.assert_array_equal(run(h, [px], x)[0], x.astype(np.float16).astype(np.float32))


def test_interpolate_eval():
    x = rng.standard_normal((1, 2, 4, 5)).astype(np.float32)
    px = P([1, 2, 4, 5])
    n = ops.interpolate(px, np.array([8, 10], dtype=np.int64), np.array([2, 3], dtype=np.int64), "nearest", "sizes", [0] * 4, [0] * 4, "asymmetric", "floor")
    np.testing.assert_array_equal(run(n, [px], x)[0], F.interpolate(torch.tensor(x), size=(8, 10), mode="nearest").numpy())
    lin = ops.interpolate(px, np.array([7, 9], dtype=np.int64), np.array([2, 3], dtype=np.int64), "linear_onnx", "sizes", [0] * 4, [0] * 4, "pytorch_half_pixel")
    np.testing.assert_allclose(run(lin, [px], x)[0], F.interpolate(torch.tensor(x), size=(7, 9), mode="bilinear", align_corners=False).numpy(), rtol=1e-4, atol=1e-5)
    ac = ops.interpolate(px, np.array([7, 9], dtype=np.int64), np.array([2, 3], dtype=np.int64), "linear_onnx", "sizes", [0] * 4, [0] * 4, "align_corners")
    np.testing.assert_allclose(run(ac, [px], x)[0], F.interpolate(torch.tensor(x), size=(7, 9), mode="bilinear", align_corners=True).numpy(), rtol=1e-4, atol=1e-5)


def test_sdpa_eval():
    q = rng.standard_normal((2, 4, 6, 8)).astype(np.float32)
    k = rng.standard_normal((2, 4, 9, 8)).astype(np.float32)
    v = rng.standard_normal((2, 4, 9, 8)).astype(np.float32)
    pq, pk, pv = P(list(q.shape)), P(list(k.shape)), P(list(v.shape))
    ref = F.scaled_dot_product_attention(torch.tensor(q), torch.tensor(k), torch.tensor(v)).numpy()
    np.testing.assert_allclose(run(ops.scaled_dot_product_attention(pq, pk, pv), [pq, pk, pv], q, k, v)[0], ref, rtol=1e-4, atol=1e-5)
    k2, v2 = k[:, :, :6], v[:, :, :6]
    pk2, pv2 = P(list(k2.shape)), P(list(v2.shape))
    ref = F.scaled_dot_product_attention(torch.tensor(q), torch.tensor(k2), torch.tensor(v2), is_causal=True).numpy()
    got = run(ops.scaled_dot_product_attention(pq, pk2, pv2, causal=True), [pq, pk2, pv2], q, k2, v2)[0]
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)
    mask = rng.standard_normal((6, 9)).astype(np.float32)
    ref = F.scaled_dot_product_attention(torch.tensor(q), torch.tensor(k), torch.tensor(v), attn_mask=torch.tensor(mask)).numpy()
    got = run(ops.scaled_dot_product_attention(pq, pk, pv, mask), [pq, pk, pv], q, k, v)[0]
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)


def test_dynamic_shapes_evaluate_with_actual_sizes():
    p = P([-1, -1])
    y = ops.matmul(ops.relu(p), ops.transpose(p, [1, 0]))
    for n, k in ((2, 3), (5, 1)):
        x = rng.standard_normal((n, k)).astype(np.float32)
        np.testing.assert_allclose(run(y, [p], x)[0], np.maximum(x, 0) @ x.T, rtol=1e-5, atol=1e-6)


def test_if_and_loop_eval():
    # If: cond ? x + 1 : x * 2
    x = P([3]); cond = P([], "boolean")
    tp = P([3]); then_body = Model([ops.add(tp, np.float32(1))], [tp], "then")
    ep = P([3]); else_body = Model([ops.multiply(ep, np.float32(2))], [ep], "else")
    b = ops.if_op(cond)
    b.set_then_body(then_body); b.set_else_body(else_body)
    b.set_input(x, tp, ep)
    b.set_output(then_body.get_results()[0], else_body.get_results()[0])
    node = b.build()
    v = np.array([1, 2, 3], dtype=np.float32)
    np.testing.assert_array_equal(run(node, [cond, x], np.array(True), v)[0], v + 1)
    np.testing.assert_array_equal(run(node, [cond, x], np.array(False), v)[0], v * 2)
    # Loop: acc = acc + x, 4 times
    acc_p, x_p = P([3]), P([3])
    new_acc = ops.add(acc_p, x_p)
    body = Model([ops.constant(np.array(True)), new_acc], [acc_p, x_p], "body")
    lb = ops.loop(np.array(4, dtype=np.int64), np.array(True))
    lb.set_function(body)
    lb.set_special_body_ports(-1, 0)
    lb.set_merged_input(acc_p, np.zeros(3, np.float32), new_acc)
    lb.set_invariant_input(x_p, x)
    lb.get_iter_value(new_acc, -1)
    loop = lb.build()
    np.testing.assert_array_equal(run(loop, [x], v)[0], 4 * v)
