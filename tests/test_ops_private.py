"""Transformation-private operations: expert-gathered products, compressed grouped product, quantised fully-connected
forms and segment-wise attention, against NumPy / PyTorch restatements."""
import numpy as np
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops


def run(outputs, params, feeds):
    m = ov.Model(outputs, params, "t")
    xml, weights = ov._ovcore.serialize(m._m)
    back = ov.Model._wrap(ov._ovcore.deserialize(xml.decode(), np.frombuffer(weights, dtype=np.uint8)))
    res = ov.compile_model(back, "CPU")(feeds)
    return [res[i] for i in range(len(outputs))]


def P(shape, name, dt="f32"):
    return ops.parameter(list(shape), dt, name)


def test_gather_matmul_plain_and_compressed():
    rng = np.random.default_rng(0)
    E, Nn, Kk, T, top = 4, 6, 8, 5, 2
    a = rng.standard_normal((top, T, Kk)).astype(np.float32)
    b = rng.standard_normal((E, Nn, Kk)).astype(np.float32)
    idx = rng.integers(0, E, (T, top)).astype(np.int32)
    bias = rng.standard_normal((Nn,)).astype(np.float32)
    ps = [P(a.shape, "a"), P(b.shape, "b"), P(idx.shape, "i", "i32"), P(bias.shape, "bias")]
    n = ops.gather_matmul(*ps)
    assert list(n.get_output_shape(0)) == [top, T, Nn]
    ref = np.stack([np.stack([a[s, t] @ b[idx[t, s]].T + bias for t in range(T)]) for s in range(top)])
    np.testing.assert_allclose(run([n], ps, [a, b, idx, bias])[0], ref, rtol=1e-5, atol=1e-5)
    # one shared activation for all slots; weights u8 with per-group scales and zero points [E, N, G, gs]
    G = 2
    q = rng.integers(0, 256, (E, Nn, G, Kk // G)).astype(np.uint8)
    sc = (rng.random((E, Nn, G, 1)) * 0.02 + 0.01).astype(np.float32)
    zp = rng.integers(100, 156, (E, Nn, G, 1)).astype(np.float32)
    a1 = a[:1]
    ps = [P(a1.shape, "a"), P(q.shape, "q", "u8"), P(idx.shape, "i", "i32"), P([0], "nb"), P(sc.shape, "s"), P(zp.shape, "z")]
    n = ops.gather_matmul_compressed(*ps)
    w = ((q.astype(np.float32) - zp) * sc).reshape(E, Nn, Kk)
    ref = np.stack([np.stack([a1[0, t] @ w[idx[t, s]].T for t in range(T)]) for s in range(top)])
    got = run([n], ps, [a1, q, idx, np.zeros((0,), np.float32), sc, zp])[0]
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)


def test_grouped_matmul_compressed_with_offsets():
    rng = np.random.default_rng(1)
    G, Nn, Kk = 3, 4, 8
    a = rng.standard_normal((7, Kk)).astype(np.float32)
    q = rng.integers(-8, 8, (G, Nn, Kk)).astype(np.int8)
    sc = (rng.random((G, Nn, 1)) * 0.1 + 0.05).astype(np.float32)
    offs = np.array([2, 2, 7], np.int32)                   # group 1 is empty
    ps = [P(a.shape, "a"), P(q.shape, "q", "i8"), P([G], "o", "i32"), P(sc.shape, "s")]
    n = ops.grouped_matmul_compressed(ps)
    w = q.astype(np.float32) * sc
    ref = np.concatenate([a[:2] @ w[0].T, a[2:7] @ w[2].T])
    np.testing.assert_allclose(run([n], ps, [a, q, offs, sc])[0], ref, rtol=1e-5, atol=1e-5)
    a3 = rng.standard_normal((G, 2, Kk)).astype(np.float32)
    ps = [P(a3.shape, "a"), P(q.shape, "q", "i8"), P(sc.shape, "s")]
    n3 = ops.grouped_matmul_compressed(ps)
    np.testing.assert_allclose(run([n3], ps, [a3, q, sc])[0], np.einsum("gmk,gnk->gmn", a3, w), rtol=1e-5, atol=1e-5)


def test_fully_connected_quantized_forms():
    rng = np.random.default_rng(2)
    x = rng.integers(0, 256, (3, 8)).astype(np.uint8)
    w = rng.integers(-127, 128, (5, 8)).astype(np.int8)
    bias = rng.standard_normal((5,)).astype(np.float32)
    deq = (rng.random((5,)) * 0.01 + 0.001).astype(np.float32)
    ps = [P(x.shape, "x", "u8"), P(w.shape, "w", "i8"), P([5], "b"), P([5], "d")]
    n = ops.fully_connected_quantized_legacy(*ps, output_type="f32")
    ref = (x.astype(np.float32) @ w.astype(np.float32).T) * deq + bias
    np.testing.assert_allclose(run([n], ps, [x, w, bias, deq])[0], ref, rtol=1e-5, atol=1e-4)
    ws, wz = (rng.random((5,)) * 0.02 + 0.01).astype(np.float32), np.zeros((5,), np.float32)
    xs, xz = np.array([0.05], np.float32), np.array([128.0], np.float32)
    os_, oz = np.array([0.1], np.float32), np.array([3.0], np.float32)
    ps = [P(x.shape, "x", "u8"), P(w.shape, "w", "i8"), P([5], "b"), P([5], "ws"), P([5], "wz"), P([1], "xs"), P([1], "xz"), P([1], "os"), P([1], "oz")]
    n = ops.fully_connected_quantized(*ps, output_type="f32")
    real = ((x.astype(np.float32) - 128) * 0.05) @ (w.astype(np.float32) * ws[:, None]).T + bias
    np.testing.assert_allclose(run([n], ps, [x, w, bias, ws, wz, xs, xz, os_, oz])[0], real / 0.1 + 3, rtol=1e-4, atol=1e-4)


def test_vl_sdpa_attends_inside_segments():
    torch.manual_seed(3)
    L, H, S = 9, 2, 8
    q, k, v = torch.randn(L, H, S), torch.randn(L, H, S), torch.randn(L, H, S)
    cu = np.array([0, 4, 9], np.int32)
    ps = [P(q.shape, "q"), P(k.shape, "k"), P(v.shape, "v"), P([3], "c", "i32")]
    n = ops.vl_sdpa(*ps, order_q=[1, 0, 2], order_k=[1, 0, 2], order_v=[1, 0, 2], order_out=[1, 0, 2])
    got = run([n], ps, [q.numpy(), k.numpy(), v.numpy(), cu])[0]
    ref = torch.zeros(L, H, S)
    for b, e in ((0, 4), (4, 9)):
        o = torch.nn.functional.scaled_dot_product_attention(q[b:e].transpose(0, 1), k[b:e].transpose(0, 1), v[b:e].transpose(0, 1))
        ref[b:e] = o.transpose(0, 1)
    np.testing.assert_allclose(got, ref.numpy(), rtol=1e-4, atol=1e-5)


def test_static_shape_suppression_forms_pad_the_dynamic_ones():
    from openvino_b200._graph import make_op
    rng = np.random.default_rng(5)
    B, M, Cn = 1, 6, 2
    xy = rng.random((B, M, 2)).astype(np.float32) * 0.5
    boxes = np.concatenate([xy, xy + 0.3], -1).astype(np.float32)
    scores = rng.random((B, Cn, M)).astype(np.float32)
    pb, ps = P(boxes.shape, "b"), P(scores.shape, "s")
    dyn = ops.non_max_suppression(pb, ps, np.int64(3), np.float32(0.4), np.float32(0.1))
    d_idx, d_sc, d_valid = run([dyn.output(0), dyn.output(1), dyn.output(2)], [pb, ps], [boxes, scores])
    st = make_op("NonMaxSuppressionIEInternal", [pb, ps, ops.constant(np.int64(3)), ops.constant(np.float32(0.4)), ops.constant(np.float32(0.1))],
                 {"center_point_box": 0, "sort_result_descending": True, "output_type": "i64", "score_output_type": "f32", "rotation": 0}, version="ie_internal_opset")
    assert list(st.get_output_shape(0)) == [3 * Cn * B, 3]
    s_idx, s_sc, s_valid = run([st.output(0), st.output(1), st.output(2)], [pb, ps], [boxes, scores])
    k = int(d_valid[0])
    assert int(s_valid[0]) == k and s_idx.shape == (6, 3)
    np.testing.assert_array_equal(s_idx[:k], d_idx[:k])
    np.testing.assert_allclose(s_sc[:k], d_sc[:k])
    assert (s_idx[k:] == -1).all() and (s_sc[k:] == -1).all()
    # multiclass form
    mc_dyn = ops.multiclass_nms(pb, ps, iou_threshold=0.4, score_threshold=0.2, keep_top_k=4)
    d_sel, d_i, d_n = run([mc_dyn.output(0), mc_dyn.output(1), mc_dyn.output(2)], [pb, ps], [boxes, scores])
    mc_st = make_op("MulticlassNmsIEInternal", [pb, ps], {"iou_threshold": 0.4, "score_threshold": 0.2, "keep_top_k": 4}, version="ie_internal_opset")
    assert list(mc_st.get_output_shape(0)) == [4, 6] and list(mc_st.get_output_shape(1)) == [4, 1]
    s_sel, s_i, s_n = run([mc_st.output(0), mc_st.output(1), mc_st.output(2)], [pb, ps], [boxes, scores])
    k = int(d_n[0])
    np.testing.assert_allclose(s_sel[:k], d_sel, rtol=1e-6)
    np.testing.assert_array_equal(s_i[:k], d_i)
    assert (s_sel[k:] == -1).all() and int(s_n[0]) == k


def test_einsum_reference_evaluation():
    rng = np.random.default_rng(7)
    a, b, c = rng.standard_normal((2, 3, 4)).astype(np.float32), rng.standard_normal((2, 4, 5)).astype(np.float32), rng.standard_normal((5,)).astype(np.float32)
    pa, pb, pc = P(a.shape, "a"), P(b.shape, "b"), P(c.shape, "c")
    for eq, ins, feeds in (("bij,bjk->bik", [pa, pb], [a, b]), ("...ij,...jk,k->...i", [pa, pb, pc], [a, b, c]), ("bij->jb", [pa], [a]), ("bij,bjk", [pa, pb], [a, b])):
        n = ops.einsum(ins, eq)
        got = run([n], ins, feeds)[0]
        np.testing.assert_allclose(got, np.einsum(eq, *feeds), rtol=1e-4, atol=1e-5)
    sq = rng.standard_normal((4, 4)).astype(np.float32)
    ps = P(sq.shape, "s")
    np.testing.assert_allclose(run([ops.einsum([ps], "ii->i")], [ps], [sq])[0], np.diag(sq), rtol=1e-6)
