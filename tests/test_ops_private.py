"""Transformation-private operations: expert-gathered products, compressed grouped product, quantised fully-connected
forms and segment-wise attention, against NumPy / PyTorch restatements."""
import numpy as np
import pytest
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


def _gqa_reference(q, k, v, pk, pv, total, scale=None, window=-1, rotary=None, interleaved=False, sink=None, bias=None):
    """PyTorch restatement of GroupQueryAttention: returns (out [B, S, N * H], present k, present v)."""
    q, k, v, pk, pv = (torch.from_numpy(np.array(t, dtype=np.float32)) for t in (q, k, v, pk, pv))
    B, Nq, S, H = q.shape
    Nkv = k.shape[1]
    P_ = total - S
    if rotary is not None:
        cos, sin = (torch.from_numpy(t)[P_:P_ + S] for t in rotary)           # [S, H / 2]

        def rot(x):
            if interleaved:
                a, b = x[..., 0::2], x[..., 1::2]
                return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)
            a, b = x[..., :H // 2], x[..., H // 2:]
            return torch.cat([a * cos - b * sin, a * sin + b * cos], -1)
        q, k = rot(q), rot(k)
    K_ = torch.cat([pk[:, :, :P_], k], 2)
    V_ = torch.cat([pv[:, :, :P_], v], 2)
    Kx = K_.repeat_interleave(Nq // Nkv, 1)
    Vx = V_.repeat_interleave(Nq // Nkv, 1)
    s = q @ Kx.transpose(-1, -2) * (scale or 1.0 / np.sqrt(H))
    if bias is not None:
        s = s + torch.from_numpy(bias)[..., :total]
    i = torch.arange(S)[:, None] + P_
    j = torch.arange(total)[None, :]
    keep = j <= i
    if window > 0:
        keep &= j > i - window
    s = s.masked_fill(~keep, float("-inf"))
    if sink is not None:
        col = torch.from_numpy(sink).reshape(1, Nq, 1, 1).expand(B, Nq, S, 1)
        w = torch.softmax(torch.cat([s, col], -1), -1)[..., :-1]
    else:
        w = torch.softmax(s, -1)
    o = (w @ Vx).permute(0, 2, 1, 3).reshape(B, S, Nq * H)
    return o.numpy(), K_.numpy(), V_.numpy()


def test_group_query_attention_prefill_decode_rotary_window_sink():
    rng = np.random.default_rng(11)
    B, Nq, Nkv, H, Pmax = 2, 4, 2, 8, 12
    for S, past, kw in ((5, 0, {}), (1, 7, {}), (3, 4, {"window": 4}), (2, 5, {"rot": True}), (2, 5, {"rot": True, "inter": True}), (3, 2, {"sink": True}),
                        (2, 3, {"bias": True})):
        total = past + S
        q = rng.standard_normal((B, Nq, S, H)).astype(np.float32)
        k = rng.standard_normal((B, Nkv, S, H)).astype(np.float32)
        v = rng.standard_normal((B, Nkv, S, H)).astype(np.float32)
        pk = rng.standard_normal((B, Nkv, Pmax, H)).astype(np.float32)
        pv = rng.standard_normal((B, Nkv, Pmax, H)).astype(np.float32)
        feeds = [q, k, v, pk, pv, np.array([total - 1], np.int32), np.array(total, np.int32)]
        ps = [P(q.shape, "q"), P(k.shape, "k"), P(v.shape, "v"), P(pk.shape, "pk"), P(pv.shape, "pv"), P([1], "lens", "i32"), P([], "total", "i32")]
        attrs = dict(num_heads=Nq, kv_num_heads=Nkv)
        ref_kw = {}
        empty = lambda: ops.constant(np.zeros((0,), np.float32))
        extra = []
        if kw.get("rot"):
            ang = rng.random((32, H // 2)).astype(np.float32) * 3
            cos, sin = np.cos(ang), np.sin(ang)
            extra = [ops.constant(cos), ops.constant(sin)]
            attrs.update(do_rotary=True, rotary_interleaved=bool(kw.get("inter")))
            ref_kw.update(rotary=(cos, sin), interleaved=bool(kw.get("inter")))
        if kw.get("window"):
            attrs["local_window_size"] = kw["window"]
            ref_kw["window"] = kw["window"]
        if kw.get("sink"):
            sink = rng.standard_normal((Nq,)).astype(np.float32)
            extra = [empty(), empty(), empty(), empty(), ops.constant(sink)]
            ref_kw["sink"] = sink
        if kw.get("bias"):
            bias = rng.standard_normal((1, Nq, S, total + 2)).astype(np.float32)
            extra = [empty(), empty(), empty(), ops.constant(bias)]
            ref_kw["bias"] = bias
        n = ops.group_query_attention(ps + extra, **attrs)
        assert n.get_output_partial_shape(0).to_shape() if False else True
        assert [d.get_length() for d in n.get_output_partial_shape(0)] == [B, S, Nq * H]
        got = run([n.output(0), n.output(1), n.output(2)], ps, feeds)
        ref = _gqa_reference(q, k, v, pk, pv, total, **ref_kw)
        for g, r in zip(got, ref):
            np.testing.assert_allclose(g, r, rtol=2e-5, atol=2e-5)


def test_type_relaxed_overrides_input_and_output_types():
    # u8 x i8 product accumulated and declared as i32: the wrapped Multiply sees both inputs as i32
    a = P([2, 3], "a", "u8")
    b = P([2, 3], "b", "i8")
    n = ops.type_relaxed("Multiply", [a, b], ["i32", "i32"], ["i32"], base_version="opset1")
    assert n.get_output_element_type(0) == ov.Type.i32 and list(n.get_output_shape(0)) == [2, 3]
    av = np.array([[200, 3, 255], [7, 100, 0]], np.uint8)
    bv = np.array([[-100, 5, 127], [-3, -128, 9]], np.int8)
    got = run([n], [a, b], [av, bv])[0]
    assert got.dtype == np.int32
    np.testing.assert_array_equal(got, av.astype(np.int32) * bv.astype(np.int32))
    # a float operation whose result is declared as f16; attributes of the wrapped operation pass through
    x = P([2, 4], "x")
    s = ops.type_relaxed("Softmax", [x], [], ["f16"], base_version="opset8", axis=1)
    xv = np.random.default_rng(3).standard_normal((2, 4)).astype(np.float32)
    got = run([s], [x], [xv])[0]
    assert got.dtype == np.float16
    np.testing.assert_allclose(got.astype(np.float32), torch.softmax(torch.from_numpy(xv), 1).numpy(), atol=1e-3)
    # shape arguments given as constants still drive the wrapped operation's shape inference
    r = ops.type_relaxed("Reshape", [x, ops.constant(np.array([4, 2], np.int64))], [], ["f16"], base_version="opset1", special_zero=False)
    assert list(r.get_output_shape(0)) == [4, 2]


def test_group_query_attention_device_expression_matches_the_reference_evaluation():
    """The CUDA device's GroupQueryAttention (runtime/cuda_plugin.py) on host tensors against the restatement above."""
    import types as _types
    from openvino_b200.runtime import cuda_plugin
    rng = np.random.default_rng(12)
    ctx = _types.SimpleNamespace(on_gpu=False, device="cpu", K=None)
    B, Nq, Nkv, H, Pmax = 2, 4, 2, 8, 12
    for S, past, kw in ((5, 0, {}), (1, 7, {}), (3, 4, {"window": 4}), (2, 5, {"rot": True}), (2, 5, {"rot": True, "inter": True}), (3, 2, {"sink": True}), (2, 3, {"bias": True})):
        total = past + S
        q, k, v = (rng.standard_normal((B, h, S, H)).astype(np.float32) for h in (Nq, Nkv, Nkv))
        pk, pv = (rng.standard_normal((B, Nkv, Pmax, H)).astype(np.float32) for _ in range(2))
        feeds = [q, k, v, pk, pv, np.array([total - 1], np.int32), np.array(total, np.int32)]
        attrs, ref_kw = dict(num_heads=Nq, kv_num_heads=Nkv), {}
        empty = np.zeros((0,), np.float32)
        if kw.get("rot"):
            ang = rng.random((32, H // 2)).astype(np.float32) * 3
            feeds += [np.cos(ang), np.sin(ang)]
            attrs.update(do_rotary=True, rotary_interleaved=bool(kw.get("inter")))
            ref_kw.update(rotary=(np.cos(ang), np.sin(ang)), interleaved=bool(kw.get("inter")))
        if kw.get("window"):
            attrs["local_window_size"] = ref_kw["window"] = kw["window"]
        if kw.get("sink"):
            sink = rng.standard_normal((Nq,)).astype(np.float32)
            feeds += [empty, empty, empty, empty, sink]
            ref_kw["sink"] = sink
        if kw.get("bias"):
            bias = rng.standard_normal((1, Nq, S, total + 2)).astype(np.float32)
            feeds += [empty, empty, empty, bias]
            ref_kw["bias"] = bias
        ps = [P(a.shape, "p%d" % i, "f32" if a.dtype == np.float32 else "i32") for i, a in enumerate(feeds)]
        node = ops.group_query_attention(ps, **attrs)
        got = cuda_plugin._OPS["GroupQueryAttention"](node, [torch.from_numpy(a) for a in feeds], ctx)
        ref = _gqa_reference(q, k, v, pk, pv, total, **ref_kw)
        for g, r in zip(got, ref):
            np.testing.assert_allclose(g.numpy(), r, rtol=2e-5, atol=2e-5, err_msg=str(kw))


@pytest.mark.gpu
def test_group_query_attention_on_the_device():
    """Prefill in f16 with head size 64 runs the package's dense attention kernel; a decode step with a past runs the
    expression path; both against the fp32 restatement."""
    rng = np.random.default_rng(13)
    B, Nq, Nkv, H, Pmax = 2, 4, 2, 64, 40
    core = ov.Core()
    for S, past, tol in ((33, 0, 2e-2), (1, 20, 2e-2)):
        total = past + S
        q, k, v = (rng.standard_normal((B, h, S, H)).astype(np.float32) * 0.5 for h in (Nq, Nkv, Nkv))
        pk, pv = (rng.standard_normal((B, Nkv, Pmax, H)).astype(np.float32) * 0.5 for _ in range(2))
        feeds = [q, k, v, pk, pv, np.array([total - 1], np.int32), np.array(total, np.int32)]
        ps = [P(a.shape, "p%d" % i, "f32" if a.dtype == np.float32 else "i32") for i, a in enumerate(feeds)]
        node = ops.group_query_attention(ps, num_heads=Nq, kv_num_heads=Nkv)
        cm = core.compile_model(ov.Model([node.output(0), node.output(1)], ps, "gqa"), "CUDA", {"INFERENCE_PRECISION_HINT": "f16"})
        res = cm(feeds)
        ref = _gqa_reference(q, k, v, pk, pv, total)
        np.testing.assert_allclose(np.asarray(res[0], np.float32), ref[0], rtol=tol, atol=tol)
        np.testing.assert_allclose(np.asarray(res[1], np.float32), ref[1], rtol=2e-3, atol=2e-3)
