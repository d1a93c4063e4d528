"""Second part of the ONNX translator table (frontend/onnx_more.py) on models written by the test-side encoder of
tests/test_frontend_onnx.py, against NumPy / PyTorch."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import openvino_b200 as ov   # noqa: E402
from openvino_b200.frontend import onnx as fe   # noqa: E402
import test_frontend_onnx as W   # noqa: E402
from test_frontend_onnx import model, node   # noqa: E402

_ELEM = {np.dtype("float32"): 1, np.dtype("uint8"): 2, np.dtype("int8"): 3, np.dtype("int32"): 6, np.dtype("int64"): 7, np.dtype("bool"): 9}


def _tensor(name, arr):
    arr = np.ascontiguousarray(arr)
    return b"".join(W._int(1, d) for d in arr.shape) + W._int(2, _ELEM[arr.dtype]) + W._ld(8, name.encode()) + W._ld(9, arr.tobytes())


W.tensor = _tensor            # the encoder's initialisers may now be 8-bit as well


def run(nodes, inits, inputs, outputs, feeds):
    data = model(nodes, inits, inputs, outputs)
    m = fe.convert(data)
    res = ov.compile_model(m, "CPU")(feeds)
    return [res[i] for i in range(len(outputs))]


def test_activations_indexing_and_reductions():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 4, 5)).astype(np.float32)
    nodes = [node("Selu", ["x"], ["a"]), node("HardSigmoid", ["a"], ["b"], alpha=0.25, beta=0.4), node("Celu", ["b"], ["c"], alpha=1.5),
             node("ReduceLogSumExp", ["c"], ["d"], axes=[2], keepdims=1), node("Trilu", ["x", "k"], ["t"], upper=0),
             node("ReduceSumSquare", ["t"], ["e"], axes=[1, 2], keepdims=0), node("Hardmax", ["x"], ["hm"], axis=-1),
             node("Reciprocal", ["d"], ["rec"]), node("Round", ["x"], ["rnd"]), node("Size", ["x"], ["sz"])]
    d, e, hm, rec, rnd, sz = run(nodes, {"k": np.array(1, np.int64)}, [("x", 1, [3, 4, 5])],
                                 [("d", 1, [3, 4, 1]), ("e", 1, [3]), ("hm", 1, [3, 4, 5]), ("rec", 1, [3, 4, 1]), ("rnd", 1, [3, 4, 5]), ("sz", 7, [])], [x])
    t = torch.tensor(x)
    c = torch.nn.functional.celu(torch.clamp(0.25 * torch.selu(t) + 0.4, 0, 1), alpha=1.5)
    np.testing.assert_allclose(d, torch.logsumexp(c, 2, keepdim=True).numpy(), rtol=1e-5)
    np.testing.assert_allclose(e, (torch.tril(t, 1) ** 2).sum((1, 2)).numpy(), rtol=1e-5)
    np.testing.assert_array_equal(hm, torch.nn.functional.one_hot(t.argmax(-1), 5).float().numpy())
    np.testing.assert_allclose(rec, 1 / d, rtol=1e-6)
    np.testing.assert_array_equal(rnd, np.round(x))
    assert int(sz) == 60
    # OneHot / GatherND / ScatterND(add) / Compress
    idx = np.array([[0, 2], [3, 1]], np.int64)
    data = rng.standard_normal((4, 3, 2)).astype(np.float32)
    nodes = [node("OneHot", ["idx", "depth", "vals"], ["oh"], axis=-1), node("GatherND", ["data", "gidx"], ["g"]),
             node("ScatterND", ["data", "sidx", "upd"], ["s"], reduction=b"add"), node("Compress", ["data", "cond"], ["cp"], axis=0)]
    inits = {"depth": np.array(4, np.int64), "vals": np.array([-1.0, 2.0], np.float32), "gidx": np.array([[1, 2], [3, 0]], np.int64),
             "sidx": np.array([[0], [0]], np.int64), "upd": np.ones((2, 3, 2), np.float32), "cond": np.array([True, False, False, True])}
    oh, g, s, cp = run(nodes, inits, [("idx", 7, [2, 2]), ("data", 1, [4, 3, 2])], [("oh", 1, [2, 2, 4]), ("g", 1, [2, 2]), ("s", 1, [4, 3, 2]), ("cp", 1, [2, 3, 2])], [idx, data])
    np.testing.assert_array_equal(oh, np.where(np.eye(4)[idx] > 0, 2.0, -1.0))
    np.testing.assert_array_equal(g, np.stack([data[1, 2], data[3, 0]]))
    ref = data.copy()
    ref[0] += 2
    np.testing.assert_allclose(s, ref, rtol=1e-6)
    np.testing.assert_array_equal(cp, data[[0, 3]])


def test_quantisation_family():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((4, 6)).astype(np.float32) * 3
    nodes = [node("QuantizeLinear", ["x", "s", "z"], ["q"]), node("DequantizeLinear", ["q", "s", "z"], ["dq"]),
             node("DynamicQuantizeLinear", ["x"], ["y", "ys", "yz"]),
             node("DequantizeLinear", ["w", "ws"], ["wd"], axis=0), node("MatMulInteger", ["q", "wq", "z", "wz"], ["mi"])]
    w = rng.integers(-100, 100, (3, 6)).astype(np.int8)
    wq = rng.integers(0, 255, (6, 2)).astype(np.uint8)
    inits = {"s": np.array(0.05, np.float32), "z": np.array(120, np.uint8), "w": w, "ws": np.array([0.1, 0.2, 0.3], np.float32), "wq": wq, "wz": np.array(7, np.uint8)}
    q, dq, y, ys, yz, wd, mi = run(nodes, inits, [("x", 1, [4, 6])], [("q", 2, [4, 6]), ("dq", 1, [4, 6]), ("y", 2, [4, 6]), ("ys", 1, []), ("yz", 2, []), ("wd", 1, [3, 6]), ("mi", 6, [4, 2])], [x])
    qr = np.clip(np.round(x / 0.05) + 120, 0, 255)
    np.testing.assert_array_equal(q, qr.astype(np.uint8))
    np.testing.assert_allclose(dq, (qr - 120) * 0.05, rtol=1e-6)
    scale = (max(x.max(), 0) - min(x.min(), 0)) / 255
    zp = np.clip(np.round(-min(x.min(), 0) / scale), 0, 255)
    np.testing.assert_allclose(ys, scale, rtol=1e-6)
    assert int(yz) == int(zp)
    np.testing.assert_array_equal(y, np.clip(np.round(x / scale) + zp, 0, 255).astype(np.uint8))
    np.testing.assert_allclose(wd, w.astype(np.float32) * np.array([[0.1], [0.2], [0.3]], np.float32), rtol=1e-6)
    np.testing.assert_array_equal(mi, (qr.astype(np.int32) - 120) @ (wq.astype(np.int32) - 7))


def test_conv_transpose_and_lstm():
    torch.manual_seed(2)
    x = torch.randn(1, 4, 5, 5)
    w = torch.randn(4, 3, 3, 3)
    b = torch.randn(6)
    wg = torch.randn(4, 3, 3, 3)                         # two groups: [C, O / G, k, k]
    nodes = [node("ConvTranspose", ["x", "w"], ["y"], strides=[2, 2], pads=[1, 1, 1, 1], output_padding=[1, 1]),
             node("ConvTranspose", ["x", "wg", "b"], ["yg"], strides=[1, 1], group=2)]
    y, yg = run(nodes, {"w": w.numpy(), "wg": wg.numpy(), "b": b.numpy()}, [("x", 1, [1, 4, 5, 5])], [("y", 1, [1, 3, 10, 10]), ("yg", 1, [1, 6, 7, 7])], [x.numpy()])
    np.testing.assert_allclose(y, torch.nn.functional.conv_transpose2d(x, w, stride=2, padding=1, output_padding=1).numpy(), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(yg, torch.nn.functional.conv_transpose2d(x, wg, b, groups=2).numpy(), rtol=1e-4, atol=1e-4)
    # LSTM: ONNX gate order i o f c, torch order i f g o
    S, B, I, H = 5, 2, 3, 4
    lstm = torch.nn.LSTM(I, H)
    xs = torch.randn(S, B, I)
    with torch.no_grad():
        ref, (hn, cn) = lstm(xs)

    def regate(t):
        i_, f_, g_, o_ = t.chunk(4, 0)
        return torch.cat([i_, o_, f_, g_], 0)
    Wn, Rn = regate(lstm.weight_ih_l0.detach())[None].numpy(), regate(lstm.weight_hh_l0.detach())[None].numpy()
    Bn = torch.cat([regate(lstm.bias_ih_l0.detach()), regate(lstm.bias_hh_l0.detach())])[None].numpy()
    nodes = [node("LSTM", ["x", "W", "R", "B"], ["Y", "Yh", "Yc"], hidden_size=H)]
    Y, Yh, Yc = run(nodes, {"W": Wn, "R": Rn, "B": Bn}, [("x", 1, [S, B, I])], [("Y", 1, [S, 1, B, H]), ("Yh", 1, [1, B, H]), ("Yc", 1, [1, B, H])], [xs.numpy()])
    np.testing.assert_allclose(Y[:, 0], ref.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(Yh, hn.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(Yc, cn.numpy(), rtol=1e-4, atol=1e-5)


def test_transformer_contrib_operations():
    rng = np.random.default_rng(3)
    B, S, H = 2, 4, 8
    x, skip = rng.standard_normal((B, S, H)).astype(np.float32), rng.standard_normal((B, S, H)).astype(np.float32)
    gamma, beta, bias = rng.random(H).astype(np.float32) + 0.5, rng.standard_normal(H).astype(np.float32), rng.standard_normal(H).astype(np.float32)
    nodes = [node("SkipLayerNormalization", ["x", "skip", "gamma", "beta", "bias"], ["y", "", "", "sum"], epsilon=1e-5),
             node("BiasGelu", ["y", "bias"], ["bg"]), node("FastGelu", ["y"], ["fg"]), node("SimplifiedLayerNormalization", ["sum", "gamma"], ["rms"], epsilon=1e-6),
             node("FusedMatMul", ["x", "skip"], ["fm"], transB=1, alpha=0.5)]
    y, s, bg, fg, rms, fm = run(nodes, {"gamma": gamma, "beta": beta, "bias": bias}, [("x", 1, [B, S, H]), ("skip", 1, [B, S, H])],
                                [("y", 1, [B, S, H]), ("sum", 1, [B, S, H]), ("bg", 1, [B, S, H]), ("fg", 1, [B, S, H]), ("rms", 1, [B, S, H]), ("fm", 1, [B, S, S])], [x, skip])
    st = torch.tensor(x + skip + bias)
    ref = torch.nn.functional.layer_norm(st, [H], torch.tensor(gamma), torch.tensor(beta), 1e-5)
    np.testing.assert_allclose(s, st.numpy(), rtol=1e-6)
    np.testing.assert_allclose(y, ref.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(bg, torch.nn.functional.gelu(ref + torch.tensor(bias)).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(fg, torch.nn.functional.gelu(ref, approximate="tanh").numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(rms, (st / torch.sqrt((st ** 2).mean(-1, keepdim=True) + 1e-6) * torch.tensor(gamma)).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(fm, 0.5 * (x @ skip.transpose(0, 2, 1)), rtol=1e-4, atol=1e-5)
    # MatMulNBits: 4-bit blocks of 16 along K = 32, N = 5
    K, N, bs = 32, 5, 16
    qv = rng.integers(0, 16, (N, K)).astype(np.uint8)
    scales = (rng.random((N, K // bs)) * 0.1 + 0.01).astype(np.float32)
    zps = rng.integers(0, 16, (N, K // bs)).astype(np.uint8)
    packed = (qv[:, 0::2] | (qv[:, 1::2] << 4)).reshape(N, K // bs, bs // 2)
    zp_packed = (zps[:, 0::2] | (zps[:, 1::2] << 4)).reshape(N, -1)
    a = rng.standard_normal((3, K)).astype(np.float32)
    nodes = [node("MatMulNBits", ["a", "Bq", "sc", "zp"], ["y"], K=K, N=N, bits=4, block_size=bs)]
    got = run(nodes, {"Bq": packed, "sc": scales.reshape(-1), "zp": zp_packed}, [("a", 1, [3, K])], [("y", 1, [3, N])], [a])[0]
    wd = (qv.astype(np.float32) - np.repeat(zps, bs, 1)) * np.repeat(scales, bs, 1)
    np.testing.assert_allclose(got, a @ wd.T, rtol=2e-3, atol=2e-3)
    # RotaryEmbedding, half-rotate, [B, S, heads * D]
    heads, D = 2, 4
    xr = rng.standard_normal((B, S, heads * D)).astype(np.float32)
    pos = np.tile(np.arange(S, dtype=np.int64), (B, 1))
    ang = np.outer(np.arange(16), 1.0 / (10000 ** (np.arange(0, D, 2) / D))).astype(np.float32)
    nodes = [node("RotaryEmbedding", ["x", "pos", "cos", "sin"], ["y"], num_heads=heads)]
    got = run(nodes, {"cos": np.cos(ang), "sin": np.sin(ang)}, [("x", 1, [B, S, heads * D]), ("pos", 7, [B, S])], [("y", 1, [B, S, heads * D])], [xr, pos])[0]
    x4 = xr.reshape(B, S, heads, D)
    c, sn = np.cos(ang)[pos][:, :, None], np.sin(ang)[pos][:, :, None]
    a_, b_ = x4[..., :D // 2], x4[..., D // 2:]
    ref = np.concatenate([a_ * c - b_ * sn, a_ * sn + b_ * c], -1).reshape(B, S, heads * D)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


def test_group_query_attention_contrib():
    """com.microsoft GroupQueryAttention with separate and with packed q / k / v, a past of 3 positions and rotary caches."""
    rng = np.random.default_rng(21)
    B, S, N, Nkv, H, P = 1, 2, 4, 2, 8, 3
    total = P + S
    q = rng.standard_normal((B, S, N * H)).astype(np.float32)
    k = rng.standard_normal((B, S, Nkv * H)).astype(np.float32)
    v = rng.standard_normal((B, S, Nkv * H)).astype(np.float32)
    pk = rng.standard_normal((B, Nkv, P, H)).astype(np.float32)
    pv = rng.standard_normal((B, Nkv, P, H)).astype(np.float32)
    ang = rng.random((16, H // 2)).astype(np.float32)
    inits = {"lens": np.array([total - 1], np.int32), "total": np.array(total, np.int32), "cos": np.cos(ang), "sin": np.sin(ang)}

    def reference(rot):
        t = lambda x, h: torch.tensor(x).reshape(B, S, h, H).transpose(1, 2)
        qh, kh, vh = t(q, N), t(k, Nkv), t(v, Nkv)
        if rot:
            c, s = torch.tensor(inits["cos"][P:total]), torch.tensor(inits["sin"][P:total])
            r = lambda x: torch.cat([x[..., :H // 2] * c - x[..., H // 2:] * s, x[..., :H // 2] * s + x[..., H // 2:] * c], -1)
            qh, kh = r(qh), r(kh)
        K_ = torch.cat([torch.tensor(pk), kh], 2)
        V_ = torch.cat([torch.tensor(pv), vh], 2)
        sc = qh @ K_.repeat_interleave(N // Nkv, 1).transpose(-1, -2) / np.sqrt(H)
        keep = torch.arange(total)[None, :] <= torch.arange(S)[:, None] + P
        w = torch.softmax(sc.masked_fill(~keep, float("-inf")), -1)
        return (w @ V_.repeat_interleave(N // Nkv, 1)).transpose(1, 2).reshape(B, S, N * H).numpy(), K_.numpy()

    outs = [("y", 1, [B, S, N * H]), ("nk", 1, [B, Nkv, total, H]), ("nv", 1, [B, Nkv, total, H])]
    ins = [("q", 1, list(q.shape)), ("k", 1, list(k.shape)), ("v", 1, list(v.shape)), ("pk", 1, list(pk.shape)), ("pv", 1, list(pv.shape))]
    y, nk, _ = run([node("GroupQueryAttention", ["q", "k", "v", "pk", "pv", "lens", "total"], ["y", "nk", "nv"], num_heads=N, kv_num_heads=Nkv)],
                   inits, ins, outs, [q, k, v, pk, pv])
    ref_y, ref_k = reference(False)
    np.testing.assert_allclose(y, ref_y, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(nk, ref_k, rtol=1e-6)
    packed = np.concatenate([q, k, v], -1)
    ins = [("qkv", 1, list(packed.shape)), ("pk", 1, list(pk.shape)), ("pv", 1, list(pv.shape))]
    y, nk, _ = run([node("GroupQueryAttention", ["qkv", "", "", "pk", "pv", "lens", "total", "cos", "sin"], ["y", "nk", "nv"], num_heads=N, kv_num_heads=Nkv,
                         do_rotary=1)], inits, ins, outs, [packed, pk, pv])
    ref_y, ref_k = reference(True)
    np.testing.assert_allclose(y, ref_y, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(nk, ref_k, rtol=2e-5, atol=2e-5)


def test_contrib_attention_qlinear_and_fused_ops():
    rng = np.random.default_rng(31)
    B, S, Hd, N = 2, 5, 16, 4
    x = rng.standard_normal((B, S, Hd)).astype(np.float32)
    w = (rng.standard_normal((Hd, 3 * Hd)) * 0.3).astype(np.float32)
    bias = rng.standard_normal((3 * Hd,)).astype(np.float32)
    mask = np.array([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]], np.int32)
    t = torch.tensor

    def sdpa(q, k, v, add=None, causal=False):
        sp = lambda a: a.reshape(B, -1, N, Hd // N).transpose(1, 2)
        o = torch.nn.functional.scaled_dot_product_attention(sp(q), sp(k), sp(v), attn_mask=add, is_causal=causal)
        return o.transpose(1, 2).reshape(B, -1, Hd).numpy()
    qkv = t(x) @ t(w) + t(bias)
    q, k, v = qkv.split(Hd, -1)
    add = ((1 - t(mask).float()) * -10000.0)[:, None, None, :]
    y, = run([node("Attention", ["x", "w", "b", "m"], ["y"], num_heads=N)], {"w": w, "b": bias}, [("x", 1, [B, S, Hd]), ("m", 6, [B, S])], [("y", 1, [B, S, Hd])], [x, mask])
    np.testing.assert_allclose(y, sdpa(q, k, v, add), rtol=1e-4, atol=1e-5)
    y, = run([node("Attention", ["x", "w", "b"], ["y"], num_heads=N, unidirectional=1)], {"w": w, "b": bias}, [("x", 1, [B, S, Hd])], [("y", 1, [B, S, Hd])], [x])
    np.testing.assert_allclose(y, sdpa(q, k, v, None, True), rtol=1e-4, atol=1e-5)

    kx = rng.standard_normal((B, 7, Hd)).astype(np.float32)
    vx = rng.standard_normal((B, 7, Hd)).astype(np.float32)
    rel = rng.standard_normal((1, N, S, 7)).astype(np.float32)
    y, = run([node("MultiHeadAttention", ["q", "k", "v", "b", "", "rel"], ["y"], num_heads=N)], {"b": bias, "rel": rel},
             [("q", 1, [B, S, Hd]), ("k", 1, [B, 7, Hd]), ("v", 1, [B, 7, Hd])], [("y", 1, [B, S, Hd])], [x, kx, vx])
    bq, bk, bv = t(bias).split(Hd)
    np.testing.assert_allclose(y, sdpa(t(x) + bq, t(kx) + bk, t(vx) + bv, t(rel)), rtol=1e-4, atol=1e-5)

    # quantised element-wise family
    a = rng.integers(0, 255, (3, 4)).astype(np.uint8)
    b = rng.integers(0, 255, (3, 4)).astype(np.uint8)
    inits = {"as": np.array(0.02, np.float32), "az": np.array(128, np.uint8), "bs": np.array(0.03, np.float32), "bz": np.array(120, np.uint8),
             "cs": np.array(0.05, np.float32), "cz": np.array(100, np.uint8)}
    nodes = [node("QLinearAdd", ["a", "as", "az", "b", "bs", "bz", "cs", "cz"], ["s"]), node("QLinearMul", ["a", "as", "az", "b", "bs", "bz", "cs", "cz"], ["p"]),
             node("QLinearSigmoid", ["a", "as", "az", "cs", "cz"], ["g"]), node("QLinearLeakyRelu", ["a", "as", "az", "cs", "cz"], ["l"], alpha=0.1),
             node("QLinearConcat", ["cs", "cz", "a", "as", "az", "b", "bs", "bz"], ["c"], axis=1)]
    s, p, g, l, c = run(nodes, inits, [("a", 2, [3, 4]), ("b", 2, [3, 4])], [("s", 2, [3, 4]), ("p", 2, [3, 4]), ("g", 2, [3, 4]), ("l", 2, [3, 4]), ("c", 2, [3, 8])], [a, b])
    fa, fb = (a.astype(np.float32) - 128) * 0.02, (b.astype(np.float32) - 120) * 0.03
    quant = lambda v: np.clip(np.round(v / 0.05) + 100, 0, 255).astype(np.uint8)
    for got, ref in ((s, fa + fb), (p, fa * fb), (g, 1 / (1 + np.exp(-fa))), (l, np.where(fa >= 0, fa, 0.1 * fa)), (c, np.concatenate([fa, fb], 1))):
        assert got.dtype == np.uint8 and np.abs(got.astype(np.int32) - quant(ref).astype(np.int32)).max() <= 1

    # fused float ops and the integer products with float scales
    gx = rng.standard_normal((3, 6)).astype(np.float32)
    gw = rng.standard_normal((6, 5)).astype(np.float32)
    gb = rng.standard_normal((5,)).astype(np.float32)
    skip = rng.standard_normal((B, S, Hd)).astype(np.float32)
    bi = rng.integers(-100, 100, (6, 5)).astype(np.int8)
    nodes = [node("FusedGemm", ["gx", "gw", "gb"], ["fg"], activation=b"LeakyRelu", activation_params=[0.2]), node("BiasAdd", ["x", "hb", "skip"], ["ba"]),
             node("MatMulIntegerToFloat", ["ai", "bi", "sa", "sb", "za", "", "gb"], ["mf"]), node("DynamicQuantizeMatMul", ["gx", "bi", "sb", "", "gb"], ["dq"])]
    ai = rng.integers(0, 255, (3, 6)).astype(np.uint8)
    inits = {"gw": gw, "gb": gb, "hb": bias[:Hd].copy(), "bi": bi, "sa": np.array(0.01, np.float32), "sb": np.array(0.02, np.float32), "za": np.array(127, np.uint8)}
    fg, ba, mf, dq = run(nodes, inits, [("gx", 1, [3, 6]), ("x", 1, [B, S, Hd]), ("skip", 1, [B, S, Hd]), ("ai", 2, [3, 6])],
                         [("fg", 1, [3, 5]), ("ba", 1, [B, S, Hd]), ("mf", 1, [3, 5]), ("dq", 1, [3, 5])], [gx, x, skip, ai])
    np.testing.assert_allclose(fg, torch.nn.functional.leaky_relu(t(gx) @ t(gw) + t(gb), 0.2).numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(ba, x + bias[:Hd] + skip, rtol=1e-6)
    np.testing.assert_allclose(mf, ((ai.astype(np.float32) - 127) * 0.01) @ (bi.astype(np.float32) * 0.02) + gb, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(dq, gx @ (bi.astype(np.float32) * 0.02) + gb, atol=0.15)          # A goes through 8 bits first

    # channels-last group normalisation with Swish
    im = rng.standard_normal((2, 3, 3, 8)).astype(np.float32)
    gamma, beta = rng.standard_normal(8).astype(np.float32), rng.standard_normal(8).astype(np.float32)
    gn, = run([node("GroupNorm", ["im", "gamma", "beta"], ["gn"], groups=2, activation=1, epsilon=1e-5)], {"gamma": gamma, "beta": beta}, [("im", 1, [2, 3, 3, 8])],
              [("gn", 1, [2, 3, 3, 8])], [im])
    ref = torch.nn.functional.silu(torch.nn.functional.group_norm(t(im).permute(0, 3, 1, 2), 2, t(gamma), t(beta), 1e-5)).permute(0, 2, 3, 1).numpy()
    np.testing.assert_allclose(gn, ref, rtol=1e-4, atol=1e-5)
