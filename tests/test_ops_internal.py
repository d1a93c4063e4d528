"""Internal-opset operations (compressed gather, dynamic quantisation, experts with compressed weights) and
ExtractImagePatches / RegionYolo / CTCLoss / STFT: shape inference, evaluation on the CPU device, IR round trip."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops
from openvino_b200._graph import make_op


def run(outputs, params, feeds):
    m = ov.Model(outputs, params, "t")
    xml, weights = ov._ovcore.serialize(m._m)
    back = ov.Model._wrap(ov._ovcore.deserialize(xml.decode(), np.frombuffer(weights, dtype=np.uint8)))      # IR round trip first
    return ov.compile_model(back, "CPU")(feeds)


def test_extract_image_patches_matches_unfold():
    x = np.arange(2 * 3 * 10 * 9, dtype=np.float32).reshape(2, 3, 10, 9)
    p = ops.parameter([2, 3, 10, 9], "f32", "x")
    for sizes, strides, rates in (([3, 3], [2, 2], [1, 1]), ([2, 3], [1, 2], [2, 1])):
        n = ops.extract_image_patches(p, sizes, strides, rates, "valid")
        out = run([n], [p], [x])[0]
        # torch.unfold orders channels (c, kh, kw); the operation orders them (kh, kw, c)
        u = torch.nn.functional.unfold(torch.from_numpy(x), sizes, dilation=rates, stride=strides)
        oh = (10 - (sizes[0] + (rates[0] - 1) * (sizes[0] - 1))) // strides[0] + 1
        ow = (9 - (sizes[1] + (rates[1] - 1) * (sizes[1] - 1))) // strides[1] + 1
        u = u.reshape(2, 3, sizes[0], sizes[1], oh, ow).permute(0, 2, 3, 1, 4, 5).reshape(2, -1, oh, ow).numpy()
        assert list(n.get_output_shape(0)) == list(u.shape)
        np.testing.assert_array_equal(out, u)
    same = ops.extract_image_patches(p, [3, 3], [2, 2], [1, 1], "same_upper")
    out = run([same], [p], [x])[0]
    assert out.shape == (2, 27, 5, 5)
    u = torch.nn.functional.unfold(torch.nn.functional.pad(torch.from_numpy(x), [1, 1, 0, 1]), [3, 3], stride=[2, 2])      # W: 2 cells split 1/1, H: 1 cell after
    u = u.reshape(2, 3, 3, 3, 5, 5).permute(0, 2, 3, 1, 4, 5).reshape(2, 27, 5, 5).numpy()
    np.testing.assert_array_equal(out, u)


def test_region_yolo_both_forms():
    rng = np.random.default_rng(0)
    coords, classes, num = 4, 3, 2
    x = rng.standard_normal((1, num * (coords + classes + 1), 4, 5)).astype(np.float32)
    p = ops.parameter(list(x.shape), "f32", "x")
    sig = lambda t: 1 / (1 + np.exp(-t))
    n = ops.region_yolo(p, coords, classes, num, True, [0, 1], 1, 3)
    out = run([n], [p], [x])[0]
    assert out.shape == (1, x.size)
    ref = x.copy().reshape(num, coords + classes + 1, 20)
    ref[:, 0:2] = sig(ref[:, 0:2])
    ref[:, coords] = sig(ref[:, coords])
    e = np.exp(ref[:, coords + 1:] - ref[:, coords + 1:].max(1, keepdims=True))
    ref[:, coords + 1:] = e / e.sum(1, keepdims=True)
    np.testing.assert_allclose(out.reshape(-1), ref.reshape(-1), rtol=1e-5, atol=1e-6)
    n2 = ops.region_yolo(p, coords, classes, 5, False, [1], 1, 3)
    out2 = run([n2], [p], [x])[0]
    assert out2.shape == (1, coords + classes + 1, 4, 5)
    ref2 = x[0, :coords + classes + 1].copy().reshape(coords + classes + 1, 20)
    ref2[0:2] = sig(ref2[0:2])
    ref2[coords:] = sig(ref2[coords:])
    np.testing.assert_allclose(out2.reshape(-1), ref2.reshape(-1), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("blank", [0, 5])
def test_ctc_loss_matches_torch(blank):
    rng = np.random.default_rng(1)
    B, T, Cc = 3, 12, 6
    logits = rng.standard_normal((B, T, Cc)).astype(np.float32)
    logit_len = np.array([12, 9, 7], np.int32)
    label_len = np.array([4, 3, 2], np.int32)
    labels = np.zeros((B, T), np.int32)
    cand = [c for c in range(Cc) if c != blank]
    for b in range(B):
        labels[b, :label_len[b]] = rng.choice(cand, label_len[b])
    labels[0, :4] = [cand[0], cand[0], cand[1], cand[0]]           # a repeated label needs a blank in between
    ps = [ops.parameter(list(a.shape), "f32" if a.dtype == np.float32 else "i32") for a in (logits, logit_len, labels, label_len)]
    n = ops.ctc_loss(ps[0], ps[1], ps[2], ps[3], np.int32(blank))
    out = run([n], ps, [logits, logit_len, labels, label_len])[0]
    lp = torch.log_softmax(torch.from_numpy(logits), -1).transpose(0, 1)
    targets = torch.cat([torch.from_numpy(labels[b, :label_len[b]]).long() for b in range(B)])
    ref = torch.nn.functional.ctc_loss(lp, targets, torch.from_numpy(logit_len).long(), torch.from_numpy(label_len).long(), blank=blank, reduction="none")
    np.testing.assert_allclose(out, ref.numpy(), rtol=1e-4)


@pytest.mark.parametrize("transpose", [False, True])
def test_stft_matches_torch(transpose):
    rng = np.random.default_rng(2)
    sig = rng.standard_normal((2, 64)).astype(np.float32)
    win = np.hanning(12).astype(np.float32)
    p, w = ops.parameter([2, 64], "f32"), ops.parameter([12], "f32")
    n = ops.stft(p, w, np.int64(16), np.int64(5), transpose)
    out = run([n], [p, w], [sig, win])[0]
    ref = torch.stft(torch.from_numpy(sig), n_fft=16, hop_length=5, win_length=12, window=torch.from_numpy(win), center=False, return_complex=True)
    ref = torch.view_as_real(ref).numpy()                     # [B, bins, frames, 2]
    if not transpose:
        ref = ref.transpose(0, 2, 1, 3)
    assert list(n.get_output_shape(0)) == list(ref.shape)
    np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-4)


def test_gather_compressed_dequantises_the_gathered_rows():
    rng = np.random.default_rng(3)
    q = rng.integers(0, 255, (10, 4, 8), dtype=np.uint8)
    scale = rng.uniform(0.01, 0.1, (10, 4, 1)).astype(np.float16)
    zp = rng.integers(100, 150, (10, 4, 1)).astype(np.uint8)
    idx = np.array([[3, 9], [0, 3]], np.int32)
    pi = ops.parameter([2, 2], "i32", "idx")
    n = make_op("GatherCompressed", [ops.constant(q), pi, ops.constant(np.int64(0)), ops.constant(scale), ops.constant(zp)], {"batch_dims": 0},
                "ie_internal_opset")
    assert list(n.get_output_shape(0)) == [2, 2, 32] and n.get_output_element_type(0).name == "f16"
    out = run([n], [pi], [idx])[0]
    table = ((q.astype(np.float32) - zp.astype(np.float32)) * scale.astype(np.float32)).reshape(10, 32)
    np.testing.assert_allclose(out, table[idx], rtol=2e-3, atol=1e-3)


@pytest.mark.parametrize("qtype", ["Symmetric", "Asymmetric"])
def test_dynamic_quantize_round_trip(qtype):
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((3, 5, 64)) * 3).astype(np.float32)
    p = ops.parameter([3, 5, 64], "f32", "x")
    attrs = {"quantization_type": qtype, "quantization_dt": ov.Type.i8 if qtype == "Symmetric" else ov.Type.u8, "scale_dt": ov.Type.f32,
             "zp_dt": ov.Type.u8 if qtype == "Asymmetric" else ov.Type.dynamic, "group_sizes": [1, 1, 32], "output_storage_type": "Planar"}
    n = make_op("DynamicQuantize", [p], attrs, "ie_internal_opset")
    assert n.get_output_size() == (3 if qtype == "Asymmetric" else 2)
    assert list(n.get_output_shape(1)) == [3, 5, 2]
    outs = run([n.output(i) for i in range(n.get_output_size())], [p], [x])
    q, scale = outs[0].astype(np.float32).reshape(3, 5, 2, 32), outs[1].reshape(3, 5, 2, 1)
    zp = outs[2].astype(np.float32).reshape(3, 5, 2, 1) if qtype == "Asymmetric" else 0.0
    back = ((q - zp) * scale).reshape(3, 5, 64)
    assert np.abs(back - x).max() <= 0.51 * scale.max() + 1e-6
    # one group over the whole last axis (all bits set)
    n2 = make_op("DynamicQuantize", [p], dict(attrs, group_sizes=[1, 1, -1]), "ie_internal_opset")
    assert list(n2.get_output_shape(1)) == [3, 5, 1]


def test_moe_compressed_equals_moe_on_dequantised_weights():
    rng = np.random.default_rng(5)
    E, F, H, T, k, gs = 4, 16, 32, 6, 2, 16
    def qw(n_, kd):
        q = rng.integers(0, 15, (E, n_, kd // gs, gs), dtype=np.uint8)
        s = rng.uniform(0.01, 0.05, (E, n_, kd // gs, 1)).astype(np.float16)
        z = rng.integers(6, 10, (E, n_, kd // gs, 1)).astype(np.uint8)
        return q, s, z, ((q.astype(np.float32) - z) * s.astype(np.float32)).reshape(E, n_, kd)
    g, u, d = qw(F, H), qw(F, H), qw(H, F)
    x = rng.standard_normal((T, H)).astype(np.float32)
    rw = rng.uniform(0.2, 0.8, (T, k)).astype(np.float32)
    idx = np.stack([rng.choice(E, k, replace=False) for _ in range(T)]).astype(np.int32)
    px, pr, pi = ops.parameter([T, H], "f32"), ops.parameter([T, k], "f32"), ops.parameter([T, k], "i32")
    cins = [ops.constant(a) for t in (g, u, d) for a in t[:3]]
    attrs = {"expert_type": "GEMM3_SWIGLU", "activation_type": "SWISH", "hidden_size": H, "inter_size": F, "num_expert": E, "top_k": k, "group_size": gs, "has_zp": True}
    mc = make_op("MOECompressed", [px, pr, pi] + cins, attrs, "")
    mf = make_op("MOE", [px, pr, pi, ops.constant(g[3]), ops.constant(u[3]), ops.constant(d[3])], {"expert_type": "GEMM3_SWIGLU", "activation_type": "SWISH"}, "internal")
    a = run([mc], [px, pr, pi], [x, rw, idx])[0]
    b = ov.compile_model(ov.Model([mf], [px, pr, pi], "f"), "CPU")([x, rw, idx])[0]
    np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-5)


def _yuv_ref(y, u, v):
    c, d, e = y - 16.0, u - 128.0, v - 128.0
    clip = lambda a: np.clip(np.round(a), 0, 255)
    return clip(1.164 * c + 1.596 * e), clip(1.164 * c - 0.391 * d - 0.813 * e), clip(1.164 * c + 2.018 * d)


def test_colour_conversions_from_nv12_and_i420():
    rng = np.random.default_rng(6)
    H, W = 4, 6
    y = rng.integers(16, 235, (1, H, W, 1), dtype=np.uint8)
    u = rng.integers(16, 240, (1, H // 2, W // 2, 1), dtype=np.uint8)
    v = rng.integers(16, 240, (1, H // 2, W // 2, 1), dtype=np.uint8)
    uu, vv = np.repeat(np.repeat(u, 2, 1), 2, 2).astype(np.float32), np.repeat(np.repeat(v, 2, 1), 2, 2).astype(np.float32)
    r, g, b = _yuv_ref(y.astype(np.float32), uu, vv)
    rgb = np.concatenate([r, g, b], -1).astype(np.uint8)
    py, pu, pv = ops.parameter([1, H, W, 1], "u8"), ops.parameter([1, H // 2, W // 2, 1], "u8"), ops.parameter([1, H // 2, W // 2, 1], "u8")
    np.testing.assert_array_equal(run([ops.i420_to_rgb(py, pu, pv)], [py, pu, pv], [y, u, v])[0], rgb)
    np.testing.assert_array_equal(run([ops.i420_to_bgr(py, pu, pv)], [py, pu, pv], [y, u, v])[0], rgb[..., ::-1])
    puv = ops.parameter([1, H // 2, W // 2, 2], "u8")
    uv = np.concatenate([u, v], -1)
    np.testing.assert_array_equal(run([ops.nv12_to_rgb(py, puv)], [py, puv], [y, uv])[0], rgb)
    # one plane holding the whole frame: Y rows, then the interleaved UV rows
    frame = np.concatenate([y.reshape(1, H, W), uv.reshape(1, H // 2, W)], 1)[..., None]
    pf = ops.parameter([1, H * 3 // 2, W, 1], "u8")
    n = ops.nv12_to_bgr(pf)
    assert list(n.get_output_shape(0)) == [1, H, W, 3]
    np.testing.assert_array_equal(run([n], [pf], [frame])[0], rgb[..., ::-1])


def test_prior_box_clustered():
    n = ops.prior_box_clustered(np.array([2, 3], np.int64), np.array([20, 30], np.int64), [4.0, 8.0], [6.0, 2.0], offset=0.5, variance=[0.1, 0.1, 0.2, 0.2])
    assert list(n.get_output_shape(0)) == [2, 2 * 3 * 2 * 4]
    out = run([n], [], [])[0].reshape(2, 2, 3, 2, 4)
    # cell (h=1, w=2), second prior: centre (2.5 * 10, 1.5 * 10) in a 30 x 20 image
    np.testing.assert_allclose(out[0, 1, 2, 1], [(25 - 4) / 30, (15 - 1) / 20, (25 + 4) / 30, (15 + 1) / 20], rtol=1e-6)
    np.testing.assert_allclose(out[1, 0, 0, 0], [0.1, 0.1, 0.2, 0.2], rtol=1e-6)
    assert out[0].min() >= 0 and out[0].max() <= 1


def test_psroi_pooling_average():
    rng = np.random.default_rng(7)
    G, Cout = 2, 3
    x = rng.standard_normal((1, Cout * G * G, 8, 8)).astype(np.float32)
    rois = np.array([[0, 0, 0, 7, 7], [0, 2, 2, 5, 5]], np.float32)
    px, pr = ops.parameter(list(x.shape), "f32"), ops.parameter([2, 5], "f32")
    n = ops.psroi_pooling(px, pr, Cout, G, 1.0)
    out = run([n], [px, pr], [x, rois])[0]
    assert out.shape == (2, Cout, G, G)
    # first ROI covers the whole map: bin (ph, pw) of output channel c averages a 4 x 4 quadrant of input channel (c * G + ph) * G + pw
    for c in range(Cout):
        for ph in range(G):
            for pw in range(G):
                want = x[0, (c * G + ph) * G + pw, ph * 4:(ph + 1) * 4, pw * 4:(pw + 1) * 4].mean()
                assert abs(out[0, c, ph, pw] - want) < 1e-5
    want = x[0, (1 * G + 1) * G + 0, 4:6, 2:4].mean()          # second ROI (2..5 -> 4 cells per side), channel 1, bin (1, 0)
    assert abs(out[1, 1, 1, 0] - want) < 1e-5


def test_fake_convert_is_an_fp8_round_trip():
    x = np.array([[0.3, -1.7, 100.0, 1e-3], [5.5, 7.3, -0.02, 200.0]], np.float32)
    p = ops.parameter([2, 4], "f32")
    out = run([ops.fake_convert(p, np.array([2.0], np.float32))], [p], [x])[0]
    want = torch.from_numpy(x * 2).to(torch.float8_e4m3fn).float().numpy() / 2
    np.testing.assert_allclose(out, want, rtol=1e-6)
    out5 = run([ops.fake_convert(p, np.array([1.0], np.float32), np.array([0.0], np.float32), "f8e5m2")], [p], [x])[0]
    np.testing.assert_allclose(out5, torch.from_numpy(x).to(torch.float8_e5m2).float().numpy(), rtol=1e-6)


def test_sparse_fill_empty_rows():
    vals = np.array([1.0, 2.0, 3.0], np.float32)
    idx = np.array([[0, 1], [3, 0], [0, 3]], np.int64)
    pv, pi = ops.parameter([3], "f32"), ops.parameter([3, 2], "i64")
    n = ops.sparse_fill_empty_rows(pv, np.array([5, 4], np.int64), pi, np.float32(-1))
    res = run([n.output(0), n.output(1), n.output(2)], [pv, pi], [vals, idx])
    oi, ov_, empty = res[0], res[1], res[2]
    np.testing.assert_array_equal(oi, [[0, 1], [0, 3], [1, 0], [2, 0], [3, 0], [4, 0]])
    np.testing.assert_array_equal(ov_, [1, 3, -1, -1, 2, -1])
    np.testing.assert_array_equal(empty, [False, True, True, False, True])
