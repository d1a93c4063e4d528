"""Second part of the TensorFlow Lite translator table (frontend/tflite_more.py) on flatbuffers written by the test-side
builder of tests/test_frontend_tflite.py."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import openvino_b200 as ov   # noqa: E402
from fb_writer import Tab   # noqa: E402
from test_frontend_tflite import F32, I32, TfliteBuilder   # noqa: E402

BOOL, I64 = 6, 4


def test_selection_reduction_and_indexing_operators():
    rng = np.random.default_rng(0)
    b = TfliteBuilder()
    x = b.tensor("x", [4, 6])
    ax1 = b.tensor("ax1", [1], I32, np.array([1], np.int32))
    half = b.tensor("half", [], F32, np.array(0.5, np.float32))
    gt = b.tensor("gt", [4, 6], BOOL)
    b.op(61, [x, half], [gt])                                                  # GREATER
    sq = b.tensor("sq", [4, 6])
    b.op(92, [x], [sq])                                                        # SQUARE
    sel = b.tensor("sel", [4, 6])
    b.op(123, [gt, sq, x], [sel])                                              # SELECT_V2
    s = b.tensor("sum", [4, 1])
    b.op(74, [sel, ax1], [s], 27, Tab([("b", 1)]))                             # SUM keep_dims
    cs = b.tensor("cs", [4, 6])
    b.op(128, [sel, b.tensor("ax_s", [], I32, np.array(1, np.int32))], [cs], 108, Tab([("b", 0), ("b", 1)]))    # CUMSUM reverse
    am = b.tensor("am", [4], I64)
    b.op(56, [x, b.tensor("ax_c", [], I32, np.array(1, np.int32))], [am], 40, Tab([("b", I64)]))           # ARG_MAX
    k = b.tensor("k", [], I32, np.array(2, np.int32))
    tv, ti = b.tensor("tv", [4, 2]), b.tensor("ti", [4, 2], I32)
    b.op(48, [x, k], [tv, ti])                                                 # TOPK_V2
    begin, size = b.tensor("b", [2], I32, np.array([1, 2], np.int32)), b.tensor("s", [2], I32, np.array([2, -1], np.int32))
    sl = b.tensor("sl", [2, 4])
    b.op(65, [x, begin, size], [sl])                                           # SLICE
    p0, p1 = b.tensor("p0", [4, 3]), b.tensor("p1", [4, 3])
    b.op(49, [b.tensor("ax_sp", [], I32, np.array(1, np.int32)), x], [p0, p1], 35, Tab([("i", 2)]))          # SPLIT
    pk = b.tensor("pk", [2, 4, 3])
    b.op(83, [p0, p1], [pk], 59, Tab([("i", 2), ("i", 0)]))                    # PACK
    data = b.finish([x], [s, cs, am, tv, ti, sl, pk])
    m = ov.convert_model(data)
    xv = rng.standard_normal((4, 6)).astype(np.float32)
    res = ov.compile_model(m, "CPU")([xv])
    sel_r = np.where(xv > 0.5, xv * xv, xv)
    np.testing.assert_allclose(res[0], sel_r.sum(1, keepdims=True), rtol=1e-5)
    np.testing.assert_allclose(res[1], np.flip(np.cumsum(np.flip(sel_r, 1), 1), 1), rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(res[2], xv.argmax(1))
    order = np.argsort(-xv, 1, kind="stable")[:, :2]
    np.testing.assert_allclose(res[3], np.take_along_axis(xv, order, 1))
    np.testing.assert_array_equal(res[4], order)
    np.testing.assert_array_equal(res[5], xv[1:3, 2:])
    np.testing.assert_array_equal(res[6], np.stack([xv[:, :3], xv[:, 3:]]))


def test_image_operators():
    rng = np.random.default_rng(1)
    b = TfliteBuilder()
    x = b.tensor("img", [1, 4, 4, 8])
    d2s = b.tensor("d2s", [1, 8, 8, 2])
    b.op(5, [x], [d2s], 94, Tab([("i", 2)]))                                   # DEPTH_TO_SPACE
    rs = b.tensor("size", [2], I32, np.array([6, 6], np.int32))
    rb = b.tensor("rb", [1, 6, 6, 2])
    b.op(23, [d2s, rs], [rb], 15, Tab([None, None, ("b", 0), ("b", 1)]))       # RESIZE_BILINEAR half_pixel_centers
    w = rng.standard_normal((2, 3, 3, 8)).astype(np.float32)                   # [O, kh, kw, I]
    tw = b.tensor("w", list(w.shape), data=w)
    osz = b.tensor("osz", [4], I32, np.array([1, 8, 8, 2], np.int32))
    tc = b.tensor("tc", [1, 8, 8, 2])
    b.op(67, [osz, tw, x], [tc], 49, Tab([("b", 0), ("i", 2), ("i", 2), ("b", 0)]))         # TRANSPOSE_CONV SAME stride 2
    mp = b.tensor("mp", [1, 6, 6, 8])
    pads = b.tensor("pads", [4, 2], I32, np.array([[0, 0], [1, 1], [1, 1], [0, 0]], np.int32))
    b.op(100, [x, pads], [mp], 61, Tab([("b", 0)]))                            # MIRROR_PAD REFLECT
    data = b.finish([x], [rb, tc, mp])
    m = ov.convert_model(data)
    img = rng.standard_normal((1, 4, 4, 8)).astype(np.float32)
    res = ov.compile_model(m, "CPU")([img])
    t = torch.tensor(img).permute(0, 3, 1, 2)
    b_, c_, h_, w_ = t.shape
    d = t.reshape(b_, 2, 2, c_ // 4, h_, w_).permute(0, 3, 4, 1, 5, 2).reshape(b_, c_ // 4, h_ * 2, w_ * 2)
    np.testing.assert_allclose(res[0], torch.nn.functional.interpolate(d, size=(6, 6), mode="bilinear", align_corners=False).permute(0, 2, 3, 1).numpy(), rtol=1e-4, atol=1e-5)
    wt = torch.tensor(w).permute(3, 0, 1, 2)
    ref_tc = torch.nn.functional.conv_transpose2d(t, wt, stride=2, padding=0)[:, :, :8, :8].permute(0, 2, 3, 1).numpy()
    np.testing.assert_allclose(res[1], ref_tc, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(res[2], np.pad(img, [(0, 0), (1, 1), (1, 1), (0, 0)], mode="reflect"))
