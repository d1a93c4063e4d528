"""Second part of the TensorFlow translator table (frontend/tensorflow_more.py) on GraphDefs written by the test-side
encoder of tests/test_frontend_tensorflow.py, against NumPy / PyTorch."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import openvino_b200 as ov   # noqa: E402
from openvino_b200.frontend import tensorflow as fe   # noqa: E402
from test_frontend_tensorflow import const, node   # noqa: E402


def run(graph, feeds, names=None):
    m = fe.convert(graph)
    res = ov.compile_model(m, "CPU")(feeds)
    if names is None:
        return [res[i] for i in range(len(m.outputs))]
    return [res[n] for n in names]


def test_elementwise_selection_and_indexing():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 6)).astype(np.float32)
    graph = b"".join([
        node("x", "Placeholder", dtype=("type", 1), shape=("shape", [4, 6])),
        const("lo", np.array(-0.5, np.float32)), const("hi", np.array(0.75, np.float32)), const("two", np.array(2.0, np.float32)),
        const("ax1", np.array(1, np.int32)), const("k", np.array(2, np.int32)), const("begin", np.array([1, 2], np.int32)), const("size", np.array([2, -1], np.int32)),
        node("clip", "ClipByValue", ["x", "lo", "hi"]),
        node("fd", "FloorDiv", ["x", "two"]),
        node("cs", "Cumsum", ["clip", "ax1"], exclusive=False, reverse=True),
        node("gt", "GreaterEqual", ["x", "lo"]),
        node("sel", "SelectV2", ["gt", "cs", "fd"]),
        node("sp", "Split", ["ax1", "sel"], num_split=2),
        node("sum", "AddN", ["sp", "sp:1"], N=2),
        node("top", "TopKV2", ["sum", "k"], sorted=True),
        node("am", "ArgMax", ["x", "ax1"], output_type=("type", 9)),
        node("sl", "Slice", ["x", "begin", "size"]),
        node("l1p", "Log1p", ["clip"]),
        node("out0", "Identity", ["top"]), node("out1", "Identity", ["top:1"]), node("out2", "Identity", ["am"]), node("out3", "Identity", ["sl"]),
        node("out4", "Identity", ["l1p"]),
    ])
    vals, idx, am, sl, l1p = run(graph, [x])
    clip = np.clip(x, -0.5, 0.75)
    cs = np.flip(np.cumsum(np.flip(clip, 1), 1), 1)
    sel = np.where(x >= -0.5, cs, np.floor(x / 2))
    s = sel[:, :3] + sel[:, 3:]
    order = np.argsort(-s, 1, kind="stable")[:, :2]
    np.testing.assert_allclose(vals, np.take_along_axis(s, order, 1), rtol=1e-5)
    np.testing.assert_array_equal(idx, order)
    np.testing.assert_array_equal(am, x.argmax(1))
    np.testing.assert_array_equal(sl, x[1:3, 2:])
    np.testing.assert_allclose(l1p, np.log1p(clip), rtol=1e-5, atol=1e-6)


def test_generation_rearrangement_and_convolutions():
    rng = np.random.default_rng(1)
    img = rng.standard_normal((1, 4, 4, 8)).astype(np.float32)          # NHWC
    w = rng.standard_normal((3, 3, 2, 8)).astype(np.float32)            # HWOI of the transposed convolution: 8 in, 2 out
    graph = b"".join([
        node("img", "Placeholder", dtype=("type", 1), shape=("shape", [1, 4, 4, 8])),
        const("w", w), const("osz", np.array([1, 8, 8, 2], np.int32)), const("rs", np.array([6, 6], np.int32)),
        const("dims", np.array([2, 3], np.int32)), const("val", np.array(1.5, np.float32)), const("r0", np.array(0, np.int32)), const("r1", np.array(6, np.int32)),
        const("r2", np.array(2, np.int32)), const("depth", np.array(4, np.int32)), const("on", np.array(1.0, np.float32)), const("off", np.array(0.0, np.float32)),
        node("d2s", "DepthToSpace", ["img"], block_size=2, data_format=b"NHWC"),
        node("rb", "ResizeBilinear", ["d2s", "rs"], align_corners=False, half_pixel_centers=True),
        node("tc", "Conv2DBackpropInput", ["osz", "w", "img"], strides=[1, 2, 2, 1], padding=b"SAME", data_format=b"NHWC"),
        node("fill", "Fill", ["dims", "val"]),
        node("rng", "Range", ["r0", "r1", "r2"]),
        node("oh", "OneHot", ["rng", "depth", "on", "off"], axis=-1),
        node("ein", "Einsum", ["fill", "fill"], equation=b"ij,kj->ik", N=2),
        node("up", "Unpack", ["fill"], axis=0, num=2),
        node("o0", "Identity", ["rb"]), node("o1", "Identity", ["tc"]), node("o2", "Identity", ["oh"]), node("o3", "Identity", ["ein"]), node("o4", "Identity", ["up:1"]),
    ])
    rb, tc, oh, ein, up1 = run(graph, [img])
    t = torch.tensor(img).permute(0, 3, 1, 2)
    # TensorFlow's depth_to_space reads the channel as (block_h, block_w, depth): DCR order
    b_, c_, h_, w_ = t.shape
    d2s = t.reshape(b_, 2, 2, c_ // 4, h_, w_).permute(0, 3, 4, 1, 5, 2).reshape(b_, c_ // 4, h_ * 2, w_ * 2)
    ref_rb = torch.nn.functional.interpolate(d2s, size=(6, 6), mode="bilinear", align_corners=False).permute(0, 2, 3, 1).numpy()
    np.testing.assert_allclose(rb, ref_rb, rtol=1e-4, atol=1e-5)
    wt = torch.tensor(w).permute(3, 2, 0, 1)                             # [in = 8, out = 2, kh, kw]
    # SAME padding of the forward convolution (8 -> 4, kernel 3, stride 2) pads one row / column at the end only
    ref_tc = torch.nn.functional.conv_transpose2d(t, wt, stride=2, padding=0)[:, :, :8, :8].permute(0, 2, 3, 1).numpy()
    assert tc.shape == (1, 8, 8, 2)
    np.testing.assert_allclose(tc, ref_tc, rtol=1e-4, atol=1e-4)
    np.testing.assert_array_equal(oh, np.eye(4, dtype=np.float32)[[0, 2, 0]] * np.array([[1], [1], [0]], np.float32) + np.array([[0, 0, 0, 0], [0, 0, 0, 0], [0, 0, 0, 0]], np.float32))
    np.testing.assert_allclose(ein, np.full((2, 2), 1.5 * 1.5 * 3, np.float32))
    np.testing.assert_allclose(up1, np.full((3,), 1.5, np.float32))
