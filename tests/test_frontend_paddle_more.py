"""Second part of the Paddle translator table (frontend/paddle_more.py) on programs written by the test-side encoder of
tests/test_frontend_paddle.py."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import openvino_b200 as ov   # noqa: E402
from test_frontend_paddle import op, params_file, program, var   # noqa: E402


def test_more_paddle_operators(tmp_path):
    rng = np.random.default_rng(0)
    w = {"wt": rng.standard_normal((4, 3, 3, 3)).astype(np.float32) * 0.3, "gamma": (rng.random(4) + 0.5).astype(np.float32), "beta": rng.standard_normal(4).astype(np.float32)}
    vars_ = [var("x", [2, 4, 6, 6]), var("gn", [2, 4, 6, 6]), var("tc", [2, 3, 12, 12]), var("up", [2, 3, 24, 24]), var("cl", [2, 3, 24, 24]),
             var("s0", [2, 1, 24, 24]), var("s1", [2, 2, 24, 24]), var("st", [2, 2, 1, 24, 24]), var("am", [2, 24, 24], 3), var("cs", [2, 2, 24, 24]),
             var("gt", [2, 2, 24, 24], 0), var("wh", [2, 2, 24, 24]), var("fill", [2, 2, 24, 24]), var("tv", [2, 2, 24, 2]), var("ti", [2, 2, 24, 2], 3)]
    vars_ += [var(k, list(v.shape), persistable=True) for k, v in w.items()]
    ops_ = [op("feed", {"X": ["feed"]}, {"Out": ["x"]}, col=0),
            op("group_norm", {"X": ["x"], "Scale": ["gamma"], "Bias": ["beta"]}, {"Y": ["gn"]}, groups=2, epsilon=1e-5),
            op("conv2d_transpose", {"Input": ["gn"], "Filter": ["wt"]}, {"Output": ["tc"]}, strides=[2, 2], paddings=[1, 1], dilations=[1, 1], groups=1, output_padding=[1, 1],
               padding_algorithm="EXPLICIT"),
            op("nearest_interp_v2", {"X": ["tc"]}, {"Out": ["up"]}, out_h=24, out_w=24, align_corners=False, data_layout="NCHW"),
            op("clip", {"X": ["up"]}, {"Out": ["cl"]}, min=-0.5, max=0.75),
            op("split", {"X": ["cl"]}, {"Out": ["s0", "s1"]}, axis=1, sections=[1, 2], num=0),
            op("stack", {"X": ["s1"]}, {"Y": ["st"]}, axis=2),
            op("arg_max", {"X": ["cl"]}, {"Out": ["am"]}, axis=1, keepdims=False, flatten=False, dtype=3),
            op("cumsum", {"X": ["s1"]}, {"Out": ["cs"]}, axis=3, exclusive=False, reverse=False),
            op("fill_any_like", {"X": ["s1"]}, {"Out": ["fill"]}, value=0.1),
            op("greater_than", {"X": ["s1"], "Y": ["fill"]}, {"Out": ["gt"]}, axis=-1),
            op("where", {"Condition": ["gt"], "X": ["cs"], "Y": ["s1"]}, {"Out": ["wh"]}),
            op("top_k_v2", {"X": ["wh"]}, {"Out": ["tv"], "Indices": ["ti"]}, k=2, axis=-1, largest=True, sorted=True),
            op("fetch", {"X": ["st"]}, {"Out": ["fetch"]}, col=0), op("fetch", {"X": ["am"]}, {"Out": ["fetch"]}, col=1),
            op("fetch", {"X": ["tv"]}, {"Out": ["fetch"]}, col=2), op("fetch", {"X": ["ti"]}, {"Out": ["fetch"]}, col=3)]
    (tmp_path / "m.pdmodel").write_bytes(program(vars_, ops_))
    (tmp_path / "m.pdiparams").write_bytes(params_file(w))
    m = ov.convert_model(str(tmp_path / "m.pdmodel"))
    xv = rng.standard_normal((2, 4, 6, 6)).astype(np.float32)
    res = ov.compile_model(m, "CPU")([xv])
    t = torch.tensor(xv)
    gn = torch.nn.functional.group_norm(t, 2, torch.tensor(w["gamma"]), torch.tensor(w["beta"]), 1e-5)
    tc = torch.nn.functional.conv_transpose2d(gn, torch.tensor(w["wt"]), stride=2, padding=1, output_padding=1)
    up = torch.nn.functional.interpolate(tc, size=(24, 24), mode="nearest")
    cl = up.clamp(-0.5, 0.75)
    s1 = cl[:, 1:]
    np.testing.assert_allclose(res[0], s1.unsqueeze(2).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_array_equal(res[1], cl.argmax(1).numpy())
    wh = torch.where(s1 > 0.1, torch.cumsum(s1, 3), s1)
    tv, ti = torch.topk(wh, 2, -1)
    np.testing.assert_allclose(res[2], tv.numpy(), rtol=1e-4, atol=1e-5)
    assert res[3].shape == (2, 2, 24, 2)
