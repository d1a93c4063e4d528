"""InputModel / Place editing and the frontend extensions (frontend/input_model.py), on a Paddle program written by the
test-side encoder of tests/test_frontend_paddle.py."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import openvino_b200 as ov   # noqa: E402
from openvino_b200 import opset as ops   # noqa: E402
from openvino_b200.frontend.input_model import ConversionExtension, ProgressReporterExtension, TelemetryExtension   # noqa: E402
from test_frontend_paddle import op, params_file, program, var   # noqa: E402


def _write(tmp_path, extra_op=None):
    rng = np.random.default_rng(0)
    w = {"w1": rng.standard_normal((8, 6)).astype(np.float32), "w2": rng.standard_normal((6, 3)).astype(np.float32)}
    vars_ = [var("x", [-1, 8]), var("h", [-1, 6]), var("a", [-1, 6]), var("s", [-1, 6]), var("y", [-1, 3])]
    vars_ += [var(k, list(v.shape), persistable=True) for k, v in w.items()]
    ops_ = [op("feed", {"X": ["feed"]}, {"Out": ["x"]}, col=0),
            op("matmul_v2", {"X": ["x"], "Y": ["w1"]}, {"Out": ["h"]}, trans_x=False, trans_y=False),
            op(extra_op or "relu", {"X": ["h"]}, {"Out": ["a"]}),
            op("scale", {"X": ["a"]}, {"Out": ["s"]}, scale=2.0, bias=1.0, bias_after_scale=True),
            op("matmul_v2", {"X": ["s"], "Y": ["w2"]}, {"Out": ["y"]}, trans_x=False, trans_y=False),
            op("fetch", {"X": ["y"]}, {"Out": ["fetch"]}, col=0)]
    (tmp_path / "m.pdmodel").write_bytes(program(vars_, ops_))
    (tmp_path / "m.pdiparams").write_bytes(params_file(w))
    return w


def test_places_shapes_and_cuts(tmp_path):
    w = _write(tmp_path)
    fe = ov.FrontEndManager().load_by_framework("paddle")
    assert fe.get_name() == "paddle" and fe.supported(str(tmp_path / "m.pdmodel"))
    im = fe.load(str(tmp_path / "m.pdmodel"))
    assert [p.get_names() for p in im.get_inputs()] == [["x"]] and [p.get_names() for p in im.get_outputs()] == [["y"]]
    x = im.get_inputs()[0]
    im.set_partial_shape(x, [4, 8])
    assert im.get_partial_shape(x).to_shape() == [4, 8]
    a = im.get_place_by_tensor_name("a")
    assert a is not None and not a.is_input() and a.get_producing_operation().get_names() == ["a"]
    cons = a.get_consuming_operations()                    # "scale" is a Multiply followed by an Add named "s"
    assert len(cons) == 1 and cons[0]._node.get_type_name() == "Multiply"
    xin = np.random.default_rng(1).standard_normal((4, 8)).astype(np.float32)
    # head of the model: x -> a
    head = fe.load(str(tmp_path / "m.pdmodel"))
    head.override_all_outputs([head.get_place_by_tensor_name("a")])
    np.testing.assert_allclose(ov.compile_model(fe.convert(head), "CPU")([xin])[0], np.maximum(xin @ w["w1"], 0), rtol=1e-5, atol=1e-6)
    # tail of the model: s -> y, with "s" as a new input
    tail = fe.load(str(tmp_path / "m.pdmodel"))
    tail.extract_subgraph([tail.get_place_by_tensor_name("s")], [tail.get_place_by_tensor_name("y")])
    m = fe.convert(tail)
    assert [p.get_friendly_name() for p in m.get_parameters()] == ["s"]
    s_in = np.random.default_rng(2).standard_normal((4, 6)).astype(np.float32)
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([s_in])[0], s_in @ w["w2"], rtol=1e-5, atol=1e-6)
    # the unedited model still converts to the whole graph
    full = ov.compile_model(fe.convert(fe.load(str(tmp_path / "m.pdmodel"))), "CPU")([xin])[0]
    np.testing.assert_allclose(full, (np.maximum(xin @ w["w1"], 0) * 2 + 1) @ w["w2"], rtol=1e-5, atol=1e-5)


def test_conversion_telemetry_and_progress_extensions(tmp_path):
    w = _write(tmp_path, extra_op="my_square")
    fe = ov.FrontEndManager().load_by_framework("paddle")
    try:
        fe.convert(fe.load(str(tmp_path / "m.pdmodel")))
    except RuntimeError as e:
        assert "my_square" in str(e)
    else:
        raise AssertionError("the operator has no translator yet")
    events, progress, errors = [], [], []
    fe.add_extension(ConversionExtension("my_square", lambda o, g: {"Out": [ops.multiply(g.get(o.inp("X")[0]), g.get(o.inp("X")[0])).output(0)]}))
    fe.add_extension(TelemetryExtension("test", lambda cat, action, label, value=1: events.append((cat, action, label, value)),
                                        lambda cat, msg: errors.append(msg)))
    fe.add_extension(ProgressReporterExtension(lambda p, total, done: progress.append((p, total, done))))
    m = fe.convert(fe.load(str(tmp_path / "m.pdmodel")))
    xin = np.random.default_rng(3).standard_normal((2, 8)).astype(np.float32)
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xin])[0], ((xin @ w["w1"]) ** 2 * 2 + 1) @ w["w2"], rtol=1e-4, atol=1e-4)
    assert ("test", "conversion", "paddle", 1) in events and ("test", "op_count", "paddle_MatMul", 2) in events
    assert progress[0] == (0.0, 1, 0) and progress[-1] == (1.0, 1, 1) and not errors
    from openvino_b200.frontend import paddle
    del paddle._T["my_square"]
