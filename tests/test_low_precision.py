"""Low-precision passes and pruning: the rewritten graph computes what the original does."""
import numpy as np

import openvino_b200 as ov
from openvino_b200 import opset as ops
from openvino_b200.passes import low_precision as lp
from openvino_b200.passes.pruning import Pruning
from openvino_b200 import _offline_transformations as off


def _types(m):
    return [n.get_type_name() for n in m.get_ops()]


def _quantized_net(rng):
    x = ops.parameter([2, 3, 8, 8], "f32", "x")
    xq = ops.fake_quantize(x, np.float32(-1.0), np.float32(1.0), np.float32(-1.0), np.float32(1.0), 256)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32) * 0.2
    lim = np.abs(w).reshape(4, -1).max(1).reshape(4, 1, 1, 1).astype(np.float32)
    wq = ops.fake_quantize(w, -lim, lim, -lim, lim, 255)
    conv = ops.convolution(xq, wq, [1, 1], [1, 1], [1, 1], [1, 1])
    act = ops.relu(conv)
    aq = ops.fake_quantize(act, np.float32(0.0), np.float32(4.0), np.float32(0.0), np.float32(4.0), 256)
    pooled = ops.max_pool(aq, [2, 2], [1, 1], [0, 0], [0, 0], [2, 2])
    flat = ops.reshape(pooled.output(0), np.array([2, -1], dtype=np.int64), False)
    w2 = rng.standard_normal((5, 64)).astype(np.float32) * 0.1
    w2q = ops.fake_quantize(w2, np.float32(-0.4), np.float32(0.4), np.float32(-0.4), np.float32(0.4), 255)
    fc = ops.matmul(flat, w2q, False, True)
    return ov.Model([ops.result(fc)], [x], "qnet")


def test_low_precision_pipeline_keeps_the_numbers():
    rng = np.random.default_rng(0)
    m = _quantized_net(rng)
    x = rng.uniform(-1.2, 1.2, (2, 3, 8, 8)).astype(np.float32)
    ref = ov.compile_model(m.clone(), "CPU")(x)[0]
    assert lp.is_quantized(m)
    assert lp.LowPrecision().run_on_model(m)
    types = _types(m)
    # weights are integer constants now, activations are quantised to u8 / i8, FakeQuantize stays on activations only
    assert types.count("FakeQuantize") == 2
    const_types = {n.get_output_element_type(0).get_type_name() for n in m.get_ops() if n.get_type_name() == "Constant"}
    assert "i8" in const_types
    conv = [n for n in m.get_ops() if n.get_type_name() == "Convolution"][0]
    # the convolution reads integer-valued tensors: Convert(i8/u8) (minus zero point), no Multiply in front of it
    assert conv.input_value(1).get_node().get_type_name() == "Convert"
    assert conv.input_value(0).get_node().get_type_name() in ("Convert", "Subtract")
    mm = [n for n in m.get_ops() if n.get_type_name() == "MatMul"][0]
    assert mm.input_value(0).get_node().get_type_name() == "Reshape" and mm.input_value(1).get_node().get_type_name() == "Convert"
    got = ov.compile_model(m, "CPU")(x)[0]
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)


def test_compress_quantize_weights_offline_entry_point():
    rng = np.random.default_rng(1)
    x = ops.parameter([1, 16], "f32", "x")
    w = rng.standard_normal((8, 16)).astype(np.float32)
    wq = ops.fake_quantize(w, np.float32(-2.0), np.float32(2.5), np.float32(-2.0), np.float32(2.5), 256)   # asymmetric: zero point
    m = ov.Model([ops.result(ops.matmul(x, wq, False, True))], [x], "fc")
    xv = rng.standard_normal((1, 16)).astype(np.float32)
    ref = ov.compile_model(m.clone(), "CPU")(xv)[0]
    off.compress_quantize_weights_transformation(m)
    assert "FakeQuantize" not in _types(m) and "Subtract" in _types(m)
    assert any(n.get_type_name() == "Constant" and n.get_output_element_type(0).get_type_name() == "u8" for n in m.get_ops())
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(xv)[0], ref, rtol=1e-5, atol=1e-5)


def test_pruning_removes_zero_channels():
    rng = np.random.default_rng(2)
    x = ops.parameter([1, 3, 8, 8], "f32", "x")
    w1 = rng.standard_normal((8, 3, 3, 3)).astype(np.float32)
    w1[[1, 4, 6]] = 0
    b1 = rng.standard_normal((1, 8, 1, 1)).astype(np.float32)
    b1[0, [1, 4, 6]] = 0
    g = rng.uniform(0.5, 2, (1, 8, 1, 1)).astype(np.float32)
    y = ops.relu(ops.multiply(ops.add(ops.convolution(x, w1, [1, 1], [1, 1], [1, 1], [1, 1]), b1), g))
    w2 = rng.standard_normal((4, 8, 3, 3)).astype(np.float32)
    z = ops.convolution(y, w2, [1, 1], [1, 1], [1, 1], [1, 1])
    m = ov.Model([ops.result(z)], [x], "prunable")
    xv = rng.standard_normal((1, 3, 8, 8)).astype(np.float32)
    ref = ov.compile_model(m.clone(), "CPU")(xv)[0]
    off.apply_pruning_transformation(m)
    convs = [n for n in m.get_ops() if n.get_type_name() == "Convolution"]
    assert list(convs[0].get_output_shape(0)) == [1, 5, 8, 8] and list(convs[1].input_value(1).get_shape()) == [4, 5, 3, 3]
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(xv)[0], ref, rtol=1e-5, atol=1e-5)
    # a bias that revives a dead channel blocks the rewrite
    b_bad = b1.copy()
    b_bad[0, 1] = 0.5
    y2 = ops.relu(ops.add(ops.convolution(x, w1, [1, 1], [1, 1], [1, 1], [1, 1]), b_bad))
    m2 = ov.Model([ops.result(ops.convolution(y2, w2, [1, 1], [1, 1], [1, 1], [1, 1]))], [x], "kept")
    assert not Pruning().run_on_model(m2)
