"""Repeated-block folding, the weights bank and the NPUW device (runtime/npuw.py)."""
import numpy as np
import pytest

import openvino_b200 as ov
from openvino_b200 import opset as ops
from openvino_b200.runtime.npuw import WeightsBank, dedupe_constants, find_repeated_blocks, fold_repeated_blocks


def _stack(layers=4, H=16, seed=0, tied=False):
    rng = np.random.default_rng(seed)
    x = ops.parameter([-1, H], "f32", "x")
    h = ops.relu(x)
    shared = rng.standard_normal((2 * H,)).astype(np.float32)
    for _ in range(layers):
        w1 = rng.standard_normal((H, 2 * H)).astype(np.float32) * 0.2
        b1 = shared.copy() if tied else rng.standard_normal((2 * H,)).astype(np.float32)
        w2 = rng.standard_normal((2 * H, H)).astype(np.float32) * 0.2
        t = ops.gelu(ops.add(ops.matmul(h, w1, False, False), b1), "ERF")
        h = ops.mvn(ops.add(h, ops.matmul(t, w2, False, False)), np.array([-1], np.int64), True, 1e-5, "inside_sqrt")
    return ov.Model([ops.sigmoid(h)], [x], "stack")


def test_fold_compiles_the_block_once_and_keeps_the_numbers():
    m = _stack(layers=5)
    xv = np.random.default_rng(1).standard_normal((3, 16)).astype(np.float32)
    ref = ov.compile_model(m.clone(), "CPU")([xv])[0]
    blocks = find_repeated_blocks(m)
    assert (blocks.count, blocks.length) == (5, 6)
    f = fold_repeated_blocks(m)
    types = [n.get_type_name() for n in m.get_ops() if n.get_type_name() != "Constant"]
    assert types == ["Parameter", "Relu"] + ["FunctionCall"] * 5 + ["Sigmoid", "Result"]
    assert (f.n_external, f.n_closure) == (1, 3)                 # the residual stream; two weight matrices and a bias
    assert [p.get_friendly_name() for p in f.body.get_parameters()] == ["ext0", "w0", "w1", "w2"]
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xv])[0], ref, rtol=1e-6, atol=1e-6)
    assert f.compiles == 1 and f.calls == 5
    # dynamic batch flows through the calls
    xv2 = np.random.default_rng(2).standard_normal((7, 16)).astype(np.float32)
    assert ov.compile_model(m, "CPU")([xv2])[0].shape == (7, 16)


def test_blocks_with_state_are_not_folded():
    x = ops.parameter([1, 8], "f32", "x")
    h = x
    sinks = []
    for l in range(3):
        rv = ops.read_value(ops.constant(np.zeros((1, 8), np.float32)), "v%d" % l, "f32", [1, 8])
        s = ops.add(rv, ops.multiply(h, np.full((1, 8), 0.5 + l, np.float32)))
        sinks.append(ops.assign(s, "v%d" % l))
        h = ops.tanh(ops.add(ops.relu(s), ops.multiply(h, np.full((1, 8), 0.25, np.float32))))
    m = ov.Model([h], [x], "stateful", sinks)
    before = [n.get_type_name() for n in m.get_ops()]
    f = fold_repeated_blocks(m, min_ops=2)
    after = [n.get_type_name() for n in m.get_ops()]
    assert after.count("ReadValue") == 3 and after.count("Assign") == before.count("Assign")
    if f is not None:                                     # whatever was folded holds neither ReadValue nor Assign
        assert not any(n.get_type_name() in ("ReadValue", "Assign") for n in f.body.get_ops())
    req = ov.compile_model(m, "CPU").create_infer_request()
    one = np.ones((1, 8), np.float32)
    a = req.infer([one])[0].copy()
    b = req.infer([one])[0].copy()
    assert not np.allclose(a, b)                          # the states moved between the two inferences


def test_weights_bank_and_device():
    m = _stack(layers=3, tied=True, seed=5)
    bank = WeightsBank("test")
    assert dedupe_constants(m, bank) == 2 and len(bank) >= 7            # three equal biases become one
    core = ov.Core()
    xv = np.random.default_rng(3).standard_normal((2, 16)).astype(np.float32)
    ref = ov.compile_model(_stack(layers=3, tied=True, seed=5), "CPU")([xv])[0]
    cm = core.compile_model(_stack(layers=3, tied=True, seed=5), "NPUW", {"NPUW_DEVICES": "CPU"})
    assert cm.get_property("NPUW_FOLDED_BLOCKS") == 3 and cm.get_property("EXECUTION_DEVICES") == ["NPUW", "CPU"]
    np.testing.assert_allclose(cm([xv])[0], ref, rtol=1e-6, atol=1e-6)
    dev_bank = WeightsBank.for_device("CPU/shared")
    hits = dev_bank.hits
    core.compile_model(_stack(layers=3, tied=True, seed=5), "NPUW:CPU")      # a second model over the same weights
    assert dev_bank.hits >= hits + 7
    off = core.compile_model(_stack(layers=3), "NPUW", {"NPUW_DEVICES": "CPU", "NPUW_FOLD": "NO"})
    assert off.get_property("NPUW_FOLDED_BLOCKS") == 0


@pytest.mark.gpu
def test_folded_stack_on_cuda():
    core = ov.Core()
    xv = np.random.default_rng(4).standard_normal((5, 16)).astype(np.float32)
    ref = ov.compile_model(_stack(layers=6, seed=9), "CPU")([xv])[0]
    cm = core.compile_model(_stack(layers=6, seed=9), "NPUW", {"NPUW_DEVICES": "CUDA"})
    assert cm.get_property("NPUW_FOLDED_BLOCKS") == 6
    np.testing.assert_allclose(cm([xv])[0], ref, rtol=2e-3, atol=2e-3)
    assert cm.function.compiles == 1 and cm.function.calls == 6
