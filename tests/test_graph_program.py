"""The device graph program (operation table + executor of the CUDA device), exercised on the host with CPU tensors:
every model must give what the native reference executor gives."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import Model, Tensor, _ovcore as _c
from openvino_b200 import opset as ops
from openvino_b200.models import llama
from openvino_b200.models.llm_config import TINY_LLAMA
from openvino_b200.models.ov_builders import build_llama
from openvino_b200.models.torch_zoo import ResNet18, bert_tiny
from openvino_b200.runtime.cuda_plugin import GraphProgram, supported_op_types


def both(m: Model, arrays, transform=True, rtol=1e-4, atol=1e-4):
    want = ov.compile_model(m, "CPU")(list(arrays))
    rm = m.clone()
    if transform:
        _c.run_moc_transformations(rm._m, True)
        _c.run_llm_fusions(rm._m)
        from openvino_b200.runtime import cuda_fusions
        cuda_fusions.run(rm)          # bias / activation into FullyConnected, LayerNorm as one operation
    prog = GraphProgram(rm, "cpu")
    got = prog.run([torch.from_numpy(np.ascontiguousarray(a)) for a in arrays])
    assert len(got) == len(want)
    for i, g in enumerate(got):
        np.testing.assert_allclose(g.float().numpy() if g.dtype.is_floating_point else g.numpy(), want[i], rtol=rtol, atol=atol)
    return prog


def test_resnet_and_bert_graphs():
    torch.manual_seed(0)
    net = ResNet18(num_classes=10, width=8).eval()
    m = ov.convert_model(net, example_input=(torch.randn(1, 3, 64, 64),))
    both(m, [np.random.default_rng(0).standard_normal((1, 3, 64, 64)).astype(np.float32)], rtol=1e-3, atol=1e-3)
    bert = bert_tiny().eval()
    ids = torch.randint(0, 100, (2, 10))
    mask = torch.ones(2, 10, dtype=torch.int64)
    mask[0, 7:] = 0
    m = ov.convert_model(bert, example_input=(ids, mask, torch.zeros(2, 10, dtype=torch.int64)))
    fused = m.clone()
    _c.run_moc_transformations(fused._m, True)
    _c.run_llm_fusions(fused._m)
    from openvino_b200.runtime import cuda_fusions
    assert cuda_fusions.run(fused) >= 12
    types = [n.get_type_name() for n in fused.get_ops()]
    assert "LayerNormFused" in types and "MVN" not in types and "Gelu" not in types
    both(m, [ids.numpy(), mask.numpy(), np.zeros((2, 10), np.int64)], rtol=1e-3, atol=1e-3)


def test_fused_llama_graph_with_state():
    cfg = TINY_LLAMA.with_(vocab_size=64, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=64, ffn_size=256, group_size=64)
    state = llama.random_float_state(cfg, seed=1, std=0.1)
    for compress in (None, "int4"):
        m = build_llama(cfg, state, compress=compress)
        rm = m.clone()
        _c.run_moc_transformations(rm._m, True)
        _c.run_llm_fusions(rm._m)
        prog = GraphProgram(rm, "cpu")
        assert not prog.fallback_nodes
        req = ov.compile_model(m, "CPU").create_infer_request()
        ids = np.array([[3, 9, 27, 5]], np.int64)
        feeds = [[ids, np.ones((1, 4), np.int64), np.arange(4)[None], np.zeros(1, np.int32)],
                 [np.array([[11]], np.int64), np.ones((1, 5), np.int64), np.array([[4]], np.int64), np.zeros(1, np.int32)]]
        for feed in feeds:       # prefill, then one decode step from the state
            want = req.infer(feed)[0]
            got = prog.run([torch.from_numpy(a) for a in feed])[0].numpy()
            np.testing.assert_allclose(got, want, rtol=2e-2 if compress else 1e-3, atol=2e-2 if compress else 1e-4)


def test_misc_ops_match_reference():
    rng = np.random.default_rng(2)
    x = ops.parameter([2, 6, 5], "f32")
    i = ops.parameter([3], "i64")
    parts = ops.variadic_split(x, 1, [2, -1])
    y = ops.concat([ops.relu(parts.output(0)).output(0), ops.sigmoid(parts.output(1)).output(0)], 1)
    g = ops.gather(y, i, 1)
    s = ops.slice(g, [4], [0], [-2], [2])
    t = ops.transpose(ops.reshape(s, [0, -1], True), [1, 0])
    r = ops.reduce_sum(ops.multiply(t, t), [0], True)
    tk = ops.topk(ops.squeeze(r, [0]), 2, 0, "max", "value", "i64")
    cs = ops.cumsum(ops.pad(x, [0, 1, 0], [0, 0, 2], np.float32(0.5), "constant"), 2, False, True)
    sel = ops.select(ops.greater(x, np.float32(0)), x, ops.negative(x))
    st = ops.strided_slice(x, [0, 1, 0], [0, 5, 0], [1, 2, 1], [1, 0, 1], [1, 0, 1])
    m = Model([tk.output(0), tk.output(1), cs.output(0), sel.output(0), st.output(0), ops.softmax(ops.mvn(x, [-1], True, 1e-6, "inside_sqrt"), 1).output(0)], [x, i], "misc")
    both(m, [rng.standard_normal((2, 6, 5)).astype(np.float32), np.array([5, 0, 2], np.int64)], transform=False)


def test_dynamic_shapes_and_host_fallback():
    x = ops.parameter([-1, 4], "f32")
    b = ops.gather(ops.shape_of(x), [0], 0)
    y = ops.reshape(ops.multiply(x, np.float32(2)), ops.concat([b.output(0), ops.constant(np.array([2, 2], np.int64)).output(0)], 0), False)
    e = ops.einsum([y.output(0), y.output(0)], "bij,bjk->bik")
    e = ops.selu(e, np.float32(1.5), np.float32(1.0))               # no device implementation: host fallback
    m = Model([e], [x], "dyn")
    rm = m.clone()
    prog = GraphProgram(rm, "cpu")
    assert prog.fallback_nodes == [e.get_friendly_name()]
    for n in (1, 3):
        a = np.random.default_rng(n).standard_normal((n, 4)).astype(np.float32)
        got = prog.run([torch.from_numpy(a)])[0].numpy()
        y_ = (2 * a).reshape(n, 2, 2)
        z = y_ @ y_
        np.testing.assert_allclose(got, np.where(z > 0, z, 1.5 * (np.exp(z) - 1)), rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError, match="no device implementation"):
        GraphProgram(rm, "cpu", host_fallback=False)
    assert {"FullyConnectedCompressed", "PagedAttentionExtension", "RMS", "RoPE", "Convolution"} <= set(supported_op_types())
