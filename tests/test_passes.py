"""Graph passes: infrastructure (Manager, MatcherPass, patterns from Python) and the named transformations,
checked structurally and by comparing evaluation before and after (the reference's TransformationTestsF pattern,
src/tests/test_utils/common_test_utils/include/common_test_utils/ov_test_utils.hpp)."""
from collections import Counter

import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import Model, PartialShape, Tensor, Type
from openvino_b200 import _offline_transformations as offline
from openvino_b200 import opset as ops
from openvino_b200 import passes
from openvino_b200.models import llama
from openvino_b200.models.llm_config import TINY_LLAMA
from openvino_b200.models.ov_builders import build_llama

CFG = TINY_LLAMA.with_(vocab_size=128, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=64, ffn_size=256, group_size=64, num_layers=2)


def types(m):
    return Counter(n.get_type_name() for n in m.get_ops())


def infer(m, *arrays):
    return ov.compile_model(m, "CPU")(list(arrays))


def test_constant_folding_and_nop_elimination():
    x = ops.parameter([2, 3], "f32")
    c = ops.add(ops.constant(np.ones((2, 3), np.float32)), ops.multiply(np.float32(2), np.float32(3)))
    y = ops.add(x, c)
    y = ops.reshape(y, [2, 3], False)            # no-op reshape
    y = ops.convert(y, "f32")                    # no-op convert
    y = ops.transpose(y, [0, 1])                 # identity transpose
    m = Model([y], [x], "cf")
    before = infer(m, np.zeros((2, 3), np.float32))[0]
    pm = passes.Manager()
    pm.register_pass(passes.ConstantFolding())
    pm.register_pass("NopElimination")
    assert pm.run_passes(m)
    t = types(m)
    assert t["Add"] == 1 and t["Multiply"] == 0 and t["Reshape"] == 0 and t["Convert"] == 0 and t["Transpose"] == 0
    np.testing.assert_array_equal(infer(m, np.zeros((2, 3), np.float32))[0], before)
    assert [name for name, ms, changed in pm.get_timings()] == ["ConstantFolding", "NopElimination"]


def test_python_matcher_pass_rewrites_graph():
    x = ops.parameter([4], "f32")
    y = ops.relu(ops.add(x, np.float32(1)))
    m = Model([ops.exp(y)], [x], "mp")
    add_p = passes.WrapType("opset1.Add", [passes.AnyInput(), passes.WrapType("Constant")])
    relu_p = passes.WrapType("Relu", [add_p], passes.consumers_count(1))
    seen = []

    def callback(matcher):
        root = matcher.get_match_root()
        pmap = matcher.get_pattern_value_map()
        assert add_p in pmap and pmap[relu_p].get_node() == root
        seen.append(root.get_type_name())
        new = ops.sigmoid(pmap[add_p])
        root.output(0).replace(new.output(0))
        return True
    p = passes.MatcherPass(passes.Matcher(relu_p, "ReluToSigmoid"), callback)
    pm = passes.Manager()
    pm.register_pass(p)
    assert pm.run_passes(m) and seen == ["Relu"]
    assert types(m)["Relu"] == 0 and types(m)["Sigmoid"] == 1
    v = np.array([0.0, 1.0, -1.0, 2.0], np.float32)
    np.testing.assert_allclose(infer(m, v)[0], np.exp(1 / (1 + np.exp(-(v + 1)))), rtol=1e-6)


def test_matcher_or_optional_and_predicates():
    x = ops.parameter([2, 2], "f32")
    a = ops.relu(ops.convert(x, "f32"))
    b = ops.sigmoid(x)
    pat = passes.Or([passes.WrapType("Relu", [passes.Optional("Convert", [passes.AnyInput()])]), passes.WrapType("Tanh")])
    mt = passes.Matcher(pat, "m")
    assert mt.match(a.output(0)) and not mt.match(b.output(0))
    assert passes.Matcher(passes.WrapType("Relu", [passes.AnyInput(passes.rank_equals(3))])).match(a.output(0)) is False
    assert passes.Matcher(passes.AnyInput(passes.type_matches(Type.f32))).match(b.output(0))


def test_custom_model_pass_and_disable():
    class Count(passes.ModelPass):
        def __init__(self):
            super().__init__("Count")
            self.n = 0

        def run_on_model(self, model):
            self.n = len(model.get_ops())
            return False
    x = ops.parameter([1], "f32")
    m = Model([ops.add(x, ops.multiply(np.float32(2), np.float32(3)))], [x], "c")
    cnt = Count()
    pm = passes.Manager()
    pm.register_pass("ConstantFolding")
    pm.register_pass(cnt)
    pm.disable("ConstantFolding")
    assert pm.run_passes(m) is False and cnt.n == 6 and types(m)["Multiply"] == 1
    pm.enable("ConstantFolding")
    assert pm.run_passes(m) and cnt.n == 4


def test_batch_norm_decomposition_and_fp16_compression():
    rng = np.random.default_rng(0)
    x = ops.parameter([1, 4, 5, 5], "f32")
    g, b, mu, var = (rng.uniform(0.5, 1.5, 4).astype(np.float32) for _ in range(4))
    y = ops.batch_norm_inference(ops.convolution(x, rng.standard_normal((4, 4, 3, 3)).astype(np.float32), [1, 1], [1, 1], [1, 1], [1, 1]), g, b, mu, var, 1e-5)
    m = Model([y], [x], "bn")
    inp = rng.standard_normal((1, 4, 5, 5)).astype(np.float32)
    before = infer(m, inp)[0]
    offline.apply_moc_transformations(m)
    assert types(m)["BatchNormInference"] == 0
    np.testing.assert_allclose(infer(m, inp)[0], before, rtol=1e-4, atol=1e-5)
    offline.compress_model_transformation(m)
    consts = [n for n in m.get_ops() if n.get_type_name() == "Constant" and n.get_output_shape(0) == [4, 4, 3, 3]]
    assert consts and consts[0].get_output_element_type(0) == Type.f16
    conv = [n for n in m.get_ops() if n.get_type_name() == "Convert"][0]
    assert "decompression" in " ".join(conv.rt_info.keys()).lower()
    np.testing.assert_allclose(infer(m, inp)[0], before, rtol=2e-2, atol=2e-2)


def test_convert_precision():
    x = ops.parameter([2, 2], "f32")
    m = Model([ops.add(x, np.ones((2, 2), np.float32))], [x], "p")
    passes.ConvertPrecision("f32", "f16").run_on_model(m)
    assert m.input(0).get_element_type() == Type.f16 and m.output(0).get_element_type() == Type.f16


def test_weight_compression_int4_and_int8():
    rng = np.random.default_rng(1)
    x = ops.parameter([3, 256], "f32")
    w = rng.standard_normal((64, 256)).astype(np.float32)
    m = Model([ops.matmul(x, w, False, True)], [x], "wc")
    inp = rng.standard_normal((3, 256)).astype(np.float32)
    ref = inp @ w.T
    for mode, tol in (("int8_asym", 0.02), ("int4_asym", 0.15)):
        c = m.clone()
        assert passes.CompressWeights(mode=mode, group_size=64, all_layers=True).run_on_model(c)
        lp = [n for n in c.get_ops() if n.get_type_name() == "Constant" and n.get_output_element_type(0) in (Type.u4, Type.u8)]
        assert lp, mode
        out = infer(c, inp)[0]
        assert np.linalg.norm(out - ref) / np.linalg.norm(ref) < tol


def test_make_stateful_and_back():
    x = ops.parameter([1, 4], "f32", "x")
    past = ops.parameter([1, 4], "f32", "past")
    past.output(0).set_names({"past"})
    s = ops.add(past, x)
    s.output(0).set_names({"present"})
    m = Model([ops.result(ops.relu(s), "out"), ops.result(s, "present")], [x, past], "st")
    offline.apply_make_stateful_transformation(m, {"past": "present"})
    t = types(m)
    assert t["ReadValue"] == 1 and t["Assign"] == 1 and len(m.get_parameters()) == 1 and len(m.get_results()) == 1
    assert [v.get_info().variable_id for v in m.get_variables()] == ["pastpresent"]
    req = ov.compile_model(m, "CPU").create_infer_request()
    one = np.ones((1, 4), np.float32)
    assert (req.infer([one])[0] == 1).all() and (req.infer([one])[0] == 2).all()
    offline.stateful_to_stateless_transformation(m)
    t = types(m)
    assert t["ReadValue"] == 0 and t["Assign"] == 0 and len(m.get_parameters()) == 2 and len(m.get_results()) == 2


@pytest.fixture(scope="module")
def llama_state():
    return llama.random_float_state(CFG, seed=0, std=0.1)


def run_stateful(m, ids):
    req = ov.compile_model(m, "CPU").create_infer_request()
    n = len(ids)
    return req.infer({"input_ids": np.asarray(ids)[None], "attention_mask": np.ones((1, n), np.int64),
                      "position_ids": np.arange(n)[None], "beam_idx": np.zeros(1, np.int32)})[0][0]


def test_llm_fusions_keep_numerics(llama_state):
    ids = list(range(3, 12))
    ref = llama.reference_logits(CFG, llama_state, torch.tensor(ids)).numpy()
    m = build_llama(CFG, llama_state)
    np.testing.assert_allclose(run_stateful(m, ids), ref, rtol=1e-3, atol=1e-4)
    pm = passes.Manager()
    for name in ("RMSFusion", "RoPEFusion", "ConvertMatMulToFullyConnected"):
        pm.register_pass(name)
    pm.run_passes(m)
    t = types(m)
    assert t["RMS"] == 2 * CFG.num_layers + 1 and t["RoPE"] == 2 * CFG.num_layers and t["FullyConnected"] == 7 * CFG.num_layers + 1
    assert t["Power"] == 0 and t["Sqrt"] == 0 and t["MatMul"] == 0
    np.testing.assert_allclose(run_stateful(m, ids), ref, rtol=1e-3, atol=1e-4)


def test_compressed_llm_becomes_fully_connected_compressed(llama_state):
    ids = [5, 9, 1, 77, 30]
    m = build_llama(CFG, llama_state, compress="int4")
    eff = llama.effective_state(CFG, llama_state)
    # the graph keeps norms and embeddings in fp32: compare against weights dequantised the same way
    eff = {k: (v if v.dim() == 2 and not k.endswith("embed_tokens") else llama_state[k]) for k, v in eff.items()}
    ref = llama.reference_logits(CFG, eff, torch.tensor(ids)).numpy()
    before = run_stateful(m, ids)
    np.testing.assert_allclose(before, ref, rtol=2e-2, atol=2e-2)
    pm = passes.Manager()
    for name in ("RMSFusion", "RoPEFusion", "ConvertMatMulToFullyConnected", "ConvertFullyConnectedToFullyConnectedCompressed"):
        pm.register_pass(name)
    pm.run_passes(m)
    t = types(m)
    assert t["FullyConnectedCompressed"] == 7 * CFG.num_layers + 1 and t["FullyConnected"] == 0
    fc = [n for n in m.get_ops() if n.get_type_name() == "FullyConnectedCompressed"][0]
    assert fc.input_value(1).get_element_type() == Type.u4
    # the unfused graph rounds (q - zp) * scale to fp16 before the product, the fused op keeps fp32
    np.testing.assert_allclose(run_stateful(m, ids), before, rtol=1e-2, atol=1e-2)


def test_sdpa_to_paged_attention(llama_state):
    m = build_llama(CFG, llama_state)
    offline.paged_attention_transformation(m)
    t = types(m)
    assert t["PagedAttentionExtension"] == CFG.num_layers and t["ScaledDotProductAttention"] == 0
    assert t["ReadValue"] == 0 and t["Assign"] == 0 and not m.get_sinks()
    names = {p.get_friendly_name() for p in m.get_parameters()}
    assert {"input_ids", "position_ids", "past_lens", "subsequence_begins", "block_indices", "block_indices_begins", "max_context_len",
            "key_cache.0", "value_cache.0", "key_cache.1", "value_cache.1"} <= names
    assert "beam_idx" not in names and "attention_mask" not in names
    pa = [n for n in m.get_ops() if n.get_type_name() == "PagedAttentionExtension"][0]
    assert pa.get_input_size() == 28 and pa.get_output_size() == 3
    assert m.input("input_ids").get_partial_shape().to_string() == "[?]"

    # run two sequences as one ragged batch against block caches and compare with the dense reference
    seqs = [[3, 7, 11, 19, 23], [2, 4, 6]]
    bs, Hkv, D = 16, CFG.num_kv_heads, CFG.head_dim
    caches = {}
    for l in range(CFG.num_layers):
        caches["key_cache.%d" % l] = np.zeros((4, Hkv, bs, D), np.float32)
        caches["value_cache.%d" % l] = np.zeros((4, Hkv, bs, D), np.float32)
    feed = {"input_ids": np.array(sum(seqs, []), np.int64), "position_ids": np.array([0, 1, 2, 3, 4, 0, 1, 2], np.int64),
            "past_lens": np.array([0, 0], np.int32), "subsequence_begins": np.array([0, 5, 8], np.int32),
            "block_indices": np.array([2, 0], np.int32), "block_indices_begins": np.array([0, 1, 2], np.int32),
            "max_context_len": np.array(5, np.int32)}
    feed.update(caches)
    cm = ov.compile_model(m, "CPU")
    logits = cm(feed)["logits"]
    logits = logits.reshape(-1, CFG.vocab_size)
    for s, (a, b) in zip(seqs, ((0, 5), (5, 8))):
        ref = llama.reference_logits(CFG, llama_state, torch.tensor(s)).numpy()
        np.testing.assert_allclose(logits[a:b], ref, rtol=1e-3, atol=1e-4)
    # the caches were written in place: decode one more token of sequence 0 from the cache
    assert np.abs(caches["key_cache.0"][2]).sum() > 0
    feed2 = dict(feed, input_ids=np.array([29], np.int64), position_ids=np.array([5], np.int64), past_lens=np.array([5], np.int32),
                 subsequence_begins=np.array([0, 1], np.int32), block_indices=np.array([2], np.int32),
                 block_indices_begins=np.array([0, 1], np.int32), max_context_len=np.array(6, np.int32))
    logits2 = cm(feed2)["logits"].reshape(-1, CFG.vocab_size)
    ref2 = llama.reference_logits(CFG, llama_state, torch.tensor(seqs[0] + [29])).numpy()
    np.testing.assert_allclose(logits2[0], ref2[-1], rtol=1e-3, atol=1e-4)


def test_sdpa_to_paged_attention_reads_sliding_window_and_alibi_from_the_mask():
    cfg = CFG.with_(sliding_window=3)
    state = llama.random_float_state(cfg, seed=3, std=0.05)
    m = build_llama(cfg, state)
    offline.paged_attention_transformation(m)
    pas = [n for n in m.get_ops() if n.get_type_name() == "PagedAttentionExtension"]
    assert all(int(p.input_value(10).get_node().get_data()) == 3 for p in pas)
    # prefill of 6 tokens: every query sees itself and the two keys before it, like the dense reference with the same window
    seq = [3, 7, 11, 19, 23, 5]
    bs = 16
    feed = {"input_ids": np.array(seq, np.int64), "position_ids": np.arange(6, dtype=np.int64), "past_lens": np.array([0], np.int32),
            "subsequence_begins": np.array([0, 6], np.int32), "block_indices": np.array([1], np.int32), "block_indices_begins": np.array([0, 1], np.int32),
            "max_context_len": np.array(6, np.int32)}
    for l in range(cfg.num_layers):
        feed["key_cache.%d" % l] = np.zeros((2, cfg.num_kv_heads, bs, cfg.head_dim), np.float32)
        feed["value_cache.%d" % l] = np.zeros((2, cfg.num_kv_heads, bs, cfg.head_dim), np.float32)
    logits = ov.compile_model(m, "CPU")(feed)["logits"].reshape(-1, cfg.vocab_size)
    ref = llama.reference_logits(cfg, state, torch.tensor(seq)).numpy()
    np.testing.assert_allclose(logits, ref, rtol=1e-3, atol=1e-4)
    full = llama.reference_logits(CFG, state, torch.tensor(seq)).numpy()
    assert np.abs(full[-1] - ref[-1]).max() > 1e-4                  # the window matters for the later tokens
    # ALiBi: slopes [H, 1, 1] times a position term, added to a causal mask
    H, D = 4, 8
    q, k, v = (ops.parameter([1, H, -1, D], "f32", n) for n in "qkv")
    past_k = ops.read_value(ops.constant(np.zeros((1, H, 0, D), np.float32)), "pk", "f32", [1, H, -1, D])
    past_v = ops.read_value(ops.constant(np.zeros((1, H, 0, D), np.float32)), "pv", "f32", [1, H, -1, D])
    kk, vv = ops.concat([past_k, k], 2), ops.concat([past_v, v], 2)
    ids = ops.parameter([1, -1], "i64", "input_ids")
    L = ops.gather(ops.shape_of(ids), np.array([1], np.int64), np.int64(0))
    pos = ops.convert(ops.range(np.int64(0), ops.squeeze(L), np.int64(1), "i64"), "f32")
    slopes = np.array([0.5, 0.25, 0.125, 0.0625], np.float32).reshape(H, 1, 1)
    bias = ops.multiply(slopes, ops.unsqueeze(pos, np.array([0, 1], np.int64)))                       # [H, 1, L]
    causal = ops.select(ops.less_equal(ops.unsqueeze(pos, np.array([0], np.int64)), ops.unsqueeze(pos, np.array([1], np.int64))), np.float32(0), np.float32(-65504))
    mask = ops.add(ops.unsqueeze(bias, np.array([0], np.int64)), ops.unsqueeze(causal, np.array([0, 1], np.int64)))
    att = ops.scaled_dot_product_attention(q, kk, vv, mask)
    ma = Model([att], [q, k, v, ids], "alibi", [ops.assign(kk, "pk"), ops.assign(vv, "pv")])
    offline.paged_attention_transformation(ma)
    pa = next(n for n in ma.get_ops() if n.get_type_name() == "PagedAttentionExtension")
    folded = ov.compile_model(Model([pa.input_value(11)], [], "s"), "CPU")([])[0]
    np.testing.assert_allclose(folded, slopes.reshape(-1))
    assert int(pa.input_value(10).get_node().get_data()) == 0


def test_visualize_and_serialize_passes(tmp_path):
    x = ops.parameter([1], "f32")
    m = Model([ops.relu(x)], [x], "v")
    pm = passes.Manager()
    pm.register_pass(passes.VisualizeTree(str(tmp_path / "g.dot")))
    pm.register_pass(passes.Serialize(str(tmp_path / "m.xml"), str(tmp_path / "m.bin")))
    pm.run_passes(m)
    assert "digraph" in open(tmp_path / "g.dot").read() and (tmp_path / "m.xml").exists()
    assert "ConstantFolding" in passes.available_passes()


def test_low_latency2_makes_recurrent_state_persistent():
    """A TensorIterator with a back edge accumulates over the sequence; after LowLatency2 the accumulator is model state
    that survives between inferences until reset_state."""
    import openvino_b200 as ov
    from openvino_b200 import opset as ops
    from openvino_b200.passes import LowLatency2
    xt = ops.parameter([1, 1, 4], "f32", "xt")
    h = ops.parameter([1, 4], "f32", "h")
    hn = ops.add(h, ops.squeeze(xt, np.array([1], dtype=np.int64)))
    body = ov.Model([ops.result(hn)], [xt, h], "body")
    x = ops.parameter([1, 3, 4], "f32", "x")
    h0 = ops.constant(np.full((1, 4), 10.0, np.float32))
    ti = ops.tensor_iterator()
    ti.set_body(body)
    ti.set_sliced_input(xt, x, axis=1)
    ti.set_merged_input(h, h0, body.get_results()[0])
    out_idx = ti.get_iter_value(body.get_results()[0])
    node = ti.build()
    m = ov.Model([ops.result(node.output(out_idx))], [x], "rnn")
    data = np.arange(12, dtype=np.float32).reshape(1, 3, 4)
    np.testing.assert_allclose(ov.compile_model(m.clone(), "CPU")(data)[0], 10.0 + data.sum(1))
    assert LowLatency2(use_const_initializer=False).run_on_model(m)
    types = [n.get_type_name() for n in m.get_ops()]
    assert "ReadValue" in types and len(m.get_sinks()) == 1
    req = ov.compile_model(m, "CPU").create_infer_request()
    first = req.infer([data])[0].copy()
    second = req.infer([data])[0].copy()
    np.testing.assert_allclose(first, 10.0 + data.sum(1))
    np.testing.assert_allclose(second, 10.0 + 2 * data.sum(1))          # the state carried over
    req.reset_state()
    np.testing.assert_allclose(req.infer([data])[0], 10.0 + data.sum(1))
    assert not LowLatency2().run_on_model(m)                              # idempotent


def _run_pass(m, p):
    mgr = passes.Manager()
    mgr.register_pass(p)
    mgr.run_passes(m)
    return m


def _rope_tables(L, D, repeat):
    inv = 10000.0 ** (-np.arange(0, D, 2, dtype=np.float32) / D)
    ang = np.arange(L, dtype=np.float32)[:, None] * inv[None]
    ang = np.repeat(ang, 2, axis=1) if repeat == "interleave" else np.concatenate([ang, ang], 1)
    return np.cos(ang)[None, None].astype(np.float32), np.sin(ang)[None, None].astype(np.float32)


def test_rope_fusion_interleaved_form():
    """GPT-J "rotate every two": pairs (2i, 2i + 1) are rotated; the tables repeat every angle twice."""
    B, H, L, D = 2, 3, 5, 8
    i64 = lambda v: ops.constant(np.array(v, dtype=np.int64))
    x = ops.parameter([B, H, L, D], "f32", "x")
    cos, sin = _rope_tables(L, D, "interleave")
    odd = ops.slice(x, i64([1]), i64([D]), i64([2]), i64([3]))
    even = ops.slice(x, i64([0]), i64([D]), i64([2]), i64([3]))
    stacked = ops.concat([ops.unsqueeze(ops.negative(odd), i64([4])).output(0), ops.unsqueeze(even, i64([4])).output(0)], 4)
    rot = ops.reshape(stacked, i64([B, H, L, D]), False)
    y = ops.add(ops.multiply(x, ops.constant(cos)), ops.multiply(rot, ops.constant(sin)))
    m = ov.Model([y], [x], "gptj")
    xin = np.random.default_rng(0).standard_normal((B, H, L, D)).astype(np.float32)
    want = ov.compile_model(m, "CPU")([xin])[0]
    _run_pass(m, passes.RoPEFusion())
    rope = [n for n in m.get_ops() if n.get_type_name() == "RoPE"]
    assert len(rope) == 1 and rope[0].get_attribute("is_interleaved") and rope[0].get_attribute("rotary_ndims") == D
    assert not any(n.get_type_name() in ("Slice", "Concat", "Negative") for n in m.get_ops())
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xin])[0], want, rtol=1e-5, atol=1e-6)


def test_rope_fusion_partial_rotary():
    """Only the first `rot` channels of every head are rotated (GPT-NeoX / Phi); the rest passes through."""
    B, H, L, D, rot = 1, 2, 6, 16, 8
    i64 = lambda v: ops.constant(np.array(v, dtype=np.int64))
    x = ops.parameter([B, H, L, D], "f32", "x")
    cos, sin = _rope_tables(L, rot, "halves")
    head = ops.slice(x, i64([0]), i64([rot]), i64([1]), i64([3]))
    tail = ops.slice(x, i64([rot]), i64([D]), i64([1]), i64([3]))
    lo = ops.slice(head, i64([0]), i64([rot // 2]), i64([1]), i64([3]))
    hi = ops.slice(head, i64([rot // 2]), i64([rot]), i64([1]), i64([3]))
    rotated = ops.concat([ops.negative(hi).output(0), lo.output(0)], 3)
    emb = ops.add(ops.multiply(head, ops.constant(cos)), ops.multiply(rotated, ops.constant(sin)))
    y = ops.concat([emb.output(0), tail.output(0)], 3)
    m = ov.Model([y], [x], "neox")
    xin = np.random.default_rng(1).standard_normal((B, H, L, D)).astype(np.float32)
    want = ov.compile_model(m, "CPU")([xin])[0]
    _run_pass(m, passes.RoPEFusion())
    rope = [n for n in m.get_ops() if n.get_type_name() == "RoPE"]
    assert len(rope) == 1 and rope[0].get_attribute("rotary_ndims") == rot and rope[0].get_attribute("head_size") == D
    assert rope[0].input_value(0).get_node().get_type_name() == "Parameter"           # the slices are gone: RoPE reads the whole head
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xin])[0], want, rtol=1e-5, atol=1e-6)


def test_rope_fusion_qwen_fused_qkv():
    """Qwen: heads cut out of the fused QKV projection, [B, L, H, S] order, halves swapped through reshape / split, tables
    [1, positions, 1, S] already cut to the tokens at hand -> RoPE {is_qwen} reading the projection itself."""
    B, L, H, S = 2, 5, 3, 8
    i64 = lambda v: ops.constant(np.array(v, dtype=np.int64))
    qkv = ops.parameter([B, L, 3 * H * S], "f32", "qkv")
    cos, sin = _rope_tables(L, S, "halves")
    cos, sin = cos.reshape(1, L, 1, S), sin.reshape(1, L, 1, S)
    parts = ops.variadic_split(qkv, i64(2), i64([H * S, H * S, H * S]))
    outs = []
    for k in (0, 1):
        x = ops.reshape(parts.output(k), i64([0, 0, H, S]), True)
        halves = ops.split(ops.reshape(x, i64([0, 0, 0, 2, S // 2]), True), i64(-2), 2)
        rot = ops.concat([ops.squeeze(ops.multiply(halves.output(1), np.float32(-1.0)), i64(-2)).output(0), ops.squeeze(halves.output(0), i64(-2)).output(0)], -1)
        outs.append(ops.add(ops.multiply(x, ops.constant(cos)), ops.multiply(rot, ops.constant(sin))))
    m = ov.Model(outs, [qkv], "qwen")
    xin = np.random.default_rng(3).standard_normal((B, L, 3 * H * S)).astype(np.float32)
    want = ov.compile_model(m, "CPU")([xin])
    want = [want[0], want[1]]
    _run_pass(m, passes.RoPEFusion())
    rope = [n for n in m.get_ops() if n.get_type_name() == "RoPE"]
    assert len(rope) == 2 and all(r.get_attribute("is_qwen") and r.get_attribute("head_cnt") == H and r.get_attribute("head_size") == S for r in rope)
    assert sorted(r.get_attribute("slice_start") for r in rope) == [0, H * S]
    assert all(r.input_value(0).get_node().get_type_name() == "Parameter" for r in rope)
    assert not any(n.get_type_name() in ("VariadicSplit", "Split", "Squeeze") for n in m.get_ops())
    got = ov.compile_model(m, "CPU")([xin])
    for k in (0, 1):
        assert list(got[k].shape) == [B, L, H, S]
        np.testing.assert_allclose(got[k], want[k], rtol=1e-5, atol=1e-6)


def test_rope_fusion_chatglm_fused_qkv():
    """ChatGLM: [L, B, W] projection, neighbouring pairs of the first `rot` values of each head rotated by a combined
    (cos, sin) cache [L, 1, 1, rot / 2, 2], the rest of the head passes through -> RoPE {is_chatglm}."""
    L, B, H, S, rot = 4, 2, 3, 16, 8
    i64 = lambda v: ops.constant(np.array(v, dtype=np.int64))
    qkv = ops.parameter([L, B, H * S + 2 * 2 * S], "f32", "qkv")          # multi-query: 3 query heads, 2 key and 2 value heads
    ang = np.arange(L, dtype=np.float32)[:, None] * (10000.0 ** (-np.arange(0, rot, 2, dtype=np.float32) / rot))[None]
    cache = np.stack([np.cos(ang), np.sin(ang)], -1).reshape(L, 1, 1, rot // 2, 2).astype(np.float32)
    parts = ops.variadic_split(qkv, i64(-1), i64([H * S, 2 * S, 2 * S]))
    x = ops.reshape(parts.output(0), i64([0, 0, H, S]), True)
    head = ops.slice(x, i64([0]), i64([rot]), i64([1]), i64([3]))
    tail = ops.slice(x, i64([rot]), i64([S]), i64([1]), i64([3]))
    pairs = ops.reshape(head, i64([0, 0, H, rot // 2, 2]), True)
    cc = ops.constant(cache)
    p0, p1 = ops.gather(pairs, i64(0), i64(-1)), ops.gather(pairs, i64(1), i64(-1))
    c, s_ = ops.gather(cc, i64(0), i64(-1)), ops.gather(cc, i64(1), i64(-1))
    o0 = ops.subtract(ops.multiply(p0, c), ops.multiply(p1, s_))
    o1 = ops.add(ops.multiply(p1, c), ops.multiply(p0, s_))
    stack = ops.concat([ops.unsqueeze(o0, i64(-1)).output(0), ops.unsqueeze(o1, i64(-1)).output(0)], -1)
    y = ops.concat([ops.reshape(stack, i64([0, 0, H, rot]), True).output(0), tail.output(0)], -1)
    m = ov.Model([y], [qkv], "chatglm")
    xin = np.random.default_rng(4).standard_normal((L, B, H * S + 4 * S)).astype(np.float32)
    want = ov.compile_model(m, "CPU")([xin])[0]
    _run_pass(m, passes.RoPEFusion())
    rope = [n for n in m.get_ops() if n.get_type_name() == "RoPE"]
    assert len(rope) == 1 and rope[0].get_attribute("is_chatglm") and rope[0].get_attribute("rotary_ndims") == rot
    assert rope[0].get_attribute("slice_start") == 0 and rope[0].get_attribute("slice_stop") == H * S
    assert not any(n.get_type_name() in ("Gather", "Slice", "VariadicSplit") for n in m.get_ops())
    got = ov.compile_model(m, "CPU")([xin])[0]
    assert list(got.shape) == [L, B, H, S]
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


def test_rope_fusion_leaves_blhs_tables_alone():
    """x in [B, L, H, S] order with tables [1, L, 1, S] and slice-built halves is not the [B, H, L, S] form RoPE reads: no fusion."""
    B, L, H, S = 1, 4, 2, 8
    i64 = lambda v: ops.constant(np.array(v, dtype=np.int64))
    x = ops.parameter([B, L, H, S], "f32", "x")
    cos, sin = _rope_tables(L, S, "halves")
    cos, sin = cos.reshape(1, L, 1, S), sin.reshape(1, L, 1, S)
    lo = ops.slice(x, i64([0]), i64([S // 2]), i64([1]), i64([3]))
    hi = ops.slice(x, i64([S // 2]), i64([S]), i64([1]), i64([3]))
    y = ops.add(ops.multiply(x, ops.constant(cos)), ops.multiply(ops.concat([ops.negative(hi).output(0), lo.output(0)], 3), ops.constant(sin)))
    m = ov.Model([y], [x], "blhs")
    xin = np.random.default_rng(5).standard_normal((B, L, H, S)).astype(np.float32)
    want = ov.compile_model(m, "CPU")([xin])[0]
    _run_pass(m, passes.RoPEFusion())
    assert not any(n.get_type_name() == "RoPE" for n in m.get_ops())
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xin])[0], want, rtol=1e-6)


def test_lora_subgraph_fusion_keeps_adapters_switchable():
    rng = np.random.default_rng(2)
    din, dout, r = 16, 12, 4
    x = ops.parameter([3, din], "f32", "x")
    w = rng.standard_normal((dout, din)).astype(np.float32)
    a0, b0 = rng.standard_normal((r, din)).astype(np.float32), rng.standard_normal((dout, r)).astype(np.float32)
    al0 = np.full((1, r), 0.5, np.float32)
    main = ops.matmul(x, w, False, True, name="proj")
    A = ops.read_value(ops.constant(a0), "lora_A", "f32", ov.PartialShape([-1, din]))
    AL = ops.read_value(ops.constant(al0), "lora_alpha", "f32", ov.PartialShape([1, -1]))
    Bm = ops.read_value(ops.constant(b0), "lora_B", "f32", ov.PartialShape([dout, -1]))
    low = ops.matmul(ops.multiply(ops.matmul(x, A, False, True), AL), Bm, False, True)
    y = ops.add(main, low)
    m = ov.Model([y], [x], "lora")
    xin = rng.standard_normal((3, din)).astype(np.float32)
    want = xin @ w.T + ((xin @ a0.T) * al0) @ b0.T
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xin])[0], want, rtol=1e-4, atol=1e-5)
    _run_pass(m, passes.LoraSubgraphFusion())
    fused = [n for n in m.get_ops() if n.get_type_name() == "LoraSubgraph"]
    assert len(fused) == 1 and sum(1 for n in m.get_ops() if n.get_type_name() == "MatMul") == 1
    cm = ov.compile_model(m, "CPU")
    req = cm.create_infer_request()
    np.testing.assert_allclose(req.infer([xin])[0], want, rtol=1e-4, atol=1e-5)
    # another adapter (another rank) through the states
    a1, b1 = rng.standard_normal((2, din)).astype(np.float32), rng.standard_normal((dout, 2)).astype(np.float32)
    for st in req.query_state():
        st.state = ov.Tensor({"lora_A": a1, "lora_alpha": np.ones((1, 2), np.float32), "lora_B": b1}[st.name])
    np.testing.assert_allclose(req.infer([xin])[0], xin @ w.T + (xin @ a1.T) @ b1.T, rtol=1e-4, atol=1e-5)


def test_symbols_travel_with_dynamic_dimensions():
    """Dynamic dimensions carry symbols through shape inference; where operands must agree their symbols become one."""
    a = ops.parameter(ov.PartialShape([-1, 16]), "f32", "a")
    b = ops.parameter(ov.PartialShape([-1, 16]), "f32", "b")
    w = np.ones((8, 16), np.float32)
    ya = ops.matmul(ops.relu(a), w, False, True)                       # [?, 8]: keeps a's batch symbol
    yb = ops.reshape(b, np.array([0, 4, 4], np.int64), True)           # [?, 4, 4]: keeps b's batch symbol
    cat = ops.concat([a.output(0), b.output(0)], 1)                    # rows must agree: a's and b's symbols become equal
    m = ov.Model([ya, yb, cat], [a, b], "sym")
    assert not m.input(0).get_partial_shape()[0].has_symbol()
    _run_pass(m, passes.SymbolicPropagation())
    sa, sb = m.input(0).get_partial_shape()[0].get_symbol(), m.input(1).get_partial_shape()[0].get_symbol()
    assert sa is not None and sb is not None
    assert m.output(0).get_partial_shape()[0].get_symbol() == sa and not m.output(0).get_partial_shape()[1].has_symbol()
    assert m.output(1).get_partial_shape()[0].get_symbol() == sb
    assert ov.symbol.are_equal(sa, sb)                                  # through the Concat
    assert m.output(2).get_partial_shape()[0].get_symbol() == sa
    # fresh symbols are unrelated until they are declared equal
    s1, s2 = ov.Symbol(), ov.Symbol()
    assert s1 != s2 and not ov.symbol.are_equal(s1, s2)
    ov.symbol.set_equal(s1, s2)
    assert s1 == s2 and ov.symbol.ancestor_of(s2) == s1
    # static dimensions never carry one; serialisation ignores symbols
    d = ov.Dimension(4)
    d.set_symbol(s1)
    assert not d.has_symbol()
    xml, _ = ov._ovcore.serialize(m._m)
    assert b"Symbol" not in xml


def test_precision_sensitive_islands_stay_in_fp32():
    """Soft-max written out (exp / sum / divide) overflows in fp16 for large logits; the marking pass keeps that island in
    fp32 while the projections around it are converted."""
    from openvino_b200 import rt_info as rt
    rng = np.random.default_rng(3)
    x = ops.parameter([2, 8], "f32", "x")
    w1 = rng.standard_normal((16, 8)).astype(np.float32)
    w2 = rng.standard_normal((4, 16)).astype(np.float32) * 0.1
    h = ops.matmul(x, w1, False, True, name="proj_in")
    e = ops.exp(h, name="exp")
    ssum = ops.reduce_sum(e, np.array([1], np.int64), True, name="sum")
    p = ops.divide(e, ssum, name="normalise")
    y = ops.matmul(p, w2, False, True, name="proj_out")
    m = ov.Model([y], [x], "softmax_written_out")
    xin = (rng.standard_normal((2, 8)) * 6).astype(np.float32)             # exp() of these sums leaves the fp16 range
    want = ov.compile_model(m, "CPU")([xin])[0]
    plain = m.clone()
    _run_pass(plain, passes.ConvertPrecision("f32", "f16"))
    lossy = ov.compile_model(plain, "CPU")([xin.astype(np.float16)])[0].astype(np.float32)
    assert not np.isfinite(lossy).all() or np.abs(lossy - want).max() > 1e-2       # without the island the result is ruined
    _run_pass(m, passes.MarkSugraphsToKeepInMixedPrecision())
    by_name = {n.get_friendly_name(): n for n in m.get_ops()}
    assert all(rt.fp16_compression_is_disabled(by_name[k]) for k in ("exp", "sum", "normalise"))
    assert not rt.fp16_compression_is_disabled(by_name["proj_in"]) and not rt.fp16_compression_is_disabled(by_name["proj_out"])
    _run_pass(m, passes.ConvertPrecision("f32", "f16"))
    by_name = {n.get_friendly_name(): n for n in m.get_ops()}
    assert by_name["proj_in"].get_output_element_type(0).name == "f16" and by_name["proj_out"].get_output_element_type(0).name == "f16"
    assert all(by_name[k].get_output_element_type(0).name == "f32" for k in ("exp", "sum", "normalise"))
    got = ov.compile_model(m, "CPU")([xin.astype(np.float16)])[0].astype(np.float32)
    assert np.isfinite(got).all() and np.abs(got - want).max() < 2e-2 * max(1.0, np.abs(want).max())
    # attribute helpers
    c = ops.constant(np.ones(4, np.float32))
    rt.enable_keep_const_precision(c)
    assert rt.is_keep_const_precision(c)
    rt.disable_keep_const_precision(c)
    assert not rt.is_keep_const_precision(c)
    cv = ops.convert(c, "f16")
    rt.mark_as_decompression(cv)
    assert rt.is_decompression(cv)


def test_device_rope_expression_matches_the_reference_evaluation():
    """The CUDA device's RoPE (tensor expressions in runtime/cuda_plugin.py) against the native reference evaluation, on
    host tensors: plain, partial, interleaved, transposed, position ids, and the fused-QKV forms."""
    import types as _types
    import torch
    from openvino_b200.runtime import cuda_plugin
    rng = np.random.default_rng(9)
    ctx = _types.SimpleNamespace(on_gpu=False, device="cpu", K=None)
    B, H, L, S = 2, 3, 5, 8

    def check(x, cos, sin, pos=None, **cfg):
        ps = [ops.parameter(list(a.shape), "f32" if a.dtype == np.float32 else "i64", "p%d" % i) for i, a in enumerate([x, cos, sin] + ([pos] if pos is not None else []))]
        node = ops.rope(ps[0], ps[1], ps[2], ps[3] if pos is not None else None, **cfg)
        feeds = [x, cos, sin] + ([pos] if pos is not None else [])
        want = ov.compile_model(ov.Model([node], ps, "rope"), "CPU")(feeds)[0]
        got = cuda_plugin._OPS["RoPE"](node, [torch.from_numpy(a) for a in feeds], ctx)
        assert got is not NotImplemented, cfg
        np.testing.assert_allclose(got[0].numpy(), want, rtol=1e-5, atol=1e-6, err_msg=str(cfg))

    x = rng.standard_normal((B, H, L, S)).astype(np.float32)
    cos, sin = _rope_tables(L, S, "halves")
    check(x, cos, sin, rotary_ndims=S)
    check(x, cos[..., :S // 2].copy(), sin[..., :S // 2].copy(), rotary_ndims=S)                     # half-width tables
    cos4, sin4 = _rope_tables(L, 4, "halves")
    check(x, cos4, sin4, rotary_ndims=4)                                                              # partial rotary
    ci, si = _rope_tables(L, S, "interleave")
    check(x, ci, si, rotary_ndims=S, is_interleaved=True)
    check(x.transpose(0, 2, 1, 3).copy(), cos, sin, rotary_ndims=S, input_trans0213=True)
    check(x, cos, sin, rotary_ndims=S, output_trans0213=True)
    big_c, big_s = _rope_tables(16, S, "halves")
    check(x, big_c, big_s, pos=np.array([[3, 4, 9, 1, 0], [2, 2, 15, 7, 5]], np.int64), rotary_ndims=S)
    # fused QKV forms
    qkv = rng.standard_normal((B, L, 3 * H * S)).astype(np.float32)
    tc, ts = _rope_tables(L + 3, S, "halves")
    check(qkv, tc.reshape(1, L + 3, 1, S), ts.reshape(1, L + 3, 1, S), is_qwen=True, slice_start=H * S, slice_stop=2 * H * S, head_cnt=H, head_size=S, rotary_ndims=S)
    glm = rng.standard_normal((L, B, H * S + 16)).astype(np.float32)
    ang = rng.random((L, 1, 1, 2, 1)).astype(np.float32)
    cache = np.concatenate([np.cos(ang), np.sin(ang)], -1)
    check(glm, cache, cache, is_chatglm=True, is_interleaved=True, slice_start=0, slice_stop=H * S, head_cnt=H, head_size=S, rotary_ndims=4)
