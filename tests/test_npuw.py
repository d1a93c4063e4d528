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


def _tiny_llm():
    import torch
    from openvino_b200.models import llama
    from openvino_b200.models.llm_config import TINY_LLAMA
    from openvino_b200.models.ov_builders import build_llama
    cfg = TINY_LLAMA.with_(vocab_size=96, hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=128, group_size=32, num_layers=2)
    state = llama.random_float_state(cfg, seed=3, std=0.1)
    return cfg, state, build_llama(cfg, state), llama, torch


def test_llm_pipeline_static_prefill_and_generate_variants():
    """The stateful decoder behind static sub-models: chunked prefill, KV rows copied between the prefill model and the
    generate variants, the smallest variant that holds the sequence, reset_state, prefix caching."""
    cfg, state, model, llama, torch = _tiny_llm()
    core = ov.Core()
    cm = core.compile_model(model, "NPUW", {"NPUW_LLM": "YES", "NPUW_LLM_MAX_PROMPT_LEN": 16, "NPUW_LLM_MIN_RESPONSE_LEN": 8, "NPUW_LLM_PREFILL_CHUNK_SIZE": 8,
                                            "NPUW_LLM_GENERATE_VARIANTS": "12,16", "NPUW_LLM_PREFIX_CACHING": "YES"})
    assert cm.get_property("NPUW_LLM_GENERATE_VARIANTS") == [12, 16, 24] and cm.get_property("NPUW_LLM_PREFILL_CHUNK_SIZE") == 8
    assert [i.get_any_name() for i in cm.inputs] == ["input_ids", "attention_mask", "position_ids", "beam_idx"]
    req = cm.create_infer_request()

    def feed(ids, past):
        n = len(ids)
        return {"input_ids": np.asarray(ids, np.int64)[None], "attention_mask": np.ones((1, past + n), np.int64),
                "position_ids": np.arange(past, past + n)[None], "beam_idx": np.zeros(1, np.int32)}
    prompt = [5, 9, 1, 77, 30, 2, 41, 8, 63, 12, 7]                 # 11 tokens: one full chunk and a ragged one
    seq = list(prompt)
    logits = req.infer(feed(prompt, 0))[0]
    ref = llama.reference_logits(cfg, state, torch.tensor(seq)).numpy()
    np.testing.assert_allclose(logits[0], ref, rtol=2e-3, atol=2e-4)
    for _ in range(8):                                              # rows 12 ... 19: variants 12, then 16, then the full 24
        tok = int(logits[0, -1].argmax())
        seq.append(tok)
        logits = req.infer(feed([tok], len(seq) - 1))[0]
        ref = llama.reference_logits(cfg, state, torch.tensor(seq)).numpy()
        np.testing.assert_allclose(logits[0, -1], ref[-1], rtol=2e-3, atol=2e-4)
    names = [t[0] for t in req.npuw_trace]
    assert names[:2] == ["prefill", "prefill"] and names[2] == "generate/12" and "generate/16" in names and names[-1] == "generate/24"
    kv = req.query_state()
    assert len(kv) == 2 * cfg.num_layers and list(kv[0].state.shape) == [1, 2, len(seq), 16]

    # a new prompt that repeats the first chunk of the conversation: that chunk is served from the cache
    before = len(req.npuw_trace)
    again = prompt[:8] + [3, 4, 6]
    logits = req.infer(feed(again, 0))[0]
    assert [t for t in req.npuw_trace[before:]] == [("prefill", 3)]
    ref = llama.reference_logits(cfg, state, torch.tensor(again)).numpy()
    np.testing.assert_allclose(logits[0, 8:], ref[8:], rtol=2e-3, atol=2e-4)

    # reset_state starts over: the same prompt now runs both chunks
    req.reset_state()
    before = len(req.npuw_trace)
    logits = req.infer(feed(again, 0))[0]
    assert [t for t in req.npuw_trace[before:]] == [("prefill", 8), ("prefill", 3)]
    np.testing.assert_allclose(logits[0], ref, rtol=2e-3, atol=2e-4)
    with pytest.raises(RuntimeError, match="longer than"):
        req.infer(feed(list(range(1, 19)), 0))
    with pytest.raises(RuntimeError, match="stateful decoder"):
        x = ops.parameter([1, 4], "f32", "x")
        core.compile_model(ov.Model([ops.relu(x)], [x], "plain"), "NPUW", {"NPUW_LLM": "YES"})
