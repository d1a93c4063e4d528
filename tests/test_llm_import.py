"""Structural recognition of decoder-only LLM graphs (runtime/llm_import.py): node names play no part."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import passes
from openvino_b200.models import llama
from openvino_b200.models.llm_config import TINY_LLAMA, TINY_MOE
from openvino_b200.models.ov_builders import build_llama, build_llama_random_int4
from openvino_b200.runtime import llm_import


def _cfg(layers=2):
    return TINY_LLAMA.with_(vocab_size=320, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=128, ffn_size=512, group_size=128, num_layers=layers)


def _to_paged(m):
    mgr = passes.Manager()
    mgr.register_pass(passes.SDPAToPagedAttention())
    mgr.run_passes(m)
    return m


@pytest.mark.parametrize("compress", [None, "int4", "int8"])
@pytest.mark.parametrize("paged", [False, True])
def test_renamed_graph_is_still_recognised(compress, paged, tmp_path):
    cfg = _cfg()
    state = llama.random_float_state(cfg, seed=7, std=0.05)
    m = build_llama(cfg, state, compress=compress)
    if paged:
        _to_paged(m)
    for i, n in enumerate(m.get_ops()):
        if n.get_type_name() not in ("Parameter", "Result"):
            n.set_friendly_name("op_%d" % i)                 # nothing is called q_proj / layers.N / lm_head any more
    ov.save_model(m, str(tmp_path / "m.xml"), compress_to_fp16=False)
    back = ov.Core().read_model(str(tmp_path / "m.xml"))
    got, parts = llm_import.analyze(back)
    assert (got.num_layers, got.num_heads, got.num_kv_heads, got.head_dim, got.ffn_size, got.hidden_size, got.vocab_size) == (2, 4, 2, 128, 512, 256, 320)
    assert got.weight_format == {None: "bf16", "int4": "int4", "int8": "int8"}[compress]
    assert abs(got.rope_theta - cfg.rope_theta) / cfg.rope_theta < 1e-3 and abs(got.rms_eps - cfg.rms_eps) < 1e-9
    # the right constants ended up in the right roles
    if compress is None:
        for l in range(2):
            for key in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
                assert torch.allclose(parts["lin"][(l, key)].w, state["layers.%d.%s" % (l, key)].float(), atol=1e-6), (l, key)
            assert torch.allclose(parts["norms"][(l, "input_layernorm")], state["layers.%d.input_layernorm" % l].float())
            assert torch.allclose(parts["norms"][(l, "post_attention_layernorm")], state["layers.%d.post_attention_layernorm" % l].float())
        assert torch.allclose(parts["lm_head"].w, state["lm_head"].float(), atol=1e-6)
        assert torch.allclose(parts["final_norm"], state["norm"].float()) and torch.allclose(parts["embed"], state["embed_tokens"].float(), atol=1e-6)
    else:
        assert parts["lin"][(0, "q_proj")].compressed and parts["lin"][(1, "down_proj")].G == 512 // 128


@pytest.mark.parametrize("paged", [False, True])
def test_mixture_of_experts_decoder_is_recognised_by_structure(paged, tmp_path):
    """Router projection -> softmax -> top-k -> MOE: the experts, their number and the top-k come from the graph."""
    cfg = TINY_MOE.with_(vocab_size=320)
    state = llama.random_float_state(cfg, seed=9, std=0.05)
    m = build_llama(cfg, state)
    assert sum(1 for n in m.get_ops() if n.get_type_name() == "MOE") == cfg.num_layers
    # the graph computes what the reference model computes
    ids = np.array([[5, 9, 200, 17, 3]], dtype=np.int64)
    feed = {"input_ids": ids, "attention_mask": np.ones_like(ids), "position_ids": np.arange(5, dtype=np.int64)[None], "beam_idx": np.zeros(1, np.int32)}
    logits = ov.Core().compile_model(m, "CPU")(feed)[0]
    eff = llama.effective_state(cfg, state)
    want = llama.reference_logits(cfg, eff, torch.tensor(ids[0])).numpy()
    assert np.abs(logits[0] - want).max() < 1e-2 * np.abs(want).max()      # the reference model rounds its weights to bf16
    if paged:
        _to_paged(m)
    for i, n in enumerate(m.get_ops()):
        if n.get_type_name() not in ("Parameter", "Result"):
            n.set_friendly_name("op_%d" % i)
    ov.save_model(m, str(tmp_path / "moe.xml"), compress_to_fp16=False)
    got, parts = llm_import.analyze(ov.Core().read_model(str(tmp_path / "moe.xml")))
    assert (got.num_experts, got.experts_top_k, got.ffn_size, got.num_layers) == (cfg.num_experts, cfg.experts_top_k, cfg.ffn_size, cfg.num_layers)
    for l in range(cfg.num_layers):
        assert torch.allclose(parts["lin"][(l, "router")].w, state["layers.%d.router" % l].float(), atol=1e-6)
        for e in range(cfg.num_experts):
            for key, role in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
                assert torch.allclose(parts["experts"][l][role][e], state["layers.%d.experts.%d.%s" % (l, e, key)].float(), atol=1e-6)


def test_graphs_that_are_not_decoders_are_refused():
    from openvino_b200 import opset as ops
    x = ops.parameter([1, 8], "f32", "x")
    m = ov.Model([ops.result(ops.relu(x))], [x], "m")
    with pytest.raises(llm_import.NotAnLlm):
        llm_import.analyze(m)


def test_random_int4_builder_writes_compressed_constants_directly():
    cfg = _cfg(layers=1)
    m = _to_paged(build_llama_random_int4(cfg, seed=3))
    got, parts = llm_import.analyze(m)
    assert got.weight_format == "int4" and got.num_layers == 1 and got.group_size == 128
    q = parts["lin"][(0, "q_proj")]
    assert q.q.shape == (512, 256 // 2) and q.q.dtype == torch.uint8 and int(q.zp.min()) == 8 and int(q.zp.max()) == 8
    w = (torch.stack([q.q & 0xF, q.q >> 4], -1).reshape(512, 256).float() - 8.0) * q.scales.repeat_interleave(128, 1)
    assert 0.012 < float(w.std()) < 0.03                    # about the 0.02 that float initialisation would give
    emb = parts["embed"]
    assert emb.shape == (320, 256) and 0.015 < float(emb.abs().min()) and float(emb.abs().max()) < 0.032


def test_sliding_window_reaches_the_serving_configuration():
    """A windowed mask in the SDPA form becomes the sliding_window input of the paged form and then a field of the
    configuration that the serving program is built from."""
    cfg = _cfg().with_(sliding_window=5)
    m = _to_paged(build_llama(cfg, llama.random_float_state(cfg, seed=2, std=0.05)))
    got, _ = llm_import.analyze(m)
    assert got.sliding_window == 5
    plain, _ = llm_import.analyze(_to_paged(build_llama(_cfg(), llama.random_float_state(_cfg(), seed=2, std=0.05))))
    assert plain.sliding_window == 0
