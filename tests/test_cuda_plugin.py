"""The "CUDA" device through the public API: compile, infer, precision hints, states, remote tensors, AUTO/HETERO."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import Model, Tensor, Type
from openvino_b200 import opset as ops
from openvino_b200 import properties as props
from openvino_b200.models import llama
from openvino_b200.models.llm_config import TINY_LLAMA
from openvino_b200.models.ov_builders import build_llama
from openvino_b200.models.torch_zoo import ResNet18, bert_tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def core():
    return ov.Core()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-12)


def test_device_is_listed_and_describes_itself(core):
    assert any(d.startswith("CUDA") for d in core.available_devices)
    assert "B200" in core.get_property("CUDA", props.device.full_name) or core.get_property("CUDA", props.device.full_name)
    assert core.get_property("CUDA", props.device.architecture).startswith("sm_")
    assert "INT4" in core.get_property("CUDA", props.device.capabilities)


def test_resnet_fp32_and_fp16(core):
    torch.manual_seed(0)
    net = ResNet18(num_classes=10, width=16).eval()
    x = torch.randn(4, 3, 64, 64)
    with torch.no_grad():
        want = net(x).numpy()
    m = ov.convert_model(net, example_input=(x,))
    out = core.compile_model(m, "CUDA")(x.numpy())[0]
    assert rel(out, want) < 1e-3
    out16 = core.compile_model(m, "CUDA", {props.hint.inference_precision: "f16"})(x.numpy())[0]
    assert out16.dtype == np.float32 and rel(out16, want) < 3e-2
    assert core.compile_model(m, "GPU").get_property(props.execution_devices) == ["CUDA.0"]


def test_bert_fp16_uses_own_kernels(core):
    torch.manual_seed(0)
    net = bert_tiny().eval()
    ids = torch.randint(0, 100, (2, 16))
    mask = torch.ones(2, 16, dtype=torch.int64)
    typ = torch.zeros(2, 16, dtype=torch.int64)
    with torch.no_grad():
        want = net(ids, mask, typ).numpy()
    m = ov.convert_model(net, example_input=(ids, mask, typ))
    cm = core.compile_model(m, "CUDA", {props.hint.inference_precision: "f16", props.enable_profiling: True})
    req = cm.create_infer_request()
    out = req.infer([ids.numpy(), mask.numpy(), typ.numpy()])[0]
    assert rel(out, want) < 3e-2
    prof = req.get_profiling_info()
    assert any(p.node_type == "FullyConnected" for p in prof) and all(p.exec_type == "cuda" for p in prof)


def test_static_graphs_replay_a_cuda_graph(core):
    """The third inference of a request with unchanged shapes replays a captured CUDA graph; results equal the eager walk,
    new input values are picked up, and another batch size gets a graph of its own."""
    torch.manual_seed(1)
    net = ResNet18(num_classes=10, width=16).eval()
    x1, x2 = torch.randn(2, 3, 64, 64), torch.randn(2, 3, 64, 64)
    with torch.no_grad():
        want1, want2 = net(x1).numpy(), net(x2).numpy()
    m = ov.convert_model(net, example_input=(x1,), input=[[-1, 3, 64, 64]])
    req = core.compile_model(m, "CUDA").create_infer_request()
    eager = req.infer([x1.numpy()])[0].copy()                          # first call: eager warm-up
    captured = req.infer([x1.numpy()])[0].copy()                       # second: capture + replay
    replayed = req.infer([x2.numpy()])[0].copy()                       # third: replay with new data
    assert rel(eager, want1) < 1e-3 and np.array_equal(eager, captured) and rel(replayed, want2) < 1e-3
    entries = list(req._cuda_graphs.values())
    assert len(entries) == 1 and isinstance(entries[0], tuple), entries
    x3 = torch.randn(5, 3, 64, 64)
    for _ in range(3):
        out3 = req.infer([x3.numpy()])[0]
    with torch.no_grad():
        assert rel(out3, net(x3).numpy()) < 1e-3
    assert sum(isinstance(e, tuple) for e in req._cuda_graphs.values()) == 2
    # switched off by the property
    req_off = core.compile_model(m, "CUDA", {props.cuda.use_cuda_graphs: False}).create_infer_request()
    for _ in range(3):
        out_off = req_off.infer([x1.numpy()])[0]
    assert not req_off._cuda_graphs and rel(out_off, want1) < 1e-3


def test_stateful_llm_int4_on_device(core):
    cfg = TINY_LLAMA.with_(vocab_size=256, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=128, ffn_size=512, group_size=128)
    state = llama.random_float_state(cfg, seed=2, std=0.05)
    m = build_llama(cfg, state, compress="int4")
    cpu = core.compile_model(m, "CPU").create_infer_request()
    gpu = core.compile_model(m, "CUDA", {props.hint.inference_precision: "bf16"}).create_infer_request()
    feeds = [{"input_ids": np.array([[3, 9, 27, 5, 100, 7]], np.int64), "attention_mask": np.ones((1, 6), np.int64),
              "position_ids": np.arange(6)[None], "beam_idx": np.zeros(1, np.int32)},
             {"input_ids": np.array([[42]], np.int64), "attention_mask": np.ones((1, 7), np.int64),
              "position_ids": np.array([[6]], np.int64), "beam_idx": np.zeros(1, np.int32)}]
    for feed in feeds:
        want, got = cpu.infer(feed)[0], gpu.infer(feed)[0]
        assert rel(got, want) < 5e-2
        assert (got[0, -1].argmax() == want[0, -1].argmax()) or rel(got, want) < 2e-2
    st = gpu.query_state()
    assert len(st) == 2 * cfg.num_layers and st[0].state.shape[2] == 7
    gpu.reset_state()
    assert rel(gpu.infer(feeds[0])[0], cpu.infer(feeds[0])[0]) < 1.0    # runs again from an empty state


def test_remote_tensors_and_async(core):
    x = ops.parameter([4, 8], "f32", "x")
    m = Model([ops.relu(ops.add(x, np.float32(-0.5)))], [x], "r")
    cm = core.compile_model(m, "CUDA", {props.num_streams: 2})
    ctx = core.get_default_context("CUDA")
    rin = ctx.create_tensor(Type.f32, [4, 8])
    rout = ctx.create_tensor(Type.f32, [4, 8])
    rin.torch().copy_(torch.arange(32, dtype=torch.float32).reshape(4, 8) / 16)
    req = cm.create_infer_request()
    req.set_input_tensor(rin)
    req.set_output_tensor(rout)
    req.infer()
    assert req.get_output_tensor() is rout and rout.is_remote
    np.testing.assert_allclose(rout.data, np.maximum(np.arange(32).reshape(4, 8) / 16 - 0.5, 0), rtol=1e-6)
    q = ov.AsyncInferQueue(cm, 4)
    got = {}
    q.set_callback(lambda r, i: got.__setitem__(i, r.results[0].copy()))
    xs = [np.full((4, 8), float(i), np.float32) for i in range(8)]
    for i, a in enumerate(xs):
        q.start_async({"x": a}, userdata=i)
    q.wait_all()
    for i, a in enumerate(xs):
        np.testing.assert_allclose(got[i], np.maximum(a - 0.5, 0))
    host = ctx.create_host_tensor(Type.f32, [4, 8])
    assert host.data.shape == (4, 8)


def test_auto_prefers_cuda_and_hetero_splits(core):
    x = ops.parameter([2, 4], "f32", "x")
    y = ops.selu(ops.relu(x), np.float32(1.5), np.float32(1.0), name="selu")      # Selu has no device implementation
    m = Model([ops.add(y, np.float32(1), name="tail")], [x], "h")
    assert core.compile_model(m, "AUTO").get_property(props.execution_devices)[0].startswith("CUDA")
    q = core.query_model(m, "CUDA")
    assert "selu" not in q and "tail" in q
    cm = core.compile_model(m, "HETERO:CUDA,CPU")
    assert [s.device for s in cm.subs] == ["CUDA", "CPU", "CUDA"]
    a = np.array([[-1, 0.5, 2, -3], [1, 1, -1, 0]], np.float32)
    r = np.maximum(a, 0)
    np.testing.assert_allclose(cm(a)[0], np.where(r > 0, r, 1.5 * (np.exp(r) - 1)) + 1, rtol=1e-5)
    # the device alone still runs the model: unsupported operations fall back to the host
    np.testing.assert_allclose(core.compile_model(m, "CUDA")(a)[0], cm(a)[0], rtol=1e-5)


def test_llm_pipeline_from_ir_directory(tmp_path):
    """IR on disk -> graph analysis -> serving program: tokens must follow the fp32 reference of the same weights."""
    from openvino_b200.genai import ByteTokenizer, GenerationConfig, LLMPipeline
    cfg = TINY_LLAMA.with_(vocab_size=320, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=128, ffn_size=512, group_size=128)
    state = llama.random_float_state(cfg, seed=7, std=0.05)
    m = build_llama(cfg, state, compress="int4")
    ov.save_model(m, str(tmp_path / "openvino_model.xml"))
    pipe = LLMPipeline(str(tmp_path), "CUDA", tokenizer=ByteTokenizer(), max_num_seqs=4, max_num_batched_tokens=256, max_model_len=128)
    got_cfg = pipe.config
    assert (got_cfg.num_layers, got_cfg.num_heads, got_cfg.num_kv_heads, got_cfg.head_dim, got_cfg.ffn_size, got_cfg.weight_format) == \
           (cfg.num_layers, 4, 2, 128, 512, "int4")
    assert abs(got_cfg.rope_theta - cfg.rope_theta) / cfg.rope_theta < 1e-3
    prompts = [[5, 17, 200, 31, 8], [300, 2, 2, 9]]
    outs = pipe.generate(prompts, GenerationConfig(max_new_tokens=5))
    eff = llama.effective_state(cfg, state)
    for p, o in zip(prompts, outs):
        seq = p + o
        logits = llama.reference_logits(cfg, eff, torch.tensor(seq[:-1]))
        for i, tok in enumerate(o):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 0.05 * row.abs().max()
    text = pipe.generate("hi", max_new_tokens=3)
    assert isinstance(text, str)


def test_mixture_of_experts_ir_runs_on_the_serving_program(tmp_path):
    """A decoder with MOE layers, saved as IR: recognised by structure, experts run through the grouped GEMM; the
    KV_CACHE_PRECISION property selects the u8 cache of the serving program."""
    from openvino_b200.genai import ByteTokenizer, GenerationConfig, LLMPipeline
    from openvino_b200.models.llm_config import TINY_MOE
    cfg = TINY_MOE.with_(vocab_size=320)
    state = llama.random_float_state(cfg, seed=11, std=0.05)
    ov.save_model(build_llama(cfg, state), str(tmp_path / "openvino_model.xml"), compress_to_fp16=False)
    eff = llama.effective_state(cfg, state)
    prompts = [[5, 17, 200, 31, 8, 9, 1, 44, 90], [300, 2, 2, 9]]
    for extra in ({}, {props.hint.kv_cache_precision: "u8"}):
        pipe = LLMPipeline(str(tmp_path), "CUDA", tokenizer=ByteTokenizer(), max_num_seqs=4, max_num_batched_tokens=256, max_model_len=128, **extra)
        assert (pipe.config.num_experts, pipe.config.experts_top_k) == (cfg.num_experts, cfg.experts_top_k)
        outs = pipe.generate(prompts, GenerationConfig(max_new_tokens=5))
        for p, o in zip(prompts, outs):
            seq = p + o
            logits = llama.reference_logits(cfg, eff, torch.tensor(seq[:-1]))
            for i, tok in enumerate(o):
                row = logits[len(p) - 1 + i]
                assert row[tok] >= row.max() - 0.05 * row.abs().max()
