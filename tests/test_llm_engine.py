"""End-to-end numerics of the CUDA LLM program against the PyTorch fp32 reference model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["bf16", "int4", "moe", "moe-gather", "bf16-u8kv"])
def test_tiny_llama_generate_matches_reference(fmt, monkeypatch):
    from openvino_b200.genai.pipeline import ContinuousBatchingPipeline, GenerationConfig
    from openvino_b200.genai.scheduler import SchedulerConfig
    from openvino_b200.models import llama
    from openvino_b200.models.llm_config import TINY_LLAMA, TINY_MOE
    from openvino_b200.ops import cuda as K
    from openvino_b200.runtime.cuda_llm import CudaLlmExecutor, LlmWeights, StepShape

    if fmt == "moe-gather":
        # prefill batches take the path that runs every expert on its own (gathered) tokens only
        from openvino_b200.runtime import cuda_llm
        monkeypatch.setattr(cuda_llm, "MOE_GATHER_MIN_TOKENS", 8)
    cfg = TINY_MOE if fmt.startswith("moe") else TINY_LLAMA.with_(weight_format=fmt.split("-")[0])
    state = llama.random_float_state(cfg, seed=3, std=0.05)
    eff = {k: v.cuda() for k, v in llama.effective_state(cfg, state).items()}
    w = LlmWeights.from_float(cfg, state, "cuda")
    # "-u8kv": KV_CACHE_PRECISION = u8 (rows quantised per token and head by the cache-write kernel)
    ex = CudaLlmExecutor(cfg, w, num_kv_blocks=64, max_batch_tokens=256, max_seqs=4, kv_cache_precision="u8" if fmt.endswith("u8kv") else "bf16")
    sc = SchedulerConfig(max_num_batched_tokens=48, max_num_seqs=4, num_kv_blocks=64)   # forces chunked prefill
    pipe = ContinuousBatchingPipeline(ex, sc)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 37, 70, 16)]
    res = pipe.generate(prompts, GenerationConfig(max_new_tokens=6), lookahead=1 if fmt == "int4" else 0)
    K.check_status("llm")
    assert pipe.metrics.prefill_steps >= 3 and pipe.metrics.decode_steps >= 5
    for p, r in zip(prompts, res):
        # teacher-forced check: at every generated position the engine's token must be the reference
        # argmax, or a near-tie of it (bf16 activations vs fp32 reference)
        seq = p + r.tokens
        logits = llama.reference_logits(cfg, eff, torch.tensor(seq[:-1], device="cuda"))
        for i, tok in enumerate(r.tokens):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 0.05 * row.abs().max(), (i, tok, int(row.argmax()))


def test_logits_close_to_reference():
    from openvino_b200.models import llama
    from openvino_b200.models.llm_config import TINY_LLAMA
    from openvino_b200.runtime.cuda_llm import CudaLlmExecutor, LlmWeights, StepShape
    import numpy as np

    cfg = TINY_LLAMA.with_(weight_format="int4")
    state = llama.random_float_state(cfg, seed=5, std=0.05)
    eff = {k: v.cuda() for k, v in llama.effective_state(cfg, state).items()}
    ex = CudaLlmExecutor(cfg, LlmWeights.from_float(cfg, state, "cuda"), num_kv_blocks=16, max_batch_tokens=128, max_seqs=2,
                         use_cuda_graphs=False)
    ids = torch.randint(0, cfg.vocab_size, (50,))
    sb = ex.prefill
    v = {n: sb.view(n, host=0).numpy() for n in sb.offsets}
    v["ids"][:50] = ids.numpy()
    v["positions"][:50] = np.arange(50)
    v["slot_map"][:50] = np.arange(50) + 16 * 3          # blocks 3,4,5,6
    v["tok_src"][:50] = -1
    v["tok_dst"][0] = -1
    v["logit_idx"][0] = 49
    v["past_lens"][0] = 0
    v["subsequence_begins"][:2] = [0, 50]
    v["block_indices_begins"][:2] = [0, 4]
    v["block_indices"][:4] = [3, 4, 5, 6]
    ex.upload(sb)
    ex.run(sb, StepShape(50, 1, 50, 50))
    torch.cuda.synchronize()
    ref = llama.reference_logits(cfg, eff, ids.cuda())[-1]
    got = sb.logits[0].float()
    rel = ((got - ref).norm() / ref.norm()).item()
    assert rel < 3e-2, rel


@pytest.mark.parametrize("native", [True, False])
def test_python_and_native_scheduler_generate_the_same_tokens(native):
    from openvino_b200.genai.pipeline import ContinuousBatchingPipeline, GenerationConfig
    from openvino_b200.genai.scheduler import SchedulerConfig
    from openvino_b200.models import llama
    from openvino_b200.models.llm_config import TINY_LLAMA
    from openvino_b200.ops import cuda as K
    from openvino_b200.runtime.cuda_llm import CudaLlmExecutor, LlmWeights

    cfg = TINY_LLAMA
    state = llama.random_float_state(cfg, seed=9, std=0.05)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 9, 25)]
    out = []
    for use_native in (native, not native):
        ex = CudaLlmExecutor(cfg, LlmWeights.from_float(cfg, state, "cuda"), num_kv_blocks=64, max_batch_tokens=128, max_seqs=4)
        sc = SchedulerConfig(max_num_batched_tokens=32, max_num_seqs=4, num_kv_blocks=64, use_native=use_native)
        out.append([r.tokens for r in ContinuousBatchingPipeline(ex, sc).generate(prompts, GenerationConfig(max_new_tokens=6), lookahead=1)])
        K.check_status("generate")
    assert out[0] == out[1]


def test_prefix_caching_reuses_kv_blocks_and_keeps_the_tokens():
    from openvino_b200.genai.pipeline import ContinuousBatchingPipeline, GenerationConfig
    from openvino_b200.genai.scheduler import SchedulerConfig
    from openvino_b200.models import llama
    from openvino_b200.models.llm_config import TINY_LLAMA
    from openvino_b200.ops import cuda as K
    from openvino_b200.runtime.cuda_llm import CudaLlmExecutor, LlmWeights

    cfg = TINY_LLAMA
    state = llama.random_float_state(cfg, seed=11, std=0.05)
    g = torch.Generator().manual_seed(4)
    system = torch.randint(0, cfg.vocab_size, (70,), generator=g).tolist()          # shared "system prompt": four full blocks
    prompts = [system + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 11, 3)]
    gen = GenerationConfig(max_new_tokens=5)
    results = {}
    for caching in (False, True):
        ex = CudaLlmExecutor(cfg, LlmWeights.from_float(cfg, state, "cuda"), num_kv_blocks=64, max_batch_tokens=128, max_seqs=4)
        sc = SchedulerConfig(max_num_batched_tokens=128, max_num_seqs=4, num_kv_blocks=64, enable_prefix_caching=caching)
        pipe = ContinuousBatchingPipeline(ex, sc)
        first = pipe.generate(prompts[:1], gen, lookahead=0)          # fills the cache
        rest = pipe.generate(prompts[1:], gen, lookahead=0)           # later requests with the same prefix
        K.check_status("prefix caching")
        results[caching] = ([r.tokens for r in first + rest], pipe.metrics.scheduled_tokens,
                            getattr(pipe.scheduler, "prefix_hit_tokens", 0))
    assert results[True][0] == results[False][0]
    assert results[True][2] == 2 * 64                                  # two later requests x four cached blocks of 16 tokens
    assert results[True][1] == results[False][1] - 2 * 64
