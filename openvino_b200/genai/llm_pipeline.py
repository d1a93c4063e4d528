"""``LLMPipeline``: text generation from a model object or an IR directory, the way ``openvino_genai.LLMPipeline`` is used.

    pipe = LLMPipeline("model_dir_or_xml", "CUDA")            # or LLMPipeline(ov_model, "CUDA")
    out = pipe.generate([[1, 15043, 29892]], max_new_tokens=32)

The model graph is analysed and lifted into the device's serving program (paged KV cache, continuous batching, CUDA
graphs; see runtime/llm_import.py); under tensor parallelism every rank constructs the pipeline with its communicator.
Prompts are token-id lists; a tokenizer object with ``encode`` / ``decode`` may be supplied for text in, text out (a
byte-level one ships here for tests; real vocabularies come from the model's own tokenizer files).
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Union

import torch

from .._graph import Model
from ..frontend import read_model
from .pipeline import ContinuousBatchingPipeline, GenerationConfig, GenerationResult
from .scheduler import SchedulerConfig


class ByteTokenizer:
    """UTF-8 bytes as token ids (offset by 3 for pad / bos / eos)."""

    pad_token_id, bos_token_id, eos_token_id = 0, 1, 2

    def encode(self, text: str) -> List[int]:
        return [self.bos_token_id] + [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i - 3 for i in ids if 3 <= i < 259).decode("utf-8", errors="replace")


class LLMPipeline:
    def __init__(self, model: Union[str, Model], device: str = "CUDA", tokenizer=None, comm=None, tp_rank: int = 0, tp_size: int = 1,
                 max_num_seqs: int = 64, max_num_batched_tokens: int = 8192, max_model_len: int = 4096, block_size: int = 16,
                 kv_cache_blocks: int = 0, **properties):
        """``properties``: further device properties for ``compile_model`` (e.g. ``KV_CACHE_PRECISION="u8"``)."""
        if device.split(".")[0] not in ("CUDA", "GPU"):
            raise RuntimeError("LLMPipeline runs on the CUDA device; use compile_model for '%s'" % device)
        if not isinstance(model, Model):
            path = str(model)
            if os.path.isdir(path):
                path = os.path.join(path, "openvino_model.xml")
            model = read_model(path)
        from .. import passes, properties as props
        from ..runtime.core import Core
        # the stateful form that exporters write becomes the PagedAttention form the serving program is compiled from
        if not any(n.get_type_name() == "PagedAttentionExtension" for n in model.get_ops()):
            model = model.clone()
            mgr = passes.Manager()
            mgr.register_pass(passes.SDPAToPagedAttention())
            mgr.run_passes(model)
        dev_index = int(device.split(".")[1]) if "." in device else (torch.cuda.current_device() if torch.cuda.is_available() else 0)
        config = {props.cuda.serving_program: True}
        config.update(properties)
        if tp_size > 1:
            config[props.hint.model_distribution_policy] = "TENSOR_PARALLEL"
        self.compiled_model = Core().compile_model(model, "CUDA.%d" % dev_index, config)
        if tp_size > 1 and (self.compiled_model.tp_rank, self.compiled_model.tp_size) != (tp_rank, tp_size):
            raise RuntimeError("tensor-parallel rank / size (%d / %d) differ from the process group's (%d / %d)"
                               % (tp_rank, tp_size, self.compiled_model.tp_rank, self.compiled_model.tp_size))
        self.config = self.compiled_model.llm_config
        self.executor, self.scheduler_config = self.compiled_model.create_llm_executor(
            max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens, max_model_len=max_model_len, block_size=block_size,
            kv_cache_blocks=kv_cache_blocks, comm=comm)
        self.pipeline = ContinuousBatchingPipeline(self.executor, self.scheduler_config)
        self.tokenizer = tokenizer

    def get_tokenizer(self):
        return self.tokenizer

    def get_generation_config(self) -> GenerationConfig:
        return GenerationConfig()

    def generate(self, inputs, generation_config: Optional[GenerationConfig] = None, **kwargs):
        """inputs: a prompt or a list of prompts; a prompt is a token-id list or (with a tokenizer) a string.
        Returns token-id lists (or strings when the prompts were strings)."""
        cfg = generation_config or GenerationConfig()
        for k, v in kwargs.items():
            if not hasattr(cfg, k):
                raise TypeError("unknown generation parameter %s" % k)
            setattr(cfg, k, v)
        single = isinstance(inputs, str) or (isinstance(inputs, (list, tuple)) and inputs and isinstance(inputs[0], int))
        prompts = [inputs] if single else list(inputs)
        text = any(isinstance(p, str) for p in prompts)
        if text and self.tokenizer is None:
            raise RuntimeError("string prompts need a tokenizer")
        ids = [self.tokenizer.encode(p) if isinstance(p, str) else list(p) for p in prompts]
        results: List[GenerationResult] = self.pipeline.generate(ids, cfg)
        outs = [self.tokenizer.decode(r.tokens) if text else r.tokens for r in results]
        return outs[0] if single else outs
