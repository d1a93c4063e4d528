"""NPUW LLM pipeline: a stateful decoder (``input_ids`` / ``attention_mask`` / ``position_ids`` / ``beam_idx`` with the KV
cache in variables) served by STATIC-shape sub-models, the way devices without dynamic shapes serve LLMs.

``NpuwLlmCompiledModel`` keeps the caller's stateful interface and, behind it,

* turns the model stateless (KV cache as explicit ``past_key_values.*`` inputs and ``present.*`` outputs) and cuts every
  ``present`` output down to the rows of the NEW tokens, so that a step returns one KV row per token and not the cache;
* compiles one *prefill* model of ``NPUW_LLM_PREFILL_CHUNK_SIZE`` tokens (the whole ``NPUW_LLM_MAX_PROMPT_LEN`` when the
  chunk size is 0) over a past of ``max prompt - chunk`` rows, and one *generate* model of one token per KV size in
  ``NPUW_LLM_GENERATE_VARIANTS`` (by default powers of two from 256 rows up to ``max prompt + NPUW_LLM_MIN_RESPONSE_LEN``):
  a step runs the smallest variant that still holds the sequence, so short conversations never pay for the longest;
* holds the KV cache on the host, left-aligned, ONE buffer per layer sized for the largest variant; every sub-model gets
  a view of its own size, and padded rows are switched off through the attention mask;
* prompts longer than one chunk run chunk by chunk (chunked prefill); a prompt that starts with the tokens of the
  previous conversation of the request continues from the rows already in the cache (prefix caching) when
  ``NPUW_LLM_PREFIX_CACHING`` is on;
* shares constants between all sub-models through the device's ``WeightsBank``.

Reference: src/plugins/intel_npu/src/plugin/npuw/llm_compiled_model.cpp (reshape to static prefill / generate models, KV
size variants), llm_infer_request.cpp (prefill / generate dispatch, KV copy between the models, chunked prefill),
llm_prefix_caching.cpp.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

from .. import _offline_transformations as offline
from .. import opset as ops
from .. import properties as props
from .._graph import Model
from .._tensor import Tensor
from .._types import PartialShape
from .core import CompiledModel, VariableState


def is_llm(model: Model) -> bool:
    names = {p.get_friendly_name() for p in model.get_parameters()}
    return {"input_ids", "attention_mask", "position_ids"} <= names and bool(model.get_sinks())


def _cut_present_to_new_rows(model: Model) -> None:
    """present.* [B, H, past + L, D] -> its last L rows, L read from input_ids at run time."""
    ids = next(p for p in model.get_parameters() if p.get_friendly_name() == "input_ids")
    i64 = lambda v: ops.constant(np.array(v, dtype=np.int64))
    length = ops.gather(ops.shape_of(ids), i64([1]), i64(0))
    start = ops.negative(length)
    for r in model.get_results():
        if not r.get_friendly_name().startswith("present."):
            continue
        src = r.input_value(0)
        cut = ops.slice(src, start, i64([np.iinfo(np.int64).max]), i64([1]), i64([2]))
        r.input(0).replace_source_output(cut.output(0))


def _static_variant(stateless: Model, tokens: int, past: int) -> Model:
    m = stateless.clone()
    shapes = {}
    for p in m.get_parameters():
        n = p.get_friendly_name()
        if n in ("input_ids", "position_ids"):
            shapes[n] = PartialShape([1, tokens])
        elif n == "attention_mask":
            shapes[n] = PartialShape([1, past + tokens])
        elif n == "beam_idx":
            shapes[n] = PartialShape([1])
        elif n.startswith("past_key_values."):
            ps = p.get_output_partial_shape(0)
            shapes[n] = PartialShape([1, ps[1].get_length(), past, ps[3].get_length()])
    m.reshape(shapes)
    return m


class _Conversation:
    """KV cache and token history of one request."""

    def __init__(self, layers: Dict[str, tuple], capacity: int, dtype):
        self.kv = {name: np.zeros((1, h, capacity, d), dtype) for name, (h, d) in layers.items()}
        self.rows = 0
        self.tokens: List[int] = []

    def reset(self):
        self.rows = 0
        self.tokens = []


class NpuwLlmCompiledModel(CompiledModel):
    def __init__(self, plugin, model: Model, config: dict, device: str, inner_config: dict, bank=None):
        from .npuw import dedupe_constants
        stateless = model.clone()
        offline.stateful_to_stateless_transformation(stateless)
        _cut_present_to_new_rows(stateless)
        super().__init__(plugin, model, config, stateless)
        self.max_prompt = int(config.get("NPUW_LLM_MAX_PROMPT_LEN", 1024))
        self.min_response = int(config.get("NPUW_LLM_MIN_RESPONSE_LEN", 128))
        chunk = int(config.get("NPUW_LLM_PREFILL_CHUNK_SIZE", 0))
        self.chunk = chunk if 0 < chunk < self.max_prompt else self.max_prompt
        if self.max_prompt % self.chunk:
            raise RuntimeError("[NPUW] NPUW_LLM_MAX_PROMPT_LEN (%d) must be a multiple of NPUW_LLM_PREFILL_CHUNK_SIZE (%d)" % (self.max_prompt, self.chunk))
        self.capacity = self.max_prompt + self.min_response
        given = config.get("NPUW_LLM_GENERATE_VARIANTS")
        if given:
            sizes = sorted({int(s) for s in (given.split(",") if isinstance(given, str) else given)})
        else:
            sizes, s = [], 256
            while s < self.capacity:
                sizes.append(s)
                s *= 2
        self.variants = [s for s in sizes if s < self.capacity] + [self.capacity]
        self.prefix_caching = str(config.get("NPUW_LLM_PREFIX_CACHING", "NO")).upper() in ("YES", "TRUE", "1")
        self.layers: Dict[str, tuple] = {}
        self.kv_dtype = np.float32
        for p in stateless.get_parameters():
            n = p.get_friendly_name()
            if n.startswith("past_key_values."):
                ps = p.get_output_partial_shape(0)
                self.layers[n] = (ps[1].get_length(), ps[3].get_length())
                self.kv_dtype = p.get_output_element_type(0).to_dtype()
        self.present_of = {n: "present." + n[len("past_key_values."):] for n in self.layers}
        core = plugin.core
        self.constants_shared = 0

        def build(tokens, past):
            m = _static_variant(stateless, tokens, past)
            if bank is not None:
                self.constants_shared += dedupe_constants(m, bank)
            return core.compile_model(m, device, inner_config)
        self.prefill = build(self.chunk, self.max_prompt - self.chunk)
        self.generate = {k: build(1, k - 1) for k in self.variants}
        self.out_names = {}
        for cm in [self.prefill] + list(self.generate.values()):
            self.out_names[id(cm)] = [o.get_node().get_friendly_name() for o in cm.outputs]

    # ---- properties
    def get_property(self, name):
        n = str(name)
        if n == props.execution_devices:
            return ["NPUW"] + list(self.prefill.get_property(props.execution_devices))
        if n == "NPUW_LLM_GENERATE_VARIANTS":
            return list(self.variants)
        if n == "NPUW_LLM_PREFILL_CHUNK_SIZE":
            return self.chunk
        return super().get_property(name)

    # ---- requests
    def _make_runner(self, request):
        conv = _Conversation(self.layers, self.capacity, self.kv_dtype)
        request._conversation = conv
        request.npuw_trace = []                     # (sub-model, tokens) per executed step: tests and tuning read it
        reqs = {id(self.prefill): self.prefill.create_infer_request()}
        for cm in self.generate.values():
            reqs[id(cm)] = cm.create_infer_request()
        order = [p.get_node().get_friendly_name() for p in self._inputs]

        def step(cm, ids, positions, past_rows, past_cap):
            """Run `ids` (already padded to the sub-model's token count; `valid` real ones first) over the first `past_rows` cache rows."""
            tokens = len(ids)
            mask = np.zeros((1, past_cap + tokens), np.int64)
            mask[0, :past_rows] = 1
            mask[0, past_cap:past_cap + step.valid] = 1
            feed = {"input_ids": np.asarray(ids, np.int64)[None], "attention_mask": mask, "position_ids": np.asarray(positions, np.int64)[None],
                    "beam_idx": np.zeros(1, np.int32)}
            for n in self.layers:
                feed[n] = np.ascontiguousarray(conv.kv[n][:, :, :past_cap])
            res = reqs[id(cm)].infer(feed)
            outs = {name: res[i] for i, name in enumerate(self.out_names[id(cm)])}
            for n, pn in self.present_of.items():
                conv.kv[n][:, :, past_rows:past_rows + step.valid] = outs[pn][:, :, :step.valid]
            return outs["logits"][:, :step.valid]
        step.valid = 0

        def run(req, ins):
            by_name = {n: t for n, t in zip(order, ins)}
            ids = [int(v) for v in np.asarray(by_name["input_ids"].data).reshape(-1)]
            if np.asarray(by_name["input_ids"].data).shape[0] != 1:
                raise RuntimeError("[NPUW] the LLM pipeline serves batch 1")
            if len(ids) > 1:                                         # a prompt: keep the common prefix when asked to, else start over
                keep = 0
                if self.prefix_caching:
                    while keep < min(len(conv.tokens), len(ids) - 1, conv.rows) and conv.tokens[keep] == ids[keep]:
                        keep += 1
                    keep -= keep % self.chunk                        # chunks start on chunk boundaries of the cache
                conv.rows, conv.tokens = keep, conv.tokens[:keep]
                if len(ids) > self.max_prompt:
                    raise RuntimeError("[NPUW] prompt of %d tokens is longer than NPUW_LLM_MAX_PROMPT_LEN = %d" % (len(ids), self.max_prompt))
                logits = []
                todo = ids[keep:]
                for c0 in range(0, len(todo), self.chunk):
                    part = todo[c0:c0 + self.chunk]
                    step.valid = len(part)
                    padded = part + [0] * (self.chunk - len(part))
                    pos = list(range(conv.rows, conv.rows + len(part))) + [0] * (self.chunk - len(part))
                    logits.append(step(self.prefill, padded, pos, conv.rows, self.max_prompt - self.chunk))
                    conv.rows += len(part)
                    req.npuw_trace.append(("prefill", len(part)))
                conv.tokens = list(ids)
                out = np.concatenate(logits, 1)
                if keep:                                             # rows served from the cache have no logits: the caller samples from the last row
                    out = np.concatenate([np.zeros((1, keep, out.shape[2]), out.dtype), out], 1)
            else:
                if conv.rows + 1 > self.capacity:
                    raise RuntimeError("[NPUW] the conversation outgrew the KV cache of %d rows" % self.capacity)
                k = next(v for v in self.variants if v >= conv.rows + 1)
                step.valid = 1
                out = step(self.generate[k], ids, [conv.rows], conv.rows, k - 1)
                conv.rows += 1
                conv.tokens.append(ids[0])
                req.npuw_trace.append(("generate/%d" % k, 1))
            return [Tensor(np.ascontiguousarray(out))]
        return run

    def _variables(self, request):
        conv = request._conversation

        def refuse(_):
            raise RuntimeError("[NPUW] the KV cache of the LLM pipeline is written by inference only; reset_state() starts a new conversation")
        return [VariableState(n, lambda n=n: Tensor(np.ascontiguousarray(conv.kv[n][:, :, :conv.rows])), refuse, conv.reset) for n in self.layers]
