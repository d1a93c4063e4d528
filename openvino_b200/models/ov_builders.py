"""``Model`` builders for the benchmark architectures, written the way exporters write them.

``build_llama`` emits the stateful decoder that optimum-style exports of Llama-family models contain: inputs
``input_ids`` / ``attention_mask`` / ``position_ids`` / ``beam_idx``, per-layer ReadValue -> Gather(beam_idx) ->
Concat -> Assign KV state, decomposed RMSNorm and half-rotate RoPE, ScaledDotProductAttention with a causal mask,
gate/up/down MLP, and (optionally) int4/int8 group-compressed weights as Constant(u4) -> Convert -> Subtract(zp) ->
Multiply(scale) -> Reshape. The graph-level fusions and the SDPA -> PagedAttention rewrite are tested on it, and the
CUDA device turns it into its LLM program.

The same topology is described by the reference's GGUF builder (src/frontends/gguf/src/builder/blocks/attention.cpp:51-250,
blocks/ffn.cpp, arch/decoder_builder.cpp).
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from .. import opset as ops
from .._graph import make_op, Model, Node, Output, constant, parameter, result
from .._tensor import Tensor
from .._types import PartialShape, Type
from ..utils import quant
from .llm_config import LlmConfig


def _f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def _i64(v) -> Node:
    return constant(np.array(v, dtype=np.int64))


def _linear_weight(name: str, w: torch.Tensor, cfg: LlmConfig, compress: Optional[str]) -> Output:
    """[N, K] weight as an fp32 value: plain Constant, or the decompression sub-graph of a compressed one."""
    if compress is None:
        return constant(_f32(w), name=name).output(0)
    N, Kd = w.shape
    if not isinstance(w, torch.Tensor):         # a placeholder of build_llama_random_int4: draw the compressed constants directly
        return _random_compressed_weight(name, N, Kd, cfg, _linear_weight.rng)
    g = cfg.group_size
    G = Kd // g
    if compress == "int4":
        q, s, z = quant.quantize_u4_asym(w.float(), g)            # q [N, K] uint8 values 0..15, s/z [N, G]
        qt = Tensor(q.reshape(N, G, g).cpu().numpy().astype(np.float32)).astype(Type.u4)
        zt = Tensor(z.reshape(N, G, 1).cpu().numpy().astype(np.float32)).astype(Type.u4)
    elif compress == "int8":
        q, s, z = quant.quantize_u8_asym(w.float(), g)
        qt = Tensor(q.reshape(N, G, g).cpu().numpy().astype(np.uint8))
        zt = Tensor(z.reshape(N, G, 1).cpu().numpy().astype(np.uint8))
    else:
        raise ValueError("compress must be None, 'int4' or 'int8'")
    wq = constant(qt, name=name + "/compressed")
    zp = constant(zt, name=name + "/zero_point")
    sc = constant(s.reshape(N, G, 1).cpu().numpy().astype(np.float16), name=name + "/scale")
    x = ops.subtract(ops.convert(wq, "f16"), ops.convert(zp, "f16"))
    x = ops.multiply(x, sc)
    x = ops.reshape(x, _i64([N, Kd]), False)
    return ops.convert(x, "f32", name=name + "/decompressed").output(0)


def _random_compressed_weight(name: str, N: int, Kd: int, cfg: LlmConfig, rng: np.random.Generator, std: float = 0.02) -> Output:
    """A random int4 (u4, asymmetric, group-wise) weight written straight into its compressed constants: no float copy of
    the weight ever exists, which keeps the construction of multi-billion-parameter benchmark graphs to seconds. Nibbles
    are uniform, zero points 8, one fp16 scale per group chosen so that the de-quantised weights have about ``std``."""
    g = cfg.group_size
    G = Kd // g
    packed = np.frombuffer(rng.bytes(N * Kd // 2), dtype=np.uint8)
    wq = constant(Tensor(packed, shape=[N, G, g], type=Type.u4, shared_memory=True), name=name + "/compressed")
    zp = constant(Tensor(np.full(max(N * G // 2, 1), 0x88, dtype=np.uint8), shape=[N, G, 1], type=Type.u4, shared_memory=True), name=name + "/zero_point")
    # uniform nibbles minus 8 have a standard deviation of about 4.6
    sc = constant(((std / 4.6) * (0.75 + 0.5 * rng.random((N, G, 1)))).astype(np.float16), name=name + "/scale")
    x = ops.subtract(ops.convert(wq, "f16"), ops.convert(zp, "f16"))
    x = ops.multiply(x, sc)
    x = ops.reshape(x, _i64([N, Kd]), False)
    return ops.convert(x, "f32", name=name + "/decompressed").output(0)


class _RandomState(dict):
    """Stands in for the float state dict of ``build_llama`` when the weights are drawn directly in compressed form: norm
    scales are ones, the embedding a small fp16 table; projections are made by ``_random_compressed_weight``."""


def build_llama_random_int4(cfg: LlmConfig, seed: int = 0) -> Model:
    """The stateful decoder of ``build_llama`` with random int4-compressed projections, for benchmarks of architectures too
    large to quantise from float on the host in reasonable time. Same graph, same node names, same compression sub-graphs."""
    rng = np.random.default_rng(seed)
    shapes = {"q_proj": (cfg.num_heads * cfg.head_dim, cfg.hidden_size), "k_proj": (cfg.num_kv_heads * cfg.head_dim, cfg.hidden_size),
              "v_proj": (cfg.num_kv_heads * cfg.head_dim, cfg.hidden_size), "o_proj": (cfg.hidden_size, cfg.num_heads * cfg.head_dim),
              "gate_proj": (cfg.ffn_size, cfg.hidden_size), "up_proj": (cfg.ffn_size, cfg.hidden_size), "down_proj": (cfg.hidden_size, cfg.ffn_size),
              "lm_head": (cfg.vocab_size, cfg.hidden_size)}

    class _Lazy:                # a weight that is generated when the builder asks for it
        def __init__(self, key):
            self.shape = shapes[key]

    state = _RandomState()
    ones = torch.ones(cfg.hidden_size)
    for l in range(cfg.num_layers):
        p = "layers.%d." % l
        state[p + "input_layernorm"] = ones
        state[p + "post_attention_layernorm"] = ones
        for key in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
            state[p + key] = _Lazy(key)
    state["norm"] = ones
    state["lm_head"] = _Lazy("lm_head")
    # fp16 values with random sign and mantissa and the exponent of 2^-6: magnitudes in [0.0156, 0.0313)
    bits = np.frombuffer(rng.bytes(cfg.vocab_size * cfg.hidden_size * 2), dtype=np.uint16)
    state["embed_tokens"] = torch.from_numpy(((bits & np.uint16(0x83FF)) | np.uint16(0x2400)).view(np.float16).reshape(cfg.vocab_size, cfg.hidden_size))
    state["_rng"] = rng
    return build_llama(cfg, state, compress="int4")


def _rms(x: Output, gamma: np.ndarray, eps: float, name: str) -> Output:
    sq = ops.power(x, np.float32(2.0))
    var = ops.reduce_mean(sq, _i64([-1]), True)
    inv = ops.divide(np.float32(1.0), ops.sqrt(ops.add(var, np.float32(eps))))
    return ops.multiply(ops.multiply(x, inv), constant(gamma, name=name + ".weight"), name=name).output(0)


def _rope(x: Output, cos: Output, sin: Output, D: int) -> Output:
    """x [B, H, L, D]; cos/sin [B, 1, L, D]: x * cos + rotate_half(x) * sin."""
    lo = ops.slice(x, _i64([0]), _i64([D // 2]), _i64([1]), _i64([3]))
    hi = ops.slice(x, _i64([D // 2]), _i64([D]), _i64([1]), _i64([3]))
    rot = ops.concat([ops.negative(hi).output(0), lo.output(0)], 3)
    return ops.add(ops.multiply(x, cos), ops.multiply(rot, sin)).output(0)


def build_llama(cfg: LlmConfig, state: Dict[str, torch.Tensor], compress: Optional[str] = None, stateful: bool = True) -> Model:
    """Stateful decoder ``Model`` with fp32 activations. ``compress``: None | "int4" | "int8" (group-wise, asymmetric)."""
    H, D, Hq, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    _linear_weight.rng = state.get("_rng")
    input_ids = parameter(PartialShape([-1, -1]), "i64", "input_ids")
    attention_mask = parameter(PartialShape([-1, -1]), "i64", "attention_mask")
    position_ids = parameter(PartialShape([-1, -1]), "i64", "position_ids")
    beam_idx = parameter(PartialShape([-1]), "i32", "beam_idx")
    for p in (input_ids, attention_mask, position_ids, beam_idx):
        p.output(0).set_names({p.get_friendly_name()})

    if state["embed_tokens"].dtype == torch.float16:     # fp16 table + Convert, as exporters of compressed models write it
        embed = ops.convert(constant(state["embed_tokens"].numpy(), name="model.embed_tokens.weight"), "f32")
    else:
        embed = constant(_f32(state["embed_tokens"]), name="model.embed_tokens.weight")
    h = ops.gather(embed, input_ids, _i64(0), name="embed").output(0)             # [B, L, H]

    # rotary tables from position ids: [B, L] -> cos/sin [B, 1, L, D]
    inv_freq = (cfg.rope_theta ** (-np.arange(0, D, 2, dtype=np.float32) / D)).astype(np.float32)
    pos = ops.convert(ops.unsqueeze(position_ids, _i64([2])), "f32")               # [B, L, 1]
    ang = ops.multiply(pos, constant(inv_freq.reshape(1, 1, -1)))                  # [B, L, D/2]
    ang = ops.concat([ang.output(0), ang.output(0)], 2)
    cos = ops.unsqueeze(ops.cos(ang), _i64([1])).output(0)
    sin = ops.unsqueeze(ops.sin(ang), _i64([1])).output(0)

    # additive causal + padding mask [B, 1, L, S]: position of key j must be <= position of query i and mask[j] == 1
    shape_ids = ops.shape_of(input_ids)
    L = ops.gather(shape_ids, _i64([1]), _i64(0))
    S = ops.gather(ops.shape_of(attention_mask), _i64([1]), _i64(0))
    past = ops.subtract(S, L)
    q_pos = ops.add(ops.range(_i64(0), ops.squeeze(L), _i64(1), "i64"), ops.squeeze(past))
    k_pos = ops.range(_i64(0), ops.squeeze(S), _i64(1), "i64")
    causal = ops.less_equal(ops.unsqueeze(k_pos, _i64([0])), ops.unsqueeze(q_pos, _i64([1])))   # [L, S]
    if cfg.sliding_window > 0:          # only the last `sliding_window` keys stay visible: k_pos > q_pos - W
        near = ops.greater(ops.unsqueeze(k_pos, _i64([0])), ops.subtract(ops.unsqueeze(q_pos, _i64([1])), _i64(cfg.sliding_window)))
        causal = ops.logical_and(causal, near)
    pad_ok = ops.unsqueeze(ops.not_equal(attention_mask, _i64(0)), _i64([1, 2]))                # [B, 1, 1, S]
    allowed = ops.logical_and(ops.unsqueeze(causal, _i64([0, 1])), pad_ok)
    mask = ops.select(allowed, np.float32(0.0), np.float32(-65504.0), name="attention_bias").output(0)

    batch = ops.gather(shape_ids, _i64([0]), _i64(0))
    sinks = []
    for l in range(cfg.num_layers):
        p = "layers.%d." % l
        n = "model.layers.%d." % l
        x = _rms(h, _f32(state[p + "input_layernorm"]), cfg.rms_eps, n + "input_layernorm")

        def proj(name, inp, key):
            return ops.matmul(inp, _linear_weight(n + name + ".weight", state[p + key], cfg, compress), False, True, name=n + name).output(0)

        def heads(t: Output, nh: int) -> Output:   # [B, L, nh*D] -> [B, nh, L, D]
            r = ops.reshape(t, _i64([0, 0, nh, D]), True)
            return ops.transpose(r, _i64([0, 2, 1, 3])).output(0)

        q = _rope(heads(proj("self_attn.q_proj", x, "q_proj"), Hq), cos, sin, D)
        k = _rope(heads(proj("self_attn.k_proj", x, "k_proj"), Hkv), cos, sin, D)
        v = heads(proj("self_attn.v_proj", x, "v_proj"), Hkv)

        if stateful:
            init_shape = ops.concat([batch.output(0), _i64([Hkv, 0, D]).output(0)], 0)
            k_init = ops.broadcast(np.float32(0.0), init_shape)
            v_init = ops.broadcast(np.float32(0.0), init_shape)
            kid, vid = "past_key_values.%d.keypresent.%d.key" % (l, l), "past_key_values.%d.valuepresent.%d.value" % (l, l)
            k_past = ops.gather(ops.read_value(k_init, kid, "f32", PartialShape([-1, Hkv, -1, D])), beam_idx, _i64(0))
            v_past = ops.gather(ops.read_value(v_init, vid, "f32", PartialShape([-1, Hkv, -1, D])), beam_idx, _i64(0))
            k_all = ops.concat([k_past.output(0), k], 2, name=n + "self_attn.k_cache")
            v_all = ops.concat([v_past.output(0), v], 2, name=n + "self_attn.v_cache")
            sinks += [ops.assign(k_all, kid), ops.assign(v_all, vid)]
            k_use, v_use = k_all.output(0), v_all.output(0)
        else:
            k_use, v_use = k, v
        if Hq != Hkv:   # grouped-query attention: repeat every KV head Hq / Hkv times
            G = Hq // Hkv

            def expand(t: Output) -> Output:
                u = ops.unsqueeze(t, _i64([2]))                                             # [B, Hkv, 1, S, D]
                bshape = ops.concat([batch.output(0), _i64([Hkv, G]).output(0), ops.gather(ops.shape_of(t), _i64([2]), _i64(0)).output(0),
                                     _i64([D]).output(0)], 0)
                b = ops.broadcast(u, bshape)
                return ops.reshape(b, _i64([0, Hq, -1, D]), True).output(0)
            k_use, v_use = expand(k_use), expand(v_use)
        attn = ops.scaled_dot_product_attention(q, k_use, v_use, mask, name=n + "self_attn.sdpa")
        a = ops.reshape(ops.transpose(attn, _i64([0, 2, 1, 3])), _i64([0, 0, Hq * D]), True)
        h = ops.add(h, proj("self_attn.o_proj", a, "o_proj")).output(0)

        x = _rms(h, _f32(state[p + "post_attention_layernorm"]), cfg.rms_eps, n + "post_attention_layernorm")
        if cfg.num_experts:
            # mixture of experts: router -> softmax -> top-k -> renormalise -> MOE (batched expert weights [E, F, H] / [E, H, F])
            E, k = cfg.num_experts, cfg.experts_top_k
            router = ops.matmul(x, constant(_f32(state[p + "router"]), name=n + "block_sparse_moe.gate.weight"), False, True,
                                name=n + "block_sparse_moe.gate")
            probs = ops.softmax(router, -1)
            top = ops.topk(probs, _i64(k), -1, "max", "value", "i32")
            wsum = ops.reduce_sum(top.output(0), _i64([-1]), True)
            rw = ops.divide(top.output(0), wsum)

            def stack(key):
                return constant(np.stack([_f32(state[p + "experts.%d.%s" % (e, key)]) for e in range(E)]), name=n + "block_sparse_moe.experts." + key)
            moe = make_op("MOE", [x, rw.output(0), top.output(1), stack("gate_proj").output(0), stack("up_proj").output(0), stack("down_proj").output(0)],
                          {"expert_type": "GEMM3_SWIGLU", "activation_type": "SWISH"}, "internal", n + "block_sparse_moe")
            h = ops.add(h, moe.output(0)).output(0)
            continue
        gate = ops.swish(proj("mlp.gate_proj", x, "gate_proj"))
        up = proj("mlp.up_proj", x, "up_proj")
        h = ops.add(h, proj("mlp.down_proj", ops.multiply(gate, up), "down_proj")).output(0)

    x = _rms(h, _f32(state["norm"]), cfg.rms_eps, "model.norm")
    logits = ops.matmul(x, _linear_weight("lm_head.weight", state["lm_head"], cfg, compress), False, True, name="lm_head")
    logits.output(0).set_names({"logits"})
    m = Model([result(logits, "logits")], [input_ids, attention_mask, position_ids, beam_idx], cfg.name, sinks)
    m.set_rt_info("llama", ["model_info", "architecture"])
    return m
