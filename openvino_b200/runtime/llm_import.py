"""``Model`` -> LLM program: recognise a decoder-only transformer graph and lift it into the serving executor.

The CUDA device runs any graph through its graph program; a Llama-family decoder additionally gets the serving
program (``CudaLlmExecutor``: paged KV cache, ragged batches, CUDA graphs, tensor parallelism). This module reads the
architecture (hidden size, heads, head size, RoPE base, norm epsilon, vocabulary) and the weights out of the graph
after the device's fusion passes: RMS / RoPE / FullyConnected / FullyConnectedCompressed nodes named by the usual
exporter convention (``...layers.<i>.self_attn.q_proj`` and so on). Compressed weights are taken in their IR form
(u4/u8 Constant + fp16 scales + zero points) and re-packed for the kernels without ever being expanded to float.

This is the step the reference performs inside its device plugins when a PagedAttention model is compiled
(src/plugins/intel_gpu/src/plugin/ops/paged_attention.cpp, transformations_pipeline.cpp); the topology matched here is
the one the reference's own LLM builders emit (src/frontends/gguf/src/builder/arch/decoder_builder.cpp).
"""
from __future__ import annotations

import re
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .. import _ovcore as _c
from .._graph import Model, Node
from .._types import Type
from ..models.llm_config import LlmConfig

_PROJ = re.compile(r"layers\.(\d+)\.(self_attn\.(?:q|k|v|o)_proj|mlp\.(?:gate|up|down)_proj)$")
_NORM = re.compile(r"layers\.(\d+)\.(input_layernorm|post_attention_layernorm)$")


class NotAnLlm(RuntimeError):
    pass


def _const_f32(node: Node) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(node.get_tensor_view().to_float32()))


class _Linear:
    """One projection as found in the graph: dense float weight, or compressed weight + scales + zero points."""

    def __init__(self, fc: Node):
        t = fc.get_type_name()
        w = fc.input_value(1).get_node()
        if w.get_type_name() == "Convert":
            w = w.input_value(0).get_node()
        if w.get_type_name() != "Constant":
            raise NotAnLlm("weight of %s is not a constant" % fc.get_friendly_name())
        self.compressed = t == "FullyConnectedCompressed"
        view = w.get_tensor_view()
        self.N = view.shape[0]
        self.K = int(np.prod(view.shape[1:]))
        if self.compressed:
            self.kind = view.element_type.name                                     # u4 | u8
            if self.kind not in ("u4", "u8"):
                raise NotAnLlm("compressed weight type %s is not supported by the serving program" % self.kind)
            self.q = torch.from_numpy(np.ascontiguousarray(view.data).reshape(-1).view(np.uint8).copy()).reshape(self.N, -1)
            self.scales = _const_f32(fc.input_value(3).get_node()).reshape(self.N, -1)
            self.G = self.scales.shape[1]
            zp_node = fc.input_value(4).get_node() if fc.get_input_size() > 4 else None
            zp = _const_f32(zp_node).reshape(-1) if zp_node is not None and zp_node.get_type_name() == "Constant" and zp_node.get_tensor_view().size else None
            if zp is None:
                zp = torch.full((1,), 8.0 if self.kind == "u4" else 128.0)
            self.zp = (zp.expand(self.N * self.G) if zp.numel() == 1 else zp).reshape(self.N, self.G).to(torch.uint8)
        else:
            self.w = _const_f32(w).reshape(self.N, self.K)

    # tensor-parallel slices: rows [r0, r1) (column parallel) or columns [k0, k1) (row parallel)
    def rows(self, r0: int, r1: int) -> "_Linear":
        o = _Linear.__new__(_Linear)
        o.compressed, o.N, o.K = self.compressed, r1 - r0, self.K
        if self.compressed:
            o.kind, o.G = self.kind, self.G
            o.q, o.scales, o.zp = self.q[r0:r1], self.scales[r0:r1], self.zp[r0:r1]
        else:
            o.w = self.w[r0:r1]
        return o

    def cols(self, k0: int, k1: int) -> "_Linear":
        o = _Linear.__new__(_Linear)
        o.compressed, o.N, o.K = self.compressed, self.N, k1 - k0
        if self.compressed:
            g = self.K // self.G
            if k0 % g or k1 % g:
                raise NotAnLlm("a tensor-parallel cut of the K axis must fall on quantisation group borders")
            bpk = 2 if self.kind == "u4" else 1                                    # elements per byte
            o.kind, o.G = self.kind, (k1 - k0) // g
            o.q = self.q[:, k0 // bpk:k1 // bpk]
            o.scales, o.zp = self.scales[:, k0 // g:k1 // g], self.zp[:, k0 // g:k1 // g]
        else:
            o.w = self.w[:, k0:k1]
        return o

    @staticmethod
    def stack(parts) -> "_Linear":
        o = _Linear.__new__(_Linear)
        p0 = parts[0]
        o.compressed, o.K, o.N = p0.compressed, p0.K, sum(p.N for p in parts)
        if p0.compressed:
            o.kind, o.G = p0.kind, p0.G
            o.q, o.scales, o.zp = torch.cat([p.q for p in parts]), torch.cat([p.scales for p in parts]), torch.cat([p.zp for p in parts])
        else:
            o.w = torch.cat([p.w for p in parts])
        return o

    def pack(self, device):
        from ..ops import cuda as K
        if not self.compressed:
            return K.PackedWeight.from_dense(self.w.to(device).to(torch.bfloat16).contiguous())
        g = self.K // self.G
        q = self.q.contiguous().to(device)
        s = self.scales.to(torch.float16).contiguous().to(device)
        z = self.zp.contiguous().to(device)
        if self.kind == "u4":
            return K.PackedWeight.from_ir_u4(q.reshape(-1), s, z, self.N, self.K, g, zp_is_u8=True)
        return K.PackedWeight.from_ir_u8(q.reshape(self.N, self.K), s, z, self.N, self.K, g)


def analyze(model: Model) -> Tuple[LlmConfig, Dict]:
    """Fused graph -> (architecture, {name: _Linear | tensor}). Raises ``NotAnLlm`` when the graph does not look like one."""
    m = model.clone()
    _c.run_moc_transformations(m._m, True)
    _c.run_llm_fusions(m._m)
    ops = m.get_ops()
    lin: Dict[Tuple[int, str], _Linear] = {}
    norms: Dict[Tuple[int, str], torch.Tensor] = {}
    lm_head = final_norm = embed = None
    eps = 1e-6
    for n in ops:
        t = n.get_type_name()
        name = n.get_friendly_name()
        if t in ("FullyConnected", "FullyConnectedCompressed"):
            mm = _PROJ.search(name)
            if mm:
                lin[(int(mm.group(1)), mm.group(2).split(".")[1])] = _Linear(n)
            elif name.endswith("lm_head"):
                lm_head = _Linear(n)
        elif t == "RMS":
            gamma = n.input_value(1).get_node()
            if gamma.get_type_name() == "Convert":
                gamma = gamma.input_value(0).get_node()
            mm = _NORM.search(name)
            eps = float(n.get_attribute("epsilon"))
            if mm:
                norms[(int(mm.group(1)), mm.group(2))] = _const_f32(gamma).reshape(-1)
            elif name.endswith("model.norm") or name.endswith("norm"):
                final_norm = _const_f32(gamma).reshape(-1)
        elif t == "Gather" and embed is None:
            src = n.input_value(0).get_node()
            if src.get_type_name() == "Convert":
                src = src.input_value(0).get_node()
            if src.get_type_name() == "Constant" and len(src.get_output_shape(0)) == 2 and src.get_output_shape(0)[0] > 16:
                embed = _const_f32(src)
    layers = sorted({k[0] for k in lin})
    if not layers or lm_head is None or embed is None or final_norm is None:
        raise NotAnLlm("the graph has no decoder layers / embedding / final norm / lm_head with the expected names")
    for l in layers:
        for p in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
            if (l, p) not in lin:
                raise NotAnLlm("layer %d lacks %s" % (l, p))
    # head geometry from the attention op: query [B, Hq, L, D]
    att = [n for n in ops if n.get_type_name() in ("ScaledDotProductAttention", "PagedAttentionExtension")]
    if not att:
        raise NotAnLlm("no attention operation found")
    H = embed.shape[1]
    if att[0].get_type_name() == "ScaledDotProductAttention":
        qs = att[0].input_value(0).get_partial_shape()
        Hq, D = qs[1].get_length(), qs[3].get_length()
    else:
        D = int(att[0].rt_info.get("k_head_size"))
        Hq = lin[(layers[0], "q_proj")].N // D
    Hkv = lin[(layers[0], "k_proj")].N // D
    # RoPE base from the inverse-frequency table: inv_freq[1] = theta^(-2/D)
    theta = 10000.0
    for n in ops:
        if n.get_type_name() == "Constant" and n.get_output_element_type(0).is_real():
            shp = n.get_output_shape(0)
            if int(np.prod(shp or [1])) == D // 2 and D >= 4:
                v = n.get_tensor_view().to_float32().reshape(-1)
                if abs(float(v[0]) - 1.0) < 1e-6 and 0 < v[1] < 1:
                    theta = float(v[1]) ** (-D / 2.0)
                    break
    first = lin[(layers[0], "q_proj")]
    fmt = {"u4": "int4", "u8": "int8"}[first.kind] if first.compressed else "bf16"
    cfg = LlmConfig(name=model.get_friendly_name() or "llm", vocab_size=embed.shape[0], hidden_size=H, num_layers=len(layers), num_heads=Hq,
                    num_kv_heads=Hkv, head_dim=D, ffn_size=lin[(layers[0], "gate_proj")].N, rope_theta=theta, rms_eps=eps,
                    weight_format=fmt, group_size=(first.K // first.G) if first.compressed else 128)
    return cfg, {"lin": lin, "norms": norms, "lm_head": lm_head, "final_norm": final_norm, "embed": embed, "layers": layers}


def build_weights(cfg: LlmConfig, parts: Dict, device, tp_rank: int = 0, tp_size: int = 1):
    """Shard for tensor parallelism and pack into the kernels' layouts (``LlmWeights``)."""
    from .cuda_llm import LayerWeights, LlmWeights
    D = cfg.head_dim
    hq, hkv, ffn = cfg.num_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.ffn_size // tp_size
    r = tp_rank
    lin, norms = parts["lin"], parts["norms"]
    bf = lambda t: t.to(device).to(torch.bfloat16).contiguous()
    layers = []
    for l in parts["layers"]:
        q = lin[(l, "q_proj")].rows(r * hq * D, (r + 1) * hq * D)
        k = lin[(l, "k_proj")].rows(r * hkv * D, (r + 1) * hkv * D)
        v = lin[(l, "v_proj")].rows(r * hkv * D, (r + 1) * hkv * D)
        gate = lin[(l, "gate_proj")].rows(r * ffn, (r + 1) * ffn)
        up = lin[(l, "up_proj")].rows(r * ffn, (r + 1) * ffn)
        layers.append(LayerWeights(norm1=bf(norms[(l, "input_layernorm")]), qkv=_Linear.stack([q, k, v]).pack(device),
                                   o=lin[(l, "o_proj")].cols(r * hq * D, (r + 1) * hq * D).pack(device),
                                   norm2=bf(norms[(l, "post_attention_layernorm")]), gate_up=_Linear.stack([gate, up]).pack(device),
                                   down=lin[(l, "down_proj")].cols(r * ffn, (r + 1) * ffn).pack(device)))
    vs = cfg.vocab_size // tp_size
    return LlmWeights(bf(parts["embed"]), layers, bf(parts["final_norm"]), parts["lm_head"].rows(r * vs, (r + 1) * vs).pack(device), tp_rank, tp_size)
