"""``Model`` -> LLM program: recognise a decoder-only transformer graph and lift it into the serving executor.

The CUDA device runs any graph through its graph program; a Llama-family decoder additionally gets the serving
program (``CudaLlmExecutor``: paged KV cache, ragged batches, CUDA graphs, tensor parallelism). This module reads the
architecture (hidden size, heads, head size, RoPE base, norm epsilon, vocabulary) and the weights out of the graph
after the device's fusion passes, following the data flow around every attention operation (node names play no part):
RMS / RoPE / FullyConnected / FullyConnectedCompressed nodes. Compressed weights are taken in their IR form
(u4/u8 Constant + fp16 scales + zero points) and re-packed for the kernels without ever being expanded to float.

This is the step the reference performs inside its device plugins when a PagedAttention model is compiled
(src/plugins/intel_gpu/src/plugin/ops/paged_attention.cpp, transformations_pipeline.cpp); the topology matched here is
the one the reference's own LLM builders emit (src/frontends/gguf/src/builder/arch/decoder_builder.cpp).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .. import _ovcore as _c
from .._graph import Model, Node
from .._types import Type
from ..models.llm_config import LlmConfig


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

    @staticmethod
    def interleave(gate: "_Linear", up: "_Linear") -> "_Linear":
        """Gate and up projections in the row order of the fused SwiGLU epilogue: every 128-row tile holds 64 gate rows
        followed by the 64 up rows of the same channels (the row count must be a multiple of 64)."""
        o = _Linear.stack([gate, up])
        F = gate.N
        order = torch.stack([torch.arange(F).reshape(F // 64, 64), F + torch.arange(F).reshape(F // 64, 64)], dim=1).reshape(-1)
        if o.compressed:
            o.q, o.scales, o.zp = o.q[order], o.scales[order], o.zp[order]
        else:
            o.w = o.w[order]
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


_FC = ("FullyConnected", "FullyConnectedCompressed")
_DEAD_ENDS = ("Parameter", "Constant", "ReadValue", "Result", "Assign")


def _nearest_fc_ancestor(out_port) -> Optional[Node]:
    """Closest FullyConnected node that feeds ``out_port`` (breadth first over all data inputs; shape plumbing, RoPE, the
    KV-state Concat and the grouped-query broadcast are walked through, parameters / constants / states end a path)."""
    seen, frontier = set(), [out_port.get_node()]
    while frontier:
        nxt = []
        for n in frontier:
            if n in seen:
                continue
            seen.add(n)
            t = n.get_type_name()
            if t in _FC:
                return n
            if t in _DEAD_ENDS or t in ("ScaledDotProductAttention", "PagedAttentionExtension", "RMS"):
                continue
            for i in range(n.get_input_size()):
                nxt.append(n.input_value(i).get_node())
        frontier = nxt
    return None


def _consumers(node: Node, port: int = 0):
    return [inp.get_node() for inp in node.output(port).get_target_inputs()]


def _nearest_fc_descendant(node: Node) -> Optional[Node]:
    """Closest FullyConnected node fed (through reshapes / transposes / converts) by ``node``."""
    seen, frontier = set(), [node]
    while frontier:
        nxt = []
        for n in frontier:
            for c in _consumers(n):
                if c in seen:
                    continue
                seen.add(c)
                t = c.get_type_name()
                if t in _FC:
                    return c
                if t in ("Reshape", "Transpose", "Convert", "Squeeze", "Unsqueeze"):
                    nxt.append(c)
        frontier = nxt
    return None


def _one(nodes, what: str) -> Node:
    if len(nodes) != 1:
        raise NotAnLlm("expected exactly one %s, found %d" % (what, len(nodes)))
    return nodes[0]


def _gamma(rms: Node) -> torch.Tensor:
    g = rms.input_value(1).get_node()
    if g.get_type_name() == "Convert":
        g = g.input_value(0).get_node()
    if g.get_type_name() != "Constant":
        raise NotAnLlm("the scale of %s is not a constant" % rms.get_friendly_name())
    return _const_f32(g).reshape(-1)


def analyze(model: Model) -> Tuple[LlmConfig, Dict]:
    """Fused graph -> (architecture, {name: _Linear | tensor}). The decoder is recognised by its STRUCTURE, whatever the
    nodes are called: every attention operation (ScaledDotProductAttention or PagedAttentionExtension) is one layer; its
    query / key / value inputs lead back to three projections that share one RMS input; its output leads on to the output
    projection, the residual Add, the second RMS, the gate (the projection that feeds Swish) and up projections, their
    product, the down projection and the second residual Add. After the last layer come the final RMS and the projection
    onto the vocabulary; before the first one the embedding Gather. Raises ``NotAnLlm`` when the graph is not of this form."""
    m = model.clone()
    _c.run_moc_transformations(m._m, True)
    _c.run_llm_fusions(m._m)
    ops = m.get_ops()
    att = [n for n in ops if n.get_type_name() in ("ScaledDotProductAttention", "PagedAttentionExtension")]
    if not att:
        raise NotAnLlm("no attention operation found")
    lin: Dict[Tuple[int, str], _Linear] = {}
    norms: Dict[Tuple[int, str], torch.Tensor] = {}
    experts: Dict[int, Dict] = {}
    eps = 1e-6
    last_add = first_norm = None
    for l, a in enumerate(att):
        q, k, v = (_nearest_fc_ancestor(a.input_value(i)) for i in range(3))
        if q is None or k is None or v is None:
            raise NotAnLlm("attention %d is not fed by three projections" % l)
        n1 = q.input_value(0).get_node()
        if n1.get_type_name() != "RMS" or any(x.input_value(0).get_node() != n1 for x in (k, v)):
            raise NotAnLlm("the projections of attention %d do not share one RMS input" % l)
        o = _nearest_fc_descendant(a)
        if o is None:
            raise NotAnLlm("attention %d has no output projection" % l)
        add1 = _one([c for c in _consumers(o) if c.get_type_name() == "Add"], "residual Add after the attention output projection")
        n2 = _one([c for c in _consumers(add1) if c.get_type_name() == "RMS"], "RMS after the attention residual")
        mlp = [c for c in _consumers(n2) if c.get_type_name() in _FC]
        moe = [c for c in _consumers(n2) if c.get_type_name() == "MOE"]
        if moe:
            # mixture of experts: the RMS output feeds the router projection (as many rows as experts) and the MOE operation,
            # whose routing weights / expert indices come from the router through softmax and top-k
            mo = _one(moe, "MOE operation")
            if mo.get_attribute("expert_type") != "GEMM3_SWIGLU":
                raise NotAnLlm("layer %d: expert type %s is not served" % (l, mo.get_attribute("expert_type")))
            ew = []
            for i in (3, 4, 5):
                c = mo.input_value(i).get_node()
                if c.get_type_name() == "Convert":
                    c = c.input_value(0).get_node()
                if c.get_type_name() != "Constant":
                    raise NotAnLlm("layer %d: the expert weights are not constants" % l)
                ew.append(_const_f32(c))
            n_exp = ew[0].shape[0]
            router = _one([c for c in mlp if _Linear(c).N == n_exp], "router projection")
            idx_shape = mo.input_value(2).get_partial_shape()
            top_k = int(idx_shape[idx_shape.rank.get_length() - 1].get_length())
            add2 = _one([c for c in _consumers(mo) if c.get_type_name() == "Add"], "residual Add after the experts")
            for key, node in (("q_proj", q), ("k_proj", k), ("v_proj", v), ("o_proj", o), ("router", router)):
                lin[(l, key)] = _Linear(node)
            experts[l] = {"gate": ew[0], "up": ew[1], "down": ew[2], "top_k": top_k}
            norms[(l, "input_layernorm")] = _gamma(n1)
            norms[(l, "post_attention_layernorm")] = _gamma(n2)
            eps = float(n1.get_attribute("epsilon"))
            if l == 0:
                first_norm = n1
            last_add = add2
            continue
        gates = [c for c in mlp if any(x.get_type_name() == "Swish" for x in _consumers(c))]
        ups = [c for c in mlp if c not in gates]
        if len(gates) != 1 or len(ups) != 1:
            raise NotAnLlm("layer %d: expected one gate (followed by Swish) and one up projection, found %d / %d" % (l, len(gates), len(ups)))
        act = _one([x for x in _consumers(gates[0]) if x.get_type_name() == "Swish"], "Swish")
        prod = _one([x for x in _consumers(act) if x.get_type_name() == "Multiply"], "gate x up product")
        down = _nearest_fc_descendant(prod)
        if down is None:
            raise NotAnLlm("layer %d has no down projection" % l)
        add2 = _one([c for c in _consumers(down) if c.get_type_name() == "Add"], "residual Add after the MLP")
        for key, node in (("q_proj", q), ("k_proj", k), ("v_proj", v), ("o_proj", o), ("gate_proj", gates[0]), ("up_proj", ups[0]), ("down_proj", down)):
            lin[(l, key)] = _Linear(node)
        norms[(l, "input_layernorm")] = _gamma(n1)
        norms[(l, "post_attention_layernorm")] = _gamma(n2)
        eps = float(n1.get_attribute("epsilon"))
        if l == 0:
            first_norm = n1
        last_add = add2
    fn = _one([c for c in _consumers(last_add) if c.get_type_name() == "RMS"], "final RMS")
    final_norm = _gamma(fn)
    lm_head = _Linear(_one([c for c in _consumers(fn) if c.get_type_name() in _FC], "projection onto the vocabulary"))
    emb = first_norm.input_value(0).get_node()
    while emb.get_type_name() in ("Convert", "Reshape", "Squeeze", "Unsqueeze"):
        emb = emb.input_value(0).get_node()
    if emb.get_type_name() != "Gather":
        raise NotAnLlm("the first layer is not fed by an embedding Gather")
    src = emb.input_value(0).get_node()
    if src.get_type_name() == "Convert":
        src = src.input_value(0).get_node()
    if src.get_type_name() != "Constant" or len(src.get_output_shape(0)) != 2:
        raise NotAnLlm("the embedding table is not a 2-D constant")
    embed = _const_f32(src)
    layers = list(range(len(att)))
    # head geometry from the attention op: query [B, Hq, L, D]
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
                    num_kv_heads=Hkv, head_dim=D, ffn_size=experts[0]["gate"].shape[1] if experts else lin[(layers[0], "gate_proj")].N,
                    rope_theta=theta, rms_eps=eps, weight_format=fmt, group_size=(first.K // first.G) if first.compressed else 128,
                    num_experts=experts[0]["gate"].shape[0] if experts else 0, experts_top_k=experts[0]["top_k"] if experts else 0)
    if experts and len(experts) != len(layers):
        raise NotAnLlm("dense and expert layers in one model are not served")
    # the sliding window of the paged form is an input of the attention operation (0 = none); ALiBi has no kernel yet
    for n in ops:
        if n.get_type_name() == "PagedAttentionExtension" and n.get_input_size() > 11:
            w = n.input_value(10).get_node()
            if w.get_type_name() == "Constant":
                cfg = cfg.with_(sliding_window=int(np.asarray(w.get_data()).reshape(-1)[0]))
            a = n.input_value(11)
            if a.get_partial_shape().is_static and int(np.prod(list(a.get_shape()) or [1])) > 0:
                raise NotAnLlm("attention with ALiBi slopes is not served by the device program")
            break
    return cfg, {"lin": lin, "norms": norms, "lm_head": lm_head, "final_norm": final_norm, "embed": embed, "layers": layers, "experts": experts}


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
        if parts.get("experts"):
            # expert parallel: rank r holds experts [r * nloc, (r + 1) * nloc) whole; gate and up of an expert are stacked
            # ([nloc * 2F, H]), the down projections side by side along K ([H, nloc * F]); the router is replicated
            from ..ops import cuda as K
            ex = parts["experts"][l]
            nloc = cfg.num_experts // tp_size
            local = range(r * nloc, (r + 1) * nloc)
            gu = torch.cat([torch.cat([ex["gate"][e], ex["up"][e]], 0) for e in local], 0)
            down = torch.cat([ex["down"][e] for e in local], 1)
            pack16 = lambda t: K.PackedWeight.from_dense(t.to(device).to(torch.bfloat16).contiguous())
            layers.append(LayerWeights(norm1=bf(norms[(l, "input_layernorm")]), qkv=_Linear.stack([q, k, v]).pack(device),
                                       o=lin[(l, "o_proj")].cols(r * hq * D, (r + 1) * hq * D).pack(device),
                                       norm2=bf(norms[(l, "post_attention_layernorm")]), gate_up=pack16(gu), down=pack16(down),
                                       router=lin[(l, "router")].pack(device)))
            continue
        gate = lin[(l, "gate_proj")].rows(r * ffn, (r + 1) * ffn)
        up = lin[(l, "up_proj")].rows(r * ffn, (r + 1) * ffn)
        fused_gate = ffn % 64 == 0          # silu(gate) * up in the GEMM epilogue needs the interleaved row order
        gate_up = (_Linear.interleave(gate, up) if fused_gate else _Linear.stack([gate, up])).pack(device)
        gate_up.swiglu = fused_gate
        layers.append(LayerWeights(norm1=bf(norms[(l, "input_layernorm")]), qkv=_Linear.stack([q, k, v]).pack(device),
                                   o=lin[(l, "o_proj")].cols(r * hq * D, (r + 1) * hq * D).pack(device),
                                   norm2=bf(norms[(l, "post_attention_layernorm")]), gate_up=gate_up,
                                   down=lin[(l, "down_proj")].cols(r * ffn, (r + 1) * ffn).pack(device)))
    vs = cfg.vocab_size // tp_size
    return LlmWeights(bf(parts["embed"]), layers, bf(parts["final_norm"]), parts["lm_head"].rows(r * vs, (r + 1) * vs).pack(device), tp_rank, tp_size)
