"""Llama-family decoder: random-init float state, a plain PyTorch reference forward (the numerics
oracle of the CUDA program and the model used by the NCCL + cuBLAS baseline), and the
``ov.Model`` builder lives in models/ov_builders.py."""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from .llm_config import LlmConfig


def random_float_state(cfg: LlmConfig, seed: int = 0, device="cpu", std: float = 0.02) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device) * std
    H, D = cfg.hidden_size, cfg.head_dim
    st = {"embed_tokens": rn(cfg.vocab_size, H), "norm": 1.0 + rn(H), "lm_head": rn(cfg.vocab_size, H)}
    for l in range(cfg.num_layers):
        p = "layers.%d." % l
        st[p + "input_layernorm"] = 1.0 + rn(H)
        st[p + "post_attention_layernorm"] = 1.0 + rn(H)
        st[p + "q_proj"] = rn(cfg.num_heads * D, H)
        st[p + "k_proj"] = rn(cfg.num_kv_heads * D, H)
        st[p + "v_proj"] = rn(cfg.num_kv_heads * D, H)
        st[p + "o_proj"] = rn(H, cfg.num_heads * D)
        if cfg.num_experts:
            st[p + "router"] = rn(cfg.num_experts, H) * 10.0     # spread the routing logits so that the top-k is well separated
            for e in range(cfg.num_experts):
                st[p + "experts.%d.gate_proj" % e] = rn(cfg.ffn_size, H)
                st[p + "experts.%d.up_proj" % e] = rn(cfg.ffn_size, H)
                st[p + "experts.%d.down_proj" % e] = rn(H, cfg.ffn_size)
        else:
            st[p + "gate_proj"] = rn(cfg.ffn_size, H)
            st[p + "up_proj"] = rn(cfg.ffn_size, H)
            st[p + "down_proj"] = rn(H, cfg.ffn_size)
    return st


def effective_state(cfg: LlmConfig, state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The weights the compressed model actually computes with: linear weights quantised and
    dequantised per cfg.weight_format, norms/embeddings rounded to bf16."""
    from ..utils import quant
    out = {}
    for k, v in state.items():
        if v.dim() == 2 and not k.endswith("embed_tokens") and not k.endswith("router"):
            if cfg.weight_format == "int4":
                q, s, z = quant.quantize_u4_asym(v, cfg.group_size)
                out[k] = quant.dequantize_u4(q, s, z, cfg.group_size)
            elif cfg.weight_format == "int8":
                q, s, z = quant.quantize_u8_asym(v, cfg.group_size)
                N, Kd = v.shape
                out[k] = ((q.float().reshape(N, -1, cfg.group_size) - z.float().unsqueeze(-1)) * s.float().unsqueeze(-1)).reshape(N, Kd)
            else:
                out[k] = v.to(torch.bfloat16).float()
        else:
            out[k] = v.to(torch.bfloat16).float()
    return out


def _rms(x, g, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g


def _rope(x, pos, theta):
    T, Hh, D = x.shape
    inv = theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


@torch.no_grad()
def reference_logits(cfg: LlmConfig, state: Dict[str, torch.Tensor], ids: torch.Tensor) -> torch.Tensor:
    """fp32 forward of ONE sequence ``ids`` [S] with full causal attention; returns logits [S, V]."""
    S = ids.numel()
    D, Hq, Hkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    pos = torch.arange(S, device=ids.device)
    h = state["embed_tokens"][ids].float()
    mask = torch.ones(S, S, dtype=torch.bool, device=ids.device).tril()
    if cfg.sliding_window > 0:
        mask &= ~torch.ones(S, S, dtype=torch.bool, device=ids.device).tril(-cfg.sliding_window)
    for l in range(cfg.num_layers):
        p = "layers.%d." % l
        x = _rms(h, state[p + "input_layernorm"], cfg.rms_eps)
        q = _rope((x @ state[p + "q_proj"].t()).reshape(S, Hq, D), pos, cfg.rope_theta)
        k = _rope((x @ state[p + "k_proj"].t()).reshape(S, Hkv, D), pos, cfg.rope_theta)
        v = (x @ state[p + "v_proj"].t()).reshape(S, Hkv, D)
        k = k.repeat_interleave(Hq // Hkv, dim=1)
        v = v.repeat_interleave(Hq // Hkv, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        s = s.masked_fill(~mask[None], float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(S, Hq * D)
        h = h + a @ state[p + "o_proj"].t()
        x = _rms(h, state[p + "post_attention_layernorm"], cfg.rms_eps)
        if cfg.num_experts:
            probs = torch.softmax(x @ state[p + "router"].t(), -1)
            top_v, top_i = probs.topk(cfg.experts_top_k, -1)
            top_v = top_v / top_v.sum(-1, keepdim=True)
            y = torch.zeros_like(h)
            for e in range(cfg.num_experts):
                w_e = (top_v * (top_i == e)).sum(-1, keepdim=True)          # routing weight of expert e per token (0 if not chosen)
                g = torch.nn.functional.silu(x @ state[p + "experts.%d.gate_proj" % e].t()) * (x @ state[p + "experts.%d.up_proj" % e].t())
                y = y + w_e * (g @ state[p + "experts.%d.down_proj" % e].t())
            h = h + y
        else:
            g = torch.nn.functional.silu(x @ state[p + "gate_proj"].t()) * (x @ state[p + "up_proj"].t())
            h = h + g @ state[p + "down_proj"].t()
    return _rms(h, state["norm"], cfg.rms_eps) @ state["lm_head"].t()


@torch.no_grad()
def reference_generate(cfg: LlmConfig, state, prompt: List[int], max_new_tokens: int, device="cpu") -> List[int]:
    ids = list(prompt)
    for _ in range(max_new_tokens):
        logits = reference_logits(cfg, state, torch.tensor(ids, device=device))
        ids.append(int(logits[-1].argmax()))
    return ids[len(prompt):]
