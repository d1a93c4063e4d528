"""Decoder-only LLM architecture descriptions used by the model builders, the CUDA plugin and the
benchmarks. The named configurations are the ones of the serving benchmarks (Llama-3-8B,
Llama-3-70B, Mixtral-8x7B); ``tiny`` variants keep tests fast."""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class LlmConfig:
    name: str = "llama"
    vocab_size: int = 128256
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    ffn_size: int = 14336
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    num_experts: int = 0          # 0 = dense FFN
    experts_top_k: int = 2
    weight_format: str = "int4"   # "int4" (u4 asym, group scales + zero points) | "int8" | "bf16" | "fp8"
    group_size: int = 128
    sliding_window: int = 0

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def with_(self, **kw) -> "LlmConfig":
        return replace(self, **kw)


LLAMA3_8B = LlmConfig(name="llama-3-8b")
LLAMA3_70B = LlmConfig(name="llama-3-70b", hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8,
                       ffn_size=28672, weight_format="fp8")
MIXTRAL_8X7B = LlmConfig(name="mixtral-8x7b", vocab_size=32000, hidden_size=4096, num_layers=32, num_heads=32,
                         num_kv_heads=8, ffn_size=14336, rope_theta=1e6, num_experts=8, experts_top_k=2,
                         weight_format="bf16")
TINY_LLAMA = LlmConfig(name="tiny-llama", vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                       head_dim=128, ffn_size=512, group_size=128)
TINY_MOE = LlmConfig(name="tiny-moe", vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                     head_dim=128, ffn_size=256, num_experts=4, experts_top_k=2, weight_format="bf16")

NAMED = {c.name: c for c in (LLAMA3_8B, LLAMA3_70B, MIXTRAL_8X7B, TINY_LLAMA, TINY_MOE)}
