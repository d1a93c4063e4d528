"""Decoder-only LLM program of the CUDA plugin: weights in kernel layout, static step buffers,
the per-layer kernel sequence, CUDA-graph capture of decode steps, tensor-parallel sharding.

The graph form that maps onto this program is the stateless PagedAttention model
(``input_ids, position_ids, past_lens, subsequence_begins, block_indices, block_indices_begins,
max_context_len, key_cache.N, value_cache.N`` inputs; RMS -> FullyConnectedCompressed(QKV) -> RoPE ->
PagedAttentionExtension -> FullyConnectedCompressed(O) -> RMS -> gate/up -> SwiGLU -> down per layer)
produced by SDPAToPagedAttention (src/core/src/pass/sdpa_to_paged_attention.cpp) plus the LLM fusions
(rms_fusion.cpp, fuse_rotary_positional_embeddings.cpp, convert_fc_to_compressed.cpp).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..models.llm_config import LlmConfig
from ..ops import cuda as K
from ..utils import quant


# ----------------------------------------------------------------------------------------- weights
@dataclass
class LayerWeights:
    norm1: torch.Tensor
    qkv: K.PackedWeight
    o: K.PackedWeight
    norm2: torch.Tensor
    gate_up: Optional[K.PackedWeight] = None
    down: Optional[K.PackedWeight] = None
    # MoE: router [E, H]; gate_up / down hold the rank's local experts stacked ([nloc * 2F, H] and [H, nloc * F])
    router: Optional[K.PackedWeight] = None


@dataclass
class LlmWeights:
    embed: torch.Tensor
    layers: List[LayerWeights]
    final_norm: torch.Tensor
    lm_head: K.PackedWeight
    tp_rank: int = 0
    tp_size: int = 1

    @staticmethod
    def _pack(w: torch.Tensor, cfg: LlmConfig) -> K.PackedWeight:
        """Float [N, K] -> kernel layout according to cfg.weight_format (quantising when asked)."""
        N, Kd = w.shape
        if cfg.weight_format == "int4":
            q, s, z = quant.quantize_u4_asym(w, cfg.group_size)
            return K.PackedWeight.from_ir_u4(quant.pack_u4(q), s, quant.pack_u4(z), N, Kd, cfg.group_size)
        if cfg.weight_format == "int8":
            q, s, z = quant.quantize_u8_asym(w, cfg.group_size)
            return K.PackedWeight.from_ir_u8(q, s, z, N, Kd, cfg.group_size)
        if cfg.weight_format == "fp8" and Kd % 128 == 0:
            q, s = quant.quantize_f8_block(w, 128)
            return K.PackedWeight.from_f8_block(q, s, N, Kd, 128)
        return K.PackedWeight.from_dense(w.to(torch.bfloat16))

    @staticmethod
    def _random_packed(N: int, Kd: int, cfg: LlmConfig, device, seed: int) -> K.PackedWeight:
        if cfg.weight_format == "int4":
            packed, s, z = quant.random_u4_weight(N, Kd, cfg.group_size, device, seed=seed)
            return K.PackedWeight.from_ir_u4(packed, s, quant.pack_u4(z), N, Kd, cfg.group_size)
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        if cfg.weight_format == "fp8" and Kd % 128 == 0:
            # random e4m3 bytes (NaN encodings excluded) with one scale per 128 x 128 tile, values of a few hundredths
            b = torch.randint(0, 256, (N, Kd), device=device, generator=g, dtype=torch.int32)
            mag = torch.clamp(b & 0x7F, max=0x5E)                    # |value| <= 28
            w8 = ((b & 0x80) | mag).to(torch.uint8)
            scales = torch.full(((N + 127) // 128, Kd // 128), 2.0 ** -9, dtype=torch.float32, device=device)
            return K.PackedWeight.from_f8_block(w8, scales, N, Kd, 128)
        w = (torch.randn((N, Kd), device=device, generator=g, dtype=torch.float32) * 0.02)
        if cfg.weight_format == "int8":
            q, s, z = quant.quantize_u8_asym(w, cfg.group_size)
            return K.PackedWeight.from_ir_u8(q, s, z, N, Kd, cfg.group_size)
        return K.PackedWeight.from_dense(w.to(torch.bfloat16))

    @staticmethod
    def random(cfg: LlmConfig, device, seed: int = 0, tp_rank: int = 0, tp_size: int = 1) -> "LlmWeights":
        """Random-init weights generated shard by shard directly in kernel layout (no float copy of the
        full model is ever materialised). Different ranks draw different shards."""
        H, D = cfg.hidden_size, cfg.head_dim
        hq, hkv, ffn = cfg.num_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.ffn_size // tp_size
        assert cfg.num_heads % tp_size == 0 and cfg.num_kv_heads % tp_size == 0 and cfg.ffn_size % tp_size == 0
        vshard = cfg.vocab_size // tp_size
        assert cfg.vocab_size % tp_size == 0
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        embed = (torch.randn((cfg.vocab_size, H), device=device, generator=g) * 0.02).to(torch.bfloat16)
        ones = lambda: torch.ones(H, device=device, dtype=torch.bfloat16)
        layers = []
        for l in range(cfg.num_layers):
            s = seed * 100003 + l * 97 + tp_rank * 13
            lw = LayerWeights(
                norm1=ones(),
                qkv=LlmWeights._random_packed((hq + 2 * hkv) * D, H, cfg, device, s + 1),
                o=LlmWeights._random_packed(H, hq * D, cfg, device, s + 2),
                norm2=ones())
            if cfg.num_experts == 0:
                lw.gate_up = LlmWeights._random_packed(2 * ffn, H, cfg, device, s + 3)
                lw.gate_up.swiglu = ffn % 64 == 0 and lw.gate_up.bias is None     # random rows: any row order is a valid interleaving
                lw.down = LlmWeights._random_packed(H, ffn, cfg, device, s + 4)
            else:
                # expert parallel: a rank holds whole experts (nloc of them), attention stays tensor parallel
                assert cfg.num_experts % tp_size == 0, "the number of experts must be a multiple of the number of ranks"
                nloc = cfg.num_experts // tp_size
                gr = torch.Generator(device=device)
                gr.manual_seed(seed * 100003 + l * 97 + 5)       # the router is replicated: same seed on every rank
                router = (torch.randn((cfg.num_experts, H), device=device, generator=gr) * 0.02).to(torch.bfloat16)
                lw.router = K.PackedWeight.from_dense(router)
                lw.gate_up = LlmWeights._random_packed(nloc * 2 * cfg.ffn_size, H, cfg, device, s + 3)
                lw.down = LlmWeights._random_packed(H, nloc * cfg.ffn_size, cfg, device, s + 4)
            layers.append(lw)
        lm_head = LlmWeights._random_packed(vshard, H, cfg, device, seed * 100003 + 7 + tp_rank)
        return LlmWeights(embed, layers, ones(), lm_head, tp_rank, tp_size)

    @staticmethod
    def from_float(cfg: LlmConfig, state: dict, device, tp_rank: int = 0, tp_size: int = 1) -> "LlmWeights":
        """state: float tensors keyed like HF Llama (``layers.{i}.q_proj`` [N, K] ...), see
        models.llama.random_float_state. Shards for tensor parallelism and packs/quantises."""
        H, D = cfg.hidden_size, cfg.head_dim
        hq, hkv, ffn = cfg.num_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.ffn_size // tp_size
        r = tp_rank
        dev = lambda t: t.to(device)
        layers = []
        for l in range(cfg.num_layers):
            p = "layers.%d." % l
            q = state[p + "q_proj"][r * hq * D:(r + 1) * hq * D]
            k = state[p + "k_proj"][r * hkv * D:(r + 1) * hkv * D]
            v = state[p + "v_proj"][r * hkv * D:(r + 1) * hkv * D]
            o = state[p + "o_proj"][:, r * hq * D:(r + 1) * hq * D]
            router = None
            if cfg.num_experts:
                nloc = cfg.num_experts // tp_size
                local = range(r * nloc, (r + 1) * nloc)
                gu = torch.cat([torch.cat([state[p + "experts.%d.gate_proj" % e], state[p + "experts.%d.up_proj" % e]], 0) for e in local], 0)
                down = torch.cat([state[p + "experts.%d.down_proj" % e] for e in local], 1)
                gate, up = gu, gu[:0]
                router = K.PackedWeight.from_dense(dev(state[p + "router"]).to(torch.bfloat16).contiguous())
            else:
                gate = state[p + "gate_proj"][r * ffn:(r + 1) * ffn]
                up = state[p + "up_proj"][r * ffn:(r + 1) * ffn]
                down = state[p + "down_proj"][:, r * ffn:(r + 1) * ffn]
            fused_gate = cfg.num_experts == 0 and ffn % 64 == 0
            if fused_gate:          # row order of the GEMM's fused SwiGLU epilogue
                gate, up = K.interleave_gate_up(gate, up), gate[:0]
            layers.append(LayerWeights(router=router,
                norm1=dev(state[p + "input_layernorm"]).to(torch.bfloat16),
                qkv=LlmWeights._pack(dev(torch.cat([q, k, v], 0)).contiguous(), cfg),
                o=LlmWeights._pack(dev(o).contiguous(), cfg),
                norm2=dev(state[p + "post_attention_layernorm"]).to(torch.bfloat16),
                gate_up=LlmWeights._pack(dev(torch.cat([gate, up], 0)).contiguous(), cfg),
                down=LlmWeights._pack(dev(down).contiguous(), cfg)))
            layers[-1].gate_up.swiglu = fused_gate
        vshard = cfg.vocab_size // tp_size
        lm = state["lm_head"][r * vshard:(r + 1) * vshard]
        return LlmWeights(dev(state["embed_tokens"]).to(torch.bfloat16), layers, dev(state["norm"]).to(torch.bfloat16),
                          LlmWeights._pack(dev(lm).contiguous(), cfg), tp_rank, tp_size)


# ----------------------------------------------------------------------------------------- step buffers
# Batches of at least this many tokens gather the tokens of every expert instead of running every expert on every token.
MOE_GATHER_MIN_TOKENS = 1024


class StepBuffers:
    """Static device buffers of one shape bucket: the packed int32 step descriptor plus activations.

    Descriptor layout (int32 words): ids[Tcap] positions[Tcap] slot_map[Tcap] tok_src[Tcap] tok_dst[Bcap] logit_idx[Bcap]
    past_lens[Bcap] subsequence_begins[Bcap+1] block_indices_begins[Bcap+1] block_indices[Bcap*max_blocks].
    The host fills a pinned mirror and uploads it with ONE copy per step.
    """

    def __init__(self, cfg: LlmConfig, Tcap: int, Bcap: int, max_blocks_per_seq: int, device, tp_size: int = 1, comm=None):
        self.Tcap, self.Bcap, self.max_blocks = Tcap, Bcap, max_blocks_per_seq
        sizes = [("ids", Tcap), ("positions", Tcap), ("slot_map", Tcap), ("tok_src", Tcap), ("tok_dst", Bcap),
                 ("logit_idx", Bcap), ("past_lens", Bcap),
                 ("subsequence_begins", Bcap + 1), ("block_indices_begins", Bcap + 1),
                 ("block_indices", Bcap * max_blocks_per_seq)]
        self.offsets, off = {}, 0
        for name, n in sizes:
            self.offsets[name] = (off, n)
            off += (n + 3) // 4 * 4   # keep every field 16-byte aligned
        self.desc_words = off
        self.desc = torch.zeros(off, dtype=torch.int32, device=device)
        pin = (lambda t: t.pin_memory()) if torch.cuda.is_available() else (lambda t: t)
        # two pinned mirrors: the host fills one while the upload of the other may still be in flight
        self.desc_hosts = [pin(torch.zeros(off, dtype=torch.int32)) for _ in range(2)]
        H, D = cfg.hidden_size, cfg.head_dim
        hq, hkv, ffn = cfg.num_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.ffn_size // tp_size
        bf = dict(dtype=torch.bfloat16, device=device)
        # with tensor parallelism the residual stream lives in the communicator's symmetric heap: peers write into it
        self.h = comm.alloc((Tcap, H)) if comm is not None else torch.empty((Tcap, H), **bf)
        self.x = torch.empty((Tcap, H), **bf)
        self.qkv = torch.empty((Tcap, (hq + 2 * hkv) * D), **bf)
        self.attn = torch.empty((Tcap, hq * D), **bf)
        if cfg.num_experts:
            nloc = cfg.num_experts // tp_size
            self.gu = torch.empty((Tcap, nloc * 2 * cfg.ffn_size), **bf)
            self.act = torch.empty((Tcap, nloc * cfg.ffn_size), **bf)
            self.router_logits = torch.empty((Tcap, cfg.num_experts), dtype=torch.float32, device=device)
            self.route = torch.empty((Tcap, cfg.num_experts), dtype=torch.float32, device=device)
            # prefill-sized batches run every expert on its own tokens only (rows sorted by expert); see _moe_gathered
            self.moe_gather = Tcap >= MOE_GATHER_MIN_TOKENS
            if self.moe_gather:
                cap = Tcap * min(cfg.experts_top_k, nloc)          # every token in each of its local experts, at most
                self.xg = torch.empty((cap, H), **bf)
                self.gug = torch.empty((cap, 2 * cfg.ffn_size), **bf)
                self.actg = torch.empty((cap, cfg.ffn_size), **bf)
                self.outg = torch.empty((cap, H), **bf)
                # expert parallel: the local experts' contributions are summed over the ranks (symmetric heap)
                self.moe_out = comm.alloc((Tcap, H)) if comm is not None else None
                self.moe_pos = torch.zeros((Tcap, nloc), dtype=torch.int32, device=device)
                self.moe_counts = torch.zeros(nloc, dtype=torch.int32, device=device)
                self.moe_offsets = torch.zeros(nloc + 1, dtype=torch.int32, device=device)
        else:
            self.gu = torch.empty((Tcap, 2 * ffn), **bf)
            self.act = torch.empty((Tcap, ffn), **bf)
        self.last_h = torch.empty((Bcap, H), **bf)
        self.last_x = torch.empty((Bcap, H), **bf)
        self.logits = torch.empty((Bcap, cfg.vocab_size // tp_size), **bf)
        self.tokens = torch.zeros(Bcap, dtype=torch.int32, device=device)
        self.tokens_host = [pin(torch.zeros(Bcap, dtype=torch.int32)) for _ in range(2)]
        self.logit_max = torch.empty(Bcap, dtype=torch.float32, device=device)

    def view(self, name: str, host=None) -> torch.Tensor:
        """Field of the device descriptor (host=None) or of pinned mirror ``host`` (0 or 1)."""
        off, n = self.offsets[name]
        return (self.desc if host is None else self.desc_hosts[int(host)])[off:off + n]


@dataclass
class StepShape:
    T: int            # tokens in the step
    B: int            # sequences in the step
    max_q_len: int    # longest sub-sequence (1 = pure decode)
    max_ctx: int      # longest context after this step


# ----------------------------------------------------------------------------------------- executor
class CudaLlmExecutor:
    """Runs steps of a decoder-only model on one GPU (one tensor-parallel rank)."""

    def __init__(self, cfg: LlmConfig, weights: LlmWeights, num_kv_blocks: int, block_size: int = 16,
                 max_batch_tokens: int = 8192, max_seqs: int = 64, max_blocks_per_seq: int = 0, device="cuda",
                 comm=None, use_cuda_graphs: bool = True, kv_cache_precision: str = "bf16"):
        self.cfg, self.w = cfg, weights
        self.kv_u8 = str(kv_cache_precision).lower() == "u8"
        if self.kv_u8 and (cfg.head_dim != 128 or block_size != 16):
            raise ValueError("the u8 KV cache is served for head size 128 and 16-token blocks")
        self.device = torch.device(device)
        self.block_size = block_size
        self.num_kv_blocks = num_kv_blocks
        self.tp_size, self.tp_rank = weights.tp_size, weights.tp_rank
        self.comm = comm
        self.use_cuda_graphs = use_cuda_graphs
        self.hq = cfg.num_heads // self.tp_size
        self.hkv = cfg.num_kv_heads // self.tp_size
        self.max_seqs = max_seqs
        if max_blocks_per_seq <= 0:
            max_blocks_per_seq = max(1, num_kv_blocks // max(1, max_seqs)) + 1
        self.max_blocks_per_seq = max_blocks_per_seq
        # KV_CACHE_PRECISION = u8: rows are stored as bytes with one fp16 (scale, zero point) pair per (block, head, slot):
        # half the cache memory and half the decode traffic of the 16-bit cache
        self.k_cache = [torch.zeros((num_kv_blocks, self.hkv, block_size, cfg.head_dim), dtype=torch.uint8 if self.kv_u8 else torch.bfloat16,
                                    device=self.device) for _ in range(cfg.num_layers)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        self.k_meta = [torch.zeros((num_kv_blocks, self.hkv, block_size, 2), dtype=torch.float16, device=self.device) if self.kv_u8 else None
                       for _ in range(cfg.num_layers)]
        self.v_meta = [torch.zeros_like(m) if m is not None else None for m in self.k_meta]
        self.ws = K.Workspace(self.device)
        if self.tp_size > 1:
            if comm is None:
                raise ValueError("tensor-parallel weights need a communicator")
            moe_rows = max_batch_tokens + 1 if (cfg.num_experts and max_batch_tokens >= MOE_GATHER_MIN_TOKENS) else 0
            comm.setup(cfg.hidden_size, max_batch_tokens, cfg.num_layers,
                       tensor_bytes=(max_batch_tokens + max_seqs + 2 + moe_rows) * cfg.hidden_size * 2 + 8192
                       + max_seqs * cfg.vocab_size * 2 + 4096)
        self.prefill = StepBuffers(cfg, max_batch_tokens, max_seqs, max_blocks_per_seq, self.device, self.tp_size, comm if self.tp_size > 1 else None)
        self.decode = StepBuffers(cfg, max_seqs, max_seqs, max_blocks_per_seq, self.device, self.tp_size, comm if self.tp_size > 1 else None)
        # top-k / top-p under tensor parallelism need the whole row: every rank places its vocabulary shard into a zeroed
        # full-width buffer in the symmetric heap and the ranks sum the buffers (adding zeros is exact in bf16)
        self.full_logits = comm.alloc((max(max_seqs, 1), cfg.vocab_size)) if self.tp_size > 1 else None
        # token sampled last for every request slot (device-side feedback between chained steps)
        self.last_token = torch.zeros(max(max_seqs, 1) * 4, dtype=torch.int32, device=self.device)
        self._graphs = {}
        self._expert_windows = {}
        self.kernel_launches = 0
        # sampling: None = greedy; (temperature, top_k, top_p, seed) = stochastic. The step word is
        # bumped on the device before every draw, so replays of a captured decode graph keep drawing fresh numbers.
        self.sampling = None
        self.sample_step = torch.zeros(1, dtype=torch.int32, device=self.device)

    def set_sampling(self, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> None:
        new = None if temperature <= 0 else (float(temperature), int(top_k), float(top_p), int(seed))
        if new is not None and self.tp_size > 1 and (top_k > 0 or top_p < 1.0) and self.cfg.vocab_size % 8:
            raise NotImplementedError("top-k / top-p with tensor parallelism gathers the logits in 16-byte pieces: the vocabulary "
                                      "size must be a multiple of 8")
        if new != self.sampling:
            self._graphs.clear()       # captured decode graphs embed the sampling kernel
        self.sampling = new

    # -- one forward pass over the buffers of `sb`
    def _forward(self, sb: StepBuffers, shp: StepShape) -> None:
        cfg, w, ws = self.cfg, self.w, self.ws
        T, B = shp.T, shp.B
        D = cfg.head_dim
        ids = sb.view("ids")[:T]
        positions, slot_map = sb.view("positions"), sb.view("slot_map")
        h, x, qkv, attn, gu, act = sb.h[:T], sb.x[:T], sb.qkv[:T], sb.attn[:T], sb.gu[:T], sb.act[:T]
        n = 3
        if self.tp_size > 1:
            self.comm.step_begin()
            n += 1
        K.resolve_ids(ids, sb.view("tok_src")[:T], self.last_token)
        K.embedding(ids, w.embed, out=h)
        for l, lw in enumerate(w.layers):
            K.rmsnorm(h, lw.norm1, cfg.rms_eps, out=x)
            K.gemm(x, lw.qkv, out=qkv, ws=ws)
            if self.kv_u8:
                K.rope_kv_write_u8(qkv, positions, slot_map, self.k_cache[l], self.v_cache[l], self.k_meta[l], self.v_meta[l], self.hq, self.hkv, D,
                                   cfg.rope_theta, self.block_size)
            else:
                K.rope_kv_write(qkv, positions, slot_map, self.k_cache[l], self.v_cache[l], self.hq, self.hkv, D,
                                cfg.rope_theta, self.block_size)
            K.paged_attention(qkv, self.k_cache[l], self.v_cache[l], sb.view("past_lens")[:B],
                              sb.view("subsequence_begins")[:B + 1], sb.view("block_indices"),
                              sb.view("block_indices_begins")[:B + 1], self.hq, self.hkv, D,
                              max_context_len=shp.max_ctx, max_q_len=shp.max_q_len, sliding_window=cfg.sliding_window,
                              block_size=self.block_size, out=attn, ws=ws, k_meta=self.k_meta[l], v_meta=self.v_meta[l])
            self._row_parallel(attn, lw.o, h, 2 * l)
            K.rmsnorm(h, lw.norm2, cfg.rms_eps, out=x)
            if cfg.num_experts:
                # every rank holds all tokens (the residual stream is replicated), so "dispatch" is free: a rank runs its
                # experts on the tokens routed to them (others contribute zeros) and the row-parallel down projection
                # with its fused all-reduce is the "combine"
                nloc = cfg.num_experts // self.tp_size
                K.gemm(x, lw.router, out=sb.router_logits[:T], out_f32=True, ws=ws)
                K.moe_route_topk(sb.router_logits[:T], cfg.experts_top_k, out=sb.route[:T])
                if (getattr(sb, "moe_gather", False) and T >= MOE_GATHER_MIN_TOKENS and shp.max_q_len > 1
                        and lw.down.mode == lw.gate_up.mode
                        and (lw.gate_up.mode == K.W_U4 or (lw.gate_up.mode == K.W_BF16 and lw.gate_up.tiled and lw.down.tiled))):
                    n += self._moe_gathered(sb, l, T, x, h)
                    n += 7
                    continue
                K.gemm(x, lw.gate_up, out=gu, ws=ws)
                K.moe_silu_mul_scale(gu, sb.route[:T], cfg.ffn_size, nloc, self.tp_rank * nloc, out=act)
                n += 2
            elif getattr(lw.gate_up, "swiglu", False):
                K.gemm(x, lw.gate_up, out=act, act=K.ACT_SWIGLU, ws=ws)       # silu(gate) * up in the GEMM epilogue
                n -= 1
            else:
                K.gemm(x, lw.gate_up, out=gu, ws=ws)
                K.silu_mul(gu, out=act)
            self._row_parallel(act, lw.down, h, 2 * l + 1)
            n += 9
        # logits only for the last token of every sequence
        last_h, last_x = sb.last_h[:B], sb.last_x[:B]
        K.embedding(sb.view("logit_idx")[:B], h, out=last_h)
        K.rmsnorm(last_h, w.final_norm, cfg.rms_eps, out=last_x)
        logits = sb.logits[:B]
        K.gemm(last_x, w.lm_head, out=logits, ws=ws)
        self._sample(sb, B)
        self.kernel_launches += n + 5

    def _moe_gathered(self, sb: StepBuffers, l: int, T: int, x: torch.Tensor, h: torch.Tensor) -> int:
        """Experts on their own tokens only (prefill-sized batches), without a host round trip: the position of every
        routed token inside its experts' row lists and the experts' row offsets are computed on the device, the rows are
        gathered sorted by expert, ONE grouped GEMM per projection runs every expert on its rows of the stacked weights
        (the offsets are read by the kernel), and the weighted results are combined per token in expert order. Top-2 of 8
        experts does a quarter of the dense-masked work. Returns the number of kernel launches."""
        cfg = self.cfg
        lw = self.w.layers[l]
        nloc = cfg.num_experts // self.tp_size
        e0 = self.tp_rank * nloc
        rows = T * min(cfg.experts_top_k, nloc)
        route = sb.route[:T]
        xg, gug, actg, outg = sb.xg[:rows], sb.gug[:rows], sb.actg[:rows], sb.outg[:rows]
        # row tiles sized for the expected rows per expert (a group ends with a partial tile)
        bt = K.pick_block_t(max(1, rows // nloc))
        K.moe_positions(route, e0, nloc, sb.moe_pos, sb.moe_counts)
        K.moe_gather_sorted(x, sb.moe_pos, sb.moe_counts, sb.moe_offsets, xg)
        K.gemm_grouped(xg, lw.gate_up, sb.moe_offsets, nloc, 1, out=gug, ws=self.ws, block_t=bt)
        K.silu_mul(gug, out=actg, nrows=sb.moe_offsets[nloc:])
        K.gemm_grouped(actg, lw.down, sb.moe_offsets, nloc, 2, out=outg, ws=self.ws, block_t=bt)
        launches = 6
        if self.tp_size > 1:
            # expert parallel: every rank combines its experts' results, the buffers are summed over the ranks
            dst = sb.moe_out[:T]
            K.moe_combine_sorted(outg, route, sb.moe_pos, sb.moe_offsets, dst, e0, accumulate=False)
            launches += self.comm.all_reduce_large(dst)
            K.add(h, dst, out=h)
            launches += 1
        else:
            K.moe_combine_sorted(outg, route, sb.moe_pos, sb.moe_offsets, h, e0, accumulate=True)
        return launches

    def _row_parallel(self, x: torch.Tensor, wt: K.PackedWeight, h: torch.Tensor, site: int) -> None:
        """h += x @ W^T summed over tensor-parallel ranks (h is the replicated residual stream)."""
        if self.tp_size == 1:
            K.gemm(x, wt, out=h, residual=h, ws=self.ws)
        else:
            self.comm.gemm_allreduce(x, wt, h, self.ws, site)

    def _sample(self, sb: StepBuffers, B: int) -> None:
        if self.sampling is not None:
            temp, top_k, top_p, seed = self.sampling
            K.bump(self.sample_step)
            if self.tp_size > 1 and (top_k > 0 or top_p < 1.0):
                # truncated sampling needs the whole row: gather the shards (sum of zero-padded rows over the ranks), then
                # every rank runs the same draw with the same seed and step, so all ranks get the same tokens
                shard = self.cfg.vocab_size // self.tp_size
                full = self.full_logits[:B]
                full.zero_()
                full[:, self.w.tp_rank * shard:(self.w.tp_rank + 1) * shard].copy_(sb.logits[:B])
                self.kernel_launches += 2 + self.comm.all_reduce_large(full)
                K.sample(full, temp, top_k, top_p, seed, self.sample_step, out=sb.tokens[:B])
            elif self.tp_size > 1:
                # every rank perturbs its vocabulary shard with noise that depends on the global token index, then the
                # ranks exchange (best value, index): a draw from the full softmax without gathering the logits
                shard = self.cfg.vocab_size // self.tp_size
                K.sample_gumbel(sb.logits[:B], temp, seed, self.sample_step, vocab_offset=self.w.tp_rank * shard, out=sb.tokens[:B],
                                out_max=sb.logit_max[:B])
                self.comm.argmax_combine(sb.tokens[:B], sb.logit_max[:B], shard)
            else:
                K.sample(sb.logits[:B], temp, top_k, top_p, seed, self.sample_step, out=sb.tokens[:B])
            self.kernel_launches += 1
        elif self.tp_size == 1:
            K.argmax(sb.logits[:B], out=sb.tokens[:B])
        else:
            K.argmax(sb.logits[:B], out=sb.tokens[:B], out_max=sb.logit_max[:B])
            self.comm.argmax_combine(sb.tokens[:B], sb.logit_max[:B], self.cfg.vocab_size // self.tp_size)
        K.scatter_tokens(sb.tokens[:B], sb.view("tok_dst")[:B], self.last_token)

    # -- public: run one step whose descriptor already sits in sb.desc (device)
    def run(self, sb: StepBuffers, shp: StepShape) -> torch.Tensor:
        decode = sb is self.decode and shp.max_q_len == 1
        if decode and self.use_cuda_graphs:
            ctx_bucket = max(256, 1 << (max(1, shp.max_ctx) - 1).bit_length())
            key = (shp.B, ctx_bucket)
            g = self._graphs.get(key)
            if g is None:
                g = self._capture(sb, StepShape(shp.T, shp.B, 1, ctx_bucket))
                self._graphs[key] = g
            g.replay()
            self.kernel_launches += self._graph_launches
        else:
            self._forward(sb, shp)
        return sb.tokens[:shp.B]

    def _capture(self, sb: StepBuffers, shp: StepShape):
        # warm-up outside capture (first-use setup such as function attributes), then capture
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        saved, saved_last = sb.desc.clone(), self.last_token.clone()
        with torch.cuda.stream(s):
            self._forward(sb, shp)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        # undo the warm-up's side effects on the feedback state; the KV rows it wrote are rewritten with
        # the same values by the real step
        sb.desc.copy_(saved)
        self.last_token.copy_(saved_last)
        before = self.kernel_launches
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._forward(sb, shp)
        self._graph_launches = self.kernel_launches - before
        self.kernel_launches = before
        return g

    # -- host side helpers -------------------------------------------------------------------
    def upload(self, sb: StepBuffers, mirror: int = 0) -> int:
        """One H2D copy of a pinned descriptor mirror. Returns bytes copied."""
        sb.desc.copy_(sb.desc_hosts[mirror], non_blocking=True)
        return sb.desc_words * 4

    def download_tokens_async(self, sb: StepBuffers, B: int, mirror: int = 0) -> "torch.cuda.Event":
        """Queue the D2H copy of the sampled tokens into pinned buffer ``mirror``; the returned event
        completes when the values are readable on the host."""
        sb.tokens_host[mirror][:B].copy_(sb.tokens[:B], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return ev

    def download_tokens(self, sb: StepBuffers, B: int, mirror: int = 0) -> torch.Tensor:
        self.download_tokens_async(sb, B, mirror).synchronize()
        return sb.tokens_host[mirror][:B]

    def kv_cache_bytes(self) -> int:
        return sum(2 * k.numel() * k.element_size() + (2 * m.numel() * 2 if m is not None else 0) for k, m in zip(self.k_cache, self.k_meta))
