"""NCCL + cuBLAS baseline of the serving benchmark: the same architecture in plain PyTorch.

bf16 weights (library GEMMs have no int4 path), Megatron-style tensor parallelism with ``torch.distributed`` all-reduce
over NCCL after the attention-output and MLP-down projections, ``scaled_dot_product_attention`` for prefill and decode
over a dense (non-paged) KV cache, static batching: all requests are prefilled in chunks, then decoded in lock-step.
None of this framework's kernels, scheduler or executor is on this path: it is the library baseline that the fused
kernels are compared with. Prints the same JSON line as ``bench.py`` with ``"impl": "torch"``.
"""
from __future__ import annotations

import json
import math
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F


class TorchLlama:
    def __init__(self, cfg, dev, rank: int, world: int, seed: int = 0):
        self.cfg, self.dev, self.rank, self.world = cfg, dev, rank, world
        H, D = cfg.hidden_size, cfg.head_dim
        self.hq, self.hkv, self.ffn = cfg.num_heads // world, cfg.num_kv_heads // world, cfg.ffn_size // world
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1000 + rank)
        w = lambda n, k: (torch.randn((n, k), device=dev, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        self.embed = w(cfg.vocab_size, H)
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append(dict(n1=torch.ones(H, device=dev, dtype=torch.bfloat16), qkv=w((self.hq + 2 * self.hkv) * D, H),
                                    o=w(H, self.hq * D), n2=torch.ones(H, device=dev, dtype=torch.bfloat16), gu=w(2 * self.ffn, H),
                                    down=w(H, self.ffn)))
        self.norm = torch.ones(H, device=dev, dtype=torch.bfloat16)
        self.lm_head = w(cfg.vocab_size // world, H)
        inv = cfg.rope_theta ** (-torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D)
        self.inv_freq = inv

    def _rms(self, x, g):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps)).to(x.dtype) * g

    def _rope(self, x, pos):          # x [B, L, H, D], pos [B, L]
        ang = pos.float()[..., None] * self.inv_freq
        cos, sin = ang.cos()[:, :, None, :].to(x.dtype), ang.sin()[:, :, None, :].to(x.dtype)
        d = x.shape[-1] // 2
        x1, x2 = x[..., :d], x[..., d:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    def forward(self, ids, pos, k_cache, v_cache, past: int):
        """ids/pos [B, L]; caches: per layer [B, S_max, Hkv, D]; returns next-token ids [B]."""
        cfg = self.cfg
        B, L = ids.shape
        D = cfg.head_dim
        h = self.embed[ids]
        for l, w in enumerate(self.layers):
            x = self._rms(h, w["n1"])
            qkv = F.linear(x, w["qkv"]).view(B, L, self.hq + 2 * self.hkv, D)
            q = self._rope(qkv[:, :, :self.hq], pos)
            k = self._rope(qkv[:, :, self.hq:self.hq + self.hkv], pos)
            v = qkv[:, :, self.hq + self.hkv:]
            k_cache[l][:, past:past + L] = k
            v_cache[l][:, past:past + L] = v
            kk = k_cache[l][:, :past + L].transpose(1, 2)
            vv = v_cache[l][:, :past + L].transpose(1, 2)
            a = F.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, is_causal=(L > 1 and past == 0), enable_gqa=True,
                                               attn_mask=None if (L == 1 or past == 0) else self._mask(L, past + L))
            o = F.linear(a.transpose(1, 2).reshape(B, L, self.hq * D), w["o"])
            if self.world > 1:
                dist.all_reduce(o)
            h = h + o
            x = self._rms(h, w["n2"])
            gu = F.linear(x, w["gu"])
            d = F.linear(F.silu(gu[..., :self.ffn]) * gu[..., self.ffn:], w["down"])
            if self.world > 1:
                dist.all_reduce(d)
            h = h + d
        x = self._rms(h[:, -1], self.norm)
        logits = F.linear(x, self.lm_head).float()
        val, idx = logits.max(-1)
        if self.world > 1:
            vals = [torch.empty_like(val) for _ in range(self.world)]
            idxs = [torch.empty_like(idx) for _ in range(self.world)]
            dist.all_gather(vals, val)
            dist.all_gather(idxs, idx)
            best = torch.stack(vals).argmax(0)
            idx = torch.stack(idxs).gather(0, best[None])[0] + best * (self.cfg.vocab_size // self.world)
        return idx

    def _mask(self, L, S):
        q = torch.arange(S - L, S, device=self.dev)[:, None]
        k = torch.arange(S, device=self.dev)[None, :]
        return k <= q


def run_torch_baseline(args, rank: int, world: int, dev) -> int:
    from openvino_b200.models.llm_config import NAMED
    cfg = NAMED[args.model]
    if args.layers:
        cfg = cfg.with_(num_layers=args.layers)
    R, P, O = args.requests, args.prompt_len, args.output_len
    model = TorchLlama(cfg, dev, rank, world)
    g = torch.Generator().manual_seed(1234)
    prompts = torch.stack([torch.randint(0, cfg.vocab_size, (P,), generator=g) for _ in range(R)]).to(dev)
    hkv = cfg.num_kv_heads // world
    k_cache = [torch.zeros((R, P + O, hkv, cfg.head_dim), device=dev, dtype=torch.bfloat16) for _ in range(cfg.num_layers)]
    v_cache = [torch.zeros_like(k) for k in k_cache]
    chunk = max(1, 8192 // P)           # requests prefilled together (8192 tokens per step, like the serving engine)

    @torch.no_grad()
    def one_pass():
        nxt = torch.empty(R, dtype=torch.long, device=dev)
        pos = torch.arange(P, device=dev)[None]
        for r0 in range(0, R, chunk):
            sl = slice(r0, min(R, r0 + chunk))
            kc = [k[sl] for k in k_cache]
            vc = [v[sl] for v in v_cache]
            nxt[sl] = model.forward(prompts[sl], pos.expand(sl.stop - sl.start, -1), kc, vc, 0)
        for t in range(1, O):
            p = torch.full((R, 1), P + t - 1, device=dev)
            nxt = model.forward(nxt[:, None], p, k_cache, v_cache, P + t - 1)
        return nxt

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_pass()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        one_pass()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    value = R * O * args.steps / (ms / 1e3)
    if rank == 0:
        print(json.dumps({"impl": "torch", "metric": "output tokens/s", "value": value, "unit": "output tokens/s", "n_gpus": world,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                          "dtype": "bf16 (weights and activations)", "data": "synthetic: uniform random prompt ids, random-init weights",
                          "config": {"model": cfg.name, "global_batch": R, "seq_len": P, "output_len": O, "parallelism": "tp%d" % world,
                                     "stack": "PyTorch eager: cuBLAS GEMMs, SDPA, NCCL all-reduce, dense KV cache, static batching"}}))
    if world > 1:
        dist.destroy_process_group()
    return 0
