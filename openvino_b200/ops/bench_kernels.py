"""Kernel micro-benchmarks with roofline fractions: ``python -m openvino_b200.ops.bench_kernels <kernel> [options]``.

Kernels: ``gemm`` (tcgen05 GEMM, bf16 or int4/int8 weights; ``--cublas`` adds the library GEMM for comparison),
``attention`` (paged decode or prefill), ``rmsnorm``, ``rope`` (RoPE + KV-cache write), ``silu`` (SwiGLU gate),
``sample`` (top-k / top-p and perturbed arg-max), ``conv`` (im2col + GEMM). Every timed launch is preceded by an L2 flush (a 256 MB read),
timed with CUDA events on the launching stream after warm-up; the median is reported together with achieved
bandwidth / throughput and, when ``MEASURED_PEAKS.json`` sits in the working directory, the fraction of the measured
peaks. ``--iters`` small (3-5) gives a run suited to a profiler capture.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def _peaks():
    for path in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")):
        if os.path.exists(path):
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": d.get("hbm_gbs"), "bf16_tflops": d.get("bf16_tflops"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timeit(fn, iters: int, warmup: int) -> float:
    """Median device time of ``fn`` in ms. The whole sequence (L2 flush, event, launch, event) x iters is queued without
    host synchronisation in between, so the GPU never waits for the host and an interval holds kernel time only."""
    # the flush READS 256 MB: the L2 ends up full of clean lines of another buffer (a flush that writes leaves dirty
    # lines whose write-back would be charged to the kernel under test)
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    events = []
    for _ in range(iters):
        flush.sum()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        events.append((s, e))
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in events)
    return times[len(times) // 2]


def bench_gemm(a) -> dict:
    from . import cuda as K
    from ..utils import quant
    T, N, Kd = a.T, a.N, a.K
    x = torch.randn(T, Kd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    if a.wmode == "bf16":
        w = (torch.randn(N, Kd, device="cuda") * 0.02).to(torch.bfloat16)
        pw = K.PackedWeight.from_dense(w)
        wbytes = N * Kd * 2
    else:
        packed, s, z = quant.random_u4_weight(N, Kd, a.group, "cuda")
        pw = K.PackedWeight.from_ir_u4(packed, s, quant.pack_u4(z), N, Kd, a.group)
        wbytes = N * Kd // 2 + (N * Kd // a.group) * 4
    ms = timeit(lambda: K.gemm(x, pw, out=out, block_t=a.block_t), a.iters, a.warmup)
    K.check_status("gemm")
    flops = 2.0 * T * N * Kd
    bytes_ = wbytes + T * Kd * 2 + T * N * 2
    r = {"kernel": "gemm_%s" % a.wmode, "T": T, "N": N, "K": Kd, "ms": ms, "tflops": flops / ms / 1e9, "gbs": bytes_ / ms / 1e6}
    if a.cublas:
        w16 = (torch.randn(N, Kd, device="cuda") * 0.02).to(torch.bfloat16)
        r["cublas_bf16_ms"] = timeit(lambda: torch.matmul(x, w16.t(), out=out), a.iters, a.warmup)
    return r


def bench_attention(a) -> dict:
    from . import cuda as K
    B, Hq, Hkv, D, bs = a.B, a.Hq, a.Hkv, 128, 16
    ctx, q_len = a.ctx, a.q_len
    nblk = (ctx + bs - 1) // bs
    total = B * nblk
    kc = torch.randn(total, Hkv, bs, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(total, Hkv, bs, D, device="cuda").to(torch.bfloat16)
    T = B * q_len
    q = torch.randn(T, Hq * D, device="cuda").to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    past, sb = i32([ctx - q_len] * B), i32([i * q_len for i in range(B + 1)])
    bi, bib = torch.randperm(total).to(torch.int32).cuda(), i32([i * nblk for i in range(B + 1)])
    out = torch.empty(T, Hq * D, device="cuda", dtype=torch.bfloat16)
    km = vm = None
    kv_elem = 2.0
    if getattr(a, "kv_u8", False):          # byte cache with one fp16 (scale, zero point) pair per (block, head, slot)
        kc = torch.randint(0, 256, (total, Hkv, bs, D), device="cuda", dtype=torch.uint8)
        vc = torch.randint(0, 256, (total, Hkv, bs, D), device="cuda", dtype=torch.uint8)
        km = torch.stack([torch.full((total, Hkv, bs), 0.02, device="cuda"), torch.full((total, Hkv, bs), 128.0, device="cuda")], -1).to(torch.float16)
        vm = km.clone()
        kv_elem = 1.0 + 4.0 / D
    ms = timeit(lambda: K.paged_attention(q, kc, vc, past, sb, bi, bib, Hq, Hkv, D, max_context_len=ctx, max_q_len=q_len, out=out, k_meta=km, v_meta=vm),
                a.iters, a.warmup)
    K.check_status("attention")
    kv_bytes = 2 * B * ctx * Hkv * D * kv_elem
    flops = 4.0 * B * Hq * D * (q_len * (ctx - q_len) + q_len * (q_len + 1) / 2)
    return {"kernel": "paged_attention" + (" (u8 cache)" if km is not None else ""), "B": B, "ctx": ctx, "q_len": q_len, "Hq": Hq, "Hkv": Hkv, "ms": ms, "gbs": (kv_bytes + 2 * T * Hq * D * 2) / ms / 1e6,
            "tflops": flops / ms / 1e9}


def bench_rmsnorm(a) -> dict:
    from . import cuda as K
    x = torch.randn(a.T, a.N, device="cuda").to(torch.bfloat16)
    g = torch.ones(a.N, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    ms = timeit(lambda: K.rmsnorm(x, g, 1e-5, out=out), a.iters, a.warmup)
    return {"kernel": "rmsnorm", "rows": a.T, "cols": a.N, "ms": ms, "gbs": 2 * x.numel() * 2 / ms / 1e6}


def bench_rope(a) -> dict:
    """RoPE of q/k in place + write of k/v into the paged cache for T tokens (Llama-3-8B head layout by default)."""
    from . import cuda as K
    T, Hq, Hkv, D, bs = a.T, a.Hq, a.Hkv, 128, 16
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    nblk = (T + bs - 1) // bs + 1
    kc = torch.zeros(nblk, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    pos = torch.arange(T, dtype=torch.int32, device="cuda") + 1000
    slots = torch.arange(T, dtype=torch.int32, device="cuda")
    ms = timeit(lambda: K.rope_kv_write(qkv, pos, slots, kc, vc, Hq, Hkv, D, 500000.0, bs), a.iters, a.warmup)
    bytes_ = T * (Hq + Hkv) * D * 2 * 2 + T * Hkv * D * 2 * 2          # q, k read + written; v read + written
    return {"kernel": "rope_kv_write", "T": T, "Hq": Hq, "Hkv": Hkv, "ms": ms, "gbs": bytes_ / ms / 1e6}


def bench_silu(a) -> dict:
    from . import cuda as K
    gu = torch.randn(a.T, 2 * a.N, device="cuda").to(torch.bfloat16)
    out = torch.empty(a.T, a.N, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: K.silu_mul(gu, out=out), a.iters, a.warmup)
    return {"kernel": "silu_mul", "rows": a.T, "F": a.N, "ms": ms, "gbs": 3 * a.T * a.N * 2 / ms / 1e6}


def bench_sample(a) -> dict:
    from . import cuda as K
    logits = (torch.randn(a.T, a.N, device="cuda") * 3).to(torch.bfloat16)
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(a.T, dtype=torch.int32, device="cuda")
    ms = timeit(lambda: K.sample(logits, 0.8, 50, 0.9, 1, step, out=out), a.iters, a.warmup)
    ms_g = timeit(lambda: K.sample_gumbel(logits, 0.8, 1, step, out=out), a.iters, a.warmup)
    return {"kernel": "sample(top-k 50, top-p 0.9)", "rows": a.T, "vocab": a.N, "ms": ms, "gbs": a.T * a.N * 2 / ms / 1e6, "gumbel_ms": ms_g}


def bench_im2col(a) -> dict:
    """3x3 stride-1 convolution operand of a B x C x H x W image (H = W = --K)."""
    from . import cuda as K
    B, Cc, H = a.B, a.N, a.K
    x = torch.randn(B, Cc, H, H, device="cuda").to(torch.bfloat16)
    w = (torch.randn(Cc, Cc, 3, 3, device="cuda") * 0.05).to(torch.bfloat16)
    pw = K.pack_conv_weight(w)
    ms = timeit(lambda: K.conv2d(x, pw, [3, 3], [1, 1], [1, 1], [1, 1], [1, 1]), a.iters, a.warmup)
    flops = 2.0 * B * H * H * Cc * Cc * 9
    return {"kernel": "conv2d 3x3 (im2col + gemm)", "B": B, "C": Cc, "HW": H, "ms": ms, "tflops": flops / ms / 1e9,
            "gbs": (B * H * H * pw.K * 2 * 2 + x.numel() * 2) / ms / 1e6}


def bench_ssm(a) -> dict:
    """Selective state-space scan: --B sequences of --ctx tokens, --Hq heads of width --K (head_dim), state size --N, 8 groups."""
    from . import cuda as K
    B, L, H, P, S, G = a.B, a.ctx, a.Hq, a.K, a.N, min(8, a.Hq)
    A = -torch.rand(H, device="cuda")
    dt, x = torch.rand(B, L, H, device="cuda") * 0.1, torch.randn(B, L, H, P, device="cuda")
    Bm, Cm, st = torch.randn(B, L, G, S, device="cuda"), torch.randn(B, L, G, S, device="cuda"), torch.randn(B, H, P, S, device="cuda")
    ms = timeit(lambda: K.selective_ssm(A, dt, Bm, x, Cm, st), a.iters, a.warmup)
    nbytes = 4 * (dt.numel() + 2 * x.numel() + Bm.numel() + Cm.numel() + 3 * st.numel())      # the wrapper clones the state: read, write, read / write
    return {"kernel": "selective_ssm", "B": B, "L": L, "H": H, "P": P, "S": S, "ms": ms, "gbs": nbytes / ms / 1e6,
            "tokens_per_s": B * L / ms * 1e3, "gflops": 6.0 * B * L * H * P * S / ms / 1e6}


def bench_gdn(a) -> dict:
    """Gated delta rule: --B sequences of --ctx tokens, --Hkv key heads and --Hq value heads, key width --K, value width --N."""
    from . import cuda as K
    B, L, Hq, Hv, Dk, Dv = a.B, a.ctx, a.Hkv, a.Hq, a.K, a.N
    q, k = torch.randn(B, L, Hq, Dk, device="cuda") / Dk ** 0.5, torch.nn.functional.normalize(torch.randn(B, L, Hq, Dk, device="cuda"), dim=-1)
    v, st = torch.randn(B, L, Hv, Dv, device="cuda"), torch.zeros(B, Hv, Dk, Dv, device="cuda")
    g, beta = -torch.rand(B, L, Hv, device="cuda"), torch.rand(B, L, Hv, device="cuda")
    ms = timeit(lambda: K.gated_delta_rule(q, k, v, g, beta, st), a.iters, a.warmup)
    nbytes = 4 * (2 * q.numel() + 2 * v.numel() + 2 * g.numel() + 3 * st.numel())
    return {"kernel": "gated_delta_rule", "B": B, "L": L, "Hq": Hq, "Hv": Hv, "Dk": Dk, "Dv": Dv, "ms": ms, "gbs": nbytes / ms / 1e6,
            "tokens_per_s": B * L / ms * 1e3, "gflops": 7.0 * B * L * Hv * Dk * Dv / ms / 1e6}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("kernel", choices=["gemm", "attention", "rmsnorm", "rope", "silu", "sample", "conv", "ssm", "gdn"])
    ap.add_argument("--T", type=int, default=64)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--wmode", default="u4", choices=["u4", "bf16"])
    ap.add_argument("--group", type=int, default=128)
    ap.add_argument("--cublas", action="store_true")
    ap.add_argument("--block-t", dest="block_t", type=int, default=0, help="token tile of the GEMM (0 = automatic)")
    ap.add_argument("--B", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--q-len", dest="q_len", type=int, default=1)
    ap.add_argument("--Hq", type=int, default=32)
    ap.add_argument("--Hkv", type=int, default=8)
    ap.add_argument("--kv-u8", dest="kv_u8", action="store_true", help="attention: u8 KV cache with per-row scale / zero point")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    r = {"gemm": bench_gemm, "attention": bench_attention, "rmsnorm": bench_rmsnorm, "rope": bench_rope, "silu": bench_silu,
         "sample": bench_sample, "conv": bench_im2col, "ssm": bench_ssm, "gdn": bench_gdn}[a.kernel](a)
    pk = _peaks()
    if pk["hbm_gbs"]:
        r["frac_of_%s_hbm" % pk["source"]] = r["gbs"] / pk["hbm_gbs"]
    if pk["bf16_tflops"] and "tflops" in r:
        r["frac_of_%s_bf16" % pk["source"]] = r["tflops"] / pk["bf16_tflops"]
    print(json.dumps(r))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
