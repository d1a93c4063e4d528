"""Fused row-parallel GEMM + all-reduce against its roofline and against GEMM followed by an NCCL all-reduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m openvino_b200.parallel.bench_fused [--iters 20]

Shapes are the two row-parallel projections of a Llama-3-8B layer (attention output K = 4096 / N, MLP down
K = 14336 / N; int4 g128 weights, bf16 activations) at a decode batch (T = 64) and a prefill chunk (T = 8192). Every
number is device time (CUDA events, max over ranks, median of the iterations; an L2-sized read precedes every launch).
The roofline of a call is the slowest of: FLOPs / measured bf16 GEMM peak, weight bytes / measured HBM bandwidth, and the
bytes a rank must send over NVLink / 770 GB/s (one-shot, T <= 128: (N-1) copies of the bf16 tile; two-shot: 2 (N-1)/N;
in-switch reduction: 1 + 1/N).
Rank 0 prints one JSON line per shape.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import cuda as K
    from ..ops.bench_kernels import _peaks
    from ..utils import quant
    from .comm import PeerCommunicator

    H, Tmax = 4096, 8192
    comm = PeerCommunicator(rank, world, dev)
    comm.setup(H, Tmax, 2, tensor_bytes=(Tmax + 8) * H * 2 + 8192)
    h = comm.alloc((Tmax, H))
    ws = K.default_workspace(dev)
    pk = _peaks()
    flush = torch.zeros(64 << 20, dtype=torch.int32, device=dev)
    link_gbs = 770.0

    calls = [0]
    failures = []

    def timed(fn):
        for _ in range(a.warmup):
            comm.step_begin()
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        evs = []
        for _ in range(a.iters):
            flush.sum()
            comm.step_begin()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            evs.append((s, e))
        torch.cuda.synchronize()
        ts = sorted(s.elapsed_time(e) for s, e in evs)
        t = torch.tensor([ts[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for T, Kfull in ((64, 4096), (64, 14336), (8192, 4096), (8192, 14336)):
        Kd = Kfull // world
        if Kd % 128:
            continue
        x = torch.randn(T, Kd, device=dev, dtype=torch.bfloat16)
        packed, s, z = quant.random_u4_weight(H, Kd, 128, dev, seed=rank)
        pw = K.PackedWeight.from_ir_u4(packed, s, quant.pack_u4(z), H, Kd, 128)
        hv = h[:T]
        hv.zero_()
        tmp = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
        def fused():
            # consecutive one-shot calls alternate between two call sites (staging buffers), as the layers of a model do:
            # a rank may start call i+1 while a peer still reads the partials of call i
            calls[0] += 1
            comm.gemm_allreduce(x, pw, hv, ws, calls[0] & 1)
        fused_ms = timed(fused)
        K.check_status("fused gemm + all-reduce")

        def unfused():
            K.gemm(x, pw, out=tmp, ws=ws)
            dist.all_reduce(tmp)
            hv.add_(tmp)
        nccl_ms = timed(unfused)
        gemm_ms = timed(lambda: K.gemm(x, pw, out=tmp, ws=ws))
        # numerics of the fused launch (it also covers the multi-wave paths that only large T reaches): the sum over the ranks
        # against GEMM + fp32 all-reduce, and the same bits on every rank
        hv.zero_()
        comm.step_begin()
        fused()
        K.check_status("fused gemm + all-reduce, verification")
        ref = K.gemm(x, pw, out_f32=True, ws=ws)
        dist.all_reduce(ref)
        got = hv.float()
        err = float((got - ref).norm() / ref.norm().clamp_min(1e-20))
        digest = torch.stack([got.double().sum(), got.double().abs().sum(), (got.double() * torch.arange(got.numel(), device=dev, dtype=torch.float64).reshape(got.shape) % 7).sum()])
        digests = [torch.empty_like(digest) for _ in range(world)]
        dist.all_gather(digests, digest)
        identical = all(bool(torch.equal(d, digests[0])) for d in digests)
        if err > 2e-2 or not identical:
            failures.append((T, Kd, err, identical))
        flops = 2.0 * T * H * Kd
        wbytes = H * Kd // 2 + (H * Kd // 128) * 4
        tile_bytes = T * H * 2
        if comm.mc_ptr:
            # in-switch reduction: the switch pulls this rank's partial tile once and the rank stores its 1/W share of the result
            sent = (1.0 + 1.0 / world) * tile_bytes
        else:
            sent = (world - 1) * tile_bytes if T <= 128 else 2.0 * (world - 1) / world * tile_bytes
        t_compute = flops / (pk["bf16_tflops"] * 1e12) * 1e3
        t_hbm = (wbytes + T * Kd * 2 + 2 * tile_bytes) / (pk["hbm_gbs"] * 1e9) * 1e3
        t_link = sent / (link_gbs * 1e9) * 1e3
        roof = max(t_compute, t_hbm, t_link)
        if rank == 0:
            print(json.dumps({"kernel": "gemm_u4 + all-reduce (fused epilogue)", "n_gpus": world, "T": T, "N": H, "K_per_rank": Kd,
                              "mode": "in-switch (NVLS)" if comm.mc_ptr else ("one-shot" if T <= 128 else "two-shot"), "fused_ms": fused_ms, "gemm_then_nccl_ms": nccl_ms, "gemm_only_ms": gemm_ms,
                              "roofline_ms": roof, "bound": ["compute", "hbm", "nvlink"][[t_compute, t_hbm, t_link].index(roof)],
                              "fraction_of_roofline": roof / fused_ms, "peaks": pk["source"], "rel_err_vs_fp32_allreduce": err, "ranks_identical": identical,
                              "nvlink_gbs_achieved": sent / fused_ms / 1e6}), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    if failures:
        print("FUSED_ALLREDUCE_MISMATCH", failures, flush=True)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
