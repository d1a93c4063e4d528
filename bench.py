#!/usr/bin/env python
"""Serving benchmark: Llama-3-8B architecture, int4 (u4 asym, group 128, fp16 scale/zp) weights, bf16
activations, PagedAttention (block 16) + continuous batching, 64 concurrent requests x (1024 prompt
tokens, 256 greedy output tokens). Metric: output tokens/s of the whole job.

One "step" of this benchmark is one complete serving pass over the 64 requests.

  python bench.py [--gpus N --steps K --warmup W]             this framework (TP = N)
  python bench.py --impl reference ...                        the unmodified reference (unavailable offline)
  python bench.py --impl torch ...                            NCCL + cuBLAS PyTorch baseline of the same model

`value`  : device-timed (CUDA events) pass with every step descriptor staged on the device beforehand
           and sampled tokens fed back on the device: kernels only, no host in the loop.
`e2e`    : the same workload through the public API (ContinuousBatchingPipeline.generate): every step
           uploads its inputs from pinned host memory and reads the sampled tokens back.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# OVMS continuous-batching throughput of Meta-Llama-3-8B-Instruct published by the reference
# (docs/sphinx_setup/_static/benchmarks_files/data/graph-data-ovms-genai.json:201, Xeon Platinum 8580, FP16)
PUBLISHED_TOK_S = 1151.94


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--model", default="llama-3-8b",
                    help="llama-3-8b (headline) | llama-3-70b | mixtral-8x7b | tiny-llama | tiny-moe (serving); bert-large | resnet18 (graph API)")
    ap.add_argument("--requests", type=int, default=0, help="concurrent requests (default: the benchmark's number for the model)")
    ap.add_argument("--prompt-len", type=int, default=0)
    ap.add_argument("--output-len", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (result is then marked invalid)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--direct", action="store_true",
                    help="build the executor from an architecture description and packed random weights instead of going through "
                         "graph -> SDPAToPagedAttention -> save_model / read_model -> Core.compile_model (same kernels, shorter start-up)")
    return ap.parse_args()


def reference_arm(args):
    # The reference cannot be installed offline: every git submodule it needs at build time (pugixml, oneDNN,
    # xbyak, pybind11, ...) is empty in the checkout and no openvino wheel exists in the wheelhouse.
    why = "reference does not build offline: all 29 git submodules (pugixml, oneDNN, xbyak, pybind11, ...) are empty and no openvino wheel is in /opt/wheelhouse"
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    if os.path.isdir(os.path.join(ref_dir, "openvino")):
        why = "baseline/_ref holds python sources only: the native runtime (_pyopenvino) could not be built offline (empty submodules)"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


SERVING_DEFAULTS = {"mixtral-8x7b": (128, 512, 128), "llama-3-70b": (32, 2048, 512), "tiny-moe": (16, 128, 32), "tiny-llama": (16, 128, 32)}   # requests, prompt, output


def graph_api_bench(args):
    """Secondary configurations that run through convert_model / compile_model / InferRequest.

    resnet18   : the plumbing configuration (fp32, batch 1, "CPU" device): convert -> save -> read -> compile -> infer,
                 checked against eager PyTorch; reports latency.
    bert-large : encoder, fp16, batch 64 x sequence 384 on the "CUDA" device; with N GPUs every rank serves its own replica
                 (data parallel), the value is the sum over ranks.
    """
    import tempfile
    import numpy as np
    import torch
    import openvino_b200 as ov
    from openvino_b200 import properties as props
    from openvino_b200.models import torch_zoo
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    core = ov.Core()
    if args.model == "resnet18":
        torch.manual_seed(0)
        net = torch_zoo.ResNet18().eval()
        for m in net.modules():
            if isinstance(m, (torch.nn.Conv2d, torch.nn.Linear)):
                torch.nn.init.kaiming_normal_(m.weight)
        x = torch.randn(1, 3, 224, 224)
        with torch.no_grad():
            want = net(x).numpy()
        d = tempfile.mkdtemp()
        model = ov.convert_model(net, example_input=(x,))
        ov.save_model(model, os.path.join(d, "resnet18.xml"), compress_to_fp16=False)
        cm = core.compile_model(core.read_model(os.path.join(d, "resnet18.xml")), "CPU")
        req = cm.create_infer_request()
        for _ in range(args.warmup):
            req.infer([x.numpy()])
        t0 = time.perf_counter()
        for _ in range(args.steps):
            out = req.infer([x.numpy()])[0]
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
        err = float(np.abs(out - want).max() / max(np.abs(want).max(), 1e-9))
        print(json.dumps({"metric": "latency", "value": ms, "unit": "ms", "n_gpus": 0, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": ms, "higher_is_better": False, "dtype": "fp32", "data": "synthetic N(0,1) image, Kaiming-normal weights",
                          "config": {"model": "resnet18", "device": "CPU", "batch": 1, "path": "convert_model -> save_model -> read_model -> compile_model -> InferRequest"},
                          "max_rel_error_vs_torch": err, "logits_equal": err < 1e-3}))
        return 0
    # bert-large
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.manual_seed(0)
    net = torch_zoo.bert_large().eval()
    for prm in net.parameters():
        torch.nn.init.normal_(prm, 0.0, 0.02) if prm.dim() > 1 else None
    B, S = 64, 384
    ids = torch.randint(0, 30522, (B, S))
    mask = torch.ones(B, S, dtype=torch.int64)
    typ = torch.zeros(B, S, dtype=torch.int64)
    model = ov.convert_model(net, example_input=(ids, mask, typ))
    # more than one GPU: tensor parallel, every rank compiles its shard of the one model and all ranks serve the same batch
    cm = core.compile_model(model, "CUDA.%d" % local_rank, {props.hint.inference_precision: "f16",
                                                            props.hint.model_distribution_policy: "TENSOR_PARALLEL" if world > 1 else ""})
    req = cm.create_infer_request()
    feed = [ids.numpy(), mask.numpy(), typ.numpy()]
    for _ in range(args.warmup):
        req.infer(feed, share_outputs=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        req.infer(feed, share_outputs=True)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    t = torch.tensor([wall], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.destroy_process_group()
    wall = float(t.item())
    if rank == 0:
        print(json.dumps({"metric": "sequences/s", "value": B * args.steps / wall, "unit": "sequences/s", "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": wall * 1e3 / args.steps, "higher_is_better": True, "scaling": "strong", "dtype": "fp16",
                          "data": "synthetic: uniform token ids, all-ones mask, N(0,0.02) weights",
                          "config": {"model": "bert-large", "global_batch": B, "seq_len": S, "parallelism": "tp%d" % world, "device": "CUDA",
                                     "timing": "end to end through InferRequest.infer (host inputs in, host output out)"}}))
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.model in ("resnet18", "bert-large"):
        return graph_api_bench(args)
    dr, dp, do = SERVING_DEFAULTS.get(args.model, (64, 1024, 256))
    args.requests, args.prompt_len, args.output_len = args.requests or dr, args.prompt_len or dp, args.output_len or do

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # re-launch under torchrun, one rank per GPU
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
                   "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000)] + sys.argv
            return subprocess.call(cmd)
        raise SystemExit("WORLD_SIZE=%d does not match --gpus %d" % (world, args.gpus))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.impl == "torch":
        from baseline.torch_llm import run_torch_baseline
        return run_torch_baseline(args, rank, world, dev)

    from openvino_b200.genai.pipeline import ContinuousBatchingPipeline, GenerationConfig
    from openvino_b200.genai.scheduler import SchedulerConfig
    from openvino_b200.models.llm_config import NAMED
    from openvino_b200.ops import cuda as K
    from openvino_b200.runtime.cuda_llm import CudaLlmExecutor, LlmWeights

    cfg = NAMED[args.model]
    if args.layers:
        cfg = cfg.with_(num_layers=args.layers)
    comm = None
    if world > 1:
        from openvino_b200.parallel.comm import PeerCommunicator
        comm = PeerCommunicator(rank, world, dev)
    R, P, O = args.requests, args.prompt_len, args.output_len
    bs = 16
    blocks_per_seq = (P + O + bs - 1) // bs + 1
    num_blocks = R * blocks_per_seq + 8
    via_api = not args.direct and cfg.weight_format == "int4" and not cfg.num_experts
    startup = {}
    if via_api:
        # The product path: a stateful decoder graph with int4-compressed weights (u4 constants, fp16 scales, u4 zero points,
        # the decompression sub-graph exporters write) -> SDPAToPagedAttention -> IR on disk -> read_model ->
        # Core.compile_model(model, "CUDA", {CUDA_SERVING_PROGRAM, MODEL_DISTRIBUTION_POLICY: TENSOR_PARALLEL}).
        # The device analyses the graph by structure, takes this rank's slice of heads / MLP channels / vocabulary and builds
        # the serving program; LLMPipeline wraps exactly these calls. Rank 0 writes the IR, every rank reads it.
        import shutil
        import openvino_b200 as ov
        from openvino_b200 import passes
        from openvino_b200.genai import LLMPipeline
        from openvino_b200.models.ov_builders import build_llama_random_int4
        ir_dir = os.path.join(tempfile.gettempdir(), "ovb_bench_%s_%s" % (cfg.name, os.environ.get("MASTER_PORT", str(os.getpid()))))
        t0 = time.perf_counter()
        if rank == 0:
            os.makedirs(ir_dir, exist_ok=True)
            graph = build_llama_random_int4(cfg, seed=0)
            mgr = passes.Manager()
            mgr.register_pass(passes.SDPAToPagedAttention())
            mgr.run_passes(graph)
            ov.save_model(graph, os.path.join(ir_dir, "openvino_model.xml"), compress_to_fp16=False)
            del graph
        if world > 1:
            dist.barrier()
        startup["build_and_save_s"] = time.perf_counter() - t0
        t0 = time.perf_counter()
        llm = LLMPipeline(ir_dir, "CUDA.%d" % local_rank, comm=comm, tp_rank=rank, tp_size=world, max_num_seqs=R, max_num_batched_tokens=8192,
                          max_model_len=P + O, block_size=bs, kv_cache_blocks=num_blocks)
        startup["read_compile_s"] = time.perf_counter() - t0
        if world > 1:
            dist.barrier()
        if rank == 0:
            shutil.rmtree(ir_dir, ignore_errors=True)
        ex, sc = llm.executor, llm.scheduler_config
        got = llm.config
        assert (got.num_layers, got.num_heads, got.num_kv_heads, got.head_dim, got.ffn_size, got.hidden_size, got.vocab_size, got.weight_format) == \
               (cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.ffn_size, cfg.hidden_size, cfg.vocab_size, "int4"), got
    else:
        weights = LlmWeights.random(cfg, dev, seed=0, tp_rank=rank, tp_size=world)
        ex = CudaLlmExecutor(cfg, weights, num_kv_blocks=num_blocks, block_size=bs, max_batch_tokens=8192, max_seqs=R,
                             max_blocks_per_seq=blocks_per_seq, device=dev, comm=comm)
        sc = SchedulerConfig(max_num_batched_tokens=8192, max_num_seqs=R, num_kv_blocks=num_blocks, block_size=bs,
                             max_blocks_per_seq=blocks_per_seq)
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (P,), generator=g).tolist() for _ in range(R)]
    gen = GenerationConfig(max_new_tokens=O, ignore_eos=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- kernel-only passes (device resident)
    pipe = ContinuousBatchingPipeline(ex, sc)
    plan = pipe.plan(prompts, gen)
    for _ in range(args.warmup):
        pipe.run_plan(plan)
    barrier()
    K.check_status("warm-up")
    launches0 = ex.kernel_launches
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        pipe.run_plan(plan)
    e1.record()
    barrier()
    clocks = sampler.stop()
    K.check_status("timed region")
    dev_ms = e0.elapsed_time(e1)
    launches = ex.kernel_launches - launches0
    t = torch.tensor([dev_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms = float(t.item())
    out_tokens = R * O
    value = out_tokens * args.steps / (dev_ms / 1e3)

    # ---------------------------------------------------------------- end-to-end through the public API
    e2e = None
    if not args.skip_e2e:
        for _ in range(min(args.warmup, 1)):
            pipe.generate(prompts, gen)
        barrier()
        m0 = (pipe.metrics.h2d_bytes, pipe.metrics.d2h_bytes, pipe.metrics.steps)
        t0 = time.perf_counter()
        results = []
        for _ in range(args.steps):
            results = pipe.generate(prompts, gen)
        barrier()
        wall = time.perf_counter() - t0
        tw = torch.tensor([wall], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tw, op=dist.ReduceOp.MAX)
        wall = float(tw.item())
        nsteps = max(1, pipe.metrics.steps - m0[2])
        ttft = sorted(r.ttft_s for r in results)
        tpot = sorted(r.tpot_s for r in results)
        e2e = {"value": out_tokens * args.steps / wall, "unit": "output tokens/s",
               "h2d_bytes_per_step": (pipe.metrics.h2d_bytes - m0[0]) // nsteps,
               "d2h_bytes_per_step": (pipe.metrics.d2h_bytes - m0[1]) // nsteps,
               "engine_steps_per_pass": nsteps // args.steps,
               "ttft_p50_ms": 1e3 * ttft[len(ttft) // 2], "tpot_p50_ms": 1e3 * tpot[len(tpot) // 2]}
        K.check_status("e2e")

    if rank == 0:
        line = {
            "metric": "output tokens/s", "value": value, "unit": "output tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": (value / PUBLISHED_TOK_S) if cfg.name == "llama-3-8b" else None,
            "dtype": "bf16 activations, %s weights" % {"int4": "int4 (u4 g128 asym)", "int8": "int8 (u8 g128 asym)"}.get(cfg.weight_format, cfg.weight_format),
            "data": "synthetic: uniform random prompt ids, random-init weights", "impl": "ours",
            "config": {"model": cfg.name + ("" if not args.layers else "-DEBUG-%dlayers" % args.layers),
                       "global_batch": R, "seq_len": P, "output_len": O,
                       "parallelism": ("tp%d" % world) if not cfg.num_experts else ("attention tp%d, experts ep%d" % (world, world)),
                       "kv_block_size": bs, "step": "one serving pass over all requests",
                       "l2": "working set (weights + KV cache) far larger than L2; no flush needed",
                       "published_baseline": "OVMS Meta-Llama-3-8B-Instruct FP16 on Xeon 8580: 1151.94 tok/s",
                       "path": ("graph with int4-compressed constants -> SDPAToPagedAttention -> save_model -> read_model -> "
                                "Core.compile_model(CUDA, serving program%s) -> ContinuousBatchingPipeline" % (", TENSOR_PARALLEL" if world > 1 else ""))
                               if via_api else "executor built directly from the architecture description (--direct)",
                       "startup": startup},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        }
        if args.layers:
            line["invalid"] = "debug run with a reduced layer count"
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
