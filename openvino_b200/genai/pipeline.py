"""Continuous-batching text-generation pipeline over the CUDA plugin's LLM program.

API shape follows openvino.genai's ContinuousBatchingPipeline (add_request / step / has_non_finished_requests /
generate) so that serving code written against it ports over; the reference repository itself stops at
the PagedAttention model contract (docs/articles_en/openvino-workflow-generative/inference-with-genai.rst).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

import numpy as np
import torch

from ..runtime.cuda_llm import CudaLlmExecutor, StepBuffers, StepShape
from .native_scheduler import NativeScheduler, make_layout
from .scheduler import ScheduledStep, Scheduler, SchedulerConfig, Sequence


@dataclass
class GenerationConfig:
    max_new_tokens: int = 128
    eos_token_id: int = -1
    ignore_eos: bool = True
    do_sample: bool = False       # False: greedy. True: multinomial with the transforms below (whole pipeline, not per request)
    temperature: float = 1.0
    top_k: int = 0                # 0 = off
    top_p: float = 1.0            # 1 = off
    rng_seed: int = 0


@dataclass
class GenerationResult:
    request_id: int
    tokens: List[int]
    ttft_s: float
    tpot_s: float
    token_times: List[float] = field(default_factory=list)


@dataclass
class PipelineMetrics:
    steps: int = 0
    prefill_steps: int = 0
    decode_steps: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    scheduled_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0

    def report(self, results=None, kv_blocks_total: int = 0, kv_blocks_free: int = 0) -> dict:
        """Serving counters as one JSON-able dict; with the ``GenerationResult`` list of a ``generate`` call also the
        time-to-first-token / time-per-output-token percentiles (milliseconds)."""
        out = {k: getattr(self, k) for k in ("steps", "prefill_steps", "decode_steps", "h2d_bytes", "d2h_bytes", "scheduled_tokens",
                                             "generated_tokens", "preemptions")}
        if kv_blocks_total:
            out["kv_block_utilisation"] = 1.0 - kv_blocks_free / float(kv_blocks_total)
        if results:
            import numpy as _np
            ttft = _np.array([r.ttft_s for r in results]) * 1e3
            tpot = _np.array([r.tpot_s for r in results if r.tpot_s > 0]) * 1e3
            out["ttft_ms"] = {p: float(_np.percentile(ttft, q)) for p, q in (("p50", 50), ("p90", 90), ("p99", 99))}
            if tpot.size:
                out["tpot_ms"] = {p: float(_np.percentile(tpot, q)) for p, q in (("p50", 50), ("p90", 90), ("p99", 99))}
        return out


@dataclass
class StepPlan:
    steps: list            # (StepBuffers, index into desc_dev, StepShape)
    desc_dev: dict         # id(StepBuffers) -> int32 tensor [n_steps, desc_words] on the device
    prompt_tokens: int
    output_tokens: int


from ..utils import trace as _trace

class ContinuousBatchingPipeline:
    def __init__(self, executor: CudaLlmExecutor, scheduler_config: SchedulerConfig):
        self.ex = executor
        self.cfg = scheduler_config
        self.scheduler = self._make_scheduler(scheduler_config)
        self._layouts = {id(sb): make_layout(sb.offsets, sb.Tcap, sb.Bcap, sb.max_blocks) for sb in (executor.prefill, executor.decode)}
        self._next_id = 0
        self._seqs: Dict[int, Sequence] = {}
        self.metrics = PipelineMetrics()
        self._np_views = {}
        self._flip = 0
        for sb in (executor.prefill, executor.decode):
            for k in (0, 1):
                self._np_views[(id(sb), k)] = {name: sb.view(name, host=k).numpy() for name in sb.offsets}

    @staticmethod
    def _make_scheduler(cfg: SchedulerConfig):
        """The native scheduler unless the configuration asks for the Python one."""
        if getattr(cfg, "use_native", True):
            return NativeScheduler(cfg)
        if getattr(cfg, "enable_prefix_caching", False):
            raise ValueError("prefix caching is a feature of the native scheduler (use_native=True)")
        return Scheduler(cfg)

    def _fill(self, sched, st, sb, k: int) -> None:
        if isinstance(sched, NativeScheduler):
            sched.fill_flat(st, sb.desc_hosts[k].numpy(), self._layouts[id(sb)])
        else:
            sched.fill(st, self._np_views[(id(sb), k)])

    def add_request(self, prompt_ids, gen: GenerationConfig, request_id: Optional[int] = None) -> int:
        rid = self._next_id if request_id is None else request_id
        self._next_id = max(self._next_id, rid) + 1
        seq = Sequence(rid, np.asarray(prompt_ids, dtype=np.int32), gen.max_new_tokens, gen.eos_token_id, gen.ignore_eos)
        seq.t_arrival = time.perf_counter()
        self._seqs[rid] = seq
        self.scheduler.add(seq)
        return rid

    def has_non_finished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    # ------------------------------------------------------------------------------------------
    def _launch(self):
        """Schedule one step, upload its descriptor (one H2D copy from pinned memory), launch it and queue
        the D2H copy of the sampled tokens. Does not wait for the GPU."""
        st = self.scheduler.schedule()
        if st is None:
            raise RuntimeError("scheduler could not place any sequence: KV cache too small for a single request")
        ex = self.ex
        decode = st.max_q_len == 1 and len(st.seqs) <= ex.decode.Bcap
        sb = ex.decode if decode else ex.prefill
        k = self._flip
        self._flip ^= 1
        self._fill(self.scheduler, st, sb, k)
        self.metrics.h2d_bytes += ex.upload(sb, k)
        B = len(st.seqs)
        with _trace.scope("ov::genai", "decode_step" if decode else "prefill_step"):
            ex.run(sb, StepShape(st.T, B, st.max_q_len, st.max_ctx))
        ev = ex.download_tokens_async(sb, B, k)
        self.metrics.d2h_bytes += B * 4
        m = self.metrics
        m.steps += 1
        m.decode_steps += 1 if decode else 0
        m.prefill_steps += 0 if decode else 1
        m.scheduled_tokens += st.T
        return st, sb, k, ev

    def _retire(self, produced, sb, k, ev) -> List[Sequence]:
        ev.synchronize()
        toks = sb.tokens_host[k].numpy()
        now = time.perf_counter()
        self.scheduler.patch(produced, toks)
        out = []
        for s, gi in ((p[0], p[1]) for p in produced):
            if gi < len(s.generated):
                if gi == 0:
                    s.t_first = now
                s.t_tokens.append(now)
                out.append(s)
        self.metrics.generated_tokens += len(out)
        self.metrics.preemptions = self.scheduler.num_preemptions
        return out

    # ------------------------------------------------------------------------------------------
    def plan(self, prompts: Seq[Seq[int]], gen: GenerationConfig) -> "StepPlan":
        """Dry-run the scheduler over a fixed-length workload (``ignore_eos``) and stage every step's
        descriptor on the device. ``run_plan`` then replays the steps without any host round trip: sampled
        tokens are fed back through the device-side last-token table."""
        assert gen.ignore_eos, "a plan needs output lengths that do not depend on token values"
        sched = self._make_scheduler(self.cfg)
        for i, p in enumerate(prompts):
            sched.add(Sequence(i, np.asarray(p, dtype=np.int32), gen.max_new_tokens, gen.eos_token_id, True))
        ex = self.ex
        steps = []
        descs = {id(ex.prefill): [], id(ex.decode): []}
        while sched.has_unfinished():
            st = sched.schedule()
            if st is None:
                raise RuntimeError("scheduler could not place any sequence")
            decode = st.max_q_len == 1 and len(st.seqs) <= ex.decode.Bcap
            sb = ex.decode if decode else ex.prefill
            arr = np.zeros(sb.desc_words, dtype=np.int32)
            if isinstance(sched, NativeScheduler):
                sched.fill_flat(st, arr, self._layouts[id(sb)])
            else:
                sched.fill(st, {name: arr[off:off + n] for name, (off, n) in sb.offsets.items()})
            descs[id(sb)].append(torch.from_numpy(arr))
            steps.append((sb, len(descs[id(sb)]) - 1, StepShape(st.T, len(st.seqs), st.max_q_len, st.max_ctx)))
            sched.commit(st, None)
        dev = {k: (torch.stack(v).to(ex.device) if v else None) for k, v in descs.items()}
        return StepPlan(steps, dev, sum(len(p) for p in prompts), len(prompts) * gen.max_new_tokens)

    def run_plan(self, plan: "StepPlan") -> None:
        ex = self.ex
        for sb, i, shp in plan.steps:
            sb.desc.copy_(plan.desc_dev[id(sb)][i], non_blocking=True)
            ex.run(sb, shp)

    def step(self) -> List[Sequence]:
        """One synchronous step: schedule, upload, run, read tokens back, account."""
        st, sb, k, ev = self._launch()
        produced = self.scheduler.commit(st, None)
        return self._retire(produced, sb, k, ev)

    def generate(self, prompts: Seq[Seq[int]], gen: GenerationConfig, lookahead: int = 1) -> List[GenerationResult]:
        """Serve all prompts to completion. ``lookahead`` steps may be in flight on the GPU while the host
        schedules the next one (the newest token of a sequence is fed back on the device), so host work
        overlaps GPU work; 0 = fully synchronous."""
        if gen.do_sample:
            self.ex.set_sampling(gen.temperature, gen.top_k, gen.top_p, gen.rng_seed)
        else:
            self.ex.set_sampling(0.0)
        rids = [self.add_request(p, gen) for p in prompts]
        inflight = []
        while self.has_non_finished_requests() or inflight:
            if self.has_non_finished_requests():
                st, sb, k, ev = self._launch()
                inflight.append((self.scheduler.commit(st, None), sb, k, ev))
            while inflight and (len(inflight) > lookahead or not self.has_non_finished_requests()):
                self._retire(*inflight.pop(0))
        out = []
        for rid in rids:
            s = self._seqs.pop(rid)
            if isinstance(self.scheduler, NativeScheduler):
                self.scheduler.forget(rid)
            n = len(s.generated)
            tpot = (s.t_tokens[-1] - s.t_first) / (n - 1) if n > 1 else 0.0
            out.append(GenerationResult(rid, list(s.generated), s.t_first - s.t_arrival, tpot, list(s.t_tokens)))
        return out
