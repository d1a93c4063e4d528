"""Continuous-batching scheduler and paged KV block manager (host side).

The reference keeps only the device contract in tree (PagedAttentionExtension inputs and the
reference PagedCacheManager, src/core/reference/include/openvino/reference/utils/paged_cache_manager.hpp);
the scheduler itself lives in openvino.genai. This module produces exactly the ragged-batch inputs
of the stateless PagedAttention model: ``input_ids, position_ids, past_lens, subsequence_begins,
block_indices, block_indices_begins, max_context_len`` plus the slot of every new token.

Policy: prompt chunks first (FIFO, up to ``max_num_batched_tokens`` tokens per step, a prompt may be
split over steps = chunked prefill), otherwise one decode token for every running sequence. With
``dynamic_split_fuse`` decode tokens and prompt chunks share a step. Blocks are taken from a free
list; when none is left the youngest running sequence is preempted (its blocks are freed and it is
recomputed later).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

import numpy as np


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 64
    num_kv_blocks: int = 0          # 0 = sized by the pipeline from the workload / free memory
    block_size: int = 16
    dynamic_split_fuse: bool = False
    max_blocks_per_seq: int = 0
    enable_prefix_caching: bool = False   # native scheduler only: requests share the KV blocks of a common prompt prefix
    use_native: bool = True               # csrc/core/sched.cpp; False: the Python scheduler of this module (same policy)


@dataclass
class Sequence:
    request_id: int
    prompt: np.ndarray               # int32
    max_new_tokens: int
    eos_token_id: int = -1
    ignore_eos: bool = True
    generated: List[int] = field(default_factory=list)
    num_computed: int = 0            # tokens whose KV is in the cache
    blocks: List[int] = field(default_factory=list)
    finished: bool = False
    arrival_order: int = 0
    slot: int = -1                   # index into the device-side last-token table
    # timing (filled by the pipeline)
    t_arrival: float = 0.0
    t_first: float = 0.0
    t_tokens: List[float] = field(default_factory=list)

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.generated)

    def token_at(self, i: int) -> int:
        n = len(self.prompt)
        return int(self.prompt[i]) if i < n else self.generated[i - n]


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.free: Deque[int] = deque(range(num_blocks))

    def num_free(self) -> int:
        return len(self.free)

    def blocks_needed(self, seq: Sequence, new_len: int) -> int:
        need = (new_len + self.block_size - 1) // self.block_size
        return max(0, need - len(seq.blocks))

    def grow(self, seq: Sequence, new_len: int) -> bool:
        n = self.blocks_needed(seq, new_len)
        if n > len(self.free):
            return False
        for _ in range(n):
            seq.blocks.append(self.free.popleft())
        return True

    def release(self, seq: Sequence) -> None:
        self.free.extend(seq.blocks)
        seq.blocks = []


@dataclass
class ScheduledStep:
    seqs: List[Sequence]
    num_new: List[int]      # tokens scheduled for each sequence in this step
    T: int
    max_q_len: int
    max_ctx: int


class Scheduler:
    def __init__(self, cfg: SchedulerConfig):
        self.cfg = cfg
        self.blocks = BlockManager(cfg.num_kv_blocks, cfg.block_size)
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self._order = 0
        self.num_preemptions = 0
        self._free_slots = deque(range(cfg.max_num_seqs * 4))

    # True: ids of generated tokens are uploaded by the host; False: the newest generated token of a
    # sequence is read on the device from the last-token table (lets steps be chained asynchronously)
    host_ids_for_generated = False

    def add(self, seq: Sequence) -> None:
        seq.arrival_order = self._order
        self._order += 1
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def _preempt_one(self, keep: Sequence, scheduled: List[Sequence]) -> bool:
        """Free the blocks of the youngest running sequence that is neither ``keep`` nor part of the step being
        built (a sequence already scheduled keeps its blocks: the step's block table points at them)."""
        for victim in reversed(self.running):
            if victim is not keep and victim.blocks and not any(victim is s for s in scheduled):
                self.blocks.release(victim)
                victim.num_computed = 0
                self.running.remove(victim)
                self.waiting.appendleft(victim)
                self.num_preemptions += 1
                return True
        return False

    def schedule(self) -> Optional[ScheduledStep]:
        cfg = self.cfg
        budget = cfg.max_num_batched_tokens
        seqs: List[Sequence] = []
        num_new: List[int] = []

        def pending(s: Sequence) -> int:
            # tokens that still have to pass through the model before the next token can be sampled
            return s.total_len - s.num_computed

        def decode_phase() -> None:
            nonlocal budget
            for s in [r for r in self.running if pending(r) == 1]:
                if budget <= 0 or len(seqs) >= cfg.max_num_seqs:
                    break
                if not any(s is r for r in self.running):
                    continue                       # preempted on behalf of an earlier sequence of this loop
                while not self.blocks.grow(s, s.total_len):
                    if not self._preempt_one(s, seqs):
                        break
                if self.blocks.blocks_needed(s, s.total_len) > 0:
                    continue
                seqs.append(s)
                num_new.append(1)
                budget -= 1

        def prefill_phase(may_preempt: bool) -> None:
            nonlocal budget
            # taken after the decode phase: a preemption there moves a mid-prefill sequence from `running` to `waiting`
            cands = [s for s in self.running if pending(s) > 1]
            n_running_cands = len(cands)
            while self.waiting and len(self.running) + (len(cands) - n_running_cands) < cfg.max_num_seqs:
                cands.append(self.waiting.popleft())
            back: List[Sequence] = []
            for s in cands:
                is_running = any(s is r for r in self.running)
                if budget <= 0 or len(seqs) >= cfg.max_num_seqs:
                    if not is_running:
                        back.append(s)
                    continue
                n = min(budget, s.total_len - s.num_computed)
                ok = n > 0 and self.blocks.grow(s, s.num_computed + n)
                while n > 0 and not ok and may_preempt and not seqs and self._preempt_one(s, seqs):
                    ok = self.blocks.grow(s, s.num_computed + n)      # last resort: the oldest candidate evicts younger ones
                if not ok:
                    if not is_running:
                        back.append(s)
                    continue
                if not is_running:
                    self.running.append(s)
                    if s.slot < 0:
                        s.slot = self._free_slots.popleft()
                seqs.append(s)
                num_new.append(n)
                budget -= n
            for s in reversed(back):               # keep the arrival order of what could not be placed
                self.waiting.appendleft(s)

        def want_prefill() -> bool:
            return bool(self.waiting or any(pending(s) > 1 for s in self.running))

        if cfg.dynamic_split_fuse:
            decode_phase()
            if want_prefill():
                prefill_phase(False)
        else:
            if want_prefill():
                prefill_phase(False)
            if not seqs:
                decode_phase()                     # no prompt chunk fits: keep the running sequences going (they may preempt)
        if not seqs and want_prefill():
            prefill_phase(True)
        if not seqs:
            return None
        T = sum(num_new)
        max_ctx = max(s.num_computed + n for s, n in zip(seqs, num_new))
        return ScheduledStep(seqs, num_new, T, max(num_new), max_ctx)

    # -- descriptor of a scheduled step, written into numpy views of the pinned mirror --------
    def fill(self, step: ScheduledStep, views: Dict[str, np.ndarray]) -> None:
        bs = self.cfg.block_size
        t = 0
        nb = 0
        B = len(step.seqs)
        sb, bib = views["subsequence_begins"], views["block_indices_begins"]
        sb[0] = 0
        bib[0] = 0
        for i, (s, n) in enumerate(zip(step.seqs, step.num_new)):
            c0 = s.num_computed
            pos = np.arange(c0, c0 + n, dtype=np.int32)
            np_prompt = len(s.prompt)
            if c0 + n <= np_prompt:
                views["ids"][t:t + n] = s.prompt[c0:c0 + n]
            else:
                for j in range(n):
                    views["ids"][t + j] = s.token_at(c0 + j)
            views["positions"][t:t + n] = pos
            tbl = np.asarray(s.blocks, dtype=np.int32)
            views["slot_map"][t:t + n] = tbl[pos // bs] * bs + pos % bs
            # the newest generated token is taken from the device-side table (the host may not have it yet)
            src = views["tok_src"][t:t + n]
            src[:] = -1
            if not self.host_ids_for_generated and s.generated and c0 + n == s.total_len:
                src[n - 1] = s.slot
            views["tok_dst"][i] = s.slot if c0 + n == s.total_len else -1
            views["past_lens"][i] = c0
            views["logit_idx"][i] = t + n - 1
            k = (c0 + n + bs - 1) // bs
            views["block_indices"][nb:nb + k] = tbl[:k]
            nb += k
            t += n
            sb[i + 1] = t
            bib[i + 1] = nb

    def commit(self, step: ScheduledStep, tokens: Optional[np.ndarray] = None) -> List[tuple]:
        """Account for a step that has been launched. Returns [(sequence, index into generated, row)] for
        the sequences that get a token from it. With ``tokens`` None the value is not known yet: a
        placeholder is stored and ``patch`` fills it in later (asynchronous scheduling)."""
        produced = []
        for i, (s, n) in enumerate(zip(step.seqs, step.num_new)):
            s.num_computed += n
            if s.num_computed >= s.total_len and not s.finished:   # ended on the last known token
                s.generated.append(-1 if tokens is None else int(tokens[i]))
                produced.append((s, len(s.generated) - 1, i))
                if len(s.generated) >= s.max_new_tokens:
                    self._finish(s)
        if tokens is not None:
            self._check_eos(produced)
        return produced

    def patch(self, produced: List[tuple], tokens: np.ndarray) -> None:
        """Fill in the token values of an earlier ``commit(step, None)``."""
        for s, gi, row in produced:
            if gi < len(s.generated):
                s.generated[gi] = int(tokens[row])
        self._check_eos(produced)

    def _check_eos(self, produced: List[tuple]) -> None:
        for s, gi, _ in produced:
            if not s.ignore_eos and gi < len(s.generated) and s.generated[gi] == s.eos_token_id:
                del s.generated[gi + 1:]      # drop tokens sampled by steps launched before the EOS was seen
                s.num_computed = min(s.num_computed, s.total_len)
                self._finish(s)

    def _finish(self, s: Sequence) -> None:
        if s.finished:
            return
        s.finished = True
        self.blocks.release(s)
        if s in self.running:
            self.running.remove(s)
        if s.slot >= 0:
            self._free_slots.append(s.slot)
            s.slot = -1
