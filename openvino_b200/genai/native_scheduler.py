"""The native (C++) continuous-batching scheduler behind the interface the pipeline uses.

``csrc/core/sched.cpp`` holds the policy, the paged block manager (free list, shared blocks with reference counts,
prefix cache) and the step-descriptor writer. This module keeps one Python ``Sequence`` record per request for what
the host side wants to read (generated tokens, timings) and forwards everything else. The descriptor of a step is
written by native code straight into the pinned mirror of the step buffers, in one call.

Role in the reference's terms: the scheduler and block manager of the serving layer that sits on top of the
PagedAttention model contract (src/core/reference/include/openvino/reference/utils/paged_cache_manager.hpp is the
in-tree part of it).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

from .. import _ovcore as _core
from .scheduler import ScheduledStep, SchedulerConfig, Sequence


def _native_config(cfg: SchedulerConfig) -> "_core.SchedulerConfig":
    c = _core.SchedulerConfig()
    c.max_num_batched_tokens = cfg.max_num_batched_tokens
    c.max_num_seqs = cfg.max_num_seqs
    c.num_kv_blocks = cfg.num_kv_blocks
    c.block_size = cfg.block_size
    c.dynamic_split_fuse = cfg.dynamic_split_fuse
    c.enable_prefix_caching = bool(getattr(cfg, "enable_prefix_caching", False))
    return c


def make_layout(offsets: Dict[str, tuple], Tcap: int, Bcap: int, max_blocks: int) -> "_core.DescLayout":
    """Word offsets of the descriptor fields of one ``StepBuffers`` as the native writer wants them."""
    lay = _core.DescLayout()
    for name in ("ids", "positions", "slot_map", "tok_src", "tok_dst", "logit_idx", "past_lens", "subsequence_begins",
                 "block_indices_begins", "block_indices"):
        setattr(lay, name, offsets[name][0])
    lay.Tcap, lay.Bcap, lay.blocks_cap = Tcap, Bcap, Bcap * max_blocks
    return lay


class _Step(ScheduledStep):
    """A scheduled step: the Python records of its sequences plus the native step it came from."""

    def __init__(self, native, seqs: List[Sequence]):
        super().__init__(seqs, list(native.num_new), int(native.T), int(native.max_q_len), int(native.max_ctx))
        self.native = native


class NativeScheduler:
    host_ids_for_generated = False

    def __init__(self, cfg: SchedulerConfig):
        self.cfg = cfg
        self._s = _core.Scheduler(_native_config(cfg))
        self._by_id: Dict[int, Sequence] = {}
        self._state: Dict[int, object] = {}          # request id -> native SeqState

    # -- queue ------------------------------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        st = self._s.add(int(seq.request_id), np.asarray(seq.prompt, dtype=np.int32).tolist(), int(seq.max_new_tokens),
                         int(seq.eos_token_id), bool(seq.ignore_eos))
        self._by_id[seq.request_id] = seq
        self._state[seq.request_id] = st

    def has_unfinished(self) -> bool:
        return self._s.has_unfinished()

    @property
    def num_preemptions(self) -> int:
        return int(self._s.num_preemptions())

    @property
    def prefix_hit_tokens(self) -> int:
        return int(self._s.prefix_hit_tokens())

    def num_free_blocks(self) -> int:
        return int(self._s.num_free_blocks())

    # -- steps ------------------------------------------------------------------------------------
    def schedule(self) -> Optional[_Step]:
        st = self._s.schedule()
        if st is None:
            return None
        return _Step(st, [self._by_id[s.request_id] for s in st.seqs])

    def fill_flat(self, step: _Step, desc: np.ndarray, layout) -> None:
        """Write the step's descriptor into ``desc`` (the int32 words of a pinned mirror)."""
        self._s.fill(step.native, desc, layout, self.host_ids_for_generated)

    def fill(self, step: _Step, views: Dict[str, np.ndarray]) -> None:
        raise TypeError("the native scheduler writes whole descriptors: use fill_flat(step, words, layout)")

    def _mirror(self, seq: Sequence) -> None:
        st = self._state[seq.request_id]
        n = int(st.num_generated())
        seq.num_computed = int(st.num_computed)
        if n < len(seq.generated):
            del seq.generated[n:]
        while len(seq.generated) < n:
            seq.generated.append(int(st.generated_at(len(seq.generated))))
        seq.finished = bool(st.finished)

    def commit(self, step: _Step, tokens: Optional[np.ndarray] = None) -> List[tuple]:
        prod = self._s.commit(step.native, None if tokens is None else np.ascontiguousarray(tokens, dtype=np.int32))
        out = []
        for p in prod:
            seq = self._by_id[p.seq.request_id]
            out.append((seq, int(p.gen_index), int(p.row), p))
        for seq in step.seqs:
            self._mirror(seq)
        return out

    def patch(self, produced: List[tuple], tokens: np.ndarray) -> None:
        self._s.patch([p[3] for p in produced], np.ascontiguousarray(tokens, dtype=np.int32))
        for seq, gi, row, _ in produced:
            st = self._state[seq.request_id]
            n = int(st.num_generated())
            if gi < n and gi < len(seq.generated):
                seq.generated[gi] = int(tokens[row])
            if n < len(seq.generated):            # the native side saw an end-of-sequence token and dropped what came after
                del seq.generated[n:]
            seq.finished = bool(st.finished)
            seq.num_computed = int(st.num_computed)

    def forget(self, request_id: int) -> None:
        self._by_id.pop(request_id, None)
        self._state.pop(request_id, None)
