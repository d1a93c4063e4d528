"""Continuous-batching scheduler: invariants under preemption, with and without dynamic split-fuse, for the
Python scheduler and the native one (same policy, same step descriptors)."""
import numpy as np
import pytest

from openvino_b200.genai.scheduler import Scheduler, SchedulerConfig, Sequence


def _check_step(sched, st):
    ids = [id(s) for s in st.seqs]
    assert len(ids) == len(set(ids)), "a sequence was scheduled twice in one step"
    w = [id(s) for s in sched.waiting]
    assert len(w) == len(set(w)), "a sequence sits twice in the waiting queue"
    assert not (set(ids) & set(w)), "a scheduled sequence is also waiting"
    for s, n in zip(st.seqs, st.num_new):
        assert n >= 1 and s.num_computed + n <= s.total_len
        need = (s.num_computed + n + sched.cfg.block_size - 1) // sched.cfg.block_size
        assert len(s.blocks) >= need, "scheduled sequence lost its blocks"
    used = [b for s in list(sched.running) + list(sched.waiting) for b in s.blocks]
    assert len(used) == len(set(used)) and len(used) + sched.blocks.num_free() == sched.cfg.num_kv_blocks


@pytest.mark.parametrize("split_fuse", [False, True])
def test_preemption_keeps_the_queues_consistent(split_fuse):
    cfg = SchedulerConfig(max_num_batched_tokens=24, max_num_seqs=4, num_kv_blocks=6, block_size=4, dynamic_split_fuse=split_fuse)
    sched = Scheduler(cfg)
    rng = np.random.default_rng(0)
    seqs = [Sequence(i, rng.integers(0, 100, size=n).astype(np.int32), max_new_tokens=6) for i, n in enumerate((7, 9, 5, 10, 3))]
    for s in seqs:
        sched.add(s)
    steps = 0
    while sched.has_unfinished():
        st = sched.schedule()
        assert st is not None, "nothing could be scheduled although requests are pending"
        _check_step(sched, st)
        sched.commit(st, np.arange(len(st.seqs), dtype=np.int32) + 1)
        steps += 1
        assert steps < 500
    assert sched.num_preemptions > 0, "the configuration is meant to force preemption"
    assert all(s.finished and len(s.generated) == 6 for s in seqs)
    assert sched.blocks.num_free() == cfg.num_kv_blocks


def test_mid_prefill_victim_is_not_scheduled_twice():
    # one decoding sequence needs a block while another is in the middle of its (chunked) prompt
    cfg = SchedulerConfig(max_num_batched_tokens=4, max_num_seqs=2, num_kv_blocks=4, block_size=4, dynamic_split_fuse=True)
    sched = Scheduler(cfg)
    a = Sequence(0, np.arange(4, dtype=np.int32), max_new_tokens=8)
    b = Sequence(1, np.arange(11, dtype=np.int32), max_new_tokens=2)
    sched.add(a)
    sched.add(b)
    for _ in range(40):
        if not sched.has_unfinished():
            break
        st = sched.schedule()
        assert st is not None
        _check_step(sched, st)
        sched.commit(st, np.zeros(len(st.seqs), dtype=np.int32))
    assert a.finished and b.finished


# ----------------------------------------------------------------------------------------- native scheduler
def _native(cfg):
    from openvino_b200 import _ovcore as core
    c = core.SchedulerConfig()
    c.max_num_batched_tokens, c.max_num_seqs, c.num_kv_blocks = cfg.max_num_batched_tokens, cfg.max_num_seqs, cfg.num_kv_blocks
    c.block_size, c.dynamic_split_fuse = cfg.block_size, cfg.dynamic_split_fuse
    return core.Scheduler(c)


@pytest.mark.parametrize("split_fuse", [False, True])
def test_native_scheduler_matches_python_under_preemption(split_fuse):
    cfg = SchedulerConfig(max_num_batched_tokens=24, max_num_seqs=4, num_kv_blocks=6, block_size=4, dynamic_split_fuse=split_fuse)
    py, nat = Scheduler(cfg), _native(cfg)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 100, size=n).astype(np.int32) for n in (7, 9, 5, 10, 3)]
    pseqs = [Sequence(i, p, max_new_tokens=6) for i, p in enumerate(prompts)]
    nseqs = [nat.add(i, p.tolist(), 6, -1, True) for i, p in enumerate(prompts)]
    for s in pseqs:
        py.add(s)
    steps = 0
    while py.has_unfinished():
        assert nat.has_unfinished()
        a, b = py.schedule(), nat.schedule()
        assert a is not None and b is not None
        assert [s.request_id for s in a.seqs] == [s.request_id for s in b.seqs]
        assert list(a.num_new) == list(b.num_new) and (a.T, a.max_q_len, a.max_ctx) == (b.T, b.max_q_len, b.max_ctx)
        ids = [s.request_id for s in b.seqs]
        assert len(ids) == len(set(ids))
        toks = np.arange(len(a.seqs), dtype=np.int32) + 1
        py.commit(a, toks)
        nat.commit(b, toks)
        steps += 1
        assert steps < 500
    assert not nat.has_unfinished()
    assert nat.num_preemptions() == py.num_preemptions > 0
    assert nat.num_free_blocks() == cfg.num_kv_blocks
    assert [list(s.generated) for s in nseqs] == [list(s.generated) for s in pseqs]
