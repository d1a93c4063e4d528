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


# ----------------------------------------------------------------------------------------- the pipeline's adapter
def _offsets(Tcap, Bcap, max_blocks):
    sizes = [("ids", Tcap), ("positions", Tcap), ("slot_map", Tcap), ("tok_src", Tcap), ("tok_dst", Bcap), ("logit_idx", Bcap),
             ("past_lens", Bcap), ("subsequence_begins", Bcap + 1), ("block_indices_begins", Bcap + 1), ("block_indices", Bcap * max_blocks)]
    offs, off = {}, 0
    for name, n in sizes:
        offs[name] = (off, n)
        off += (n + 3) // 4 * 4
    return offs, off


@pytest.mark.parametrize("split_fuse", [False, True])
def test_native_adapter_writes_the_same_descriptors_as_the_python_scheduler(split_fuse):
    from openvino_b200.genai.native_scheduler import NativeScheduler, make_layout
    cfg = SchedulerConfig(max_num_batched_tokens=24, max_num_seqs=4, num_kv_blocks=7, block_size=4, dynamic_split_fuse=split_fuse)
    py, nat = Scheduler(cfg), NativeScheduler(cfg)
    offs, words = _offsets(24, 4, 8)
    lay = make_layout(offs, 24, 4, 8)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 100, size=n).astype(np.int32) for n in (7, 9, 5, 10, 3, 6)]
    a_seqs = [Sequence(i, p, max_new_tokens=5) for i, p in enumerate(prompts)]
    b_seqs = [Sequence(i, p, max_new_tokens=5) for i, p in enumerate(prompts)]
    for a, b in zip(a_seqs, b_seqs):
        py.add(a)
        nat.add(b)
    step_no = 0
    while py.has_unfinished():
        sa, sb = py.schedule(), nat.schedule()
        assert sa is not None and sb is not None
        da, db = np.zeros(words, np.int32), np.zeros(words, np.int32)
        py.fill(sa, {name: da[o:o + n] for name, (o, n) in offs.items()})
        nat.fill_flat(sb, db, lay)
        # block ids may differ between the two free lists only if the policies diverge; they must not
        assert np.array_equal(da, db), "descriptor of step %d differs" % step_no
        toks = (np.arange(len(sa.seqs), dtype=np.int32) + 3 * step_no) % 50
        pa, pb = py.commit(sa, None), nat.commit(sb, None)      # asynchronous form: placeholders first
        py.patch(pa, toks)
        nat.patch(pb, toks)
        assert [(p[0].request_id, p[1], p[2]) for p in pa] == [(p[0].request_id, p[1], p[2]) for p in pb]
        step_no += 1
        assert step_no < 500
    assert not nat.has_unfinished()
    assert [s.generated for s in a_seqs] == [s.generated for s in b_seqs]
    assert all(s.finished for s in b_seqs) and nat.num_preemptions == py.num_preemptions


def test_native_adapter_stops_at_eos_and_drops_later_tokens():
    from openvino_b200.genai.native_scheduler import NativeScheduler
    cfg = SchedulerConfig(max_num_batched_tokens=16, max_num_seqs=2, num_kv_blocks=8, block_size=4)
    nat = NativeScheduler(cfg)
    s = Sequence(0, np.arange(5, dtype=np.int32), max_new_tokens=10, eos_token_id=42, ignore_eos=False)
    nat.add(s)
    st1 = nat.schedule()
    p1 = nat.commit(st1, None)            # prompt step, token not known yet
    st2 = nat.schedule()                  # look-ahead: the next decode step is launched before the token arrives
    p2 = nat.commit(st2, None)
    nat.patch(p1, np.array([42], np.int32))     # first token is EOS
    nat.patch(p2, np.array([7], np.int32))      # sampled after the EOS: dropped
    assert s.finished and s.generated == [42] and not nat.has_unfinished()


def test_prefix_caching_shares_full_prompt_blocks():
    from openvino_b200.genai.native_scheduler import NativeScheduler, make_layout
    cfg = SchedulerConfig(max_num_batched_tokens=64, max_num_seqs=4, num_kv_blocks=16, block_size=4, enable_prefix_caching=True)
    nat = NativeScheduler(cfg)
    offs, words = _offsets(64, 4, 8)
    lay = make_layout(offs, 64, 4, 8)
    common = np.arange(100, 110, dtype=np.int32)                           # 10 tokens: two full blocks and a half
    a = Sequence(0, np.concatenate([common, np.array([1, 2, 3], np.int32)]), max_new_tokens=2)
    nat.add(a)
    st = nat.schedule()
    assert st.num_new == [13]
    nat.commit(st, np.array([5], np.int32))
    blocks_a = list(nat._state[0].blocks)
    # the second request arrives while the first is still running: it takes over the two full common blocks
    b = Sequence(1, np.concatenate([common, np.array([9, 9], np.int32)]), max_new_tokens=2)
    nat.add(b)
    while True:
        st = nat.schedule()
        if any(s.request_id == 1 for s in st.seqs):
            break
        nat.commit(st, np.zeros(len(st.seqs), np.int32))
    i = [s.request_id for s in st.seqs].index(1)
    assert st.num_new[i] == 12 - 8 and nat.prefix_hit_tokens == 8
    d = np.zeros(words, np.int32)
    nat.fill_flat(st, d, lay)
    o = offs["past_lens"][0]
    assert d[o + i] == 8
    assert list(nat._state[1].blocks)[:2] == blocks_a[:2] and list(nat._state[1].blocks)[2] != blocks_a[2]
    # run everything to the end; shared blocks are released once, cached blocks stay reusable
    nat.commit(st, np.zeros(len(st.seqs), np.int32))
    for _ in range(20):
        if not nat.has_unfinished():
            break
        st = nat.schedule()
        nat.commit(st, np.zeros(len(st.seqs), np.int32))
    assert not nat.has_unfinished() and nat.num_free_blocks() == cfg.num_kv_blocks
    c = Sequence(2, np.concatenate([common, np.array([4], np.int32)]), max_new_tokens=1)
    nat.add(c)
    st = nat.schedule()
    assert st.num_new == [11 - 8] and nat.prefix_hit_tokens == 16
    # an exact multiple of the block size still computes its last prompt token
    nat.commit(st, np.zeros(1, np.int32))
    e = Sequence(3, common[:8].copy(), max_new_tokens=1)
    nat.add(e)
    st = nat.schedule()
    assert st.num_new == [4]
