"""The scheduler's decisions, driven by a fake executor (CPU, torch-free)."""

import os
import sys

import pytest

from servelab_b200.cache import CacheManager
from servelab_b200.config import SchedulerConfig
from servelab_b200.engine import Scheduler, Sequence, SequenceStatus
from servelab_b200.sampling import SamplingParams


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        self.t += 1.0
        return self.t


def make(num_pages=64, page=8, budget=24, max_seqs=4, windows=(None,), chunked=True,
         policy="fcfs", eos=(), max_len=1 << 30, slots=None):
    cache = CacheManager(list(windows), num_pages, page, slots or max_seqs)
    sched = Scheduler(SchedulerConfig(max_num_seqs=max_seqs, max_num_batched_tokens=budget,
                                      chunked_prefill=chunked, policy=policy),
                      cache, Clock(), eos_token_ids=eos, max_model_len=max_len)
    return sched, cache


def add(sched, rid, n, max_tokens=12, t=None, priority=0, **kw):
    s = Sequence(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, **kw),
                 priority=priority, arrival_time=t if t is not None else len(sched.waiting))
    sched.add_request(s)
    return s


def drive(sched, cache, token=7, max_steps=500, log=None, after=None):
    """Run to completion: 'execute' each plan by sampling ``token`` for every
    portion that wants logits.  Checks the invariants after every step."""
    finished, steps = [], 0
    while sched.has_unfinished():
        steps += 1
        assert steps <= max_steps, "scheduler does not terminate"
        plan = sched.schedule()
        finished += plan.aborted
        seen = set()
        for p in plan.portions:
            assert p.seq.request_id not in seen, "a request twice in one step"
            seen.add(p.seq.request_id)
            assert p.start == p.seq.num_computed_tokens
            assert p.start + p.num_tokens <= p.seq.get_len()
            table = cache.block_table(p.seq.request_id, 0)
            assert len(table) * cache.page_size >= p.start + p.num_tokens
        assert plan.num_batched_tokens <= sched.cfg.max_num_batched_tokens or not sched.cfg.chunked_prefill
        if log is not None:
            log.append([(p.seq.request_id, p.start, p.num_tokens) for p in plan.portions])
        sampled = {p.seq.request_id: token for p in plan.portions if p.wants_logits}
        finished += sched.update_after_exec(plan, sampled)
        cache.check_invariants()
        for s in sched.running:
            assert s.num_computed_tokens == s.get_len() - 1 or s.num_uncomputed() > 1
        if after:
            after(steps)
    return finished, steps


def test_budget_split_matches_the_reference_walkthrough():
    """Budget 24, prompts 1/9/40/70: the first steps are 1+9+14, then two decodes
    plus 22 prompt tokens, ... (the sequence the reference's scheduler produces)."""
    sched, cache = make()
    for i, n in enumerate((1, 9, 40, 70)):
        add(sched, f"r{i}", n)
    log = []
    finished, _ = drive(sched, cache, log=log)
    assert log[0] == [("r0", 0, 1), ("r1", 0, 9), ("r2", 0, 14)]
    assert log[1] == [("r0", 1, 1), ("r1", 9, 1), ("r2", 14, 22)]
    assert log[2] == [("r0", 2, 1), ("r1", 10, 1), ("r2", 36, 4), ("r3", 0, 18)]
    assert all(sum(n for _, _, n in step) <= 24 for step in log)
    assert sorted(s.request_id for s in finished) == ["r0", "r1", "r2", "r3"]
    assert all(s.num_output_tokens == 12 and s.status == SequenceStatus.FINISHED_LENGTH
               for s in finished)
    assert all(p.num_free() == p.num_pages for p in cache.pools)


def test_cross_check_with_the_reference_scheduler():
    """Same arrivals through the reference's own scheduler (if its tree is at hand):
    identical (request, start, n) lists while no preemption happens."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_root = os.environ.get("SERVELAB_REFERENCE", os.path.join(here, "baseline", "_ref"))
    if not os.path.isdir(os.path.join(ref_root, "servelab")):
        pytest.skip("reference tree not available")
    sys.path.insert(0, ref_root)
    try:
        from servelab.config import CacheConfig as RC, SchedulerConfig as RS
        from servelab.engine.sampling_params import SamplingParams as RP
        from servelab.engine.scheduler import Scheduler as RSched
        from servelab.engine.sequence import Sequence as RSeq
        from servelab.kv_cache.manager import BlockManager
    except Exception as e:                                    # pragma: no cover
        pytest.skip(f"reference not importable: {e}")
    finally:
        sys.path.remove(ref_root)
    bm = BlockManager(64, 8, enable_prefix_caching=False)
    rs = RSched(RS(max_num_seqs=4, max_num_batched_tokens=24), RC(block_size=8,
                enable_prefix_caching=False), bm, Clock(), eos_token_id=-1)
    sched, cache = make()
    for i, n in enumerate((1, 9, 40, 70)):
        add(sched, f"r{i}", n)
        rs.add_request(RSeq(f"r{i}", list(range(1, n + 1)), RP(max_tokens=12), arrival_time=i))
    ours = []
    drive(sched, cache, log=ours)
    theirs = []
    while rs.has_unfinished():
        out = rs.schedule()
        step = [(s.request_id, s.num_computed_tokens, 1) for s in out.decodes]
        step += [(p.seq.request_id, p.num_computed, p.num_new_tokens) for p in out.prefills]
        sampled = {}
        for p in out.prefills:
            p.seq.num_computed_tokens = p.num_computed + p.num_new_tokens
            if p.seq.num_computed_tokens == p.seq.num_prompt_tokens:
                sampled[p.seq.request_id] = 7
        for s in out.decodes:
            s.num_computed_tokens = s.get_len()
            sampled[s.request_id] = 7
        rs.update_after_exec(sampled)
        theirs.append(step)
    assert [sorted(s) for s in ours] == [sorted(s) for s in theirs]


def test_fcfs_and_priority_order():
    sched, cache = make(budget=8, max_seqs=1)
    add(sched, "late", 4, t=5.0)
    add(sched, "early", 4, t=1.0)
    log = []
    drive(sched, cache, log=log)
    assert log[0][0][0] == "early"
    sched, cache = make(budget=8, max_seqs=1, policy="priority")
    add(sched, "low", 4, t=1.0, priority=5)
    add(sched, "high", 4, t=2.0, priority=0)
    log = []
    drive(sched, cache, log=log)
    assert log[0][0][0] == "high"


def test_max_num_seqs_caps_running():
    sched, cache = make(budget=64, max_seqs=2)
    for i in range(5):
        add(sched, f"r{i}", 6, max_tokens=3)
    finished, _ = drive(sched, cache, after=lambda _: None)
    assert len(finished) == 5
    sched, cache = make(budget=64, max_seqs=2)
    for i in range(5):
        add(sched, f"r{i}", 6, max_tokens=3)
    while sched.has_unfinished():
        plan = sched.schedule()
        assert len(sched.running) <= 2
        sched.update_after_exec(plan, {p.seq.request_id: 7 for p in plan.portions if p.wants_logits})


def test_pages_run_out_latest_arrival_is_preempted_and_everyone_finishes():
    sched, cache = make(num_pages=10, page=4, budget=32, max_seqs=3)
    seqs = [add(sched, f"r{i}", 10, max_tokens=10, t=float(i)) for i in range(3)]
    preempted = []
    orig = sched._preempt

    def spy(seq, out):
        preempted.append(seq.request_id)
        orig(seq, out)
    sched._preempt = spy
    finished, _ = drive(sched, cache)
    assert len(finished) == 3 and preempted, "the pool is too small not to preempt"
    assert preempted[0] == "r2", "the victim is the latest arrival"
    for s in seqs:
        assert s.num_output_tokens == 10            # max_tokens counts across preemptions
        assert s.status == SequenceStatus.FINISHED_LENGTH
        assert s.token_ids[:10] == list(range(1, 11))
    assert sched.num_preemptions == len(preempted)
    assert sum(s.metrics.num_preemptions for s in seqs) == len(preempted)


def test_never_fits_is_reported_as_aborted():
    sched, cache = make(num_pages=4, page=4, budget=64)
    big = add(sched, "big", 30, t=0.0)
    ok = add(sched, "ok", 5, max_tokens=2, t=1.0)
    finished, _ = drive(sched, cache)
    assert big in finished and big.status == SequenceStatus.FINISHED_ABORTED
    assert ok.status == SequenceStatus.FINISHED_LENGTH
    # a request that outgrows the whole pool while decoding ends the same way
    sched, cache = make(num_pages=2, page=4, budget=64)
    grow = add(sched, "grow", 6, max_tokens=50)
    finished, _ = drive(sched, cache)
    assert grow.status == SequenceStatus.FINISHED_ABORTED and grow.num_output_tokens >= 2


def test_position_limit():
    sched, cache = make(max_len=10)
    too_long = add(sched, "long", 11)
    s = add(sched, "s", 6, max_tokens=50)
    drive(sched, cache)
    assert too_long.status == SequenceStatus.FINISHED_ABORTED
    assert s.status == SequenceStatus.FINISHED_LENGTH and s.get_len() == 10


def test_eos_stop_ids_and_ignore_eos():
    sched, cache = make(eos=(7,))
    a = add(sched, "a", 4)
    b = add(sched, "b", 4, ignore_eos=True, max_tokens=3)
    c = add(sched, "c", 4, stop_token_ids=(7,))
    drive(sched, cache)
    assert a.status == SequenceStatus.FINISHED_EOS and a.num_output_tokens == 1
    assert b.status == SequenceStatus.FINISHED_LENGTH and b.num_output_tokens == 3
    assert c.status == SequenceStatus.FINISHED_EOS


def test_abort_waiting_and_running():
    sched, cache = make(budget=8, max_seqs=1)
    a = add(sched, "a", 20)
    b = add(sched, "b", 5)
    sched.update_after_exec(sched.schedule(), {})
    assert sched.abort_request("b") is b and b.status == SequenceStatus.FINISHED_ABORTED
    assert sched.abort_request("a") is a and sched.abort_request("a") is None
    assert not sched.has_unfinished()
    cache.check_invariants()
    assert cache.pools[0].num_free() == cache.pools[0].num_pages


def test_unchunked_mode_runs_whole_prompts_and_holds_decodes():
    sched, cache = make(budget=16, chunked=False)
    add(sched, "a", 40, max_tokens=2, t=0.0)
    plan = sched.schedule()
    assert [(p.seq.request_id, p.num_tokens) for p in plan.portions] == [("a", 40)]
    sched.update_after_exec(plan, {"a": 7})
    add(sched, "b", 5, max_tokens=2, t=1.0)
    plan = sched.schedule()
    assert [p.seq.request_id for p in plan.portions] == ["b"], "no decode while one waits"


def test_unchunked_mode_decodes_when_the_waiting_request_cannot_get_pages():
    """8 pages of 8: 'a' (40 tokens) holds 5 of them while it decodes, 'b' (40 tokens) waits
    and cannot be admitted.  Holding the decodes back for 'b' would leave every step empty;
    'a' has to go on, finish and free its pages."""
    sched, cache = make(num_pages=8, page=8, budget=16, chunked=False)
    a = add(sched, "a", 40, max_tokens=6, t=0.0)
    plan = sched.schedule()
    sched.update_after_exec(plan, {"a": 7})
    b = add(sched, "b", 40, max_tokens=6, t=1.0)
    plan = sched.schedule()
    assert [(p.seq.request_id, p.num_tokens) for p in plan.portions] == [("a", 1)]
    sched.update_after_exec(plan, {"a": 7})
    finished, steps = drive(sched, cache, max_steps=60)
    assert {s.request_id for s in finished} == {"a", "b"}
    assert a.num_output_tokens == 6 and b.num_output_tokens == 6
    assert all(p.num_free() == p.num_pages for p in cache.pools)


def test_unchunked_mode_decodes_when_every_sequence_slot_is_taken():
    sched, cache = make(budget=16, chunked=False, max_seqs=1)
    add(sched, "a", 10, max_tokens=3, t=0.0)
    add(sched, "b", 10, max_tokens=3, t=1.0)
    finished, _ = drive(sched, cache, max_steps=40)
    assert [s.request_id for s in finished] == ["a", "b"]


def test_window_group_frees_pages_during_a_long_request():
    sched, cache = make(num_pages=12, page=4, budget=8, windows=(None, 6), max_seqs=1)
    s = add(sched, "a", 30, max_tokens=10)
    used = []
    drive(sched, cache, after=lambda _: used.append(cache.pools[1].num_pages - cache.pools[1].num_free()))
    assert s.status == SequenceStatus.FINISHED_LENGTH
    assert max(used) <= 5, "the windowed group never holds the whole request"


def test_state_slots_limit_admission():
    sched, cache = make(max_seqs=4, slots=2, budget=64)
    for i in range(4):
        add(sched, f"r{i}", 4, max_tokens=2)
    plan = sched.schedule()
    assert len(plan.portions) == 2 and len(sched.waiting) == 2
    finished, _ = drive(sched, cache)
    assert len(finished) + 0 >= 2 and not sched.has_unfinished()
