"""The cache manager and the scheduler on the CPU: no page lost, held twice or freed twice under
random orders of requests; windows give pages back; the scheduler's decisions, and what happens
when pages run out."""

import random

import pytest

from quanta_b200.cache import CacheManager, OutOfPages, OutOfSlots
from quanta_b200.engine.scheduler import Request, SamplingParams, Scheduler
from quanta_b200.parts.base import KVCacheSpec

FULL = KVCacheSpec(2, 16, None)
WIN = KVCacheSpec(2, 16, 10)


def test_pages_follow_length_and_come_back():
    m = CacheManager([FULL, FULL, None, FULL], page_size=4, num_pages=6, max_requests=2)
    assert len(m.groups) == 1 and m.groups[0].positions == [0, 1, 3]       # equal needs share pages
    m.add_request("a")
    m.reserve("a", 5)
    assert len(m.groups[0].tables["a"]) == 2
    m.advance("a", 5)
    m.reserve("a", 8)                   # still two pages
    assert m.groups[0].pool.used_count == 2
    m.reserve("a", 9)
    assert m.groups[0].pool.used_count == 3
    with pytest.raises(RuntimeError, match="past its reservation"):
        m.advance("a", 5)
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 13)              # 4 pages wanted, 3 free
    assert m.groups[0].tables["b"] == []            # nothing was taken
    with pytest.raises(OutOfSlots):
        m.add_request("c")
    m.free("a")
    m.reserve("b", 13)
    m.check_invariants()
    m.free("b")
    with pytest.raises(KeyError):
        m.free("b")
    assert m.groups[0].pool.free_count == 6
    m.check_invariants()


def test_groups_with_different_needs_have_their_own_pages():
    m = CacheManager([FULL, WIN, FULL, WIN], page_size=4, num_pages=8, max_requests=2)
    assert [g.positions for g in m.groups] == [[0, 2], [1, 3]]
    m.add_request("a")
    m.reserve("a", 30)
    m.advance("a", 30)
    full, win = m.groups
    assert len([p for p in full.tables["a"] if p >= 0]) == 8
    # window 10: a query at position >= 30 reads keys >= 21, i.e. pages from index 5 on
    assert win.tables["a"][:5] == [-1] * 5 and all(p >= 0 for p in win.tables["a"][5:])
    assert win.pool.used_count == 3
    m.check_invariants()
    m.free("a")
    assert win.pool.free_count == 8 and full.pool.free_count == 8


def test_random_orders_keep_every_page_accounted_for():
    rng = random.Random(0)
    for trial in range(30):
        m = CacheManager([FULL, WIN], page_size=rng.choice([1, 4, 16]), num_pages=rng.randint(3, 40),
                         max_requests=rng.randint(1, 5))
        live, n = {}, 0
        for _ in range(200):
            op = rng.random()
            if op < 0.3 and m.slots.free_count:
                rid = f"r{n}"
                n += 1
                m.add_request(rid)
                live[rid] = 0
            elif op < 0.8 and live:
                rid = rng.choice(list(live))
                k = rng.randint(1, 20)
                try:
                    m.reserve(rid, live[rid] + k)
                except OutOfPages:
                    continue
                m.advance(rid, k)
                live[rid] += k
                assert m.length(rid) == live[rid]
            elif live:
                rid = rng.choice(list(live))
                m.free(rid)
                del live[rid]
            m.check_invariants()
        for rid in list(live):
            m.free(rid)
        m.check_invariants()
        assert all(g.pool.free_count == g.pool.num_pages for g in m.groups)


# ---- scheduler ------------------------------------------------------------------------------------------
class FakeStepper:
    """Stands in for the step function and the sampler: reserves and advances pages as the engine does
    and 'samples' a fixed token."""

    def __init__(self, mgr):
        self.mgr = mgr
        self.steps = []

    def run(self, sched, token=1, eos_after=None):
        while True:
            plan = sched.plan()
            if not plan:
                return
            assert sum(e.count for e in plan) <= sched.max_step_tokens
            for e in plan:
                if not self.mgr.has(e.request.rid):
                    self.mgr.add_request(e.request.rid)
                assert self.mgr.length(e.request.rid) == e.start
                self.mgr.reserve(e.request.rid, e.start + e.count)          # must never raise
            for e in plan:
                self.mgr.advance(e.request.rid, e.count)
            self.steps.append([(e.request.rid, e.start, e.count, e.samples) for e in plan])
            sampled = {}
            for e in plan:
                if e.samples:
                    n = len(e.request.generated)
                    sampled[e.request.rid] = 99 if (eos_after is not None and n >= eos_after) else token
            sched.commit(plan, sampled)
            self.mgr.check_invariants()


def _mgr(pages=64, page=4, slots=4):
    return CacheManager([FULL], page_size=page, num_pages=pages, max_requests=slots)


def test_prompts_are_cut_under_the_budget_and_decoding_goes_first():
    m = _mgr()
    s = Scheduler(m, max_step_tokens=10, prefill_chunk=6)
    a = Request("a", list(range(9)), SamplingParams(max_new_tokens=3))
    b = Request("b", list(range(14)), SamplingParams(max_new_tokens=2))
    s.add(a); s.add(b)
    f = FakeStepper(m)
    f.run(s)
    # step 0: a gets 6 (chunk), b gets 4 (budget); step 1: a's last 3 (samples), b 6 more; ...
    assert f.steps[0] == [("a", 0, 6, False), ("b", 0, 4, False)]
    assert f.steps[1] == [("a", 6, 3, True), ("b", 4, 6, False)]
    assert f.steps[2][0] == ("a", 9, 1, True)                 # decode token first
    assert f.steps[2][1] == ("b", 10, 4, True)
    assert a.generated == [1, 1, 1] and b.generated == [1, 1]
    assert a.finish_reason == "length" and b.finish_reason == "length"
    assert m.stats()["live_requests"] == 0 and m.groups[0].pool.free_count == 64


def test_eos_stops_and_is_not_returned_and_slots_limit_admission():
    m = _mgr(slots=2)
    s = Scheduler(m, max_step_tokens=64, prefill_chunk=64)
    reqs = [Request(i, [1, 2, 3], SamplingParams(max_new_tokens=10, eos_token_ids=(99,))) for i in range(5)]
    for r in reqs:
        s.add(r)
    f = FakeStepper(m)
    f.run(s, eos_after=2)
    assert all(r.generated == [1, 1] and r.finish_reason == "stop" for r in reqs)
    assert max(len(st) for st in f.steps) <= 2                # never more live requests than slots
    order = [rid for st in f.steps for (rid, start, _, _) in st if start == 0]
    assert order == [0, 1, 2, 3, 4]                           # first in, first out


def test_empty_prompt_and_zero_new_tokens():
    s = Scheduler(_mgr())
    with pytest.raises(ValueError, match="empty"):
        s.add(Request("x", [], SamplingParams()))
    r = Request("y", [1], SamplingParams(max_new_tokens=0))
    s.add(r)
    assert r.status == "finished" and s.plan() == []


def test_out_of_pages_preempts_the_newest_and_recomputes():
    m = _mgr(pages=6, page=4, slots=4)           # 24 tokens of cache in all
    s = Scheduler(m, max_step_tokens=64, prefill_chunk=64)
    a = Request("a", list(range(8)), SamplingParams(max_new_tokens=12))
    b = Request("b", list(range(8)), SamplingParams(max_new_tokens=12))
    s.add(a); s.add(b)
    f = FakeStepper(m)
    f.run(s)
    # both finish with all their tokens although 2 * 20 tokens never fit at once
    assert len(a.generated) == 12 and len(b.generated) == 12
    assert a.preemptions == 0 and b.preemptions >= 1           # the newer one gave way
    assert m.preemptions == b.preemptions
    # after the preemption b came back with prompt + generated as its prompt, from position 0
    restarts = [st for st in f.steps for (rid, start, cnt, _) in st if rid == "b" and start == 0]
    assert len(restarts) == 1 + b.preemptions
    assert m.groups[0].pool.free_count == 6


def test_a_request_too_large_for_the_pool_ends_with_out_of_pages():
    m = _mgr(pages=3, page=4, slots=2)           # 12 tokens
    s = Scheduler(m, max_step_tokens=64, prefill_chunk=8)
    big = Request("big", list(range(10)), SamplingParams(max_new_tokens=8))
    small = Request("small", [1, 2], SamplingParams(max_new_tokens=2))
    s.add(big); s.add(small)
    f = FakeStepper(m)
    f.run(s)
    assert big.finish_reason == "out_of_pages" and len(big.generated) < 8
    assert small.finish_reason == "length" and small.generated == [1, 1]
    assert m.groups[0].pool.free_count == 3 and m.stats()["live_requests"] == 0
    # a prompt whose first portion alone exceeds the pool never starts
    s2 = Scheduler(_mgr(pages=1, page=4), max_step_tokens=64, prefill_chunk=64)
    r = Request("r", list(range(9)), SamplingParams(max_new_tokens=1))
    s2.add(r)
    assert s2.plan() == [] and r.finish_reason == "out_of_pages"


def test_position_limit():
    m = _mgr()
    s = Scheduler(m, max_step_tokens=64, prefill_chunk=64, max_position=6)
    r = Request("r", [1, 2, 3, 4], SamplingParams(max_new_tokens=10))
    s.add(r)
    FakeStepper(m).run(s)
    assert r.finish_reason == "length" and len(r.prompt) + len(r.generated) == 6


def test_random_workloads_always_terminate_and_free_everything():
    rng = random.Random(1)
    for trial in range(25):
        m = _mgr(pages=rng.randint(2, 30), page=rng.choice([1, 4, 16]), slots=rng.randint(1, 4))
        s = Scheduler(m, max_step_tokens=rng.randint(1, 40), prefill_chunk=rng.randint(1, 20))
        reqs = [Request(i, list(range(rng.randint(1, 30))), SamplingParams(max_new_tokens=rng.randint(1, 15)))
                for i in range(rng.randint(1, 8))]
        for r in reqs:
            s.add(r)
        FakeStepper(m).run(s)
        assert all(r.status == "finished" for r in reqs)
        assert all(len(r.generated) == r.params.max_new_tokens for r in reqs if r.finish_reason == "length")
        assert m.stats()["live_requests"] == 0
        assert all(g.pool.free_count == g.pool.num_pages for g in m.groups)


def test_a_retention_rule_of_the_mixers_own():
    """The rule is the spec's: the first six positions and a window of ten.  Pages between them go back as the
    window passes them, the sinks' pages never do, and a page is asked about only while it is held."""
    from dataclasses import dataclass
    from quanta_b200.parts.base import CacheSpec, CacheStream, Retention

    @dataclass(frozen=True)
    class SinksAndWindow(Retention):
        sinks: int = 6
        window: int = 10

        def needed_ranges(self, length):
            return [(0, self.sinks), (max(0, length - self.window + 1), None)]

    spec = CacheSpec((CacheStream("latent", 1, 24),), SinksAndWindow())
    m = CacheManager([spec, FULL], page_size=4, num_pages=40, max_requests=2)
    assert len(m.groups) == 2
    g = m.groups[0]
    m.add_request("a")
    length = 0
    for n in (3, 9, 1, 1, 14, 1, 1, 1, 30, 1):
        m.reserve("a", length + n)
        m.advance("a", n)
        length += n
        held = [i for i, p in enumerate(g.tables["a"]) if p >= 0]
        first_in_window = max(0, length - 10 + 1) // 4
        want = sorted(set(i for i in (0, 1) if i * 4 < length) | set(range(first_in_window, -(-length // 4))))
        assert held == want, (length, held, want)
        m.check_invariants()
    assert g.pool.used_count == len(held) and m.groups[1].pool.used_count == -(-length // 4)
    m.free("a")
    assert g.pool.used_count == 0
    m.check_invariants()

    @dataclass(frozen=True)
    class Broken(Retention):
        def needed_ranges(self, length):
            return [(0, 4)]
    bad = CacheManager([CacheSpec((CacheStream("x", 1, 8),), Broken())], page_size=4, num_pages=8, max_requests=1)
    bad.add_request("a")
    bad.reserve("a", 5)
    with pytest.raises(ValueError, match="open range"):
        bad.advance("a", 5)
