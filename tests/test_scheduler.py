"""The scheduler's decisions (no GPU), driven by a fake model that "samples" a fixed function of the
request.  After the reference's scheduler tests (tests/backend_tests.cpp:1109-2084)."""
import random

import pytest

from mimirmind_b200.cache import CacheManager, GroupSpec
from mimirmind_b200.engine.scheduler import Request, Scheduler, SchedulerConfig


def make(pages=64, page_size=16, budget=64, max_active=4, chunk=0, max_seq=1024, window=0):
    groups = [GroupSpec("full", (0,), 1, 16, 0)]
    if window:
        groups.append(GroupSpec("win", (1,), 1, 16, window))
    mgr = CacheManager(groups, page_size, pages, max_requests=max_active)
    return Scheduler(SchedulerConfig(budget, max_active, chunk, max_seq), mgr), mgr


def fake_token(req):
    return (len(req.tokens) * 7 + sum(req.prompt)) % 1000


def run(sched, mgr, max_steps=10000, log=None):
    steps = 0
    while sched.has_work():
        plan = sched.schedule()
        if not plan:
            assert not sched.has_work(), "an empty plan while requests wait or run"
            break
        assert sum(p.count for p in plan) <= sched.cfg.token_budget
        ids = [p.request.id for p in plan]
        assert len(set(ids)) == len(ids)
        if log is not None:
            log.append([(p.request.id, p.start, p.count, p.samples) for p in plan])
        sched.commit(plan, {p.request.id: fake_token(p.request) for p in plan if p.samples})
        mgr.check()
        steps += 1
        assert steps < max_steps
    return steps


def test_prompt_is_cut_under_the_budget_and_last_portion_samples():
    s, m = make(budget=32)
    r = Request("a", list(range(70)), max_new=3)
    s.add(r)
    log = []
    run(s, m, log=log)
    assert [e[0][1:] for e in log[:3]] == [(0, 32, False), (32, 32, False), (64, 6, True)]
    assert log[3] == [("a", 70, 1, True)] and log[4] == [("a", 71, 1, True)]
    assert r.finish_reason == "length" and len(r.generated) == 3      # max_new counts the first token
    assert m.free_pages() == m.total_pages()


def test_decodes_go_first_and_prefill_takes_the_rest():
    s, m = make(budget=16)
    a, b = Request("a", [1, 2, 3], max_new=50), Request("b", list(range(40)), max_new=2)
    s.add(a)
    run_one = s.schedule()
    s.commit(run_one, {"a": 5})
    s.add(b)
    plan = s.schedule()
    assert [(p.request.id, p.count) for p in plan] == [("a", 1), ("b", 15)]
    s.commit(plan, {"a": 6})
    plan = s.schedule()
    assert [(p.request.id, p.count) for p in plan] == [("a", 1), ("b", 15)]


def test_prefill_chunk_cap():
    s, m = make(budget=64, chunk=8)
    s.add(Request("a", list(range(20)), max_new=1))
    log = []
    run(s, m, log=log)
    assert [e[0][2] for e in log] == [8, 8, 4]


def test_fifo_admission_and_max_active():
    s, m = make(max_active=2, budget=64)
    for i in range(4):
        s.add(Request(i, [1] * 5, max_new=2))
    plan = s.schedule()
    assert [p.request.id for p in plan] == [0, 1]
    s.commit(plan, {0: 1, 1: 1})
    plan = s.schedule()
    assert [p.request.id for p in plan] == [0, 1]          # both decode; nobody new: two are active
    s.commit(plan, {0: 1, 1: 1})                          # both reach max_new and leave
    plan = s.schedule()
    assert [p.request.id for p in plan] == [2, 3]


def test_stop_id_ends_a_request_and_is_part_of_the_output():
    s, m = make()
    r = Request("a", [1, 2], max_new=10, stop_ids=(42,))
    s.add(r)
    plan = s.schedule()
    s.commit(plan, {"a": 7})
    plan = s.schedule()
    done = s.commit(plan, {"a": 42})
    assert done == [r] and r.generated == [7, 42] and r.hit_stop
    assert not m.has("a")


def test_context_full_ends_a_request():
    s, m = make(max_seq=8)
    r = Request("a", [1] * 5, max_new=100)
    s.add(r)
    run(s, m)
    assert r.finish_reason == "context" and len(r.tokens) == 8


def test_rejections():
    s, m = make(pages=2, page_size=4, max_seq=64)
    assert not s.add(Request("a", [], max_new=1))
    assert not s.add(Request("b", [1] * 64, max_new=1))             # prompt >= context
    assert not s.add(Request("c", [1] * 9, max_new=1))              # needs 3 pages of 2
    assert [r.finish_reason.split(":")[0] for r in s.finished] == ["rejected"] * 3
    assert not s.has_work()


def test_out_of_pages_preempts_the_newest_and_keeps_its_tokens():
    # 6 pages of 4 tokens; two requests of 8 tokens that each want to grow to 8 + 12
    s, m = make(pages=6, page_size=4, budget=64)
    a, b = Request("a", [1] * 8, max_new=12), Request("b", [2] * 8, max_new=12)
    s.add(a)
    s.add(b)
    log = []
    run(s, m, log=log)
    assert a.finish_reason == "length" and b.finish_reason == "length"
    assert len(a.generated) == 12 and len(b.generated) == 12
    assert b.preemptions >= 1 and a.preemptions == 0               # last in, first out
    assert s.metrics.preempted == b.preemptions
    # what b generated before it was preempted came back as part of its recomputed prompt
    restarts = [e for step in log for e in step if e[0] == "b" and e[1] == 0]
    assert len(restarts) == 1 + b.preemptions and restarts[-1][2] > 8
    assert m.free_pages() == m.total_pages()


def test_preempted_output_equals_unpreempted_output():
    def go(pages):
        s, m = make(pages=pages, page_size=4, budget=64)
        reqs = [Request(i, [i + 1] * (5 + 3 * i), max_new=20) for i in range(3)]
        for r in reqs:
            s.add(r)
        run(s, m)
        return [r.generated for r in reqs], s.metrics.preempted
    roomy, p0 = go(64)
    tight, p1 = go(12)
    assert p0 == 0 and p1 > 0 and roomy == tight


def test_a_lone_request_that_cannot_fit_fails():
    s, m = make(pages=3, page_size=4, budget=64)
    r = Request("a", [1] * 10, max_new=50)
    s.add(r)
    run(s, m)
    assert r.finish_reason == "out_of_pages" and len(r.generated) >= 1
    assert m.free_pages() == m.total_pages() and not s.has_work()


def test_a_failed_lone_request_does_not_hold_up_those_that_wait():
    # A fills the pool while B waits; A's next token finds no page, A is alone and fails; B is admitted in the
    # same call instead of the plan coming back empty with work left
    s, m = make(pages=3, page_size=4, budget=64, max_active=4)
    a, b = Request("a", [1] * 10, max_new=50), Request("b", [2] * 6, max_new=2)
    s.add(a)
    plan = s.schedule()
    assert [(p.request.id, p.count) for p in plan] == [("a", 10)]
    s.add(b)                                   # no page is free for b while a holds all three
    log = []
    while s.has_work():
        s.commit(plan, {p.request.id: fake_token(p.request) for p in plan if p.samples})
        m.check()
        plan = s.schedule()
        assert plan or not s.has_work(), "an empty plan while requests wait or run"
        log.append([(p.request.id, p.count) for p in plan])
    assert a.finish_reason == "out_of_pages" and b.finish_reason == "length" and len(b.generated) == 2
    assert any(step and step[0][0] == "b" for step in log)
    assert m.free_pages() == m.total_pages()


def test_the_serving_loop_survives_a_lone_request_that_runs_out_of_pages():
    # the same through ServingLoop, with a stand-in for the engine that "samples" the fake token
    from types import SimpleNamespace

    from mimirmind_b200.engine.engine import ServingLoop
    s, m = make(pages=3, page_size=4, budget=64, max_active=4)
    eng = SimpleNamespace(sched_cfg=s.cfg, runner=SimpleNamespace(manager=m, native=None, stage_dump=None), use_graphs=False, eos_ids=(),
                          decode_trace=None,
                          _run_plan=lambda plan: {p.request.id: fake_token(p.request) for p in plan if p.samples})
    loop = ServingLoop(eng)
    ha = loop.submit([1] * 10, max_new_tokens=50, use_eos=False)
    loop.step()
    hb = loop.submit([2] * 6, max_new_tokens=2, use_eos=False)
    loop.run_until_idle()
    assert loop.result(ha).stats.finish_reason == "out_of_pages"
    assert loop.result(hb).stats.finish_reason == "length" and len(loop.result(hb).tokens) == 2
    assert m.free_pages() == m.total_pages()


def test_cancel():
    s, m = make()
    s.add(Request("a", [1] * 5, max_new=50))
    s.add(Request("b", [1] * 5, max_new=50))
    plan = s.schedule()
    s.commit(plan, {"a": 1, "b": 1})
    assert s.cancel("a") and not s.cancel("zzz")
    assert [r.id for r in s.running] == ["b"] and not m.has("a")


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_and_leak_nothing(seed):
    rng = random.Random(seed)
    s, m = make(pages=rng.randint(8, 30), page_size=rng.choice([4, 8]), budget=rng.choice([8, 24, 64]),
                max_active=rng.randint(1, 4), chunk=rng.choice([0, 5]), max_seq=200, window=rng.choice([0, 16]))
    reqs = [Request(i, [rng.randrange(50) for _ in range(rng.randint(1, 40))], max_new=rng.randint(1, 30),
                    stop_ids=(999,)) for i in range(12)]
    pending = list(reqs)
    steps = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.4:
            s.add(pending.pop(0))
        if s.has_work():
            plan = s.schedule()
            s.commit(plan, {p.request.id: fake_token(p.request) for p in plan if p.samples})
            m.check()
        steps += 1
        assert steps < 5000
    assert all(r.state == "finished" for r in reqs)
    for g in m.groups:
        assert m.free_pages(g) == m.total_pages(g)
    for r in reqs:
        if r.finish_reason == "length":
            assert len(r.generated) == r.max_new
