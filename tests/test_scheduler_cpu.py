"""The scheduler's decisions (no GPU): admission, portions under the token budget,
decoding, and what happens when pages run out."""
import pytest

from llm_serving_engine_b200.engine.scheduler import (IterationScheduler, RequestState, plan_iteration,
                                                      resolve_page_pressure)


def request(name, prompt, new=4, **kw):
    return RequestState(request_id=name, prompt_token_ids=list(range(prompt)), max_new_tokens=new, **kw)


def test_admission_fcfs_up_to_the_batch_size():
    scheduler = IterationScheduler(2)
    for name in "abc":
        scheduler.add(request(name, 3))
    assert [r.request_id for r in scheduler.admit()] == ["a", "b"]
    assert scheduler.admit() == [] and [r.request_id for r in scheduler.waiting] == ["c"]
    scheduler.finish(scheduler.active[0])
    assert [r.request_id for r in scheduler.admit()] == ["c"] and not scheduler.empty


def test_policies_and_static_mode():
    sjf = IterationScheduler(1, "sjf")
    sjf.add(request("long", 3, new=9))
    sjf.add(request("short", 3, new=2))
    assert sjf.admit()[0].request_id == "short"
    priority = IterationScheduler(1, "priority")
    priority.add(request("low", 3, priority=0))
    priority.add(request("high", 3, priority=5))
    assert priority.admit()[0].request_id == "high"
    static = IterationScheduler(2, mode="static")
    static.add(request("first", 3))
    assert len(static.admit()) == 1
    static.add(request("late", 3))
    assert static.admit() == []                     # nothing joins a running static batch
    static.finish(static.active[0])
    assert static.admit()[0].request_id == "late"
    with pytest.raises(ValueError):
        IterationScheduler(1, "random")


def test_portions_under_the_token_budget():
    a, b, c = request("a", 40), request("b", 10), request("c", 5)
    c.processed_tokens = 5
    c.generated_token_ids = [7]                     # c decodes: one outstanding token
    plan = plan_iteration([a, b, c], max_tokens_per_step=24, prefill_chunk_size=16)
    assert [(r.request_id, n) for r, n in plan] == [("a", 16), ("b", 7), ("c", 1)]
    # every active request gets one token even when the budget is tight
    plan = plan_iteration([a, b, c], max_tokens_per_step=3, prefill_chunk_size=16)
    assert [n for _, n in plan] == [1, 1, 1]
    # a prompt is cut to what is left of it
    a.processed_tokens = 35
    assert plan_iteration([a], 100, 16)[0][1] == 5
    with pytest.raises(RuntimeError):
        plan_iteration([a, b, c], max_tokens_per_step=2, prefill_chunk_size=4)


def test_pages_run_out_the_largest_is_preempted_and_recomputes():
    a, b, c = request("a", 30), request("b", 30), request("c", 30)
    a.processed_tokens, b.processed_tokens, c.processed_tokens = 10, 25, 3
    plan = [(a, 4), (b, 1), (c, 8)]
    scheduler = IterationScheduler(3)
    scheduler.active = [a, b, c]
    free = {"pages": 9}
    holds = {"a": 1, "b": 2, "c": 0}           # pages a preempted request gives back

    def fits(p):
        return sum(n for _, n in p) <= free["pages"]

    def preempt(victim):
        free["pages"] += holds[victim.request_id]
        scheduler.preempt(victim)

    kept, victims, failed = resolve_page_pressure(plan, fits, preempt)
    # b has processed the most and goes first; the two pages it gives back do not yet suffice
    # (4 + 8 > 11), so a follows; its page counts at once and c runs
    assert [r.request_id for r in victims] == ["b", "a"] and failed is None
    assert [(r.request_id, n) for r, n in kept] == [("c", 8)] and free["pages"] == 12
    assert b.processed_tokens == 0 and b.preemptions == 1 and b.recomputed_tokens == 25
    assert [r.request_id for r in scheduler.waiting] == ["b", "a"] and scheduler.active == [c]
    # the freed pages of one victim can be enough
    free["pages"], holds["b"] = 9, 5
    a.processed_tokens, b.processed_tokens = 10, 25
    kept, victims, _ = resolve_page_pressure([(a, 4), (b, 1), (c, 8)], fits, lambda v: free.update(pages=free["pages"] + holds[v.request_id]))
    assert [r.request_id for r in victims] == ["b"] and [r.request_id for r, _ in kept] == ["a", "c"]
    # after the preemption the request replays prompt and generated tokens in portions
    b.processed_tokens = 0
    b.generated_token_ids = [1, 2]
    assert plan_iteration([b], 100, 16)[0][1] == 16


def test_one_request_that_cannot_fit_fails_alone():
    a = request("a", 30)
    kept, victims, failed = resolve_page_pressure([(a, 16)], lambda plan: False)
    assert kept == [] and victims == [] and failed is a
    kept, victims, failed = resolve_page_pressure([(a, 16)], lambda plan: True)
    assert kept == [(a, 16)] and failed is None
