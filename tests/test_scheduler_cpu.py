"""The scheduler's decisions (no GPU): admission, portions under the token budget,
decoding, and what happens when pages run out."""
import random

import pytest

from llm_serving_engine_b200.engine.scheduler import GenerationRequest, Scheduler


def request(name, prompt, new=4, **kw):
    return GenerationRequest(name, list(range(prompt)), new, **kw)


def names(requests):
    return [r.request_id for r in requests]


def test_admission_fcfs_up_to_the_batch_size():
    scheduler = Scheduler(2)
    for name in "abc":
        scheduler.enqueue(request(name, 3))
    assert names(scheduler.admit()) == ["a", "b"]
    assert scheduler.admit() == [] and names(scheduler.waiting) == ["c"] and scheduler.has_waiting
    scheduler.release(scheduler.live[0])
    assert names(scheduler.admit()) == ["c"] and not scheduler.idle and not scheduler.has_waiting
    assert names(scheduler.live) == ["b", "c"]


def test_policies_and_static_mode():
    sjf = Scheduler(1, "sjf")
    sjf.enqueue(request("long", 3, new=9))
    sjf.enqueue(request("short", 3, new=2))
    sjf.enqueue(request("short too", 3, new=2))
    assert names(sjf.waiting) == ["short", "short too", "long"]
    assert sjf.admit()[0].request_id == "short"
    priority = Scheduler(1, "priority")
    priority.enqueue(request("low", 3, priority=0))
    priority.enqueue(request("high", 3, priority=5))
    assert priority.admit()[0].request_id == "high"
    static = Scheduler(2, mode="static")
    static.enqueue(request("first", 3))
    assert len(static.admit()) == 1
    static.enqueue(request("late", 3))
    assert static.admit() == []                     # nothing joins a running static batch
    static.release(static.live[0])
    assert static.admit()[0].request_id == "late"
    with pytest.raises(ValueError):
        Scheduler(1, "random")
    with pytest.raises(ValueError):
        Scheduler(1, mode="sometimes")


def test_the_waiting_order_is_that_of_a_sort_at_admission_time():
    rng = random.Random(0)
    for policy in ("fcfs", "sjf", "priority"):
        scheduler = Scheduler(3, policy)
        pool = [request(f"r{i}", 2, new=rng.randrange(1, 5), priority=rng.randrange(3)) for i in range(40)]
        for item in pool:
            scheduler.enqueue(item)
        order = []
        while not scheduler.idle:
            admitted = scheduler.admit()
            order += names(admitted)
            for item in list(scheduler.live):
                scheduler.release(item)
        key = {"fcfs": lambda r: r.arrival, "sjf": lambda r: (r.output_left, r.arrival),
               "priority": lambda r: (-r.priority, r.arrival)}[policy]
        assert order == names(sorted(pool, key=key))


def test_portions_under_the_token_budget():
    a, b, c = request("a", 40), request("b", 10), request("c", 5)
    c.cached = 5
    c.output = [7]                                  # c decodes: one outstanding token
    scheduler = Scheduler(3)
    scheduler.live = [a, b, c]
    plan = scheduler.plan(token_budget=24, chunk=16)
    assert [(r.request_id, n) for r, n in plan] == [("a", 16), ("b", 7), ("c", 1)]
    # every live request gets one token even when the budget is tight
    assert [n for _, n in scheduler.plan(3, 16)] == [1, 1, 1]
    # a prompt is cut to what is left of it
    a.cached = 35
    scheduler.live = [a]
    assert scheduler.plan(100, 16)[0][1] == 5
    scheduler.live = [a, b, c]
    with pytest.raises(RuntimeError):
        scheduler.plan(2, 4)
    c.cached = 6                                    # nothing outstanding: a live request must have a token to run
    with pytest.raises(RuntimeError):
        scheduler.plan(10, 4)


def test_tokens_of_prompt_and_output_are_cut_anywhere():
    r = request("r", 5)
    r.output = [50, 51, 52]
    assert r.length == 8 and r.outstanding == 8 and r.in_prompt
    assert r.tokens(0, 5) == [0, 1, 2, 3, 4] and r.tokens(3, 4) == [3, 4, 50, 51]
    assert r.tokens(5, 2) == [50, 51] and r.tokens(7, 1) == [52] and r.tokens(2, 2) == [2, 3]
    r.cached = 7
    assert r.outstanding == 1 and not r.in_prompt and r.output_left == 1


def test_pages_run_out_the_largest_gives_way_and_replays():
    a, b, c = request("a", 30), request("b", 30), request("c", 30)
    a.cached, b.cached, c.cached = 10, 25, 3
    plan = [(a, 4), (b, 1), (c, 8)]
    scheduler = Scheduler(3)
    scheduler.live = [a, b, c]
    free = {"pages": 9}
    holds = {"a": 1, "b": 2, "c": 0}           # pages a request gives back when it gives way

    def fits(p):
        return sum(n for _, n in p) <= free["pages"]

    def give_way(victim):
        free["pages"] += holds[victim.request_id]
        scheduler.requeue(victim)

    kept, victims, failed = scheduler.shed(plan, fits, give_way)
    # b has cached the most and goes first; the two pages it gives back do not yet suffice
    # (4 + 8 > 11), so a follows; its page counts at once and c runs
    assert names(victims) == ["b", "a"] and failed is None
    assert [(r.request_id, n) for r, n in kept] == [("c", 8)] and free["pages"] == 12
    assert b.cached == 0 and b.evictions == 1 and b.replayed_tokens == 25
    assert names(scheduler.waiting) == ["b", "a"] and scheduler.live == [c]
    # the freed pages of one victim can be enough
    free["pages"], holds["b"] = 9, 5
    a.cached, b.cached = 10, 25
    kept, victims, _ = Scheduler.shed([(a, 4), (b, 1), (c, 8)], fits, lambda v: free.update(pages=free["pages"] + holds[v.request_id]))
    assert names(victims) == ["b"] and [r.request_id for r, _ in kept] == ["a", "c"]
    # afterwards the request feeds prompt and output again in portions
    b.cached = 0
    b.output = [1, 2]
    scheduler.live = [b]
    assert scheduler.plan(100, 16)[0][1] == 16
    # among equals the earlier one in the plan goes first
    a.cached = b.cached = c.cached = 4
    _, victims, _ = Scheduler.shed([(a, 1), (b, 1), (c, 1)], lambda p: len(p) <= 1)
    assert names(victims) == ["a", "b"]


def test_one_request_that_cannot_fit_fails_alone():
    a = request("a", 30)
    kept, victims, failed = Scheduler.shed([(a, 16)], lambda plan: False)
    assert kept == [] and victims == [] and failed is a
    kept, victims, failed = Scheduler.shed([(a, 16)], lambda plan: True)
    assert kept == [(a, 16)] and failed is None


def test_drain_forgets_everyone():
    scheduler = Scheduler(1)
    for name in "abc":
        scheduler.enqueue(request(name, 2))
    scheduler.admit()
    assert names(scheduler.drain()) == ["a", "b", "c"] and scheduler.idle
