"""Iteration-level scheduling: who is live, how many tokens each live request runs in
the next step, and who gives way when the pages run out.  Pure host code.

The behaviour is the reference's (``src/llmserve/scheduler.py:40-97``,
``src/llmserve/engine.py:256-267,372-400``); the shape is this engine's own:

* Requests wait in a heap keyed by the admission policy at the time they are queued
  (``fcfs``: arrival; ``sjf``: output tokens still to come, then arrival; ``priority``:
  higher first, then arrival).  The key of a waiting request cannot change while it
  waits, so the heap pops in the order a sort at admission time would give.
* ``admit`` moves requests from the heap to the live list until ``max_live`` are live;
  in ``static`` mode only when nobody is live.  Admission does not look at pages.
* ``plan`` gives every live request one token, then, in live order, more of what it has
  outstanding (prompt not yet cached, or prompt and output to replay), at most ``chunk``
  per request and step, while the step's token budget lasts.
* ``shed`` is called with a plan that may not fit the free pages: while it does not and
  more than one request is planned, the planned request with the most cached tokens
  gives way (``requeue``: its pages go back at once, it returns to the heap and later
  feeds prompt and output again, sampling nothing until it has caught up).  A request
  that does not fit even alone is reported as failed.
"""
from __future__ import annotations

import heapq
from typing import Any, Callable

POLICIES = ("fcfs", "sjf", "priority")
MODES = ("continuous", "static")


class GenerationRequest:
    """One request as the scheduler sees it.  ``cached`` counts the tokens (prompt first,
    then output) whose keys and values are in the cache; a request decodes when only its
    last output token is outstanding."""

    __slots__ = ("request_id", "prompt", "output", "max_new_tokens", "priority", "callback", "future",
                 "cached", "arrival", "evictions", "replayed_tokens")

    def __init__(self, request_id: str, prompt: list[int], max_new_tokens: int, callback: Callable[[int], Any] | None = None,
                 priority: int = 0, future: Any = None) -> None:
        self.request_id = request_id
        self.prompt = prompt
        self.output: list[int] = []
        self.max_new_tokens = max_new_tokens
        self.priority = priority
        self.callback = callback
        self.future = future
        self.cached = 0
        self.arrival = -1
        self.evictions = 0
        self.replayed_tokens = 0

    @property
    def length(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def outstanding(self) -> int:
        return len(self.prompt) + len(self.output) - self.cached

    @property
    def in_prompt(self) -> bool:
        return self.cached < len(self.prompt)

    @property
    def output_left(self) -> int:
        return self.max_new_tokens - len(self.output)

    def tokens(self, first: int, count: int) -> list[int]:
        """Tokens ``first .. first + count - 1`` of prompt followed by output."""
        boundary = len(self.prompt)
        if first >= boundary:
            return self.output[first - boundary:first - boundary + count]
        head = self.prompt[first:first + count]
        if len(head) < count:
            head = head + self.output[:count - len(head)]
        return head

    def __repr__(self) -> str:
        return f"GenerationRequest({self.request_id!r}, cached {self.cached}/{self.length}, output {len(self.output)}/{self.max_new_tokens})"


Plan = list  # of (GenerationRequest, number of tokens in the next step)


class Scheduler:
    def __init__(self, max_live: int, policy: str = "fcfs", mode: str = "continuous") -> None:
        if policy not in POLICIES:
            raise ValueError(f"policy must be one of {', '.join(POLICIES)}")
        if mode not in MODES:
            raise ValueError(f"mode must be one of {', '.join(MODES)}")
        self.max_live = int(max_live)
        self.policy = policy
        self.mode = mode
        self.live: list[GenerationRequest] = []
        self._heap: list[tuple] = []
        self._arrivals = 0

    # -- waiting ---------------------------------------------------------------------------
    def _rank(self, request: GenerationRequest) -> tuple:
        if self.policy == "sjf":
            return (request.output_left, request.arrival)
        if self.policy == "priority":
            return (-request.priority, request.arrival)
        return (request.arrival,)

    def enqueue(self, request: GenerationRequest) -> None:
        """A new arrival, or a request that gave way: it gets a fresh arrival number (the back of
        the line among equals)."""
        request.arrival = self._arrivals
        self._arrivals += 1
        heapq.heappush(self._heap, (self._rank(request), request))

    @property
    def waiting(self) -> list[GenerationRequest]:
        """The waiting requests in the order they would be admitted."""
        return [request for _, request in sorted(self._heap, key=lambda item: item[0])]

    @property
    def has_waiting(self) -> bool:
        return bool(self._heap)

    @property
    def idle(self) -> bool:
        return not self._heap and not self.live

    # -- live ------------------------------------------------------------------------------
    def admit(self) -> list[GenerationRequest]:
        if self.mode == "static" and self.live:
            return []                          # nothing joins a batch that is running
        admitted = []
        while self._heap and len(self.live) < self.max_live:
            _, request = heapq.heappop(self._heap)
            self.live.append(request)
            admitted.append(request)
        return admitted

    def release(self, request: GenerationRequest) -> None:
        """The request has ended (or failed): it leaves the live list."""
        self.live.remove(request)

    def requeue(self, request: GenerationRequest) -> None:
        """The request gives way: nothing of it is cached any more, and it waits again."""
        self.live.remove(request)
        request.replayed_tokens += request.cached
        request.cached = 0
        request.evictions += 1
        self.enqueue(request)

    def drain(self) -> list[GenerationRequest]:
        """Forget every request; returns them (live first, then waiting)."""
        everyone = self.live + self.waiting
        self.live = []
        self._heap = []
        return everyone

    # -- the next step ---------------------------------------------------------------------
    def plan(self, token_budget: int, chunk: int) -> Plan:
        """(request, tokens) for every live request, in live order."""
        spare = token_budget - len(self.live)      # what is left once everybody has its one token
        if spare < 0:
            raise RuntimeError("the step's token budget is below the number of live requests")
        plan = []
        for request in self.live:
            outstanding = request.outstanding
            if outstanding <= 0:
                raise RuntimeError(f"live request {request.request_id!r} has no token to run")
            more = min(min(chunk, outstanding) - 1, spare)
            spare -= more
            plan.append((request, 1 + more))
        return plan

    @staticmethod
    def shed(plan: Plan, fits: Callable[[Plan], bool], give_way: Callable[[GenerationRequest], None] = lambda request: None):
        """Make ``plan`` fit.  ``fits(plan)`` says whether the free pages suffice; ``give_way(victim)``
        is called at once for every request that is dropped from the plan, so that the pages it
        returns count for the next answer.  Returns ``(plan, victims, failed)``: what runs, who gave
        way (in the order chosen: most cached tokens first, earlier in the plan among equals) and the
        single request that does not fit even alone (or ``None``)."""
        by_size = sorted(range(len(plan)), key=lambda index: -plan[index][0].cached)   # stable
        kept = list(plan)
        victims = []
        for index in by_size:
            if len(kept) <= 1 or fits(kept):
                break
            victim = plan[index][0]
            kept = [item for item in kept if item[0] is not victim]
            victims.append(victim)
            give_way(victim)
        failed = None
        if kept and not fits(kept):
            failed = kept[0][0]
            kept = []
        return kept, victims, failed
