"""Iteration-level scheduling: admission, the cut of prompts into portions under a
token budget, and what happens when pages run out.  Pure host code.

Kept from the reference (``src/llmserve/scheduler.py:12-97``,
``src/llmserve/engine.py:256-267,372-400``):

* ``waiting`` and ``active`` lists; ``admit`` sorts the waiting requests by policy
  (fcfs: arrival; sjf: remaining output tokens, then arrival; priority: higher
  first, then arrival) and admits up to ``max_batch_size`` live requests; in
  ``static`` mode only when nothing is active.  Admission does not look at pages.
* ``plan_iteration``: every active request gets one token; then, in list order,
  each gets more of its outstanding tokens, up to ``prefill_chunk_size`` per step,
  while the step's token budget lasts.
* Pages run out: while the plan needs more pages than are free and more than one
  request is planned, the planned request that has processed the most tokens is
  preempted: its pages are freed, it goes to the back of ``waiting`` with
  ``processed_tokens = 0`` and later recomputes prompt and generated tokens,
  sampling nothing until it has caught up.  If a single request still does not
  fit, that request fails with ``CacheFullError``.
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import Any, Callable


@dataclass
class RequestState:
    request_id: str
    prompt_token_ids: list[int]
    max_new_tokens: int
    callback: Callable[[int], Any] | None = None
    priority: int = 0
    arrival_order: int = 0
    arrival_time: float = field(default_factory=time.monotonic)
    generated_token_ids: list[int] = field(default_factory=list)
    processed_tokens: int = 0
    preemptions: int = 0
    recomputed_tokens: int = 0
    future: Any = None

    @property
    def all_tokens(self) -> list[int]:
        return self.prompt_token_ids + self.generated_token_ids

    def tokens_from(self, first: int, count: int) -> list[int]:
        """Tokens first .. first+count-1 of prompt + generated, without joining the two lists."""
        prompt = self.prompt_token_ids
        n_prompt = len(prompt)
        if first >= n_prompt:
            return self.generated_token_ids[first - n_prompt:first - n_prompt + count]
        if first + count <= n_prompt:
            return prompt[first:first + count]
        return prompt[first:] + self.generated_token_ids[:first + count - n_prompt]

    @property
    def total_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.generated_token_ids)

    @property
    def remaining_output_tokens(self) -> int:
        return self.max_new_tokens - len(self.generated_token_ids)


class IterationScheduler:
    def __init__(self, max_batch_size: int, policy: str = "fcfs", mode: str = "continuous") -> None:
        if policy not in {"fcfs", "sjf", "priority"}:
            raise ValueError("policy must be fcfs, sjf, or priority")
        if mode not in {"continuous", "static"}:
            raise ValueError("mode must be continuous or static")
        self.max_batch_size = max_batch_size
        self.policy = policy
        self.mode = mode
        self.waiting: list[RequestState] = []
        self.active: list[RequestState] = []
        self._counter = itertools.count()

    def add(self, request: RequestState) -> None:
        request.arrival_order = next(self._counter)
        self.waiting.append(request)

    def _key(self, request: RequestState):
        if self.policy == "fcfs":
            return request.arrival_order
        if self.policy == "sjf":
            return (request.remaining_output_tokens, request.arrival_order)
        return (-request.priority, request.arrival_order)

    def admit(self) -> list[RequestState]:
        if self.mode == "static" and self.active:
            return []
        self.waiting.sort(key=self._key)
        count = min(self.max_batch_size - len(self.active), len(self.waiting))
        admitted = self.waiting[:count]
        del self.waiting[:count]
        self.active.extend(admitted)
        return admitted

    def finish(self, request: RequestState) -> None:
        self.active.remove(request)

    def preempt(self, request: RequestState) -> None:
        self.active.remove(request)
        request.recomputed_tokens += request.processed_tokens
        request.processed_tokens = 0
        request.preemptions += 1
        self.waiting.append(request)

    @property
    def empty(self) -> bool:
        return not self.waiting and not self.active


def plan_iteration(active: list[RequestState], max_tokens_per_step: int,
                   prefill_chunk_size: int) -> list[tuple[RequestState, int]]:
    """How many of its outstanding tokens each active request runs in this step."""
    budget = max_tokens_per_step
    planned: list[tuple[RequestState, int]] = []
    for request in active:
        if request.total_tokens - request.processed_tokens <= 0:
            raise RuntimeError("active request has no input token to process")
        planned.append((request, 1))
        budget -= 1
    if budget < 0:
        raise RuntimeError("max_tokens_per_step is below the number of active requests")
    for index, (request, count) in enumerate(planned):
        if budget <= 0:
            break
        remaining = request.total_tokens - request.processed_tokens
        extra = min(min(prefill_chunk_size, remaining) - count, budget)
        planned[index] = (request, count + extra)
        budget -= extra
    return planned


def resolve_page_pressure(planned: list[tuple[RequestState, int]],
                          fits: Callable[[list[tuple[RequestState, int]]], bool],
                          preempt: Callable[[RequestState], None] = lambda request: None):
    """Drop requests from the plan until it fits the free pages.

    ``fits(plan)`` answers whether the free pages suffice; ``preempt(victim)`` is
    called at once for every request that is dropped, so that the pages it gives
    back count for the next answer.  Returns ``(planned, victims, failed)``: the
    plan that runs, the requests that were preempted (in the order chosen) and the
    single request that cannot fit even alone (or ``None``).
    """
    planned = list(planned)
    victims: list[RequestState] = []
    while not fits(planned) and len(planned) > 1:
        victim, _ = max(planned, key=lambda item: item[0].processed_tokens)
        victims.append(victim)
        planned = [item for item in planned if item[0] is not victim]
        preempt(victim)
    failed = None
    if planned and not fits(planned):
        failed = planned[0][0]
        planned = []
    return planned, victims, failed
