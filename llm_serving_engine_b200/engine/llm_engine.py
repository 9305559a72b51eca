"""The Python entry point: ``LLMEngine``, in the reference's manner
(``src/llmserve/engine.py:108-464``).

``await engine.generate(prompt, config, callback)`` queues a request and returns
its generated token ids; a background task runs one model step per loop turn:
admit, plan, resolve page pressure, pack, run the step function, sample on the
device, call back, finish and free.  ``generate_many`` is the same loop without
asyncio, for scripts and measurement.
"""
from __future__ import annotations

import asyncio
import inspect
import time
import uuid
from typing import Any

import torch

from ..cache.manager import CacheFullError, CacheManager
from ..config.runtime_config import CacheConfig, SchedulerConfig
from ..models import cache_requirements
from ..sampling.sampler import GenerationConfig, Sampler
from .scheduler import GenerationRequest, Scheduler
from .step import StepEntry, StepRunner

PHASES = ("prefill", "decode", "mixed")


class _IterationMeter:
    """Per-phase step counts, host milliseconds and CUDA event pairs: what ``iteration_stats`` reports
    (the reference's ``collect_iteration_metrics``, ``src/llmserve/engine.py:246-254,358-370``).  A
    step is "prefill" when every live request still has prompt to feed, "decode" when none has,
    else "mixed"."""

    def __init__(self) -> None:
        self.steps = dict.fromkeys(PHASES, 0)
        self.host_ms = dict.fromkeys(PHASES, 0.0)
        self.pairs: dict[str, list] = {phase: [] for phase in PHASES}
        self._open = None

    def begin(self, live: list[GenerationRequest]) -> None:
        feeding = sum(1 for request in live if request.in_prompt)
        phase = "decode" if feeding == 0 else "prefill" if feeding == len(live) else "mixed"
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        self._open = (phase, time.perf_counter(), first, last)

    def end(self) -> None:
        phase, started, first, last = self._open
        self._open = None
        last.record()
        self.pairs[phase].append((first, last))
        self.host_ms[phase] += (time.perf_counter() - started) * 1e3
        self.steps[phase] += 1

    def device_ms(self, device) -> dict[str, float]:
        torch.cuda.synchronize(device)
        return {phase: sum(first.elapsed_time(last) for first, last in pairs) for phase, pairs in self.pairs.items()}


class LLMEngine:
    """Iteration-level engine over the paged cache and the step function.

    Arguments follow the reference (``src/llmserve/engine.py:111-125``): ``model`` (a
    ``DecoderModel``), ``tokenizer`` (may be ``None`` when prompts are token ids),
    ``cache_config``, ``scheduler_config``, ``scheduler_mode`` ("continuous" or
    "static"), ``prefill_chunk_size`` (most tokens of one prompt in a step),
    ``collect_iteration_metrics``.  Device and dtype are the model's.
    """

    def __init__(self, model, tokenizer=None, *, cache_config: CacheConfig | None = None,
                 scheduler_config: SchedulerConfig | None = None, scheduler_mode: str = "continuous",
                 prefill_chunk_size: int = 2048, collect_iteration_metrics: bool = False) -> None:
        cache_config = cache_config or CacheConfig()
        scheduler_config = scheduler_config or SchedulerConfig()
        if prefill_chunk_size <= 0:
            raise ValueError("prefill_chunk_size must be positive")
        if scheduler_config.max_tokens_per_step < scheduler_config.max_batch_size:
            raise ValueError("max_tokens_per_step must allow one token per active request")
        self.model = model
        self.tokenizer = tokenizer
        self.device = model.device
        self.scheduler_config = scheduler_config
        self.prefill_chunk_size = prefill_chunk_size
        self.collect_iteration_metrics = collect_iteration_metrics
        self.cache = CacheManager(cache_requirements(model.spec), cache_config, model.dtype, model.device,
                                  model.spec.max_position_embeddings,
                                  num_state_slots=cache_config.num_state_slots or scheduler_config.max_batch_size)
        self.runner = StepRunner(model, self.cache, scheduler_config.max_tokens_per_step,
                                 scheduler_config.max_batch_size)
        self.scheduler = Scheduler(scheduler_config.max_batch_size, scheduler_config.policy, scheduler_mode)
        self.sampler = Sampler(model.vocab_size, scheduler_config.max_batch_size, model.device)
        self._configs: dict[str, GenerationConfig] = {}
        self._incoming: asyncio.Queue | None = None
        self._worker: asyncio.Task | None = None
        self._closed = False
        self._ahead = None   # the next decode step, packed while the device ran the last one
        self.pack_ahead = True
        self.launch_ahead = True
        self._flying = None  # (requests, configs, sampling ticket) of a decode step that is queued on the device
        self._pending_callbacks: list[tuple[GenerationRequest, int]] = []
        self._ended: list[tuple[GenerationRequest, Exception | None]] = []   # resolved after the step's callbacks
        self._meter = _IterationMeter() if collect_iteration_metrics else None
        self._evictions_of_ended = 0
        self._replayed_tokens_of_ended = 0

    # -- requests ------------------------------------------------------------------
    def _new_request(self, prompt, config: GenerationConfig, callback, priority: int,
                     request_id: str | None, future=None) -> GenerationRequest:
        if self._closed:
            raise RuntimeError("engine is closed")
        if config.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer")
            tokens = self.tokenizer.encode(prompt)
        else:
            tokens = [int(token) for token in prompt]
        if not tokens:
            raise ValueError("prompt cannot be empty")
        vocab = self.model.vocab_size
        if min(tokens) < 0 or max(tokens) >= vocab:
            raise ValueError(f"prompt holds a token id outside [0, {vocab})")
        limit = self.model.spec.max_position_embeddings
        if len(tokens) + config.max_new_tokens > limit:
            raise ValueError(f"prompt ({len(tokens)}) plus max_new_tokens ({config.max_new_tokens}) "
                             f"exceeds max_position_embeddings ({limit})")
        request_id = request_id or str(uuid.uuid4())
        if request_id in self._configs:
            raise ValueError(f"request id {request_id!r} is already in use")
        self._configs[request_id] = config
        return GenerationRequest(request_id, tokens, config.max_new_tokens, callback, priority, future)

    async def generate(self, prompt, config: GenerationConfig | None = None, callback=None, *,
                       priority: int = 0, request_id: str | None = None) -> list[int]:
        """Generate for one prompt (text or token ids); ``callback(token)`` is called, and
        awaited if it is a coroutine, once per generated token."""
        config = config or GenerationConfig()
        if self._incoming is None:
            self._incoming = asyncio.Queue()
        future = asyncio.get_running_loop().create_future()
        state = self._new_request(prompt, config, callback, priority, request_id, future)
        if self._worker is None:
            self._worker = asyncio.create_task(self._run())
        await self._incoming.put(state)
        return await future

    def generate_many(self, prompts, configs=None, callbacks=None) -> list[list[int]]:
        """Synchronous form: run all ``prompts`` (token ids or text) to the end and return
        their generated ids in order.  ``configs``: one ``GenerationConfig`` or a list."""
        count = len(prompts)
        if configs is None or isinstance(configs, GenerationConfig):
            configs = [configs or GenerationConfig()] * count
        callbacks = callbacks or [None] * count
        states = []
        for prompt, config, callback in zip(prompts, configs, callbacks):
            state = self._new_request(prompt, config, callback, 0, None)
            self.scheduler.enqueue(state)
            states.append(state)
        errors: dict[str, Exception] = {}
        try:
            while not self.scheduler.idle:
                self._admit()
                if self.scheduler.live:
                    self._step()
                    for request, token in self._pending_callbacks:
                        result = request.callback(token)
                        if inspect.isawaitable(result):
                            raise TypeError("generate_many takes plain callbacks; use generate() for coroutines")
                    self._pending_callbacks.clear()
                    self._settle(errors)
        except Exception:
            self._abandon_everything(None)
            raise
        self._drop_flying()   # a step queued for requests that have all ended meanwhile
        for state in states:
            if state.request_id in errors:
                raise errors[state.request_id]
        return [state.output for state in states]

    # -- the loop ------------------------------------------------------------------
    async def _run(self) -> None:
        try:
            while not self._closed:
                if self.scheduler.idle:
                    self.scheduler.enqueue(await self._incoming.get())
                while not self._incoming.empty():
                    self.scheduler.enqueue(self._incoming.get_nowait())
                self._admit()
                if self.scheduler.live:
                    self._step()
                    for request, token in self._pending_callbacks:
                        result = request.callback(token)
                        if inspect.isawaitable(result):
                            await result
                    self._pending_callbacks.clear()
                    self._settle()
                await asyncio.sleep(0)
        except asyncio.CancelledError:
            pass
        except Exception as error:  # a failure of the loop fails every request (``src/llmserve/engine.py:241-242``)
            self._abandon_everything(error)

    def _admit(self) -> None:
        for request in self.scheduler.admit():
            self.cache.create(request.request_id)

    # -- a decode step in flight ---------------------------------------------------------
    # In a run of decode steps over the same requests the engine keeps one step queued on the device
    # ahead of the host: the step is launched before the tokens of the step before have reached the
    # host (it takes them on the device), so packing, planning and book-keeping run beside the
    # device's work.  A request that ends by a stop token is found out one step late: its row of the
    # step in flight is dropped (its pages are freed with it).  Requests that will reach their token
    # limit, waiting requests, a new page that cannot be had or iteration metrics end the run: the
    # step in flight is collected and the ordinary path goes on.
    def _may_fly(self, requests: list[GenerationRequest]) -> bool:
        return (self.pack_ahead and self.launch_ahead and self._meter is None
                and not self.scheduler.has_waiting
                and all(len(r.output) + 2 <= r.max_new_tokens for r in requests))

    def _launch_flying(self, requests: list[GenerationRequest], ticket: int):
        """Queue the next decode step of ``requests`` behind the sampling launch ``ticket`` whose tokens
        it consumes.  Returns (requests, configs, ticket of its own sampling) or None."""
        packed = self.runner.prepare_ahead([r.request_id for r in requests])
        if packed is None:
            return None
        logits = self.runner.launch_ahead(packed, self.sampler.device_tokens(ticket))
        if logits is None:
            return None
        configs = [self._configs[r.request_id] for r in requests]
        counters = [len(r.output) + 1 for r in requests]   # the token before is still on its way
        return requests, configs, self.sampler.launch(logits, configs, counters)

    def _take_tokens(self, requests, configs, tokens, fed: bool) -> None:
        """Book the sampled tokens; ``fed``: the step consumed one token of every request on the device."""
        for request, config, token in zip(requests, configs, tokens):
            if request not in self.scheduler.live:
                continue          # ended a step ago (a stop token): this row was computed for nothing
            if fed:
                request.cached += 1
            request.output.append(token)
            if request.callback:
                self._pending_callbacks.append((request, token))
            if request.output_left <= 0 or token in config.stop_token_ids:
                self._retire(request)

    def _drop_flying(self) -> None:
        flying, self._flying = self._flying, None
        if flying is not None:
            self.sampler.collect(flying[2])   # its buffers are free again; the tokens are not wanted

    @torch.inference_mode()
    def _step(self) -> None:
        if self._flying is not None:
            self._land_flying()
            return
        if self._meter is not None:
            self._meter.begin(self.scheduler.live)
        plan, ahead = self._next_plan()
        if plan:
            self._run_plan(plan, ahead)
        if self._meter is not None:
            self._meter.end()

    def _land_flying(self) -> None:
        """The step in flight ends: queue the one after it (if the same requests go on decoding), then
        read and book its tokens."""
        requests, configs, ticket = self._flying
        self._flying = None
        live = self.scheduler.live
        unchanged = len(requests) == len(live) and all(a is b for a, b in zip(requests, live))
        following = self._launch_flying(requests, ticket) if unchanged and self._may_fly(requests) else None
        self._take_tokens(requests, configs, self.sampler.collect(ticket), fed=True)
        self._flying = following

    def _next_plan(self):
        """(plan, step packed ahead or None).  The plan is the packed-ahead step when it still describes the
        live requests (the same ones, one outstanding token each: their pages are there already); else the
        scheduler's plan, cut down until it fits the free pages."""
        packed, self._ahead = self._ahead, None
        live = self.scheduler.live
        if packed is not None:
            ahead, expected = packed
            if (len(expected) == len(live) and all(a is b for a, b in zip(expected, live))
                    and all(request.outstanding == 1 for request in live)):
                return [(request, 1) for request in live], ahead
        plan = self.scheduler.plan(self.scheduler_config.max_tokens_per_step, self.prefill_chunk_size)

        def give_way(victim: GenerationRequest) -> None:
            self.cache.free(victim.request_id)        # its pages count for the next answer of ``fits``
            self.scheduler.requeue(victim)

        plan, _, failed = self.scheduler.shed(
            plan, lambda kept: self.cache.fits([(request.request_id, count) for request, count in kept]), give_way)
        if failed is not None:
            self._retire(failed, CacheFullError("one sequence exceeds total KV cache capacity"))
        return plan, None

    def _run_plan(self, plan, ahead) -> None:
        entries, sampled = [], []
        for request, count in plan:
            last = request.cached + count == request.length     # the request's newest token is among these
            entries.append(StepEntry(request.request_id, request.tokens(request.cached, count), [count - 1] if last else []))
            if last:
                sampled.append(request)
        logits = self.runner.run_ahead(ahead, entries) if ahead is not None else None
        if logits is None:
            logits = self.runner.run(entries)
        for request, count in plan:
            request.cached += count
        if not sampled:
            return
        configs = [self._configs[request.request_id] for request in sampled]
        ticket = self.sampler.launch(logits, configs, [len(request.output) for request in sampled])
        # While the device works: if the next step will be these same requests with one token each (nobody
        # waits, nobody reaches its token limit), launch it now on the tokens that are still on the device,
        # or at least pack it but for the tokens.
        following = None
        if (self.pack_ahead and len(sampled) == len(plan) and not self.scheduler.has_waiting
                and all(len(request.output) + 1 < request.max_new_tokens for request in sampled)):
            if len(sampled) == len(self.scheduler.live) and self._may_fly(sampled):
                following = self._launch_flying(sampled, ticket)
            if following is None:
                packed = self.runner.prepare_ahead([request.request_id for request in sampled])
                if packed is not None:
                    self._ahead = (packed, list(sampled))
        self._take_tokens(sampled, configs, self.sampler.collect(ticket), fed=False)
        self._flying = following

    # -- requests leave --------------------------------------------------------------
    def _retire(self, request: GenerationRequest, error: Exception | None = None) -> None:
        """The request has ended, with its tokens or with ``error``: off the live list, pages back.  Its
        caller hears of it after this step's callbacks have run (``_settle``)."""
        if request in self.scheduler.live:
            self.scheduler.release(request)
        if request.request_id in self.cache.requests:
            self.cache.free(request.request_id)
        self._configs.pop(request.request_id, None)
        self._evictions_of_ended += request.evictions
        self._replayed_tokens_of_ended += request.replayed_tokens
        self._ended.append((request, error))

    def _settle(self, errors: dict[str, Exception] | None = None) -> None:
        ended, self._ended = self._ended, []
        for request, error in ended:
            if error is not None and errors is not None:
                errors[request.request_id] = error
            future = request.future
            if future is None or future.done():
                continue
            if error is None:
                future.set_result(request.output)
            else:
                future.set_exception(error)

    def _abandon_everything(self, error: Exception | None) -> None:
        """The loop failed: nothing that was queued on the device is wanted any more, every page goes back
        and every caller that still waits gets ``error``."""
        self._ahead = None
        self._drop_flying()
        for request in self.scheduler.drain():
            if error is not None and request.future is not None and not request.future.done():
                request.future.set_exception(error)
        self.cache.free_all()
        self._configs.clear()
        self._pending_callbacks.clear()
        self._ended.clear()

    def warmup(self, batch_sizes=None) -> None:
        """Capture the CUDA graphs of decode steps ahead of time (one per batch bucket up to
        ``max_batch_size``), so that no request pays for a capture.  Uses temporary requests."""
        self.runner.warmup(batch_sizes)

    async def close(self) -> None:
        self._closed = True
        worker, self._worker = self._worker, None
        if worker is not None:
            worker.cancel()
            await asyncio.gather(worker, return_exceptions=True)
        self._ahead = None
        self._drop_flying()   # a decode step that was still queued on the device

    async def __aenter__(self) -> "LLMEngine":
        return self

    async def __aexit__(self, *_: Any) -> None:
        await self.close()

    # -- statistics (the reference's report keys, ``src/llmserve/engine.py:438-458``) ---------------
    @property
    def cache_stats(self) -> dict[str, float]:
        return self.cache.stats(self.model.spec.max_position_embeddings)

    @property
    def iteration_stats(self) -> dict[str, float | int]:
        report: dict[str, float | int] = {"preemptions": self._evictions_of_ended,
                                          "recomputed_tokens": self._replayed_tokens_of_ended}
        meter = self._meter
        device_ms = meter.device_ms(self.device) if meter is not None else dict.fromkeys(PHASES, 0.0)
        for phase in PHASES:
            report[f"{phase}_iterations"] = meter.steps[phase] if meter is not None else 0
            report[f"{phase}_cpu_ms"] = meter.host_ms[phase] if meter is not None else 0.0
            report[f"{phase}_cuda_ms"] = device_ms[phase]
        return report
