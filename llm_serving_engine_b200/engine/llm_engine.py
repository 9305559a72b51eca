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
from .scheduler import IterationScheduler, RequestState, plan_iteration, resolve_page_pressure
from .step import StepEntry, StepRunner


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
        self.scheduler = IterationScheduler(scheduler_config.max_batch_size, scheduler_config.policy, scheduler_mode)
        self.sampler = Sampler(model.vocab_size, scheduler_config.max_batch_size, model.device)
        self._configs: dict[str, GenerationConfig] = {}
        self._incoming: asyncio.Queue | None = None
        self._worker: asyncio.Task | None = None
        self._closed = False
        self._ahead = None   # the next decode step, packed while the device ran the last one
        self.pack_ahead = True
        self.launch_ahead = True
        self._flying = None  # (requests, configs, sampling ticket) of a decode step that is queued on the device
        self._pending_callbacks: list[tuple[RequestState, int]] = []
        self._just_finished: list[tuple[RequestState, Exception | None]] = []
        self._cpu_ms = {"prefill": 0.0, "decode": 0.0, "mixed": 0.0}
        self._counts = {"prefill": 0, "decode": 0, "mixed": 0}
        self._events: dict[str, list] = {"prefill": [], "decode": [], "mixed": []}
        self._completed_preemptions = 0
        self._completed_recomputed_tokens = 0

    # -- requests ------------------------------------------------------------------
    def _new_request(self, prompt, config: GenerationConfig, callback, priority: int,
                     request_id: str | None, future=None) -> RequestState:
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
        state = RequestState(request_id=request_id, prompt_token_ids=tokens, max_new_tokens=config.max_new_tokens,
                             callback=callback, priority=priority, future=future)
        self._configs[request_id] = config
        return state

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
            self.scheduler.add(state)
            states.append(state)
        errors: dict[str, Exception] = {}
        try:
            while not self.scheduler.empty:
                self._admit()
                if self.scheduler.active:
                    self._step()
                    for request, token in self._pending_callbacks:
                        result = request.callback(token)
                        if inspect.isawaitable(result):
                            raise TypeError("generate_many takes plain callbacks; use generate() for coroutines")
                    self._pending_callbacks.clear()
                    self._resolve_finished(errors)
        except Exception:
            self._fail_all(None)
            raise
        self._drop_flying()   # a step queued for requests that have all ended meanwhile
        for state in states:
            if state.request_id in errors:
                raise errors[state.request_id]
        return [state.generated_token_ids for state in states]

    # -- the loop ------------------------------------------------------------------
    async def _run(self) -> None:
        try:
            while not self._closed:
                if self.scheduler.empty:
                    self.scheduler.add(await self._incoming.get())
                while True:
                    try:
                        self.scheduler.add(self._incoming.get_nowait())
                    except asyncio.QueueEmpty:
                        break
                self._admit()
                if self.scheduler.active:
                    self._step()
                    for request, token in self._pending_callbacks:
                        result = request.callback(token)
                        if inspect.isawaitable(result):
                            await result
                    self._pending_callbacks.clear()
                    self._resolve_finished()
                await asyncio.sleep(0)
        except asyncio.CancelledError:
            pass
        except Exception as error:  # any failure fails every request, as the reference does
            self._fail_all(error)

    def _admit(self) -> None:
        for request in self.scheduler.admit():
            self.cache.create(request.request_id)

    def _phase(self) -> str:
        active = self.scheduler.active
        prefill = any(r.processed_tokens < len(r.prompt_token_ids) for r in active)
        decode = any(r.processed_tokens >= len(r.prompt_token_ids) for r in active)
        return "mixed" if prefill and decode else "prefill" if prefill else "decode"

    # -- a decode step in flight ---------------------------------------------------------
    # In a run of decode steps over the same requests the engine keeps one step queued on the device
    # ahead of the host: the step is launched before the tokens of the step before have reached the
    # host (it takes them on the device), so packing, planning and book-keeping run beside the
    # device's work.  A request that ends by a stop token is found out one step late: its row of the
    # step in flight is dropped (its pages are freed with it).  Requests that will reach their token
    # limit, waiting requests, a new page that cannot be had or iteration metrics end the run: the
    # step in flight is collected and the ordinary path goes on.
    def _may_fly(self, requests: list[RequestState]) -> bool:
        return (self.pack_ahead and self.launch_ahead and not self.collect_iteration_metrics
                and not self.scheduler.waiting
                and all(len(r.generated_token_ids) + 2 <= r.max_new_tokens for r in requests))

    def _launch_flying(self, requests: list[RequestState], ticket: int):
        """Queue the next decode step of ``requests`` behind the sampling launch ``ticket`` whose tokens
        it consumes.  Returns (requests, configs, ticket of its own sampling) or None."""
        packed = self.runner.prepare_ahead([r.request_id for r in requests])
        if packed is None:
            return None
        logits = self.runner.launch_ahead(packed, self.sampler.device_tokens(ticket))
        if logits is None:
            return None
        configs = [self._configs[r.request_id] for r in requests]
        counters = [len(r.generated_token_ids) + 1 for r in requests]   # the token before is still on its way
        return requests, configs, self.sampler.launch(logits, configs, counters)

    def _take_tokens(self, requests, configs, tokens, fed: bool) -> None:
        """Book the sampled tokens; ``fed``: the step consumed one token of every request on the device."""
        for request, config, token in zip(requests, configs, tokens):
            if request not in self.scheduler.active:
                continue          # ended a step ago (a stop token): this row was computed for nothing
            if fed:
                request.processed_tokens += 1
            request.generated_token_ids.append(token)
            if request.callback:
                self._pending_callbacks.append((request, token))
            if len(request.generated_token_ids) >= request.max_new_tokens or token in config.stop_token_ids:
                self._finish(request)

    def _drop_flying(self) -> None:
        flying, self._flying = self._flying, None
        if flying is not None:
            self.sampler.collect(flying[2])   # its buffers are free again; the tokens are not wanted

    @torch.inference_mode()
    def _step(self) -> None:
        flying, self._flying = self._flying, None
        if flying is not None:
            requests, configs, ticket = flying
            active = self.scheduler.active
            same = len(requests) == len(active) and all(a is b for a, b in zip(requests, active))
            following = self._launch_flying(requests, ticket) if same and self._may_fly(requests) else None
            self._take_tokens(requests, configs, self.sampler.collect(ticket), fed=True)
            self._flying = following
            return
        events = None
        if self.collect_iteration_metrics:
            phase = self._phase()
            started = time.perf_counter()
            events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            events[0].record()
        ahead, self._ahead = self._ahead, None
        active = self.scheduler.active
        if (ahead is not None and len(ahead[1]) == len(active) and all(a is b for a, b in zip(ahead[1], active))
                and all(r.total_tokens - r.processed_tokens == 1 for r in active)):
            # the step that was packed ahead: the same requests, one token each; their pages are there
            planned = [(request, 1) for request in active]
            ahead = ahead[0]
        else:
            ahead = None
            planned = plan_iteration(list(active), self.scheduler_config.max_tokens_per_step, self.prefill_chunk_size)

            def preempt(victim: RequestState) -> None:
                self.cache.free(victim.request_id)
                self.scheduler.preempt(victim)

            planned, _, failed = resolve_page_pressure(
                planned, lambda plan: self.cache.fits([(r.request_id, n) for r, n in plan]), preempt)
            if failed is not None:
                self._finish(failed, CacheFullError("one sequence exceeds total KV cache capacity"))
        if planned:
            entries, sampled = [], []
            for request, count in planned:
                first = request.processed_tokens
                tokens = request.tokens_from(first, count)
                done = first + count == request.total_tokens
                entries.append(StepEntry(request.request_id, tokens, [count - 1] if done else []))
                if done:
                    sampled.append(request)
            logits = self.runner.run_ahead(ahead, entries) if ahead is not None else None
            if logits is None:
                logits = self.runner.run(entries)
            for request, count in planned:
                request.processed_tokens += count
            if sampled:
                configs = [self._configs[r.request_id] for r in sampled]
                counters = [len(r.generated_token_ids) for r in sampled]
                ticket = self.sampler.launch(logits, configs, counters)
                # While the device works: if the next step will be these same requests with one token
                # each (nobody waits, nobody reaches its token limit), launch it now on the tokens that
                # are still on the device, or at least pack it but for the tokens.
                following = None
                if (self.pack_ahead and len(sampled) == len(planned) and not self.scheduler.waiting
                        and all(len(r.generated_token_ids) + 1 < r.max_new_tokens for r in sampled)):
                    if len(sampled) == len(self.scheduler.active) and self._may_fly(sampled):
                        following = self._launch_flying(sampled, ticket)
                    if following is None:
                        packed = self.runner.prepare_ahead([r.request_id for r, _ in planned])
                        if packed is not None:
                            self._ahead = (packed, [r for r, _ in planned])
                self._take_tokens(sampled, configs, self.sampler.collect(ticket), fed=False)
                self._flying = following
        if self.collect_iteration_metrics:
            events[1].record()
            self._events[phase].append(events)
            self._cpu_ms[phase] += (time.perf_counter() - started) * 1000
            self._counts[phase] += 1

    def _finish(self, request: RequestState, error: Exception | None = None) -> None:
        if request in self.scheduler.active:
            self.scheduler.finish(request)
        if request.request_id in self.cache.requests:
            self.cache.free(request.request_id)
        self._configs.pop(request.request_id, None)
        self._completed_preemptions += request.preemptions
        self._completed_recomputed_tokens += request.recomputed_tokens
        self._just_finished.append((request, error))  # resolved after this step's callbacks have run

    def _resolve_finished(self, errors: dict[str, Exception] | None = None) -> None:
        for request, error in self._just_finished:
            if errors is not None and error is not None:
                errors[request.request_id] = error
            if request.future is not None and not request.future.done():
                if error is not None:
                    request.future.set_exception(error)
                else:
                    request.future.set_result(request.generated_token_ids)
        self._just_finished.clear()

    def _fail_all(self, error: Exception | None) -> None:
        for request in self.scheduler.active + self.scheduler.waiting:
            if error is not None and request.future is not None and not request.future.done():
                request.future.set_exception(error)
        self._ahead = None
        self._drop_flying()
        self.cache.free_all()
        self.scheduler.active.clear()
        self.scheduler.waiting.clear()
        self._configs.clear()
        self._pending_callbacks.clear()
        self._just_finished.clear()

    def warmup(self, batch_sizes=None) -> None:
        """Capture the CUDA graphs of decode steps ahead of time (one per batch bucket up to
        ``max_batch_size``), so that no request pays for a capture.  Uses temporary requests."""
        self.runner.warmup(batch_sizes)

    async def close(self) -> None:
        self._closed = True
        if self._worker:
            self._worker.cancel()
            await asyncio.gather(self._worker, return_exceptions=True)
        self._ahead = None
        self._drop_flying()   # a decode step that was still queued on the device

    async def __aenter__(self) -> "LLMEngine":
        return self

    async def __aexit__(self, *_: Any) -> None:
        await self.close()

    # -- statistics ------------------------------------------------------------
    @property
    def cache_stats(self) -> dict[str, float]:
        return self.cache.stats(self.model.spec.max_position_embeddings)

    @property
    def iteration_stats(self) -> dict[str, float | int]:
        cuda_ms = {phase: 0.0 for phase in self._events}
        if self.collect_iteration_metrics:
            torch.cuda.synchronize(self.device)
            cuda_ms = {phase: sum(a.elapsed_time(b) for a, b in events) for phase, events in self._events.items()}
        result: dict[str, float | int] = {
            "preemptions": self._completed_preemptions,
            "recomputed_tokens": self._completed_recomputed_tokens,
        }
        for phase in ("prefill", "decode", "mixed"):
            result[f"{phase}_iterations"] = self._counts[phase]
            result[f"{phase}_cpu_ms"] = self._cpu_ms[phase]
            result[f"{phase}_cuda_ms"] = cuda_ms[phase]
        return result
