"""Synthetic request traffic for the command line's ``benchmark`` and for ``bench.py``.

The traffic has the statistics of the reference's generator
(``src/llmserve/benchmark/workload.py:11-79``, ``configs/benchmark-sharegpt.yaml``): prompt and
output lengths are log-normal around a median, clipped to a range; requests arrive with
exponential gaps at a given rate; token ids are uniform over the vocabulary above the four
reserved ids.  A profile file has the reference's keys (``requests``, ``arrival_rate``, ``seed``,
``vocabulary_size``, and ``prompt`` / ``output`` with ``median``, ``sigma``, ``minimum``, ``maximum``).
Everything is drawn from one NumPy generator, array by array, so a profile and a seed give the
same traffic everywhere (not the reference's own stream of numbers).

``replay_traffic`` plays such traffic against any ``async generate(request, on_token)`` and returns
one timing row per request; ``summarise`` turns the rows into the usual latency figures (time to the
first token, time per later token, total latency: median, 95th and 99th percentile).
"""
from __future__ import annotations

import asyncio
import time
from dataclasses import dataclass, field, replace
from pathlib import Path

import numpy as np

RESERVED_IDS = 4       # pad, bos, eos, unk of the byte tokenizer: traffic never uses them


@dataclass(frozen=True)
class ClippedLogNormal:
    median: int
    sigma: float
    minimum: int
    maximum: int

    def draw(self, rng: np.random.Generator, count: int) -> np.ndarray:
        values = np.rint(rng.lognormal(np.log(self.median), self.sigma, size=count)).astype(np.int64)
        return np.clip(values, self.minimum, self.maximum)


@dataclass(frozen=True)
class TrafficProfile:
    requests: int = 100
    arrival_rate: float = 2.0                  # requests per second; 0: all at once
    prompt: ClippedLogNormal = ClippedLogNormal(128, 0.9, 8, 1024)
    output: ClippedLogNormal = ClippedLogNormal(64, 0.7, 4, 256)
    seed: int = 7
    vocabulary_size: int = 32_000

    @staticmethod
    def from_file(path) -> "TrafficProfile":
        import yaml

        raw = yaml.safe_load(Path(path).read_text()) or {}
        known = {"requests", "arrival_rate", "seed", "vocabulary_size"}
        fields = {key: raw[key] for key in known if key in raw}
        for key in ("prompt", "output"):
            if key in raw:
                fields[key] = ClippedLogNormal(**raw[key])
        return TrafficProfile(**fields)

    def fitted_to(self, vocabulary_size: int, max_positions: int) -> "TrafficProfile":
        """The profile with the model's vocabulary, and prompts short enough that prompt + output fits."""
        room = max(self.prompt.minimum, max_positions - self.output.maximum)
        return replace(self, vocabulary_size=vocabulary_size,
                       prompt=replace(self.prompt, maximum=min(self.prompt.maximum, room)))


@dataclass(frozen=True)
class TrafficRequest:
    request_id: str
    arrives_at: float                          # seconds after the start
    prompt_token_ids: tuple[int, ...]
    max_new_tokens: int


def make_traffic(profile: TrafficProfile) -> list[TrafficRequest]:
    if profile.requests <= 0:
        return []
    if profile.vocabulary_size <= RESERVED_IDS:
        raise ValueError("the vocabulary has no ids beyond the reserved ones")
    rng = np.random.default_rng(profile.seed)
    count = profile.requests
    prompt_lengths = profile.prompt.draw(rng, count)
    output_lengths = profile.output.draw(rng, count)
    arrivals = np.zeros(count)
    if profile.arrival_rate > 0:
        arrivals[1:] = np.cumsum(rng.exponential(1.0 / profile.arrival_rate, size=count - 1))
    ids = rng.integers(RESERVED_IDS, profile.vocabulary_size, size=int(prompt_lengths.sum()))
    ends = np.cumsum(prompt_lengths)
    return [TrafficRequest(f"request-{index:06d}", float(arrivals[index]),
                           tuple(int(token) for token in ids[ends[index] - prompt_lengths[index]:ends[index]]),
                           int(output_lengths[index]))
            for index in range(count)]


@dataclass
class RequestTiming:
    request_id: str
    prompt_tokens: int
    wanted_tokens: int
    arrived: float
    first_token: float | None = None
    ended: float | None = None
    output_tokens: int = 0
    error: str | None = None

    def figures(self) -> dict:
        """ttft_ms, tpot_ms, e2e_ms (None where the request did not get that far)."""
        ttft = None if self.first_token is None else (self.first_token - self.arrived) * 1e3
        e2e = None if self.ended is None else (self.ended - self.arrived) * 1e3
        tpot = None
        if self.first_token is not None and self.ended is not None and self.output_tokens > 1:
            tpot = (self.ended - self.first_token) * 1e3 / (self.output_tokens - 1)
        return {"ttft_ms": ttft, "tpot_ms": tpot, "e2e_ms": e2e}


@dataclass
class TrafficResult:
    name: str
    seconds: float
    rows: list[RequestTiming]
    cache: dict = field(default_factory=dict)
    extra: dict = field(default_factory=dict)

    def as_dict(self) -> dict:
        rows = [dict(vars(row), **row.figures()) for row in self.rows]
        return {"summary": summarise(self), "metadata": self.extra, "requests": rows}


def summarise(result: TrafficResult) -> dict:
    served = [row for row in result.rows if row.error is None]
    out = {"config": result.name, "requests": len(result.rows), "successful_requests": len(served),
           "duration_s": result.seconds,
           "throughput_tokens_per_s": sum(row.output_tokens for row in served) / max(result.seconds, 1e-9)}
    figures = [row.figures() for row in served]
    for key in ("ttft_ms", "tpot_ms", "e2e_ms"):
        values = np.array([item[key] for item in figures if item[key] is not None], dtype=np.float64)
        for label, q in (("p50", 50), ("p95", 95), ("p99", 99)):
            out[f"{key}_{label}"] = float(np.percentile(values, q)) if values.size else 0.0
    for key, value in result.cache.items():
        out[f"cache_{key}"] = value
    return out


async def replay_traffic(name: str, traffic: list[TrafficRequest], generate) -> TrafficResult:
    """Send every request at its arrival time to ``await generate(request, on_token)``; a request that
    raises keeps its row, with the error's text."""
    loop = asyncio.get_running_loop()
    origin = loop.time()
    rows = {item.request_id: RequestTiming(item.request_id, len(item.prompt_token_ids), item.max_new_tokens, 0.0)
            for item in traffic}

    async def one(item: TrafficRequest) -> None:
        await asyncio.sleep(max(0.0, origin + item.arrives_at - loop.time()))
        row = rows[item.request_id]
        row.arrived = loop.time()

        def on_token(_token: int) -> None:
            row.output_tokens += 1
            if row.output_tokens == 1:
                row.first_token = loop.time()

        try:
            await generate(item, on_token)
        except Exception as error:   # the run goes on; the row says what happened
            row.error = f"{type(error).__name__}: {error}"
        row.ended = loop.time()

    await asyncio.gather(*[one(item) for item in traffic])
    return TrafficResult(name, loop.time() - origin, [rows[item.request_id] for item in traffic],
                         extra={"wall_clock_unix_s": time.time()})
