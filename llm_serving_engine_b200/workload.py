"""Synthetic open-loop workloads and the report of a run, after the reference's
benchmark package (``src/llmserve/benchmark/workload.py``, ``metrics.py``,
``runner.py``): clipped log-normal prompt and output lengths, exponential
inter-arrival times, token ids uniform in [4, vocabulary), all from one seed;
time to first token, time per output token and end-to-end latency percentiles."""
from __future__ import annotations

import asyncio
import math
import random
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path


@dataclass(frozen=True)
class LengthDistribution:
    median: int
    sigma: float
    minimum: int
    maximum: int

    def sample(self, rng: random.Random) -> int:
        value = round(rng.lognormvariate(math.log(self.median), self.sigma))
        return max(self.minimum, min(self.maximum, value))


@dataclass(frozen=True)
class LoadProfile:
    requests: int = 100
    arrival_rate: float = 2.0
    prompt: LengthDistribution = LengthDistribution(128, 0.9, 8, 1_024)
    output: LengthDistribution = LengthDistribution(64, 0.7, 4, 256)
    seed: int = 7
    vocabulary_size: int = 32_000

    @classmethod
    def from_yaml(cls, path) -> "LoadProfile":
        import yaml

        values = yaml.safe_load(Path(path).read_text())
        return cls(requests=values["requests"], arrival_rate=values["arrival_rate"],
                   prompt=LengthDistribution(**values["prompt"]), output=LengthDistribution(**values["output"]),
                   seed=values.get("seed", 7), vocabulary_size=values.get("vocabulary_size", 32_000))

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class RequestSpec:
    request_id: str
    arrival_offset_s: float
    prompt_token_ids: tuple[int, ...]
    max_new_tokens: int


def generate_workload(profile: LoadProfile) -> list[RequestSpec]:
    if profile.arrival_rate <= 0:
        raise ValueError("arrival_rate must be positive")
    rng = random.Random(profile.seed)
    elapsed = 0.0
    out = []
    for index in range(profile.requests):
        if index:
            elapsed += rng.expovariate(profile.arrival_rate)
        prompt_length = profile.prompt.sample(rng)
        output_length = profile.output.sample(rng)
        tokens = tuple(rng.randrange(4, profile.vocabulary_size) for _ in range(prompt_length))
        out.append(RequestSpec(f"request-{index:06d}", elapsed, tokens, output_length))
    return out


def percentile(values: list[float], quantile: float) -> float:
    if not values:
        return 0.0
    ordered = sorted(values)
    position = (len(ordered) - 1) * quantile
    lower, upper = math.floor(position), math.ceil(position)
    if lower == upper:
        return ordered[lower]
    return ordered[lower] * (upper - position) + ordered[upper] * (position - lower)


@dataclass
class RequestMetrics:
    request_id: str
    arrival_s: float
    prompt_tokens: int
    requested_output_tokens: int
    first_token_s: float | None = None
    finished_s: float | None = None
    output_tokens: int = 0
    error: str | None = None

    @property
    def ttft_ms(self):
        return None if self.first_token_s is None else (self.first_token_s - self.arrival_s) * 1e3

    @property
    def tpot_ms(self):
        if self.first_token_s is None or self.finished_s is None or self.output_tokens < 2:
            return None
        return (self.finished_s - self.first_token_s) * 1e3 / (self.output_tokens - 1)

    @property
    def e2e_ms(self):
        return None if self.finished_s is None else (self.finished_s - self.arrival_s) * 1e3


@dataclass
class BenchmarkReport:
    config_name: str
    duration_s: float
    requests: list[RequestMetrics]
    cache: dict = field(default_factory=dict)
    metadata: dict = field(default_factory=dict)

    @property
    def summary(self) -> dict:
        good = [row for row in self.requests if row.error is None]
        out = {
            "config": self.config_name,
            "requests": len(self.requests),
            "successful_requests": len(good),
            "duration_s": self.duration_s,
            "throughput_tokens_per_s": sum(row.output_tokens for row in good) / max(self.duration_s, 1e-9),
        }
        for name in ("ttft_ms", "tpot_ms", "e2e_ms"):
            values = [getattr(row, name) for row in good if getattr(row, name) is not None]
            for label, q in (("p50", 0.5), ("p95", 0.95), ("p99", 0.99)):
                out[f"{name}_{label}"] = percentile(values, q)
        out.update({f"cache_{key}": value for key, value in self.cache.items()})
        return out

    def to_dict(self) -> dict:
        rows = []
        for row in self.requests:
            item = asdict(row)
            item.update(ttft_ms=row.ttft_ms, tpot_ms=row.tpot_ms, e2e_ms=row.e2e_ms)
            rows.append(item)
        return {"summary": self.summary, "metadata": self.metadata, "requests": rows}


async def run_open_loop(name: str, profile: LoadProfile, generate) -> BenchmarkReport:
    """Issue the profile's requests at their arrival times; ``generate(spec, on_token)`` is
    an async callable that returns the generated ids.  Failures are kept in the rows."""
    loop = asyncio.get_running_loop()
    start = loop.time()
    rows: list[RequestMetrics] = []

    async def execute(spec: RequestSpec) -> None:
        delay = start + spec.arrival_offset_s - loop.time()
        if delay > 0:
            await asyncio.sleep(delay)
        row = RequestMetrics(spec.request_id, loop.time(), len(spec.prompt_token_ids), spec.max_new_tokens)
        rows.append(row)

        def on_token(_: int) -> None:
            if row.first_token_s is None:
                row.first_token_s = loop.time()
            row.output_tokens += 1

        try:
            await generate(spec, on_token)
        except Exception as error:
            row.error = f"{type(error).__name__}: {error}"
        row.finished_s = loop.time()

    await asyncio.gather(*(asyncio.create_task(execute(spec)) for spec in generate_workload(profile)))
    rows.sort(key=lambda row: row.request_id)
    return BenchmarkReport(name, loop.time() - start, rows,
                           metadata={"profile": profile.to_dict(), "wall_clock_unix_s": time.time()})
