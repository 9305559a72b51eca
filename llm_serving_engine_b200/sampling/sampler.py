"""Greedy, temperature and top-p sampling, on the device.

Options are the reference's ``GenerationConfig`` (``src/llmserve/engine.py:20-26``):
``temperature <= 0`` takes the argmax; otherwise softmax(logits / temperature),
cut by ``top_p`` when below 1, and one draw per token.  The draw is the inverse
CDF in vocabulary order at u = uniform(seed, index of the generated token), a
counter-based number: a request's tokens do not depend on what else is in the
batch, and a request that is recomputed after a preemption draws the same
numbers again.  (The reference draws with ``torch.multinomial`` from a
per-request generator, ``engine.py:41,218-219``; its stream is not reproduced.)
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import ops


@dataclass(frozen=True)
class GenerationConfig:
    max_new_tokens: int = 32
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 7
    stop_token_ids: tuple[int, ...] = ()


_MASK64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return x ^ (x >> 31)


def uniform01(seed: int, counter: int) -> float:
    """The number the sampling kernel draws for (seed, counter): 24 bits in [0, 1)."""
    mixed = _splitmix64(_splitmix64(seed & _MASK64) ^ ((counter * 0xD1342543DE82EF95 + 1) & _MASK64))
    return (mixed >> 40) / 16777216.0


class Sampler:
    """Reusable buffers for sampling up to ``max_rows`` rows of ``vocab`` logits."""

    def __init__(self, vocab: int, max_rows: int, device) -> None:
        self.vocab, self.max_rows = vocab, max_rows
        self.device = torch.device(device)
        pinned = self.device.type == "cuda"
        self._host_f = torch.empty((2, max_rows), dtype=torch.float32, pin_memory=pinned)
        self._host_i = torch.empty((2, max_rows), dtype=torch.int64, pin_memory=pinned)
        self._dev_f = torch.empty((2, max_rows), dtype=torch.float32, device=self.device)
        self._dev_i = torch.empty((2, max_rows), dtype=torch.int64, device=self.device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._host_out = torch.empty(max_rows, dtype=torch.int32, pin_memory=pinned)
        self._scratch = None
        self._pending_rows = 0

    def sample(self, logits: torch.Tensor, configs: list[GenerationConfig], counters: list[int]) -> list[int]:
        """One token per row of ``logits`` (float32 [R, V]); ``counters[r]`` is the index of
        the token being generated for row r's request.  One device-to-host transfer."""
        self.launch(logits, configs, counters)
        return self.collect()

    def launch(self, logits: torch.Tensor, configs: list[GenerationConfig], counters: list[int]) -> None:
        """Start sampling and the copy of the tokens to the host; :meth:`collect` waits for them.
        What the host does in between runs beside the device's work."""
        rows = logits.shape[0]
        if rows != len(configs) or rows != len(counters) or rows > self.max_rows:
            raise ValueError("batched sampling inputs must have matching rows")
        out = self._out[:rows]
        if all(config.temperature <= 0 for config in configs):
            ops.argmax(logits, out)
        else:
            if self._scratch is None:
                self._scratch = torch.empty(self.max_rows * self.vocab, dtype=torch.float32, device=self.device)
            for row, (config, counter) in enumerate(zip(configs, counters)):
                self._host_f[0, row] = config.temperature
                self._host_f[1, row] = config.top_p
                self._host_i[0, row] = config.seed
                self._host_i[1, row] = counter
            self._dev_f.copy_(self._host_f, non_blocking=True)
            self._dev_i.copy_(self._host_i, non_blocking=True)
            ops.sample(logits, self._dev_f[0, :rows], self._dev_f[1, :rows], self._dev_i[0, :rows],
                       self._dev_i[1, :rows], self._scratch, out)
        self._host_out[:rows].copy_(out, non_blocking=True)
        self._pending_rows = rows

    def collect(self) -> list[int]:
        """The tokens of the last :meth:`launch` (waits for the device)."""
        torch.cuda.current_stream().synchronize()
        return self._host_out[:self._pending_rows].tolist()
