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


class _Turn:
    """The buffers of one sampling launch.  There are two, used in turn, so that a launch may be queued
    while the tokens of the one before have not been read yet."""

    def __init__(self, max_rows: int, device, pinned: bool) -> None:
        self.host_f = torch.empty((2, max_rows), dtype=torch.float32, pin_memory=pinned)
        self.host_i = torch.empty((2, max_rows), dtype=torch.int64, pin_memory=pinned)
        self.dev_f = torch.empty((2, max_rows), dtype=torch.float32, device=device)
        self.dev_i = torch.empty((2, max_rows), dtype=torch.int64, device=device)
        self.out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self.host_out = torch.empty(max_rows, dtype=torch.int32, pin_memory=pinned)
        self.host_status = torch.zeros(2, dtype=torch.int32, pin_memory=pinned) if pinned else None
        self.done = torch.cuda.Event() if pinned else None
        self.rows = 0


class Sampler:
    """Reusable buffers for sampling up to ``max_rows`` rows of ``vocab`` logits."""

    def __init__(self, vocab: int, max_rows: int, device) -> None:
        self.vocab, self.max_rows = vocab, max_rows
        self.device = torch.device(device)
        pinned = self.device.type == "cuda"
        self._turns = [_Turn(max_rows, self.device, pinned), _Turn(max_rows, self.device, pinned)]
        self._last = 1
        self._scratch = None

    def sample(self, logits: torch.Tensor, configs: list[GenerationConfig], counters: list[int]) -> list[int]:
        """One token per row of ``logits`` (float32 [R, V]); ``counters[r]`` is the index of
        the token being generated for row r's request.  One device-to-host transfer."""
        return self.collect(self.launch(logits, configs, counters))

    def launch(self, logits: torch.Tensor, configs: list[GenerationConfig], counters: list[int]) -> int:
        """Start sampling and the copy of the tokens to the host; returns a ticket for :meth:`collect`,
        which waits for them.  What the host does in between runs beside the device's work.  At most
        two launches may be outstanding."""
        rows = logits.shape[0]
        if rows != len(configs) or rows != len(counters) or rows > self.max_rows:
            raise ValueError("batched sampling inputs must have matching rows")
        ticket = self._last ^ 1
        turn = self._turns[ticket]
        out = turn.out[:rows]
        if all(config.temperature <= 0 for config in configs):
            ops.argmax(logits, out)
        else:
            if self._scratch is None:
                self._scratch = torch.empty(self.max_rows * self.vocab, dtype=torch.float32, device=self.device)
            for row, (config, counter) in enumerate(zip(configs, counters)):
                turn.host_f[0, row] = config.temperature
                turn.host_f[1, row] = config.top_p
                turn.host_i[0, row] = config.seed
                turn.host_i[1, row] = counter
            turn.dev_f.copy_(turn.host_f, non_blocking=True)
            turn.dev_i.copy_(turn.host_i, non_blocking=True)
            ops.sample(logits, turn.dev_f[0, :rows], turn.dev_f[1, :rows], turn.dev_i[0, :rows],
                       turn.dev_i[1, :rows], self._scratch, out)
        turn.host_out[:rows].copy_(out, non_blocking=True)
        if turn.host_status is not None:
            ops.kernel_status_async(turn.host_status)     # arrives with the tokens: no synchronisation of its own
        if turn.done is not None:
            turn.done.record()
        turn.rows = rows
        self._last = ticket
        return ticket

    def device_tokens(self, ticket: int) -> torch.Tensor:
        """The tokens of that launch on the device (int32 [rows]), for a step that is queued behind it."""
        turn = self._turns[ticket]
        return turn.out[:turn.rows]

    def collect(self, ticket: int | None = None) -> list[int]:
        """The tokens of that launch (default: the last one); waits until the device has delivered them."""
        turn = self._turns[self._last if ticket is None else ticket]
        if turn.done is not None:
            turn.done.synchronize()
        if turn.host_status is not None and (turn.host_status[0] or turn.host_status[1]):
            which = " and ".join(name for name, word in zip(("the few-rows product", "the tcgen05 prompt attention"),
                                                            turn.host_status.tolist()) if word)
            turn.host_status.zero_()
            ops.kernel_status_reset()
            raise ops.KernelError(f"a bounded wait inside {which} gave up: the step's results are not valid")
        return turn.host_out[:turn.rows].tolist()
