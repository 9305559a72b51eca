"""Cache and scheduler settings, with the reference's names and defaults
(``src/llmserve/config.py:65-76``)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class CacheConfig:
    """``block_size`` tokens per page, ``num_blocks`` pages in every layer group's pool;
    ``num_state_slots`` fixed-size per-request state slots (0 = as many as the
    scheduler's ``max_batch_size``)."""

    block_size: int = 16
    num_blocks: int = 1_024
    num_state_slots: int = 0

    def __post_init__(self) -> None:
        if self.block_size <= 0 or self.num_blocks <= 0 or self.num_state_slots < 0:
            raise ValueError("block_size and num_blocks must be positive")


@dataclass(frozen=True)
class SchedulerConfig:
    """``max_batch_size`` live requests, ``max_tokens_per_step`` token budget of a
    step, admission ``policy`` (fcfs, sjf, priority) and the ``preemption``
    victim rule when pages run out (``largest``: the request that has
    processed the most tokens, as ``src/llmserve/engine.py:258`` picks it)."""

    max_batch_size: int = 16
    max_tokens_per_step: int = 2_048
    policy: str = "fcfs"
    preemption: str = "largest"

    def __post_init__(self) -> None:
        if self.max_batch_size <= 0 or self.max_tokens_per_step <= 0:
            raise ValueError("max_batch_size and max_tokens_per_step must be positive")
        if self.policy not in ("fcfs", "sjf", "priority"):
            raise ValueError("policy must be fcfs, sjf, or priority")
        if self.preemption != "largest":
            raise ValueError("preemption must be 'largest'")
