"""What a part expects of the checkpoint: a tensor's shape and its kind."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TensorSpec:
    """``kind`` decides how the tensor is held and how random weights draw it:
    ``matrix`` (held in the compute dtype; N(0, 0.02)), ``bias`` (float32 vector;
    N(0, 0.02)), ``norm`` (float32 vector; 1 + U(-0.1, 0.1)), ``table``
    (integers, held as int32)."""

    shape: tuple[int, ...]
    kind: str = "matrix"

    def __post_init__(self) -> None:
        if self.kind not in ("matrix", "bias", "norm", "table"):
            raise ValueError(f"unknown tensor kind {self.kind!r}")
