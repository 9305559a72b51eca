"""Interfaces of the parts a decoder layer is put together from, and their registries.

A part is built from ``params`` (its sizes and constants, taken from the
configuration), ``weights`` (its own tensors, by their local names) and a
``BuildContext``.  No part knows which model it is in.

* ``Norm``:            ``forward(stream, rows=None) -> x``  (adds the pending branch
                       output to the float32 residual, returns the normalised rows)
* ``PositionEncoding``: ``encode_and_store(...)`` (rotates queries and keys and
                       writes keys and values into the layer's cache pages)
* ``Mixer``:           ``forward(x, step, cache) -> y`` over the step's flat rows
                       (y is [T, H], or a float32 stack of partial sums [P, T, H]
                       that the next norm adds up; ``reduce_partials`` gives [T, H]),
                       reading and writing its layer's cache; ``cache_requirement``
                       says what it needs (pages of keys and values, or a
                       fixed-size state per request, or nothing)
* ``FeedForward``:     ``forward(x) -> y``, row-local
* ``Block``:           the arrangement of the four in a layer:
                       ``forward(stream, step, cache)``

Each class also has ``expected_tensors(params, hidden_size)``: local tensor name
-> ``TensorSpec``; the loader and the random-weights mode are driven by it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from ..weights.tensor_spec import TensorSpec


@dataclass(frozen=True)
class BuildContext:
    dtype: torch.dtype            # compute dtype: torch.bfloat16 or torch.float32
    device: torch.device
    hidden_size: int
    layer_index: int
    max_position_embeddings: int


@dataclass(frozen=True)
class PagedKV:
    """The mixer keeps keys and values of every token in pages.  ``window`` > 0:
    only the last ``window`` keys are read, older pages are given back."""

    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class RequestState:
    """The mixer keeps a state of fixed size per request: a tensor of ``shape``
    and ``dtype`` ("float32" or "bfloat16"), zeroed when the request is created."""

    shape: tuple[int, ...]
    dtype: str = "float32"


class ResidualStream:
    """The hidden state between parts: the float32 residual [T, H] and the output
    of the last branch, not yet added (the next norm adds it in float32)."""

    __slots__ = ("residual", "delta")

    def __init__(self, residual: torch.Tensor, delta: torch.Tensor | None = None) -> None:
        self.residual = residual
        self.delta = delta


class Part:
    # True when the part only launches work whose shape depends on the number of rows and reads
    # everything else (positions, segments, tables, routing decisions) from device memory, without
    # waiting for the device: a step made of such parts can be captured in a CUDA graph and
    # replayed with other contents.  A model is captured only if every part of it says so.
    graph_safe = False

    def __init__(self, params: dict[str, Any], weights: dict[str, torch.Tensor], ctx: BuildContext) -> None:
        self.params = params
        self.ctx = ctx

    @classmethod
    def expected_tensors(cls, params: dict[str, Any], hidden_size: int) -> dict[str, TensorSpec]:
        return {}


class Norm(Part):
    def forward(self, stream: ResidualStream, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv, bias, step, cache, q_out, n_q, n_kv, head_dim) -> None:
        raise NotImplementedError


class Mixer(Part):
    @classmethod
    def cache_requirement(cls, params: dict[str, Any], hidden_size: int):
        """``PagedKV``, ``RequestState`` or ``None``."""
        return None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        raise NotImplementedError

    def launch_signature(self, segment_counts: list[int]) -> tuple:
        """What of a step's shape, beyond its numbers of rows and requests, decides which kernels ``forward``
        launches (``segment_counts``: tokens of each request in the step).  Steps with different signatures
        are captured in CUDA graphs of their own; ``forward`` must choose by the same rule."""
        return ()


class FeedForward(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    graph_safe = False     # as for ``Part``: the arrangement itself launches nothing that depends on the step's contents

    def __init__(self, params, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Norm,
                 feed_forward: FeedForward) -> None:
        self.params = params
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def parts(self) -> list:
        """Every part this block runs (a mixer's position encoding included)."""
        found = [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]
        position = getattr(self.mixer, "position", None)
        if position is not None:
            found.append(position)
        return found

    def forward(self, stream: ResidualStream, step, cache) -> None:
        raise NotImplementedError


@dataclass
class _Registry:
    what: str
    entries: dict[str, type] = field(default_factory=dict)

    def register(self, name: str, cls: type | None = None):
        if cls is None:
            def decorator(inner: type) -> type:
                self.entries[name] = inner
                return inner
            return decorator
        self.entries[name] = cls
        return cls

    def get(self, name: str) -> type:
        try:
            return self.entries[name]
        except KeyError:
            raise KeyError(f"unknown {self.what} {name!r}; registered: {sorted(self.entries)}") from None


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITION_ENCODINGS = _Registry("position encoding")
BLOCKS = _Registry("block")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_block = BLOCKS.register
