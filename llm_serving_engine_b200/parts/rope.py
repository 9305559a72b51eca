"""Rotary position encoding, fused with the bias and the cache write."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope")
class RotaryEncoding(PositionEncoding):
    """params: ``theta``, ``head_dim``, ``pairing`` ("interleaved" pairs (2i, 2i+1)
    as the reference rotates, ``src/llmserve/model.py:35-43``; "half" pairs
    (i, i + D/2)).  Angles are position * 1/theta^(2i/D) in float32
    (``src/llmserve/model.py:29-31``), computed in the kernel from the position."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        head_dim = int(params["head_dim"])
        theta = float(params["theta"])
        self.pairing = {"interleaved": 0, "half": 1}[params.get("pairing", "interleaved")]
        inverse = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
        self.inv_freq = inverse.to(ctx.device)

    def encode_and_store(self, qkv, bias, step, cache, q_out, n_q, n_kv, head_dim) -> None:
        ops.rope_kv_write(qkv, bias, step.positions, cache.slot_mapping, self.inv_freq, q_out,
                          cache.keys, cache.values, n_q, n_kv, head_dim, self.pairing)
