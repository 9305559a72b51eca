"""Dense SiLU-gated feed-forward (reference ``src/llmserve/model.py:180-188``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import linear_partials


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: ``intermediate_size``.  y = down(silu(gate(x)) * up(x)), no biases; gate and up are stacked
    into one matrix when the part is built (gate rows, then up rows), and the SiLU kernel adds up the
    partial sums of their product on the way."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.inter = int(params["intermediate_size"])
        self.gate_up_weight = torch.cat([weights["gate_proj.weight"], weights["up_proj.weight"]], dim=0).contiguous()
        self.down_weight = weights["down_proj.weight"].contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        inter = int(params["intermediate_size"])
        return {
            "gate_proj.weight": TensorSpec((inter, hidden_size)),
            "up_proj.weight": TensorSpec((inter, hidden_size)),
            "down_proj.weight": TensorSpec((hidden_size, inter)),
        }

    def forward(self, x):
        gate_up = linear_partials(x, self.gate_up_weight)
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.silu_mul(gate_up, act)
        return linear_partials(act, self.down_weight)
