"""Dense SiLU-gated feed-forward (reference ``src/llmserve/model.py:180-188``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import as_tensor, fused_rows, linear_partials


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: ``intermediate_size``.  y = down(silu(gate(x)) * up(x)), no biases.

    Gate and up are stacked into one matrix when the part is built.  In bfloat16, with an intermediate size
    that is a multiple of 64, their rows alternate in blocks of 64 (64 gate rows, the 64 up rows of the same
    outputs, and so on): a block of the few-rows product then holds both halves of its outputs and applies the
    gate itself, and the SiLU kernel reads the same layout when the rows are many.
    """

    graph_safe = True
    fuses_with_stream = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.inter = int(params["intermediate_size"])
        gate, up = weights["gate_proj.weight"], weights["up_proj.weight"]
        self.interleave = 0
        if ctx.dtype == torch.bfloat16 and self.inter % ops.GATE_INTERLEAVE == 0:
            self.interleave = ops.GATE_INTERLEAVE
            self.gate_up_weight = ops.interleave_gate_up(gate, up, self.interleave)
        else:
            self.gate_up_weight = torch.cat([gate, up], dim=0).contiguous()
        self.down_weight = weights["down_proj.weight"].contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        inter = int(params["intermediate_size"])
        return {
            "gate_proj.weight": TensorSpec((inter, hidden_size)),
            "up_proj.weight": TensorSpec((inter, hidden_size)),
            "down_proj.weight": TensorSpec((hidden_size, inter)),
        }

    def forward(self, x, stream=None):
        if self.interleave and fused_rows(x, self.gate_up_weight, "gate"):
            # few rows: norm (when the rows come un-normalised), product and gate in one kernel
            act = ops.gemm_bf16_gate(x, self.gate_up_weight, block_n=2 * self.interleave)
        else:
            x = as_tensor(x, self.ctx.dtype)
            gate_up = linear_partials(x, self.gate_up_weight)
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            ops.silu_mul(gate_up, act, self.interleave)
        if stream is not None and fused_rows(act, self.down_weight, "down"):
            stream.sumsq = ops.gemm_bf16_into_residual(act, self.down_weight, stream.residual, block_n=64)
            return None
        return linear_partials(act, self.down_weight)
