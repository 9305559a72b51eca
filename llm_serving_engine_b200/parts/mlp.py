"""Dense SiLU-gated feed-forward (reference ``src/llmserve/model.py:180-188``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import SKINNY_MAX_ROWS, linear_partials


# Rows of gate and up interleaved in blocks of this many (32 or 64) let the few-rows product apply the
# gate in its epilogue; 0 keeps gate rows then up rows and a separate SiLU kernel.  Measured on the
# Qwen2.5-1.5B shape at batch 8, the separate kernel behind a two-split product is faster (more blocks
# fetch weights ahead), so the fused form is off unless the part's ``fuse_gate`` parameter asks for it.
FUSE_GATE = 0
# With at most 16 rows the gate can also be worked out inside the down product, from the partial sums of
# the gate/up product (no SiLU kernel, no activations in memory).  Measured on the same shape it is
# slower as well (1.56 against 1.48 ms a step): making the activations sits on the product's critical
# path, while the separate SiLU kernel runs beside the product's first weight loads.  Off unless
# LSE_FUSE_GATE_INTO_DOWN=1.
FUSE_GATE_INTO_DOWN = __import__("os").environ.get("LSE_FUSE_GATE_INTO_DOWN", "0") == "1"
# A third form: the gate applied by the split of the gate/up product that finishes last in its block
# column (the product keeps its splits; gate and up rows interleaved in blocks of 64).  Measured slower
# too (1.53 against 1.48 ms a step at batch 8, 2.21 against 1.95 at batch 32): the last split's extra
# round trips are serial, the SiLU kernel's are not.  Off unless LSE_FINISH_GATE=1.
FINISH_GATE = __import__("os").environ.get("LSE_FINISH_GATE", "0") == "1"


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: ``intermediate_size``, optional ``fuse_gate`` (0, 32 or 64).  y = down(silu(gate(x)) * up(x)),
    no biases; gate and up are stacked into one matrix when the part is built."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.inter = int(params["intermediate_size"])
        # bfloat16 and I a multiple of 32: gate and up rows are interleaved in blocks of 32, the layout
        # whose few-rows product applies the SiLU gate in its epilogue; else gate rows, then up rows
        self.interleave = 0
        self.arrivals = None
        wish = int(params.get("fuse_gate", FUSE_GATE))
        if (ctx.dtype == torch.bfloat16 and not wish and FINISH_GATE and not FUSE_GATE_INTO_DOWN
                and self.inter % ops.FINISH_GATE_INTERLEAVE == 0):
            self.interleave = ops.FINISH_GATE_INTERLEAVE
            self.gate_up_weight = ops.interleave_gate_up(weights["gate_proj.weight"], weights["up_proj.weight"], self.interleave)
            self.arrivals = torch.zeros(2 * self.inter // 128, dtype=torch.int32, device=ctx.device)   # this product's own
        elif ctx.dtype == torch.bfloat16 and wish and self.inter % wish == 0:
            self.interleave = wish
            self.gate_up_weight = ops.interleave_gate_up(weights["gate_proj.weight"], weights["up_proj.weight"], wish)
        else:
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
        if self.arrivals is not None and x.shape[0] <= SKINNY_MAX_ROWS and ops.gemm_bf16_skinny_ok(x, self.gate_up_weight):
            # few rows: the split that finishes last in a block column applies the gate to the column's sums
            _, act = ops.gemm_bf16_skinny_finish_gate(x, self.gate_up_weight, self.arrivals)
        elif (self.interleave and self.arrivals is None and x.shape[0] <= SKINNY_MAX_ROWS
              and ops.gemm_bf16_skinny_ok(x, self.gate_up_weight)):
            act = ops.gemm_bf16_skinny_gated(x, self.gate_up_weight, self.interleave)   # product and gate in one kernel
        else:
            gate_up = linear_partials(x, self.gate_up_weight)
            if (FUSE_GATE_INTO_DOWN and not self.interleave
                    and ops.gemm_bf16_skinny_gated_in_ok(gate_up, self.down_weight)):
                # few rows: the gate is worked out inside the down product, from the partial sums
                return ops.gemm_bf16_skinny_gated_in(gate_up, self.down_weight)
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            ops.silu_mul(gate_up, act, self.interleave)
        return linear_partials(act, self.down_weight)
