"""RMSNorm fused with the residual sum (reference ``src/llmserve/model.py:14-23``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Norm, ResidualStream, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``eps``.  y = (x * rsqrt(mean(x^2) + eps)) * weight, where x is the
    float32 residual after the pending branch output has been added to it."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.eps = float(params["eps"])
        self.weight = weights["weight"].to(torch.float32).contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        return {"weight": TensorSpec((hidden_size,), "norm")}

    def forward(self, stream: ResidualStream, rows: torch.Tensor | None = None) -> torch.Tensor:
        n_rows = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_rows, stream.residual.shape[1]), dtype=self.ctx.dtype, device=stream.residual.device)
        ops.add_rmsnorm(stream.residual, stream.delta, self.weight, self.eps, out, rows=rows,
                        write_residual=rows is None)
        if rows is None:
            stream.delta = None
        return out
