"""Matrix products of the layers: y = x W^T (+ b), W kept [out, in].

float32: the engine's own FMA kernel (true 32-bit, fixed summation order: a few rows give the same bits as a
stack of partial sums that the next kernel adds up as they do from the kernel that adds them up itself).
bfloat16, few rows (decoding): the engine's tcgen05 kernel, which streams the
weights with TMA and may cut the k range into splits; it returns a float32 stack
of partial sums [P, rows, out] that the next kernel (norm, rotary, SiLU) adds up.
bfloat16, many rows: the library product with float32 accumulation, where the
reference uses ``nn.Linear`` (``src/llmserve/model.py:51-66,183-185,248``).
"""
from __future__ import annotations

import torch

from ..kernels import ops

import os

# above this many rows the library product is faster (LSE_SKINNY_MAX_ROWS overrides, for comparisons)
SKINNY_MAX_ROWS = int(os.environ.get("LSE_SKINNY_MAX_ROWS", "32"))


# The library product (rows beyond SKINNY_MAX_ROWS) accumulates in float32 all the way: no bfloat16 partial sums
# when it splits the k range.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


def reduce_partials(y: torch.Tensor) -> torch.Tensor:
    """[rows, out] from a branch output that may be a stack of partial sums [P, rows, out]: added in index
    order, starting from zero, as the kernels that consume such stacks add them."""
    if y.dim() == 3:
        total = torch.zeros_like(y[0])
        for part in y:
            total += part
        return total
    return y


def linear_partials(x: torch.Tensor, weight: torch.Tensor, max_splits: int | None = None) -> torch.Tensor:
    """x W^T as [rows, out] or, for few bfloat16 rows, as a float32 stack of partial sums
    [P, rows, out].  For callers whose consumer kernel adds the partials itself."""
    if (x.is_cuda and weight.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_MAX_ROWS
            and ops.gemm_bf16_skinny_ok(x, weight)):
        return ops.gemm_bf16_skinny(x, weight, max_splits=max_splits)
    if x.is_cuda and weight.dtype == torch.float32 and x.dtype == torch.float32 and ops.gemm_f32_stack_ok(x, weight):
        return ops.gemm_f32_stack(x, weight)   # at most eight partial sums: what every consumer fetches in one go
    return linear(x, weight)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None) -> torch.Tensor:
    if not x.is_cuda:
        raise ops.KernelError("linear runs on CUDA tensors only; there is no CPU fallback")
    rows, out_features = x.shape[0], weight.shape[0]
    if weight.dtype == torch.float32:
        out = torch.empty((rows, out_features), dtype=torch.float32, device=x.device)
        return ops.gemm_f32_nt(x, weight, bias, out)
    if weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        raise ops.KernelError(f"linear: unsupported dtypes {x.dtype} x {weight.dtype}")
    if out_dtype == torch.float32:
        if rows <= SKINNY_MAX_ROWS and ops.gemm_bf16_skinny_ok(x, weight):
            y = reduce_partials(ops.gemm_bf16_skinny(x, weight))
        else:
            y = torch.mm(x, weight.t(), out_dtype=torch.float32)
        return y if bias is None else y + bias
    y = torch.mm(x, weight.t())
    return y if bias is None else y + bias.to(y.dtype)
