"""Matrix products of the layers: y = x W^T (+ b), W kept [out, in].

float32: the engine's own FMA kernel (true 32-bit, fixed summation order).
bfloat16: the library product with float32 accumulation, where the reference
uses ``nn.Linear`` (``src/llmserve/model.py:51-66,183-185,248``).
"""
from __future__ import annotations

import torch

from ..kernels import ops


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
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
        return y if bias is None else y + bias
    y = torch.mm(x, weight.t())
    return y if bias is None else y + bias.to(y.dtype)
