"""Weights from safetensors, by tensor name.

The reference copies tensors by name into its module tree and reports a wrong
shape or missing tensors (``src/llmserve/checkpoint.py:46-67``).  Here the
model description says which tensors it expects (name -> ``TensorSpec``); the
loader compares that with the files and raises ONE error that lists every
missing tensor, every unexpected tensor and every wrong shape.

How tensors are held: matrices in the compute dtype (bfloat16 for serving,
float32 for the 32-bit path); vectors (norm weights, biases) in float32, which
holds a bfloat16 value exactly and leaves a tensor stored in 32-bit as it is;
integer tables as int32.
"""
from __future__ import annotations

from pathlib import Path

import torch

from .tensor_spec import TensorSpec


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every mismatch."""

    def __init__(self, folder, missing, unexpected, wrong_shapes):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shapes = sorted(wrong_shapes)
        lines = [f"checkpoint {folder} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shapes:
            lines.append(f"  wrong shapes ({len(self.wrong_shapes)}): " + ", ".join(
                f"{name} is {list(got)}, expected {list(want)}" for name, got, want in self.wrong_shapes))
        super().__init__("\n".join(lines))


def held_dtype(spec: TensorSpec, stored: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.kind == "table" or not stored.is_floating_point:
        return torch.int32
    if spec.kind == "matrix":
        return compute_dtype
    return torch.float32


def load_weights(folder, expected: dict[str, TensorSpec], compute_dtype: torch.dtype, device,
                 optional: frozenset[str] = frozenset()) -> dict[str, torch.Tensor]:
    """Read every ``*.safetensors`` of ``folder`` and return name -> tensor on ``device``.

    ``optional`` names may be present without being expected (a tied LM head
    that the file repeats); they are skipped.
    """
    from safetensors import safe_open

    folder = Path(folder)
    files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {folder}")
    loaded: dict[str, torch.Tensor] = {}
    unexpected: list[str] = []
    wrong: list[tuple[str, tuple, tuple]] = []
    for filename in files:
        with safe_open(str(filename), framework="pt", device="cpu") as source:
            for name in source.keys():
                spec = expected.get(name)
                if spec is None:
                    if name not in optional:
                        unexpected.append(name)
                    continue
                shape = tuple(source.get_slice(name).get_shape())
                if shape != tuple(spec.shape):
                    wrong.append((name, shape, tuple(spec.shape)))
                    continue
                tensor = source.get_tensor(name)
                loaded[name] = tensor.to(device=device, dtype=held_dtype(spec, tensor.dtype, compute_dtype))
    wrong_names = {name for name, _, _ in wrong}
    missing = [name for name in expected if name not in loaded and name not in wrong_names]
    if missing or unexpected or wrong:
        raise WeightError(folder, missing, unexpected, wrong)
    return loaded
