"""Random-weights mode: writes a model folder from a configuration and a seed.

Each tensor is drawn from its own generator seeded by (seed, tensor name), so
its values do not depend on the order of creation or on how the engine fuses
tensors later.  Distributions: matrices and embeddings N(0, 0.02) (the
reference's initialisation, ``src/llmserve/model.py:253-258``); biases
N(0, 0.02) and norm weights 1 + U(-0.1, 0.1), not the reference's zeros and
ones, so that a wrong bias or norm shows in the logits.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .tensor_spec import TensorSpec

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: TensorSpec, seed: int) -> torch.Tensor:
    """The float32 (int32 for tables) values of tensor ``name`` under ``seed``."""
    generator = torch.Generator(device="cpu").manual_seed(tensor_seed(seed, name))
    if spec.kind in ("matrix", "bias"):
        return torch.randn(spec.shape, generator=generator, dtype=torch.float32) * 0.02
    if spec.kind == "norm":
        return 1.0 + (torch.rand(spec.shape, generator=generator, dtype=torch.float32) * 0.2 - 0.1)
    return torch.randint(0, 2**15, spec.shape, generator=generator, dtype=torch.int32)


def random_weights(expected: dict[str, TensorSpec], seed: int, matrix_dtype=torch.float32) -> dict[str, torch.Tensor]:
    out = {}
    for name, spec in expected.items():
        tensor = random_tensor(name, spec, seed)
        if spec.kind == "matrix":
            tensor = tensor.to(matrix_dtype)
        out[name] = tensor
    return out


def write_random_model(folder, config: dict, seed: int, dtype: str | None = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a config.json
    dictionary) with random weights.  ``dtype`` ("float32" or "bfloat16", default
    the configuration's ``torch_dtype``, else float32) is the stored type of the
    matrices; vectors are stored in float32."""
    from safetensors.torch import save_file

    from ..config import load_config
    from ..models import expected_tensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    config = dict(config)
    stored = dtype or config.get("torch_dtype") or "float32"
    if stored not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {stored!r}")
    config["torch_dtype"] = stored
    _, _, spec = load_config(config)
    tensors = random_weights(expected_tensors(spec), seed, _DTYPES[stored])
    (folder / "config.json").write_text(json.dumps(config, indent=2) + "\n")
    save_file({name: tensor.contiguous() for name, tensor in tensors.items()},
              str(folder / "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder
