"""Model building: config.json -> description -> weights -> ``DecoderModel``."""
from __future__ import annotations

import torch

from . import qwen2  # noqa: F401  (registers Qwen2ForCausalLM)
from .decoder import DecoderModel, cache_requirements, expected_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}") from None


def load_model(folder, dtype="bfloat16", device="cuda") -> DecoderModel:
    """Build the model that ``folder/config.json`` names and load ``folder``'s safetensors."""
    from ..config import load_config
    from ..weights import load_weights

    dtype = parse_dtype(dtype)
    _, _, spec = load_config(folder)
    optional = frozenset({spec.lm_head_name}) if spec.tie_word_embeddings else frozenset()
    weights = load_weights(folder, expected_tensors(spec), dtype, device, optional=optional)
    return DecoderModel(spec, weights, dtype, device)


def random_model(config: dict, seed: int, dtype="bfloat16", device="cuda") -> DecoderModel:
    """The same model as ``write_random_model`` + ``load_model`` would give with
    matrices stored in float32, without touching the disk."""
    from ..config import load_config
    from ..weights.loader import held_dtype
    from ..weights.random_init import random_tensor

    dtype = parse_dtype(dtype)
    _, _, spec = load_config(config)
    weights = {}
    for name, tensor_spec in expected_tensors(spec).items():
        tensor = random_tensor(name, tensor_spec, seed)
        weights[name] = tensor.to(device=device, dtype=held_dtype(tensor_spec, tensor.dtype, dtype))
    return DecoderModel(spec, weights, dtype, device)


__all__ = ["DecoderModel", "cache_requirements", "expected_tensors", "load_model", "parse_dtype",
           "random_model"]
