"""Typed model configuration and the description of a model as data.

Two levels:

* ``Qwen2Config`` is the typed form of a Qwen2/Qwen2.5 ``config.json``: every
  size and constant of the architecture comes from that file's own keys (the
  reference reads the same keys in ``src/llmserve/config.py:10-62``).
* ``ModelSpec`` is what the generic decoder is built from: a list of
  ``LayerSpec`` (which mixer, feed-forward, norm and block arrangement a layer
  uses, with their parameters) and ``order``, the list of layer indices in the
  order they run.  An architecture's builder turns its typed configuration into
  a ``ModelSpec``; nothing below the builder knows which architecture it serves.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


@dataclass(frozen=True)
class PartSpec:
    """A registered part by name, with the constants it is built with."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: its parts and the prefix of its tensors.

    ``cache_from`` names another layer whose cache this layer reads instead of
    owning one (shared keys and values); ``None`` means the layer owns its cache.
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder as data: embedding, layers, the order they run in, head."""

    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple[LayerSpec, ...]
    order: tuple[int, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_prefix: str
    lm_head_name: str
    tie_word_embeddings: bool
    max_position_embeddings: int

    def __post_init__(self) -> None:
        for index in self.order:
            if not 0 <= index < len(self.layers):
                raise ConfigError(f"order names layer {index}, model has {len(self.layers)}")
        for number, layer in enumerate(self.layers):
            if layer.cache_from is not None and not 0 <= layer.cache_from < len(self.layers):
                raise ConfigError(f"layer {number} reads the cache of unknown layer {layer.cache_from}")


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "num_key_value_heads",
    "max_position_embeddings",
    "rope_theta",
    "rms_norm_eps",
)


@dataclass(frozen=True)
class Qwen2Config:
    """Typed ``config.json`` of ``Qwen2ForCausalLM``.

    Keys and meaning follow the reference's ``ModelConfig``
    (``src/llmserve/config.py:10-62``): ``num_hidden_layers`` (alias
    ``num_layers``), ``max_position_embeddings`` (alias ``max_seq_len``),
    ``attention_bias`` defaulting to true because Qwen2 files omit it, and
    ``tie_word_embeddings`` defaulting to true.  Beyond the reference:
    ``head_dim`` may be given (default ``hidden_size / num_attention_heads``);
    ``use_sliding_window`` is read and refused when true, because the reference
    has no windowed attention; ``rope_pairing`` (this engine's own key) chooses
    how rotary pairs are formed, ``interleaved`` being the reference's
    (``src/llmserve/model.py:39-42``).
    """

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    head_dim: int = 0
    attention_bias: bool = True
    tie_word_embeddings: bool = True
    use_sliding_window: bool = False
    hidden_act: str = "silu"
    rope_pairing: str = "interleaved"
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = ("Qwen2ForCausalLM",)
    model_type: str = "qwen2"

    def __post_init__(self) -> None:
        if self.head_dim == 0:
            if self.hidden_size % self.num_attention_heads:
                raise ConfigError("hidden_size must be divisible by num_attention_heads when head_dim is absent")
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "max_position_embeddings", "head_dim"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2:
            raise ConfigError("head_dim must be even for rotary position encoding")
        if self.use_sliding_window:
            raise ConfigError("use_sliding_window=true is not supported: the architecture runs full attention")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported: the feed-forward is SiLU-gated")
        if self.rope_pairing not in ("interleaved", "half"):
            raise ConfigError(f"rope_pairing must be 'interleaved' or 'half', got {self.rope_pairing!r}")
        if not self.rope_theta > 0 or not self.rms_norm_eps > 0:
            raise ConfigError("rope_theta and rms_norm_eps must be positive")

    # -- reading ---------------------------------------------------------------
    @classmethod
    def from_dict(cls, values: dict[str, Any]) -> "Qwen2Config":
        aliases = {"num_layers": "num_hidden_layers", "max_seq_len": "max_position_embeddings"}
        normalized = {aliases.get(key, key): value for key, value in values.items()}
        missing = [key for key in _REQUIRED if key not in normalized]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if normalized.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is not supported")
        known = cls.__dataclass_fields__.keys()
        picked = {key: value for key, value in normalized.items() if key in known and value is not None}
        if "architectures" in picked:
            picked["architectures"] = tuple(picked["architectures"])
        for key in ("rope_theta", "rms_norm_eps"):
            picked[key] = float(picked[key])
        return cls(**picked)

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen2Config":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def to_dict(self) -> dict[str, Any]:
        values = {name: getattr(self, name) for name in self.__dataclass_fields__}
        values["architectures"] = list(self.architectures)
        return values
