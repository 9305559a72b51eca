"""The generic decoder: embedding, blocks run in the order the description gives,
final norm and LM head on the wanted rows only.  Built from a ``ModelSpec``; it
does not know which architecture it serves."""
from __future__ import annotations

import torch

from ..config.model_config import LayerSpec, ModelSpec, PartSpec
from ..kernels import ops
from ..parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, BuildContext, ResidualStream)
from ..parts.linear import linear
from ..weights.tensor_spec import TensorSpec

_PART_ROLES = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")


def _layer_part_prefixes(layer: LayerSpec) -> dict[str, str]:
    """Full tensor prefix of each part of a layer: the layer's own prefix followed by the part's,
    which the architecture's builder gives in ``block.params["tensor_prefixes"]`` (a role that is
    not named there is called by its role: ``mixer.``, ``feed_forward_norm.`` and so on)."""
    names = dict(layer.block.params.get("tensor_prefixes", {}))
    return {role: layer.prefix + names.get(role, role + ".") for role in _PART_ROLES}


def _layer_parts(layer: LayerSpec) -> list[tuple[str, type, PartSpec]]:
    prefixes = _layer_part_prefixes(layer)
    return [
        (prefixes["mixer_norm"], NORMS.get(layer.mixer_norm.kind), layer.mixer_norm),
        (prefixes["mixer"], MIXERS.get(layer.mixer.kind), layer.mixer),
        (prefixes["feed_forward_norm"], NORMS.get(layer.feed_forward_norm.kind), layer.feed_forward_norm),
        (prefixes["feed_forward"], FEED_FORWARDS.get(layer.feed_forward.kind), layer.feed_forward),
    ]


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Every tensor the model reads from the checkpoint, by its full name."""
    out: dict[str, TensorSpec] = {spec.embedding_name: TensorSpec((spec.vocab_size, spec.hidden_size))}
    for layer in spec.layers:
        for prefix, cls, part in _layer_parts(layer):
            for local, tensor in cls.expected_tensors(part.params, spec.hidden_size).items():
                out[prefix + local] = tensor
    norm_cls = NORMS.get(spec.final_norm.kind)
    for local, tensor in norm_cls.expected_tensors(spec.final_norm.params, spec.hidden_size).items():
        out[spec.final_norm_prefix + local] = tensor
    if not spec.tie_word_embeddings:
        out[spec.lm_head_name] = TensorSpec((spec.vocab_size, spec.hidden_size))
    return out


def cache_requirements(spec: ModelSpec) -> list:
    """What each entry of ``spec.order`` keeps between steps.

    The list runs along ``order``, not along ``layers``: a layer that is named twice
    runs twice with the same weights, and each run has a cache of its own.  An entry
    is ``PagedKV``, ``RequestState`` or ``None`` (from the mixer), or an int: the
    position in ``order`` whose cache this run reads (``LayerSpec.cache_from`` names a
    layer; its first run is meant, and it must come earlier in the order).
    """
    from ..config.model_config import ConfigError

    first_run: dict[int, int] = {}
    out = []
    for position, index in enumerate(spec.order):
        layer = spec.layers[index]
        if layer.cache_from is not None:
            if layer.cache_from not in first_run:
                raise ConfigError(f"layer {index} reads the cache of layer {layer.cache_from}, which has not run before it")
            out.append(first_run[layer.cache_from])
        else:
            out.append(MIXERS.get(layer.mixer.kind).cache_requirement(layer.mixer.params, spec.hidden_size))
        first_run.setdefault(index, position)
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights: dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.embedding = weights[spec.embedding_name].contiguous()
        self.lm_head = self.embedding if spec.tie_word_embeddings else weights[spec.lm_head_name].contiguous()
        self.blocks = []
        for index, layer in enumerate(spec.layers):
            ctx = BuildContext(dtype, self.device, spec.hidden_size, index, spec.max_position_embeddings)
            built = []
            for prefix, cls, part in _layer_parts(layer):
                local = {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}
                built.append(cls(part.params, local, ctx))
            block_cls = BLOCKS.get(layer.block.kind)
            self.blocks.append(block_cls(layer.block.params, *built))
        ctx = BuildContext(dtype, self.device, spec.hidden_size, -1, spec.max_position_embeddings)
        prefix = spec.final_norm_prefix
        local = {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, local, ctx)

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this model can be captured in a CUDA graph: every block, every part of
        every block (mixer, its position encoding, feed-forward, both norms) and the final norm say so."""
        for block in self.blocks:
            if not getattr(block, "graph_safe", False):
                return False
            if not all(getattr(part, "graph_safe", False) for part in block.parts()):
                return False
        return bool(getattr(self.final_norm, "graph_safe", False))

    def launch_signature(self, segment_counts: list[int]) -> tuple:
        """The mixers' answers to ``Mixer.launch_signature`` for a step of this shape (each distinct answer once)."""
        answers = {block.mixer.launch_signature(segment_counts) for block in self.blocks}
        return tuple(sorted(answer for answer in answers if answer))

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads once: every matrix of every layer run, and
        the LM head (the embedding rows that a step gathers are not counted)."""
        total = self.lm_head.numel() * self.lm_head.element_size()
        for index in self.spec.order:
            block = self.blocks[index]
            for part in (block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm):
                for value in vars(part).values():
                    if isinstance(value, torch.Tensor) and value.dim() >= 1 and value.is_floating_point():
                        total += value.numel() * value.element_size()
        return total

    def forward(self, step, caches) -> torch.Tensor:
        """Run the step's rows through the layers and return float32 logits
        [number of wanted rows, vocab] (an empty tensor when nothing is wanted)."""
        tokens = step.num_tokens
        residual = torch.empty((tokens, self.spec.hidden_size), dtype=torch.float32, device=self.device)
        ops.embedding(self.embedding, step.token_ids, residual)
        stream = ResidualStream(residual)
        for position, index in enumerate(self.spec.order):   # caches run along the order
            self.blocks[index].forward(stream, step, caches[position])
        if step.num_wanted == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        x = self.final_norm.forward(stream, rows=step.want_rows)
        return linear(x, self.lm_head, out_dtype=torch.float32)
