"""Qwen2 / Qwen2.5 dense decoder as a ``ModelSpec``
(the reference's ``Transformer``, ``src/llmserve/model.py:237-309``).

Tensor names are the checkpoint's own (``src/llmserve/checkpoint.py:51-53`` strips
the ``model.`` prefix that is kept here):
``model.embed_tokens.weight``, ``model.layers.{i}.input_layernorm.weight``,
``model.layers.{i}.self_attn.{q,k,v}_proj.{weight,bias}``,
``model.layers.{i}.self_attn.o_proj.weight``,
``model.layers.{i}.post_attention_layernorm.weight``,
``model.layers.{i}.mlp.{gate,up,down}_proj.weight``, ``model.norm.weight``,
``lm_head.weight`` (absent when the embeddings are tied).
"""
from __future__ import annotations

from ..config.model_config import LayerSpec, ModelSpec, PartSpec, Qwen2Config
from ..config.registry import register_architecture


def build_qwen2_spec(config: Qwen2Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": config.rms_norm_eps})
    position = {"kind": "rope", "params": {"theta": config.rope_theta, "head_dim": config.head_dim,
                                           "pairing": config.rope_pairing}}
    mixer = PartSpec("gqa_attention", {
        "num_heads": config.num_attention_heads,
        "num_kv_heads": config.num_key_value_heads,
        "head_dim": config.head_dim,
        "bias": config.attention_bias,
        "window": 0,
        "position": position,
    })
    feed_forward = PartSpec("swiglu", {"intermediate_size": config.intermediate_size})
    block = PartSpec("prenorm_residual", {"tensor_prefixes": {
        "mixer_norm": "input_layernorm.", "mixer": "self_attn.",
        "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp.",
    }})
    layers = tuple(
        LayerSpec(prefix=f"model.layers.{index}.", block=block, mixer=mixer, feed_forward=feed_forward,
                  mixer_norm=norm, feed_forward_norm=norm)
        for index in range(config.num_hidden_layers)
    )
    return ModelSpec(
        architecture="Qwen2ForCausalLM",
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        layers=layers,
        order=tuple(range(config.num_hidden_layers)),
        final_norm=norm,
        embedding_name="model.embed_tokens.weight",
        final_norm_prefix="model.norm.",
        lm_head_name="lm_head.weight",
        tie_word_embeddings=config.tie_word_embeddings,
        max_position_embeddings=config.max_position_embeddings,
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, build_qwen2_spec, model_types=("qwen2",))
