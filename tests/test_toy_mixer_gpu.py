"""(c)'s generality: a toy mixer with a state of its own, a new architecture that runs a
layer twice and mixes it with attention layers, registered, built and stepped from
this file alone, without a change to the framework's files."""
import json
import random
from dataclasses import dataclass

import pytest
import torch

from plain import qwen2_plain

pytestmark = pytest.mark.gpu

DECAY = 0.75


def register_toy():
    from llm_serving_engine_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture
    from llm_serving_engine_b200.parts import Mixer, RequestState, register_mixer
    from llm_serving_engine_b200.weights import TensorSpec

    @register_mixer("toy_decayed_sum")
    class ToyDecayedSum(Mixer):
        """state s (float32 [H] per request): s = decay * s + x_t;  y_t = W s."""

        def __init__(self, params, weights, ctx):
            super().__init__(params, weights, ctx)
            self.decay = float(params["decay"])
            self.weight = weights["mix.weight"]

        @classmethod
        def expected_tensors(cls, params, hidden_size):
            return {"mix.weight": TensorSpec((hidden_size, hidden_size))}

        @classmethod
        def cache_requirement(cls, params, hidden_size):
            return RequestState((hidden_size,), "float32")

        def forward(self, x, step, cache):
            out = torch.empty_like(x)
            for segment in step.segments:          # a request's rows in order, from the state earlier steps left
                state = cache.state[segment.state_slot]
                for row in range(segment.row_start, segment.row_start + segment.count):
                    state.mul_(self.decay).add_(x[row].float())
                    out[row] = (self.weight.float() @ state).to(x.dtype)
            return out

    @dataclass(frozen=True)
    class ToyConfig:
        values: dict

        @classmethod
        def from_dict(cls, values):
            return cls(dict(values))

    def build_spec(config):
        v = config.values
        norm = PartSpec("rmsnorm", {"eps": v["rms_norm_eps"]})
        attention = PartSpec("gqa_attention", {
            "num_heads": v["num_attention_heads"], "num_kv_heads": v["num_key_value_heads"], "head_dim": v["head_dim"],
            "bias": True, "window": 0,
            "position": {"kind": "rope", "params": {"theta": v["rope_theta"], "head_dim": v["head_dim"],
                                                    "pairing": "interleaved"}}})
        toy = PartSpec("toy_decayed_sum", {"decay": v["decay"]})
        feed_forward = PartSpec("swiglu", {"intermediate_size": v["intermediate_size"]})
        names = {"mixer_norm": "input_layernorm.", "mixer": "self_attn.", "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."}
        block = PartSpec("prenorm_residual", {"tensor_prefixes": names})
        layers = (
            LayerSpec("model.layers.0.", block, attention, feed_forward, norm, norm),
            LayerSpec("model.layers.1.", PartSpec("prenorm_residual", {"tensor_prefixes": dict(names, mixer="toy.")}),
                      toy, feed_forward, norm, norm),
        )
        return ModelSpec("ToyHybridForCausalLM", v["vocab_size"], v["hidden_size"], layers, tuple(v["layer_order"]),
                         norm, "model.embed_tokens.weight", "model.norm.", "lm_head.weight", True,
                         v["max_position_embeddings"])

    register_architecture("ToyHybridForCausalLM", ToyConfig, build_spec)


TOY = {"architectures": ["ToyHybridForCausalLM"], "vocab_size": 300, "hidden_size": 48, "intermediate_size": 80,
       "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "rope_theta": 10000.0,
       "rms_norm_eps": 1e-5, "decay": DECAY, "max_position_embeddings": 256, "layer_order": [0, 1, 0, 1],
       "num_hidden_layers": 2, "tie_word_embeddings": True}


def plain_toy_forward(cfg, w, tokens):
    """Whole sequence, no cache: the order [attention layer, toy layer, attention layer, toy layer]."""
    tokens = torch.as_tensor(tokens)
    positions = torch.arange(len(tokens))
    h = qwen2_plain.embedding(w["model.embed_tokens.weight"], tokens)
    eps = cfg["rms_norm_eps"]
    for index in cfg["layer_order"]:
        if index == 0:
            h = qwen2_plain.decoder_layer(h, positions, w, 0, cfg)
        else:
            x = qwen2_plain.rms_norm(h, w["model.layers.1.input_layernorm.weight"], eps)
            state = torch.zeros(cfg["hidden_size"])
            mixed = []
            for row in x:
                state = DECAY * state + row
                mixed.append(w["model.layers.1.toy.mix.weight"] @ state)
            h = h + torch.stack(mixed)
            h = h + qwen2_plain.swiglu(qwen2_plain.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], eps),
                                       w, "model.layers.1.mlp.")
    return qwen2_plain.linear(qwen2_plain.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


def test_toy_mixer_with_state_runs_through_the_unchanged_framework(tmp_path):
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model
    from llm_serving_engine_b200.parts import PagedKV, RequestState
    from llm_serving_engine_b200.weights import write_random_model

    register_toy()
    write_random_model(tmp_path, TOY, seed=4, dtype="float32")
    assert json.loads((tmp_path / "config.json").read_text())["decay"] == DECAY
    model = load_model(tmp_path, dtype="float32", device="cuda")
    needs = cache_requirements(model.spec)
    assert [type(n) for n in needs] == [PagedKV, RequestState, PagedKV, RequestState]   # one cache per run of a layer
    cache = CacheManager(needs, CacheConfig(8, 24), model.dtype, model.device, 256, num_state_slots=3)
    assert cache.groups[0].layers == [0, 2] and sorted(cache.states.tensors) == [1, 3]
    runner = StepRunner(model, cache, 128, 3)
    cfg, weights = qwen2_plain.load_folder(tmp_path)
    rng = random.Random(0)
    requests = {name: [rng.randrange(300) for _ in range(length)] for name, length in (("a", 37), ("b", 52), ("c", 9))}
    want = {name: plain_toy_forward(cfg, weights, tokens) for name, tokens in requests.items()}

    def run(cuts):
        """cuts: per step, {request: number of tokens}; returns the logits of every position."""
        done = {name: 0 for name in requests}
        rows = {name: [] for name in requests}
        for name in requests:
            cache.create(name)
        for step in cuts:
            entries = []
            for name, count in step.items():
                entries.append(StepEntry(name, requests[name][done[name]:done[name] + count], list(range(count))))
                done[name] += count
            logits = runner.run(entries).cpu()
            cursor = 0
            for name, count in step.items():
                rows[name].append(logits[cursor:cursor + count])
                cursor += count
        for name in requests:
            assert done[name] == len(requests[name])
            cache.free(name)
        return {name: torch.cat(parts) for name, parts in rows.items()}

    whole = run([{"a": 37}, {"b": 52}, {"c": 9}])
    mixed = run([{"a": 30, "b": 2}, {"b": 45, "c": 3, "a": 1}, {"a": 1, "c": 1}, {"c": 5, "a": 5, "b": 5}])
    for name in requests:
        assert float((whole[name] - want[name]).abs().max()) < 2e-5 * max(1.0, float(want[name].abs().max())), name
        assert float((mixed[name] - want[name]).abs().max()) < 2e-5 * max(1.0, float(want[name].abs().max())), name
    assert cache.groups[0].pool.used_pages == 0 and len(cache._free_slots) == 3
