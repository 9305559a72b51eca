"""(c)'s generality beyond the mixer: a feed-forward with routing (top-1 of several experts) and
another position encoding, defined in this file, registered, built from a configuration of their
own, given random weights by the framework's random-weights mode and stepped through the
unchanged engine (prompt portions, mixed steps, decoding), against a plain whole-sequence
computation.  Neither part is a model of anyone's: they only show that the interfaces hold."""
import math
import random
from dataclasses import dataclass

import pytest
import torch

from plain import qwen2_plain

pytestmark = pytest.mark.gpu

EXPERTS = 3
WAVE = 0.37


def wave(positions: torch.Tensor, head_dim: int) -> torch.Tensor:
    """[T, D] factors 1 + 0.25 sin(WAVE * position + d): what the toy position encoding scales keys by."""
    d = torch.arange(head_dim, device=positions.device, dtype=torch.float32)
    return 1.0 + 0.25 * torch.sin(WAVE * positions.float()[:, None] + d[None, :])


def register_toys():
    from llm_serving_engine_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture
    from llm_serving_engine_b200.parts import FeedForward, PositionEncoding, register_feed_forward, register_position_encoding
    from llm_serving_engine_b200.parts.linear import reduce_partials
    from llm_serving_engine_b200.weights import TensorSpec

    @register_feed_forward("toy_top1_experts")
    class ToyTop1Experts(FeedForward):
        """Router logits in float32; every row goes to its best expert (a small two-matrix ReLU network) and
        the result is scaled by that expert's softmax probability."""

        def __init__(self, params, weights, ctx):
            super().__init__(params, weights, ctx)
            self.experts = int(params["experts"])
            self.router = weights["router.weight"].float()
            self.up = [weights[f"experts.{e}.up.weight"] for e in range(self.experts)]
            self.down = [weights[f"experts.{e}.down.weight"] for e in range(self.experts)]

        @classmethod
        def expected_tensors(cls, params, hidden_size):
            inner = int(params["inner"])
            out = {"router.weight": TensorSpec((int(params["experts"]), hidden_size))}
            for e in range(int(params["experts"])):
                out[f"experts.{e}.up.weight"] = TensorSpec((inner, hidden_size))
                out[f"experts.{e}.down.weight"] = TensorSpec((hidden_size, inner))
            return out

        def forward(self, x):
            probabilities = torch.softmax(x.float() @ self.router.t(), dim=-1)
            best = probabilities.argmax(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.experts):
                rows = (best == e).nonzero().flatten()
                if rows.numel():
                    hidden = torch.relu(x[rows] @ self.up[e].t())
                    out[rows] = ((hidden @ self.down[e].t()).float() * probabilities[rows, e, None]).to(x.dtype)
            return out

    @register_position_encoding("toy_wave")
    class ToyWave(PositionEncoding):
        """No rotation: keys are scaled element by element by a wave of their position; queries and values
        only get their bias.  Writes keys and values into the pages by the step's slot mapping."""

        def encode_and_store(self, qkv, bias, step, cache, q_out, n_q, n_kv, head_dim):
            tokens = q_out.shape[0]
            x = reduce_partials(qkv).float()
            if bias is not None:
                x = x + bias
            q, k, v = x.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=1)
            q_out.copy_(q.view(tokens, n_q, head_dim))
            k = k.view(tokens, n_kv, head_dim) * wave(step.positions[:tokens], head_dim)[:, None, :]
            slots = cache.slot_mapping[:tokens].long()
            page_size = cache.keys.shape[2]
            cache.keys[slots // page_size, :, slots % page_size] = k.to(cache.keys.dtype)
            cache.values[slots // page_size, :, slots % page_size] = v.view(tokens, n_kv, head_dim).to(cache.values.dtype)

    @dataclass(frozen=True)
    class ToyConfig:
        values: dict

        @classmethod
        def from_dict(cls, values):
            return cls(dict(values))

    def build_spec(config):
        v = config.values
        norm = PartSpec("rmsnorm", {"eps": v["rms_norm_eps"]})

        def attention(position):
            return PartSpec("gqa_attention", {"num_heads": v["num_attention_heads"], "num_kv_heads": v["num_key_value_heads"],
                                              "head_dim": v["head_dim"], "bias": True, "window": 0, "position": position})
        rotary = {"kind": "rope", "params": {"theta": v["rope_theta"], "head_dim": v["head_dim"], "pairing": "half"}}
        names = {"mixer_norm": "input_layernorm.", "mixer": "self_attn.", "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."}
        block = PartSpec("prenorm_residual", {"tensor_prefixes": names})
        layers = (
            LayerSpec("model.layers.0.", block, attention({"kind": "toy_wave", "params": {}}),
                      PartSpec("swiglu", {"intermediate_size": v["intermediate_size"]}), norm, norm),
            LayerSpec("model.layers.1.", block, attention(rotary),
                      PartSpec("toy_top1_experts", {"experts": EXPERTS, "inner": v["expert_inner"]}), norm, norm),
        )
        return ModelSpec("ToyRoutedForCausalLM", v["vocab_size"], v["hidden_size"], layers, (0, 1), norm,
                         "model.embed_tokens.weight", "model.norm.", "lm_head.weight", False, v["max_position_embeddings"])

    register_architecture("ToyRoutedForCausalLM", ToyConfig, build_spec)


TOY = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 211, "hidden_size": 40, "intermediate_size": 56,
       "expert_inner": 24, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16, "rope_theta": 5000.0,
       "rope_pairing": "half", "rms_norm_eps": 1e-6, "max_position_embeddings": 128, "num_hidden_layers": 2,
       "tie_word_embeddings": False}


def plain_forward(cfg, w, tokens):
    """Whole sequence, no cache: layer 0 with the wave on the keys, layer 1 with rotary attention and the
    routed feed-forward."""
    tokens = torch.as_tensor(tokens)
    positions = torch.arange(len(tokens))
    n_heads, head_dim, eps = cfg["num_attention_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    h = qwen2_plain.embedding(w["model.embed_tokens.weight"], tokens)
    # layer 0
    x = qwen2_plain.rms_norm(h, w["model.layers.0.input_layernorm.weight"], eps)
    p = "model.layers.0.self_attn."
    q = qwen2_plain.linear(x, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(-1, n_heads, head_dim)
    k = qwen2_plain.linear(x, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(-1, n_heads, head_dim)
    v = qwen2_plain.linear(x, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(-1, n_heads, head_dim)
    k = k * wave(positions, head_dim).to(k.dtype)[:, None, :]
    h = h + qwen2_plain.linear(qwen2_plain.causal_attention(q, k, v).reshape(len(tokens), -1), w[p + "o_proj.weight"])
    h = h + qwen2_plain.swiglu(qwen2_plain.rms_norm(h, w["model.layers.0.post_attention_layernorm.weight"], eps), w, "model.layers.0.mlp.")
    # layer 1
    x = qwen2_plain.rms_norm(h, w["model.layers.1.input_layernorm.weight"], eps)
    h = h + qwen2_plain.attention_block(x, positions, w, "model.layers.1.self_attn.", cfg)
    x = qwen2_plain.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], eps)
    probabilities = torch.softmax(x @ w["model.layers.1.mlp.router.weight"].t(), dim=-1)
    best = probabilities.argmax(dim=-1)
    routed = torch.zeros_like(x)
    for row in range(len(tokens)):
        e = int(best[row])
        hidden = torch.relu(w[f"model.layers.1.mlp.experts.{e}.up.weight"] @ x[row])
        routed[row] = (w[f"model.layers.1.mlp.experts.{e}.down.weight"] @ hidden) * probabilities[row, e]
    h = h + routed
    return qwen2_plain.linear(qwen2_plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"]), best


def test_routed_feed_forward_and_another_position_encoding_run_through_the_unchanged_framework(tmp_path):
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model
    from llm_serving_engine_b200.weights import write_random_model

    register_toys()
    write_random_model(tmp_path, TOY, seed=9, dtype="float32")
    model = load_model(tmp_path, dtype="float32", device="cuda")
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(8, 30), model.dtype, model.device, 128, num_state_slots=3)
    runner = StepRunner(model, cache, 96, 3)
    # the toy parts are plain tensor code whose launches depend on the routing: they do not say ``graph_safe``,
    # so the model does not either, although its attention does, and no step is captured
    assert not model.graph_safe and not runner.use_graphs
    cfg, weights = qwen2_plain.load_folder(tmp_path)
    # router weights of the size of the others would send almost every row to the same expert: spread them
    rng = random.Random(1)
    requests = {name: [rng.randrange(TOY["vocab_size"]) for _ in range(length)] for name, length in (("a", 41), ("b", 29), ("c", 7))}
    want, chosen = {}, set()
    for name, tokens in requests.items():
        want[name], best = plain_forward(cfg, weights, tokens)
        chosen |= set(best.tolist())
    assert len(chosen) >= 2, "the routing never chose a second expert: the test would not see a wrong one"

    def run(cuts):
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

    whole = run([{"a": 41}, {"b": 29}, {"c": 7}])
    mixed = run([{"a": 30, "b": 2}, {"b": 20, "c": 3, "a": 1}] + [{"a": 1, "b": 1, "c": 1}] * 4 + [{"a": 6, "b": 3}])
    for name in requests:
        bound = 3e-5 * max(1.0, float(want[name].abs().max()))
        assert float((whole[name] - want[name]).abs().max()) < bound, name
        assert float((mixed[name] - want[name]).abs().max()) < bound, name
    assert cache.groups[0].pool.used_pages == 0

    # the same model through the entry point with everything at its default: greedy tokens equal the plain ones
    from llm_serving_engine_b200 import GenerationConfig, LLMEngine, SchedulerConfig

    engine = LLMEngine(model, None, cache_config=CacheConfig(8, 30), scheduler_config=SchedulerConfig(max_batch_size=3, max_tokens_per_step=32),
                       prefill_chunk_size=16)
    assert not engine.runner.use_graphs
    prompts = [requests["b"][:19], requests["c"]]
    got = engine.generate_many(prompts, GenerationConfig(max_new_tokens=5))
    for prompt, tokens in zip(prompts, got):
        sequence = list(prompt)
        for token in tokens:
            logits, _ = plain_forward(cfg, weights, sequence)
            top = torch.topk(logits[-1], 2).values
            if float(top[0] - top[1]) > 1e-4:     # a near tie may fall either way
                assert token == int(logits[-1].argmax())
            sequence.append(token)
    assert engine.runner.graph_replays == 0
