"""(c)'s generality: the order in which layers run is data, and a layer may read another layer's cache.

A toy mixer defined here has queries of its own but no keys or values: its layer names, with
``LayerSpec.cache_from``, the attention layer whose pages it reads.  The architecture runs
[attention, reader, attention, reader]: the attention layer twice (each run with pages of its own) and
the reader twice (both runs read the pages of the attention layer's first run).  Registered, built and
stepped from this file alone, without a change to the framework's files; compared with a plain
whole-sequence computation."""
import math
import random
from dataclasses import dataclass

import pytest
import torch

from plain import qwen2_plain

pytestmark = pytest.mark.gpu


def register_toy():
    from llm_serving_engine_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.parts import Mixer, register_mixer
    from llm_serving_engine_b200.parts.linear import linear
    from llm_serving_engine_b200.weights import TensorSpec

    @register_mixer("toy_reader_attention")
    class ToyReaderAttention(Mixer):
        """y = o(softmax(q k^T / sqrt(D)) v) with q = q(x), unrotated, and k, v the pages of the layer that
        ``cache_from`` names (rotated keys, as that layer stored them)."""

        graph_safe = True   # a product and the general attention kernel: both sized by the number of rows

        def __init__(self, params, weights, ctx):
            super().__init__(params, weights, ctx)
            self.n_q, self.head_dim = int(params["num_heads"]), int(params["head_dim"])
            self.q_weight, self.o_weight = weights["q.weight"], weights["o.weight"]

        @classmethod
        def expected_tensors(cls, params, hidden_size):
            width = int(params["num_heads"]) * int(params["head_dim"])
            return {"q.weight": TensorSpec((width, hidden_size)), "o.weight": TensorSpec((hidden_size, width))}

        def forward(self, x, step, cache):
            tokens = x.shape[0]
            q = linear(x, self.q_weight).view(tokens, self.n_q, self.head_dim).contiguous()
            out = torch.empty_like(q)
            ops.paged_attention_generic(q, cache.keys, cache.values, out, cache.block_tables, step.segment_of_token,
                                        step.positions, 1.0 / math.sqrt(self.head_dim), 0)
            return linear(out.view(tokens, self.n_q * self.head_dim), self.o_weight)

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
        reader = PartSpec("toy_reader_attention", {"num_heads": v["reader_heads"], "head_dim": v["head_dim"]})
        feed_forward = PartSpec("swiglu", {"intermediate_size": v["intermediate_size"]})
        names = {"mixer_norm": "input_layernorm.", "mixer": "self_attn.", "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."}
        layers = (
            LayerSpec("model.layers.0.", PartSpec("prenorm_residual", {"tensor_prefixes": names}), attention, feed_forward, norm, norm),
            LayerSpec("model.layers.1.", PartSpec("prenorm_residual", {"tensor_prefixes": dict(names, mixer="reader.")}),
                      reader, feed_forward, norm, norm, cache_from=0),
        )
        return ModelSpec("ToyReaderForCausalLM", v["vocab_size"], v["hidden_size"], layers, tuple(v["layer_order"]),
                         norm, "model.embed_tokens.weight", "model.norm.", "lm_head.weight", True,
                         v["max_position_embeddings"])

    register_architecture("ToyReaderForCausalLM", ToyConfig, build_spec)


TOY = {"architectures": ["ToyReaderForCausalLM"], "vocab_size": 211, "hidden_size": 40, "intermediate_size": 72,
       "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "reader_heads": 6, "rope_theta": 10000.0,
       "rms_norm_eps": 1e-5, "max_position_embeddings": 256, "layer_order": [0, 1, 0, 1],
       "num_hidden_layers": 2, "tie_word_embeddings": True}


def plain_forward(cfg, w, tokens):
    """Whole sequence, no cache.  The reader's keys and values are those of the attention layer's first run."""
    tokens = torch.as_tensor(tokens)
    positions = torch.arange(len(tokens))
    eps, d = cfg["rms_norm_eps"], cfg["head_dim"]
    n_kv = cfg["num_key_value_heads"]
    h = qwen2_plain.embedding(w["model.embed_tokens.weight"], tokens)
    shared = None
    for index in cfg["layer_order"]:
        if index == 0:
            if shared is None:   # what the first run of layer 0 writes into its pages
                x = qwen2_plain.rms_norm(h, w["model.layers.0.input_layernorm.weight"], eps)
                k = qwen2_plain.linear(x, w["model.layers.0.self_attn.k_proj.weight"], w["model.layers.0.self_attn.k_proj.bias"])
                v = qwen2_plain.linear(x, w["model.layers.0.self_attn.v_proj.weight"], w["model.layers.0.self_attn.v_proj.bias"])
                shared = (qwen2_plain.rope(k.view(-1, n_kv, d), positions, cfg["rope_theta"]), v.view(-1, n_kv, d))
            h = qwen2_plain.decoder_layer(h, positions, w, 0, cfg)
        else:
            x = qwen2_plain.rms_norm(h, w["model.layers.1.input_layernorm.weight"], eps)
            q = qwen2_plain.linear(x, w["model.layers.1.reader.q.weight"]).view(-1, cfg["reader_heads"], d)
            mixed = qwen2_plain.causal_attention(q, shared[0], shared[1]).reshape(len(tokens), -1)
            h = h + qwen2_plain.linear(mixed, w["model.layers.1.reader.o.weight"])
            h = h + qwen2_plain.swiglu(qwen2_plain.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], eps),
                                       w, "model.layers.1.mlp.")
    return qwen2_plain.linear(qwen2_plain.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_that_reads_another_layers_pages(tmp_path, dtype):
    import helpers
    from llm_serving_engine_b200 import CacheConfig, GenerationConfig, LLMEngine, SchedulerConfig
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.engine import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model
    from llm_serving_engine_b200.parts import PagedKV
    from llm_serving_engine_b200.weights import write_random_model

    register_toy()
    write_random_model(tmp_path, TOY, seed=9, dtype="float32")
    model = load_model(tmp_path, dtype=dtype, device="cuda")
    needs = cache_requirements(model.spec)
    assert isinstance(needs[0], PagedKV) and isinstance(needs[2], PagedKV) and needs[1] == 0 and needs[3] == 0
    cache = CacheManager(needs, CacheConfig(8, 20), model.dtype, model.device, 256, num_state_slots=3)
    assert cache.groups[0].layers == [0, 2]   # the readers hold no pages of their own
    runner = StepRunner(model, cache, 128, 3)
    cfg, weights = qwen2_plain.load_folder(tmp_path, torch.bfloat16 if dtype == "bfloat16" else None)
    rng = random.Random(2)
    requests = {name: [rng.randrange(TOY["vocab_size"]) for _ in range(length)] for name, length in (("a", 41), ("b", 58), ("c", 7))}
    want = {name: plain_forward(cfg, weights, tokens) for name, tokens in requests.items()}

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
            logits = runner.run(entries).float().cpu()
            cursor = 0
            for name, count in step.items():
                rows[name].append(logits[cursor:cursor + count])
                cursor += count
        for name in requests:
            assert done[name] == len(requests[name])
            cache.free(name)
        return {name: torch.cat(parts) for name, parts in rows.items()}

    with torch.inference_mode():
        whole = run([{"a": 41}, {"b": 58}, {"c": 7}])
        mixed = run([{"a": 33, "b": 2}, {"b": 50, "c": 3, "a": 1}, {"a": 1, "c": 1}, {"a": 1, "c": 1, "b": 1},
                     {"c": 2, "a": 5, "b": 5}])
    for name in requests:
        for label, got in (("whole", whole[name]), ("mixed", mixed[name])):
            error = float((got - want[name]).abs().max())
            assert error <= helpers.tolerance(dtype, want[name]), (name, label, error)
            assert helpers.rms_ratio(got, want[name]) <= helpers.RMS_RATIO[dtype], (name, label)
    assert cache.groups[0].pool.used_pages == 0

    # the same model through the engine, CUDA graphs at their default: greedy tokens where the plain logits leave no tie
    engine = LLMEngine(model, None, cache_config=CacheConfig(8, 40), scheduler_config=SchedulerConfig(max_batch_size=3, max_tokens_per_step=64),
                       prefill_chunk_size=16)
    prompts = [requests["a"][:20], requests["b"][:33]]
    generated = engine.generate_many(prompts, GenerationConfig(max_new_tokens=8))
    compared = 0
    for prompt, tokens in zip(prompts, generated):
        sequence = list(prompt)
        for token in tokens:
            logits = plain_forward(cfg, weights, sequence)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > 2 * helpers.tolerance(dtype, logits):
                assert token == int(logits.argmax())
                compared += 1
            sequence.append(token)
    assert compared >= 4
