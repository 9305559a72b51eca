"""(c) and (d) together: layers with different needs in one model.  A toy architecture, defined here from the
framework's own attention part, has a layer that reads all keys, a layer that reads a window of 21 keys and a
layer that reads a window of 8: three groups of pages.  The windowed groups give pages back while a request is
still running and take them again, so a long request fits a pool far smaller than its length.  Compared with
a plain whole-sequence computation with banded masks."""
import math
import random
from dataclasses import dataclass

import pytest
import torch

from plain import qwen2_plain

pytestmark = pytest.mark.gpu

WINDOWS = (0, 21, 8)


def register_toy():
    from llm_serving_engine_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture

    @dataclass(frozen=True)
    class ToyConfig:
        values: dict

        @classmethod
        def from_dict(cls, values):
            return cls(dict(values))

    def build_spec(config):
        v = config.values
        norm = PartSpec("rmsnorm", {"eps": v["rms_norm_eps"]})
        feed_forward = PartSpec("swiglu", {"intermediate_size": v["intermediate_size"]})
        names = {"mixer_norm": "input_layernorm.", "mixer": "self_attn.", "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."}
        block = PartSpec("prenorm_residual", {"tensor_prefixes": names})
        layers = []
        for index, window in enumerate(v["windows"]):
            attention = PartSpec("gqa_attention", {
                "num_heads": v["num_attention_heads"], "num_kv_heads": v["num_key_value_heads"], "head_dim": v["head_dim"],
                "bias": True, "window": window,
                "position": {"kind": "rope", "params": {"theta": v["rope_theta"], "head_dim": v["head_dim"],
                                                        "pairing": "interleaved"}}})
            layers.append(LayerSpec(f"model.layers.{index}.", block, attention, feed_forward, norm, norm))
        return ModelSpec("ToyWindowedForCausalLM", v["vocab_size"], v["hidden_size"], tuple(layers),
                         tuple(range(len(layers))), norm, "model.embed_tokens.weight", "model.norm.", "lm_head.weight",
                         True, v["max_position_embeddings"])

    register_architecture("ToyWindowedForCausalLM", ToyConfig, build_spec)


TOY = {"architectures": ["ToyWindowedForCausalLM"], "vocab_size": 173, "hidden_size": 48, "intermediate_size": 88,
       "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 16, "rope_theta": 10000.0, "windows": list(WINDOWS),
       "rms_norm_eps": 1e-5, "max_position_embeddings": 512, "num_hidden_layers": len(WINDOWS), "tie_word_embeddings": True}


def banded_attention(q, k, v, window):
    """Row i reads keys max(0, i - window + 1) .. i (all keys up to i when window is 0)."""
    seq, n_q, head_dim = q.shape
    group = n_q // k.shape[1]
    index = torch.arange(seq)
    hidden = index[None, :] > index[:, None]
    if window > 0:
        hidden |= index[None, :] < index[:, None] - window + 1
    out = torch.empty_like(q)
    for head in range(n_q):
        scores = (q[:, head] @ k[:, head // group].t()) / math.sqrt(head_dim)
        out[:, head] = torch.softmax(scores.masked_fill(hidden, float("-inf")), -1) @ v[:, head // group]
    return out


def plain_forward(cfg, w, tokens):
    tokens = torch.as_tensor(tokens)
    seq = len(tokens)
    positions = torch.arange(seq)
    eps, d, n_q, n_kv = cfg["rms_norm_eps"], cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    h = qwen2_plain.embedding(w["model.embed_tokens.weight"], tokens)
    for index, window in enumerate(cfg["windows"]):
        base = f"model.layers.{index}."
        x = qwen2_plain.rms_norm(h, w[base + "input_layernorm.weight"], eps)
        q = qwen2_plain.linear(x, w[base + "self_attn.q_proj.weight"], w[base + "self_attn.q_proj.bias"]).view(seq, n_q, d)
        k = qwen2_plain.linear(x, w[base + "self_attn.k_proj.weight"], w[base + "self_attn.k_proj.bias"]).view(seq, n_kv, d)
        v = qwen2_plain.linear(x, w[base + "self_attn.v_proj.weight"], w[base + "self_attn.v_proj.bias"]).view(seq, n_kv, d)
        q, k = qwen2_plain.rope(q, positions, cfg["rope_theta"]), qwen2_plain.rope(k, positions, cfg["rope_theta"])
        h = h + qwen2_plain.linear(banded_attention(q, k, v, window).reshape(seq, n_q * d), w[base + "self_attn.o_proj.weight"])
        h = h + qwen2_plain.swiglu(qwen2_plain.rms_norm(h, w[base + "post_attention_layernorm.weight"], eps), w, base + "mlp.")
    return qwen2_plain.linear(qwen2_plain.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_give_pages_back_while_the_request_runs(tmp_path, dtype):
    import helpers
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model
    from llm_serving_engine_b200.weights import write_random_model

    register_toy()
    write_random_model(tmp_path, TOY, seed=6, dtype="float32")
    model = load_model(tmp_path, dtype=dtype, device="cuda")
    needs = cache_requirements(model.spec)
    assert [need.window for need in needs] == list(WINDOWS)
    page = 4
    # 64 pages of 4 keys a group; the windowed groups never hold more than a window and a portion of either request
    cache = CacheManager(needs, CacheConfig(page, 64), model.dtype, model.device, 512, num_state_slots=2)
    assert len(cache.groups) == 3
    runner = StepRunner(model, cache, 64, 2)
    cfg, weights = qwen2_plain.load_folder(tmp_path, torch.bfloat16 if dtype == "bfloat16" else None)
    rng = random.Random(3)
    requests = {"a": [rng.randrange(TOY["vocab_size"]) for _ in range(150)], "b": [rng.randrange(TOY["vocab_size"]) for _ in range(80)]}
    want = {name: plain_forward(cfg, weights, tokens) for name, tokens in requests.items()}

    # a: 40 tokens, then portions of changing size beside b's, then one by one; b joins late and ends early
    schedule = [{"a": 40}, {"a": 7, "b": 30}, {"a": 2, "b": 2}, {"a": 23, "b": 19}, {"a": 1, "b": 1}]
    schedule += [{"a": 1, "b": 1} for _ in range(28)]
    schedule += [{"a": 11}] + [{"a": 1} for _ in range(150 - 40 - 7 - 2 - 23 - 1 - 28 - 11)]
    done = {name: 0 for name in requests}
    rows = {name: [] for name in requests}
    most = [0, 0, 0]
    given_back_early = False
    order = {group.need.window: index for index, group in enumerate(cache.groups)}
    with torch.inference_mode():
        for step in schedule:
            entries = []
            for name, count in step.items():
                if done[name] == 0:
                    cache.create(name)
                entries.append(StepEntry(name, requests[name][done[name]:done[name] + count], list(range(count))))
                done[name] += count
            logits = runner.run(entries).float().cpu()
            cursor = 0
            for name, count in step.items():
                rows[name].append(logits[cursor:cursor + count])
                cursor += count
            for index, group in enumerate(cache.groups):
                most[index] = max(most[index], group.pool.used_pages)
            table = cache.requests["a"].tables
            given_back_early = given_back_early or (table[order[8]][0] == -1 and table[order[0]][0] >= 0)
            if done["b"] == len(requests["b"]) and "b" in cache.requests:
                cache.free("b")
    assert done == {name: len(tokens) for name, tokens in requests.items()}
    assert given_back_early, "the narrow window never gave its first page back while the request ran"
    assert most[order[0]] >= -(-101 // page) + 80 // page            # every key of both requests when b ends (a is 101 long then)
    assert most[order[21]] <= 2 * ((21 + 23) // page + 2)            # a window and the longest later portion, twice
    assert most[order[8]] <= 2 * ((8 + 23) // page + 2)
    assert most[order[8]] < most[order[21]] < most[order[0]]
    cache.free("a")
    assert all(group.pool.used_pages == 0 for group in cache.groups)
    for name in requests:
        got = torch.cat(rows[name])
        error = float((got - want[name]).abs().max())
        assert error <= helpers.tolerance(dtype, want[name]), (name, error)
        assert helpers.rms_ratio(got, want[name]) <= helpers.RMS_RATIO[dtype], name
