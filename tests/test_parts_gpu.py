"""Each part of a layer alone (norm, position encoding + attention mixer,
feed-forward, block) against the plain implementation's function for that part."""
import pytest
import torch

import helpers
from plain import qwen2_plain
from tiny_configs import ALL

pytestmark = pytest.mark.gpu


def reduce_partials(y):
    from llm_serving_engine_b200.parts import reduce_partials as reduce
    return reduce(y)


def build(name, dtype="float32", pages=64):
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine import StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model

    config, page, _ = ALL[name]
    model = load_model(helpers.model_folder(name), dtype=dtype, device="cuda")
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(page, pages), model.dtype, model.device,
                         config["max_position_embeddings"], num_state_slots=4)
    runner = StepRunner(model, cache, 256, 4)
    cfg, weights = qwen2_plain.load_folder(helpers.model_folder(name), torch.bfloat16 if dtype == "bfloat16" else None)
    return config, model, cache, runner, cfg, weights


@pytest.mark.parametrize("name", sorted(ALL))
def test_norm_part(name):
    from llm_serving_engine_b200.parts import ResidualStream
    config, model, _, _, cfg, weights = build(name)
    hidden = config["hidden_size"]
    residual = torch.randn(6, hidden, device="cuda")
    delta = torch.randn(6, hidden, device="cuda")
    stream = ResidualStream(residual.clone(), delta)
    got = model.blocks[0].mixer_norm.forward(stream)
    want = qwen2_plain.rms_norm((residual + delta).cpu(), weights["model.layers.0.input_layernorm.weight"],
                                config["rms_norm_eps"])
    assert stream.delta is None and torch.allclose(stream.residual, residual + delta)
    assert float((got.cpu() - want).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_attention_mixer_with_its_position_encoding(name, dtype):
    from llm_serving_engine_b200.engine import StepEntry
    config, model, cache, runner, cfg, weights = build(name, dtype)
    hidden, length = config["hidden_size"], 45
    x = torch.randn(length, hidden) * 0.5
    if dtype == "bfloat16":
        x = x.bfloat16().float()
    want = qwen2_plain.attention_block(x, torch.arange(length), weights, "model.layers.0.self_attn.", cfg)
    cache.create("r")
    got = []
    for lo, hi in ((0, 20), (20, 21), (21, 45)):           # a portion, one token, another portion
        step, caches = runner.prepare([StepEntry("r", [0] * (hi - lo), [])])
        part = model.blocks[0].mixer.forward(x[lo:hi].to("cuda", model.dtype).contiguous(), step, caches[0])
        got.append(reduce_partials(part).float().cpu())
    got = torch.cat(got)
    limit = 2e-5 if dtype == "float32" else 2.0 ** -6
    assert float((got - want).abs().max()) < limit * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_feed_forward_part(name, dtype):
    config, model, _, _, cfg, weights = build(name, dtype)
    x = torch.randn(11, config["hidden_size"])
    if dtype == "bfloat16":
        x = x.bfloat16().float()
    want = qwen2_plain.swiglu(x, weights, "model.layers.0.mlp.")
    got = reduce_partials(model.blocks[0].feed_forward.forward(x.to("cuda", model.dtype))).float().cpu()
    limit = 2e-5 if dtype == "float32" else 2.0 ** -6
    assert float((got - want).abs().max()) < limit * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("name", sorted(ALL))
def test_block_arrangement(name):
    from llm_serving_engine_b200.engine import StepEntry
    from llm_serving_engine_b200.parts import ResidualStream
    config, model, cache, runner, cfg, weights = build(name)
    length = 19
    h = torch.randn(length, config["hidden_size"])
    want = qwen2_plain.decoder_layer(h, torch.arange(length), weights, 0, cfg)
    cache.create("r")
    step, caches = runner.prepare([StepEntry("r", [0] * length, [])])
    stream = ResidualStream(h.cuda())
    model.blocks[0].forward(stream, step, caches[0])
    got = (stream.residual + reduce_partials(stream.delta).float()).cpu()      # the last branch output is still pending
    assert float((got - want).abs().max()) < 2e-5 * max(1.0, float(want.abs().max()))
