"""The layer sizes of the benchmark model (Qwen2.5-1.5B: hidden 1536, 12 query and 2 key/value heads of
128, feed-forward 8960, vocabulary 151936) with two layers and random weights: the kernels run at the
shapes they were tuned for (tcgen05 product with k = 8960, tensor-core attention with six heads per
group, the wide LM head), through prompts cut into portions, decoding from CUDA graphs and a mixed
step, against the plain implementation."""
import json
import random
import tempfile
from pathlib import Path

import pytest
import torch

import helpers
from plain import qwen2_plain

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 151936, "hidden_size": 1536, "intermediate_size": 8960, "num_hidden_layers": 2,
    "num_attention_heads": 12, "num_key_value_heads": 2, "max_position_embeddings": 1024,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
}


@pytest.fixture(scope="module")
def folder():
    from llm_serving_engine_b200.weights import write_random_model
    with tempfile.TemporaryDirectory(prefix="real_shape_") as name:
        write_random_model(name, CONFIG, seed=11, dtype="bfloat16")
        yield Path(name)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_benchmark_shapes_against_the_plain_implementation(folder, dtype):
    from llm_serving_engine_b200.engine.trace_replay import replay

    rng = random.Random(4)
    a = helpers.random_tokens(rng, CONFIG["vocab_size"], 150)
    b = helpers.random_tokens(rng, CONFIG["vocab_size"], 41)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:100], "want": [0, 63, 64, 99]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[100:130], "want": [29]}, {"id": "b", "tokens": b[:40], "want": [39]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": [a[130]], "want": [0]}, {"id": "b", "tokens": [b[40]], "want": [0]}], "end": ["b"]},
    ]
    steps += [{"step": 3 + i, "entries": [{"id": "a", "tokens": [a[131 + i]], "want": [0]}], "end": []} for i in range(19)]
    with tempfile.TemporaryDirectory(prefix="real_out_") as out:
        replay(folder, dtype, out, 256, [json.dumps(step) for step in steps])
        got = helpers.collect(steps, Path(out))
    cfg, weights = qwen2_plain.load_folder(folder)          # the matrices are stored in bfloat16 already
    want_a = qwen2_plain.forward_full(cfg, weights, a)
    want_b = qwen2_plain.forward_full(cfg, weights, b)
    rows_a = [0, 63, 64, 99, 129] + list(range(130, 150))
    for name, got_rows, want_rows in (("a", got["a"], want_a[rows_a]), ("b", got["b"], want_b[[39, 40]])):
        limit = helpers.tolerance(dtype, want_rows)
        error = (got_rows - want_rows).abs().max(dim=1).values
        assert float(error.max()) <= limit, f"{name} ({dtype}): max error {float(error.max()):.3e} > {limit:.3e} at row {int(error.argmax())}"
    from llm_serving_engine_b200.kernels import ops
    assert ops.gemm_bf16_skinny_status() == 0


def test_long_portions_take_the_tcgen05_attention(folder):
    """Steps of 128 rows and more run the tcgen05 attention kernel: a prompt whole, the same prompt in
    long portions (the second with earlier keys, starting off the tile grid), and two requests in one
    step; all against the plain implementation, and no bounded wait may have given up."""
    from llm_serving_engine_b200.engine.trace_replay import replay
    from llm_serving_engine_b200.kernels import ops

    rng = random.Random(8)
    a = helpers.random_tokens(rng, CONFIG["vocab_size"], 420)
    b = helpers.random_tokens(rng, CONFIG["vocab_size"], 180)
    want_rows_a = [0, 127, 128, 300, 419]
    steps = [
        {"step": 0, "entries": [{"id": "whole", "tokens": a, "want": want_rows_a}], "end": ["whole"]},
        {"step": 1, "entries": [{"id": "cut", "tokens": a[:150], "want": [0, 127, 128]}], "end": []},
        {"step": 2, "entries": [{"id": "cut", "tokens": a[150:390], "want": [150]},
                                {"id": "b", "tokens": b[:170], "want": [0, 169]}], "end": []},
        {"step": 3, "entries": [{"id": "cut", "tokens": a[390:], "want": [29]},
                                {"id": "b", "tokens": b[170:], "want": [9]}], "end": ["cut", "b"]},
    ]
    with tempfile.TemporaryDirectory(prefix="real_out_") as out:
        replay(folder, "bfloat16", out, 1024, [json.dumps(step) for step in steps])
        got = helpers.collect(steps, Path(out))
    assert ops.attention_tc_status() == 0
    cfg, weights = qwen2_plain.load_folder(folder)
    want_a = qwen2_plain.forward_full(cfg, weights, a)
    want_b = qwen2_plain.forward_full(cfg, weights, b)
    for name, got_rows, want_rows in (("whole", got["whole"], want_a[want_rows_a]), ("cut", got["cut"], want_a[want_rows_a]),
                                      ("b", got["b"], want_b[[0, 169, 179]])):
        limit = helpers.tolerance("bfloat16", want_rows)
        error = (got_rows - want_rows).abs().max(dim=1).values
        assert float(error.max()) <= limit, f"{name}: max error {float(error.max()):.3e} > {limit:.3e} at row {int(error.argmax())}"


CONFIG_7B_LAYER = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 2048, "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 1,
    "num_attention_heads": 28, "num_key_value_heads": 4, "max_position_embeddings": 1024,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
}


def test_layer_sizes_of_a_larger_model(tmp_path):
    """One layer of the Qwen2.5-7B sizes (hidden 3584, 28 query and 4 key/value heads, feed-forward 18944; a small
    vocabulary keeps it light): sizes the kernels were not tuned on: seven heads a group, a width beyond the
    warp-per-row norm, k = 18944 in the few-rows product, in a long portion, a short one, decoding and a mixed step."""
    from llm_serving_engine_b200.engine.trace_replay import replay
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.weights import write_random_model

    write_random_model(tmp_path / "model", CONFIG_7B_LAYER, seed=5, dtype="bfloat16")
    rng = random.Random(6)
    a = helpers.random_tokens(rng, CONFIG_7B_LAYER["vocab_size"], 330)
    b = helpers.random_tokens(rng, CONFIG_7B_LAYER["vocab_size"], 50)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:300], "want": [0, 128, 299]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[300:320], "want": [19]}, {"id": "b", "tokens": b[:40], "want": [39]}], "end": []},
    ]
    steps += [{"step": 2 + i, "entries": [{"id": "a", "tokens": [a[320 + i]], "want": [0]}, {"id": "b", "tokens": [b[40 + i]], "want": [0]}],
               "end": []} for i in range(10)]
    with tempfile.TemporaryDirectory(prefix="real_out_") as out:
        replay(tmp_path / "model", "bfloat16", out, 512, [json.dumps(step) for step in steps])
        got = helpers.collect(steps, Path(out))
    assert ops.attention_tc_status() == 0 and ops.gemm_bf16_skinny_status() == 0
    cfg, weights = qwen2_plain.load_folder(tmp_path / "model")
    want_a = qwen2_plain.forward_full(cfg, weights, a)[[0, 128, 299, 319] + list(range(320, 330))]
    want_b = qwen2_plain.forward_full(cfg, weights, b)[[39] + list(range(40, 50))]
    for name, got_rows, want_rows in (("a", got["a"], want_a), ("b", got["b"], want_b)):
        limit = helpers.tolerance("bfloat16", want_rows)
        error = (got_rows - want_rows).abs().max(dim=1).values
        assert float(error.max()) <= limit, f"{name}: max error {float(error.max()):.3e} > {limit:.3e} at row {int(error.argmax())}"


def test_tcgen05_attention_replayed_from_a_portion_graph(folder):
    """Three steps of one size class (320 rows, up to 8 requests, every row wanted, a portion of 128 rows or more)
    with different cuts: the first runs launch by launch, the second is captured and replayed, the third is a
    replay of a graph that was captured for other portions (the kernel choice and the grid are frozen in the graph;
    segment starts, first positions and block tables are read from device memory).  Portions start off the tile
    grid, on top of earlier keys.  Every row against the plain implementation."""
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine import StepEntry, StepRunner
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.models import cache_requirements, load_model

    model = load_model(folder, dtype="bfloat16", device="cuda")
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(16, 64), model.dtype, model.device, 1024, num_state_slots=8)
    runner = StepRunner(model, cache, 512, 8)
    assert runner.use_graphs and runner.graph_portions
    cfg, weights = qwen2_plain.load_folder(folder)
    rng = random.Random(12)
    rounds = [[(0, 150), (37, 150)], [(5, 170), (0, 130)], [(21, 130), (0, 130), (3, 40)]]    # (earlier keys, rows of the portion)
    with torch.inference_mode():
        for number, portions in enumerate(rounds):
            sequences, entries = [], []
            for index, (before, rows) in enumerate(portions):
                name = f"r{number}_{index}"
                tokens = helpers.random_tokens(rng, CONFIG["vocab_size"], before + rows)
                sequences.append(tokens)
                cache.create(name)
                if before:
                    runner.run([StepEntry(name, tokens[:before], [])])
                entries.append(StepEntry(name, tokens[before:], list(range(rows))))
            replays = runner.portion_graph_replays
            got = runner.run(entries).float().cpu()
            assert runner.portion_graph_replays == replays + (1 if number else 0)
            cursor = 0
            for (before, rows), tokens in zip(portions, sequences):
                want = qwen2_plain.forward_full(cfg, weights, tokens)[before:]
                part = got[cursor:cursor + rows]
                cursor += rows
                limit = helpers.tolerance("bfloat16", want)
                error = (part - want).abs().max(dim=1).values
                assert float(error.max()) <= limit, f"round {number}, portion ({before}, {rows}): {float(error.max()):.3e} > {limit:.3e} at row {int(error.argmax())}"
                assert helpers.rms_ratio(part, want) <= helpers.RMS_RATIO_LARGE_LAYERS
            for entry in entries:
                cache.free(entry.request_id)
    assert runner.portion_graph_replays >= 2 and ops.attention_tc_status() == 0


def test_a_page_of_another_request_is_noticed(folder):
    """That the comparison can fail: the same decode steps run twice, the second time with one entry of one
    request's block table pointing at a page of the other live request (a host-side edit; every page is owned
    and valid, nothing faults).  Sixteen wrong keys among 150 must fail the comparison; the undamaged run passes it."""
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model

    model = load_model(folder, dtype="bfloat16", device="cuda")
    cfg, weights = qwen2_plain.load_folder(folder)
    rng = random.Random(13)
    a = helpers.random_tokens(rng, CONFIG["vocab_size"], 158)
    b = helpers.random_tokens(rng, CONFIG["vocab_size"], 150)
    want = qwen2_plain.forward_full(cfg, weights, a)[150:]
    passed = []
    for damaged in (False, True):
        cache = CacheManager(cache_requirements(model.spec), CacheConfig(16, 64), model.dtype, model.device, 1024, num_state_slots=2)
        runner = StepRunner(model, cache, 512, 2)
        rows = []
        with torch.inference_mode():
            cache.create("a")
            cache.create("b")
            runner.run([StepEntry("a", a[:150], []), StepEntry("b", b, [])])
            if damaged:
                victim, other = cache.requests["a"], cache.requests["b"]
                victim.tables[0][3], victim.tables_np[0][3] = other.tables[0][3], other.tables_np[0][3]   # keys 48 .. 63
            for token in a[150:]:
                rows.append(runner.run([StepEntry("a", [token], [0])]).float().cpu()[0])
        got = torch.stack(rows)
        passed.append(float((got - want).abs().max()) <= helpers.tolerance("bfloat16", want)
                      and helpers.rms_ratio(got, want) <= helpers.RMS_RATIO_LARGE_LAYERS)
    assert passed == [True, False], passed
