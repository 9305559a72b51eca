"""Generation through the Python entry point and the command line on the GPU."""
import asyncio
import json
import os
import random
import subprocess
import sys

import pytest
import torch

import helpers
from plain import qwen2_plain
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine_for(name, dtype="float32", pages=256, batch=4, budget=64, chunk=16, mode="continuous", page=None):
    from llm_serving_engine_b200 import CacheConfig, LLMEngine, SchedulerConfig, load_model
    model = load_model(helpers.model_folder(name), dtype=dtype, device="cuda")
    return LLMEngine(model, None, cache_config=CacheConfig(page or ALL[name][1], pages),
                     scheduler_config=SchedulerConfig(max_batch_size=batch, max_tokens_per_step=budget),
                     scheduler_mode=mode, prefill_chunk_size=chunk)


def prompts_for(name, lengths, seed=0):
    rng = random.Random(seed)
    return [helpers.random_tokens(rng, ALL[name][0]["vocab_size"], n) for n in lengths]


def plain_greedy(name, prompt, count):
    cfg, weights = qwen2_plain.load_folder(helpers.model_folder(name))
    return qwen2_plain.greedy_generate(cfg, weights, prompt, count)


@pytest.mark.parametrize("name, lengths", [("A", (5, 17, 33)), ("B", (1, 9, 24, 40))])
def test_greedy_generation_equals_the_plain_implementation(name, lengths):
    from llm_serving_engine_b200 import GenerationConfig
    prompts = prompts_for(name, lengths)
    got = engine_for(name).generate_many(prompts, GenerationConfig(max_new_tokens=8))
    assert got == [plain_greedy(name, prompt, 8) for prompt in prompts]


def test_portions_and_batching_do_not_change_the_tokens():
    from llm_serving_engine_b200 import GenerationConfig
    prompts = prompts_for("B", (30, 3, 57, 12, 41, 8), seed=4)
    config = GenerationConfig(max_new_tokens=12, temperature=0.8, seed=11)
    alone = [engine_for("B", batch=1, chunk=1).generate_many([prompt], config)[0] for prompt in prompts]
    for chunk, batch, budget in ((1, 4, 8), (7, 3, 16), (2048, 6, 256)):
        engine = engine_for("B", batch=batch, budget=budget, chunk=chunk)
        assert engine.generate_many(prompts, config) == alone, (chunk, batch, budget)
        assert not engine.cache.requests and engine.cache.groups[0].pool.used_pages == 0


def test_sampling_options():
    from llm_serving_engine_b200 import GenerationConfig
    prompts = prompts_for("A", (9, 9), seed=2)
    engine = engine_for("A")
    greedy = engine.generate_many(prompts, GenerationConfig(max_new_tokens=10))
    a = engine.generate_many(prompts, GenerationConfig(max_new_tokens=10, temperature=1.5, seed=1))
    b = engine.generate_many(prompts, GenerationConfig(max_new_tokens=10, temperature=1.5, seed=1))
    c = engine.generate_many(prompts, GenerationConfig(max_new_tokens=10, temperature=1.5, seed=2))
    assert a == b and a != c and a != greedy
    # a very small top-p keeps the most likely token only
    assert engine.generate_many(prompts, GenerationConfig(max_new_tokens=10, temperature=1.5, top_p=1e-6, seed=5)) == greedy
    # a stop token ends the request and is returned
    stop = greedy[0][3]
    stopped = engine.generate_many([prompts[0]], GenerationConfig(max_new_tokens=10, stop_token_ids=(stop,)))[0]
    assert stopped == greedy[0][:greedy[0].index(stop) + 1]
    # mixed options in one batch
    mixed = engine.generate_many(prompts, [GenerationConfig(max_new_tokens=10),
                                           GenerationConfig(max_new_tokens=10, temperature=1.5, seed=1)])
    assert mixed == [greedy[0], a[1]]


def test_pages_run_out_preemption_recomputes_and_gives_the_same_tokens():
    from llm_serving_engine_b200 import GenerationConfig
    prompts = prompts_for("A", (20, 18, 25), seed=8)
    config = GenerationConfig(max_new_tokens=24, temperature=0.9, seed=3)
    roomy = engine_for("A", pages=64, batch=3).generate_many(prompts, config)
    tight = engine_for("A", pages=7, batch=3, page=16)       # 112 token slots for 3 x ~45 tokens
    streamed = [[] for _ in prompts]
    got = tight.generate_many(prompts, config, [lst.append for lst in streamed])
    assert got == roomy and streamed == got                  # no token is emitted twice
    assert tight.iteration_stats["preemptions"] > 0 and tight.iteration_stats["recomputed_tokens"] > 0
    assert tight.cache.groups[0].pool.used_pages == 0 and not tight.cache.requests


def test_a_request_that_can_never_fit_fails_alone():
    from llm_serving_engine_b200 import GenerationConfig
    from llm_serving_engine_b200.cache import CacheFullError
    engine = engine_for("A", pages=2, batch=2)               # 32 token slots
    with pytest.raises(CacheFullError, match="one sequence exceeds"):
        engine.generate_many(prompts_for("A", (40,)), GenerationConfig(max_new_tokens=4))
    assert engine.cache.groups[0].pool.used_pages == 0
    assert len(engine.generate_many(prompts_for("A", (10,)), GenerationConfig(max_new_tokens=4))[0]) == 4
    with pytest.raises(ValueError, match="max_position_embeddings"):
        engine.generate_many([[1] * 500], GenerationConfig(max_new_tokens=100))
    with pytest.raises(ValueError, match="token id"):
        engine.generate_many([[1, 512]], GenerationConfig(max_new_tokens=2))
    with pytest.raises(ValueError, match="empty"):
        engine.generate_many([[]], GenerationConfig(max_new_tokens=2))


def test_async_entry_point_streams_and_batches_continuously():
    from llm_serving_engine_b200 import GenerationConfig
    prompts = prompts_for("B", (40, 5, 6, 7), seed=6)
    expected = [plain_greedy("B", prompt, 6) for prompt in prompts]

    async def run(mode):
        engine = engine_for("B", batch=4, budget=32, chunk=8, mode=mode)
        seen_batches = []
        original = engine.runner.run
        engine.runner.run = lambda entries: (seen_batches.append([(e.request_id, len(e.tokens)) for e in entries]),
                                             original(entries))[1]
        streams = [[] for _ in prompts]

        async def async_callback(token, index=1):
            streams[index].append(token)

        callbacks = [streams[0].append, async_callback, streams[2].append, None]
        async with engine:
            first = asyncio.create_task(engine.generate(prompts[0], GenerationConfig(max_new_tokens=6), callbacks[0],
                                                        request_id="long"))
            await asyncio.sleep(0)
            rest = [asyncio.create_task(engine.generate(prompts[i], GenerationConfig(max_new_tokens=6), callbacks[i],
                                                        request_id=f"short{i}")) for i in (1, 2, 3)]
            results = await asyncio.gather(first, *rest)
        return results, streams, seen_batches

    results, streams, batches = asyncio.run(run("continuous"))
    assert results == expected and streams[:3] == expected[:3]
    # decode tokens of some requests ran beside prompt portions of another
    assert any(len(batch) > 1 and any(n == 1 for _, n in batch) and any(n > 1 for _, n in batch) for batch in batches)
    results, _, batches = asyncio.run(run("static"))
    assert results == expected
    assert not any({"long"} < {rid for rid, _ in batch} for batch in batches)   # nobody joins the running batch


def test_command_line_generate_and_benchmark(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmserve"), "generate", "--model",
                          str(helpers.model_folder("A")), "--dtype", "float32", "--prompt-ids", "5 17 3 250 99",
                          "--max-new-tokens", "6"], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr
    record = json.loads(out.stdout.strip().splitlines()[-1])
    assert record["output_ids"] == plain_greedy("A", [5, 17, 3, 250, 99], 6)
    report = tmp_path / "bench.json"
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmserve"), "benchmark", "--requests", "6",
                          "--arrival-rate", "200", "--batch-size", "4", "--num-blocks", "512", "--output", str(report),
                          "--profile", os.path.join(ROOT, "configs", "benchmark-sharegpt.yaml")],
                         capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stderr
    summary = json.loads(report.read_text())["summary"]
    assert summary["successful_requests"] == 6 and summary["throughput_tokens_per_s"] > 0


def test_trace_run_program(tmp_path):
    """bin/trace_run as a user calls it: steps on standard input, logits in files, 'done <step>' lines."""
    name = "A"
    rng = random.Random(3)
    tokens = helpers.random_tokens(rng, ALL[name][0]["vocab_size"], 70)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": tokens[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": tokens[40:42], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": tokens[42:70], "want": [27]},
                                {"id": "b", "tokens": tokens[:3], "want": [2]}], "end": ["a", "b"]},
    ]
    for dtype in ("float32", "bfloat16"):
        out_dir = tmp_path / dtype
        run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
                              str(helpers.model_folder(name)), "--dtype", dtype, "--out", str(out_dir),
                              "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                             capture_output=True, text=True, timeout=900)
        assert run.returncode == 0, run.stderr
        assert run.stdout.split() == ["done", "0", "done", "1", "done", "2"]
        assert not (out_dir / "1.f32").exists()
        got = helpers.collect(steps, out_dir)
        reference = helpers.plain_logits(name, dtype, tokens)
        limit = helpers.tolerance(dtype, reference)
        assert float((got["a"] - reference[[0, 39, 69]]).abs().max()) <= limit
        assert float((got["b"][0] - helpers.plain_logits(name, dtype, tokens[:3])[2]).abs().max()) <= limit


def test_warmup_captures_decode_graphs_and_leaves_the_cache_empty():
    from llm_serving_engine_b200 import GenerationConfig
    engine = engine_for("D", dtype="bfloat16", batch=4, pages=128)
    engine.warmup()
    assert engine.runner.use_graphs and len(engine.runner._graphs) == 3           # batch buckets 1, 2, 4
    assert all(slot.graph is not None for slot in engine.runner._graphs.values())
    assert not engine.cache.requests and engine.cache.groups[0].pool.used_pages == 0
    prompts = prompts_for("D", (9, 30, 4), seed=5)
    replays = engine.runner.graph_replays
    warm = engine.generate_many(prompts, GenerationConfig(max_new_tokens=12))
    assert engine.runner.graph_replays > replays and len(engine.runner._graphs) == 3   # no new capture
    cold = engine_for("D", dtype="bfloat16", batch=4, pages=128)
    cold.runner.use_graphs = False
    assert cold.generate_many(prompts, GenerationConfig(max_new_tokens=12)) == warm       # graphs change nothing


def test_decode_steps_packed_ahead_give_the_same_tokens():
    """While the device runs a decode step the host packs the next one but for its tokens.  The tokens
    must be those of an engine that packs every step after reading the last one: through page edges
    (a new page is reserved by the ordinary path), requests that stop at different lengths, stop
    tokens that nobody could foresee, and sampling with a temperature."""
    from llm_serving_engine_b200 import GenerationConfig
    prompts = prompts_for("D", (9, 30, 4, 17), seed=6)
    configs = [GenerationConfig(max_new_tokens=40), GenerationConfig(max_new_tokens=23, temperature=0.7, seed=3),
               GenerationConfig(max_new_tokens=40), GenerationConfig(max_new_tokens=31)]
    plain = engine_for("D", dtype="bfloat16", batch=4, pages=128)
    plain.pack_ahead = False
    want = plain.generate_many(prompts, configs)
    assert plain.runner.ahead_steps == 0
    ahead = engine_for("D", dtype="bfloat16", batch=4, pages=128)
    assert ahead.generate_many(prompts, configs) == want
    assert ahead.runner.ahead_steps > 20 and ahead.runner.flying_steps > 20   # most of them queued before the tokens were read
    packed_only = engine_for("D", dtype="bfloat16", batch=4, pages=128)
    packed_only.launch_ahead = False
    assert packed_only.generate_many(prompts, configs) == want
    assert packed_only.runner.ahead_steps > 20 and packed_only.runner.flying_steps == 0
    assert not ahead.cache.requests and ahead.cache.groups[0].pool.used_pages == 0
    # a stop token that ends one request early: the step packed ahead for all four is dropped
    stop = want[2][10]
    configs[2] = GenerationConfig(max_new_tokens=40, stop_token_ids=(stop,))
    again = engine_for("D", dtype="bfloat16", batch=4, pages=128)
    got = again.generate_many(prompts, configs)
    cut = want[2].index(stop) + 1
    assert got == [want[0], want[1], want[2][:cut], want[3]]
    assert again.runner.flying_steps > 10 and not again.cache.requests
    assert again.cache.groups[0].pool.used_pages == 0 and again._flying is None


def test_steps_with_prompt_portions_replayed_from_graphs_give_the_same_tokens():
    """Steps with prompt portions fall into size classes (tokens, requests, wanted places rounded up, the rest
    padding); a class is captured in a CUDA graph the second time it is met.  Prompts fed in small portions
    beside decoding requests meet few classes many times: the tokens must be those of an engine that launches
    every such step kernel by kernel, and the cache must come back empty."""
    from llm_serving_engine_b200 import GenerationConfig
    prompts = prompts_for("D", (70, 33, 5, 58, 41, 64), seed=8)
    config = GenerationConfig(max_new_tokens=20, temperature=0.6, seed=5)
    plain = engine_for("D", dtype="bfloat16", batch=4, pages=160, budget=24, chunk=16)
    plain.runner.graph_portions = False
    want = plain.generate_many(prompts, config)
    assert plain.runner.portion_graph_replays == 0
    graphs = engine_for("D", dtype="bfloat16", batch=4, pages=160, budget=24, chunk=16)
    assert graphs.generate_many(prompts, config) == want
    assert graphs.runner.portion_graph_replays >= 8 and len(graphs.runner._portion_graphs) >= 2
    assert not graphs.cache.requests and graphs.cache.groups[0].pool.used_pages == 0
    # float32 too (the general attention kernel): bit for bit the same logits with and without padding rows
    one = engine_for("B", dtype="float32", batch=3, budget=20, chunk=8)
    two = engine_for("B", dtype="float32", batch=3, budget=20, chunk=8)
    two.runner.graph_portions = False
    few = prompts_for("B", (30, 9, 44), seed=2)
    assert one.generate_many(few, GenerationConfig(max_new_tokens=6)) == two.generate_many(few, GenerationConfig(max_new_tokens=6))
    assert one.runner.portion_graph_replays > 0


def test_dependent_launch_off_gives_the_same_logits(tmp_path):
    """LSE_PDL=0 launches every kernel fully serialised; the logits must not change."""
    name = "D"
    rng = random.Random(9)
    tokens = helpers.random_tokens(rng, ALL[name][0]["vocab_size"], 40)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:30], "want": [29]}], "end": []}]
    steps += [{"step": 1 + i, "entries": [{"id": "a", "tokens": [tokens[30 + i]], "want": [0]}], "end": []} for i in range(10)]
    outs = {}
    for flag in ("1", "0"):
        out_dir = tmp_path / flag
        run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
                              str(helpers.model_folder(name)), "--dtype", "bfloat16", "--out", str(out_dir),
                              "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                             capture_output=True, text=True, timeout=900, env=dict(os.environ, LSE_PDL=flag))
        assert run.returncode == 0, run.stderr
        outs[flag] = helpers.collect(steps, out_dir)["a"]
    assert torch.equal(outs["0"], outs["1"])


def test_a_wait_that_gave_up_fails_the_requests_and_leaves_the_engine_usable():
    """The few-rows product is made to give up a wait (a test hook: a tile that never arrives and a small limit; no
    fault, the kernel returns).  Its status word reaches the host with the step's tokens: the requests fail with a
    KernelError instead of getting tokens sampled from memory that nobody wrote, every page goes back, the word is
    cleared, and the same engine generates the right tokens afterwards."""
    from llm_serving_engine_b200 import GenerationConfig
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.kernels.library import KernelError

    engine = engine_for("D", dtype="bfloat16")
    prompts = prompts_for("D", (9, 21), seed=4)
    good = engine.generate_many(prompts, GenerationConfig(max_new_tokens=4))
    ops.gemm_bf16_skinny_test_hooks(spin_limit=2000, withhold=True)
    try:
        with pytest.raises(KernelError, match="bounded wait"):
            engine.generate_many(prompts, GenerationConfig(max_new_tokens=4))
    finally:
        ops.gemm_bf16_skinny_test_hooks()
    assert engine.scheduler.idle and not engine.cache.requests and engine.cache.groups[0].pool.used_pages == 0
    assert ops.gemm_bf16_skinny_status() == 0
    assert engine.generate_many(prompts, GenerationConfig(max_new_tokens=4)) == good
