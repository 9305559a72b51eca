"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step.  The default run has the layer sizes of the
Qwen2.5-1.5B shape with random weights, a batch of 8 requests that each hold a
2,048-token prompt (context limit 4,096), bfloat16.  One JSON line is printed:
``value`` is decoded tokens per second timed on the device, ``e2e`` the same
through ``LLMEngine.generate_many`` (host token ids in, host token ids out),
``prefill`` the 2,048-token prompt step, ``roofline`` the decode step's bytes
(every weight once plus the cache of the live requests) over its time against
the measured copy bandwidth, ``points`` decoding at batch 1 and 64.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN25_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 151936, "hidden_size": 1536, "intermediate_size": 8960, "num_hidden_layers": 28,
    "num_attention_heads": 12, "num_key_value_heads": 2, "max_position_embeddings": 4096,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": True,
}
# layer sizes of the larger models of the same architecture (the workloads of the `points` beyond the headline, and
# `--sizes 7b|14b --only decode|prefill`)
QWEN25_7B_SIZES = {"hidden_size": 3584, "intermediate_size": 18944, "num_attention_heads": 28, "num_key_value_heads": 4,
                   "vocab_size": 152064, "tie_word_embeddings": False}
QWEN25_14B_SIZES = {"hidden_size": 5120, "intermediate_size": 13824, "num_attention_heads": 40, "num_key_value_heads": 8,
                    "vocab_size": 152064, "tie_word_embeddings": False, "rms_norm_eps": 1e-5, "max_position_embeddings": 8192}
LAYERS_7B, LAYERS_14B, LAYERS_14B_RUN = 28, 48, 12
FULL_LAYERS = QWEN25_1P5B["num_hidden_layers"]
USE_GRAPHS = True     # --no-graphs: launch by launch (for profilers)
PROMPT = 2048
BLOCK = 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(path):
        try:
            data = json.load(open(path))
            out["hbm_gbs"] = float(data.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(data.get("bf16_tflops", out["bf16_tflops"]))
            out["source"] = "measured"
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.rows.append([item.strip() for item in out.stdout.strip().splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *_):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = sorted(int(row[0]) for row in self.rows if row and row[0].isdigit())
        maxima = [int(row[1]) for row in self.rows if len(row) > 1 and row[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [name for index, name in enumerate(names, start=2)
                   if any(len(row) > index and row[index].lower().startswith("active") for row in self.rows)]
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": reasons, "samples": len(self.rows)}


def build_model(layers: int, sizes: dict | None = None, dtype: str = "bfloat16"):
    """A model of the architecture with random weights made on the device: N(0, 0.02) matrices and biases,
    norm weights 1 + U(-0.1, 0.1), seed 0.  ``sizes`` overrides keys of the Qwen2.5-1.5B configuration."""
    import torch

    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.models import DecoderModel, expected_tensors, parse_dtype
    from llm_serving_engine_b200.weights.loader import held_dtype

    compute = parse_dtype(dtype)
    config = dict(QWEN25_1P5B, **(sizes or {}), num_hidden_layers=layers)
    _, _, spec = load_config(config)
    generator = torch.Generator(device="cuda").manual_seed(0)
    weights = {}
    for name, tensor_spec in expected_tensors(spec).items():
        if tensor_spec.kind == "norm":
            tensor = 1.0 + (torch.rand(tensor_spec.shape, generator=generator, device="cuda") * 0.2 - 0.1)
        else:
            tensor = torch.randn(tensor_spec.shape, generator=generator, device="cuda") * 0.02
        weights[name] = tensor.to(held_dtype(tensor_spec, tensor.dtype, compute))
    return DecoderModel(spec, weights, compute, "cuda"), config


def time_decode(model, batch: int, steps: int, warmup: int, repeats: int = 1, prompt: int = 0):
    """Device time of decode steps at ``batch`` requests that hold ``prompt`` (default PROMPT) tokens each:
    ``repeats`` runs of ``steps`` steps, each between a pair of CUDA events.  Returns (median milliseconds a
    step, the bytes of keys and values a step of the median run reads, launches of one run, every run's
    milliseconds a step)."""
    import torch

    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.kernels import library, ops
    from llm_serving_engine_b200.models import cache_requirements

    prompt = prompt or PROMPT
    context = model.spec.max_position_embeddings
    pages = batch * (context // BLOCK)
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, pages), model.dtype, model.device,
                         context, num_state_slots=batch)
    runner = StepRunner(model, cache, max_tokens_per_step=max(PROMPT, batch), max_segments=batch,
                        use_graphs=USE_GRAPHS)
    generator = torch.Generator().manual_seed(1)
    ids = [f"d{index}" for index in range(batch)]
    runs = []
    with torch.inference_mode():
        for rid in ids:
            cache.create(rid)
            tokens = torch.randint(0, model.vocab_size, (prompt,), generator=generator).tolist()
            for lo in range(0, prompt, PROMPT):          # a long prompt goes in portions of PROMPT tokens
                runner.run([StepEntry(rid, tokens[lo:lo + PROMPT], [])])
        tokens = torch.randint(0, model.vocab_size, (batch,), generator=generator).tolist()
        out = torch.empty(batch, dtype=torch.int32, device=model.device)

        def one_step():
            logits = runner.run([StepEntry(rid, [token], [0]) for rid, token in zip(ids, tokens)])
            ops.argmax(logits, out)

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        launches = 0
        for _ in range(repeats):
            before = library.launches() + runner.graph_kernel_launches
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                one_step()
            end.record()
            torch.cuda.synchronize()
            launches = library.launches() + runner.graph_kernel_launches - before
            runs.append(start.elapsed_time(end) / steps)
    order = sorted(range(repeats), key=lambda index: runs[index])
    median_run = order[repeats // 2]
    kv_bytes = batch * (prompt + warmup + median_run * steps + steps // 2) * cache.kv_bytes_per_token()
    cache.free_all()
    del runner, cache
    torch.cuda.empty_cache()
    return runs[median_run], kv_bytes, launches, runs


def time_prefill(model, repeats: int = 5):
    import torch

    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements

    context = model.spec.max_position_embeddings
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, context // BLOCK), model.dtype,
                         model.device, context, num_state_slots=1)
    runner = StepRunner(model, cache, max_tokens_per_step=PROMPT, max_segments=1)
    generator = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, model.vocab_size, (PROMPT,), generator=generator).tolist()
    times = []
    with torch.inference_mode():
        for index in range(repeats + 2):
            cache.create("p")
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.run([StepEntry("p", prompt, [PROMPT - 1])])
            end.record()
            torch.cuda.synchronize()
            cache.free("p")
            if index >= 2:
                times.append(start.elapsed_time(end))
    times.sort()
    return times[len(times) // 2]


def prefill_flops(config: dict, layers: int, tokens: int) -> float:
    h, inter = config["hidden_size"], config["intermediate_size"]
    n_q, n_kv = config["num_attention_heads"], config["num_key_value_heads"]
    d = h // n_q
    linear = (n_q + 2 * n_kv) * d * h + n_q * d * h + 3 * inter * h
    attention = 4 * n_q * d * tokens * (tokens + 1) / 2
    return layers * (2.0 * tokens * linear + attention) + 2.0 * config["vocab_size"] * h


def time_e2e(model, batch: int, new_tokens: int):
    """Decode tokens per second through the Python entry point: host token ids in, host token ids
    out (``LLMEngine.generate_many`` with per-token callbacks).  The clock runs over the steps in
    which all ``batch`` requests decode together: from the moment the last of them has its first
    token to the moment the first of them ends."""
    import torch

    from llm_serving_engine_b200 import CacheConfig, GenerationConfig, LLMEngine, SchedulerConfig

    context = model.spec.max_position_embeddings
    engine = LLMEngine(model, None, cache_config=CacheConfig(BLOCK, batch * (context // BLOCK)),
                       scheduler_config=SchedulerConfig(max_batch_size=batch, max_tokens_per_step=max(PROMPT, batch)),
                       prefill_chunk_size=PROMPT)
    engine.warmup()
    generator = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, model.vocab_size, (PROMPT,), generator=generator).tolist() for _ in range(batch)]
    stamps: list[tuple[float, int]] = []

    def make_callback(index: int):
        def callback(_token: int) -> None:
            stamps.append((time.perf_counter(), index))
        return callback

    engine.generate_many(prompts, GenerationConfig(max_new_tokens=new_tokens + 2 * batch),
                         [make_callback(index) for index in range(batch)])
    torch.cuda.synchronize()
    counts = [0] * batch
    window_start = window_end = None
    for stamp, index in stamps:
        counts[index] += 1
        if window_start is None and min(counts) >= 1:
            window_start = stamp           # the last request got its first token
        if window_end is None and max(counts) >= new_tokens + 2 * batch:
            window_end = stamp             # the first request got its last token
    decoded = sum(1 for stamp, _ in stamps if window_start < stamp <= window_end)
    seconds = window_end - window_start
    h2d = engine.runner.last_h2d_bytes
    del engine
    torch.cuda.empty_cache()
    return decoded / max(seconds, 1e-9), h2d, 4 * batch, decoded // batch


REPEATS = 5     # runs of the timed decode region; the median is reported, the spread beside it


def time_mixed_traffic(model, requests: int = 32, seed: int = 0):
    """Continuous batching of ``requests`` requests through the Python entry point: prompt lengths log-normal
    (median 512, clipped to 64 .. 4,096), 128 to 512 output tokens each, all waiting at the start.  Returns
    (generated tokens a second over the whole run, generated tokens, prompt tokens, seconds)."""
    import torch

    from llm_serving_engine_b200 import CacheConfig, GenerationConfig, LLMEngine, SchedulerConfig
    from llm_serving_engine_b200.workload import ClippedLogNormal, TrafficProfile, make_traffic

    limit = model.spec.max_position_embeddings
    profile = TrafficProfile(requests=requests, arrival_rate=0.0, prompt=ClippedLogNormal(512, 1.0, 64, 4096),
                             output=ClippedLogNormal(256, 0.5, 128, 512), seed=seed,
                             vocabulary_size=model.vocab_size).fitted_to(model.vocab_size, limit)
    traffic = make_traffic(profile)
    engine = LLMEngine(model, None, cache_config=CacheConfig(BLOCK, requests * (limit // BLOCK)),
                       scheduler_config=SchedulerConfig(max_batch_size=requests, max_tokens_per_step=PROMPT),
                       prefill_chunk_size=PROMPT)
    engine.warmup()
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate_many([list(item.prompt_token_ids) for item in traffic],
                                   [GenerationConfig(max_new_tokens=item.max_new_tokens) for item in traffic])
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    generated = sum(len(output) for output in outputs)
    del engine
    torch.cuda.empty_cache()
    return generated / seconds, generated, sum(len(item.prompt_token_ids) for item in traffic), seconds


def time_short_requests(model, batch: int, prompt: int = 128, new_tokens: int = 32, chunk: int = 32, repeats: int = 3):
    """The workload of the reference's committed T4 results (``artifacts/checkpoint3-t4.json``): ``batch`` prompts of
    ``prompt`` tokens, ``new_tokens`` generated tokens each, prompts fed in portions of ``chunk`` tokens, through the
    Python entry point.  Returns generated tokens a second over the whole run (the median of ``repeats`` runs)."""
    import torch

    from llm_serving_engine_b200 import CacheConfig, GenerationConfig, LLMEngine, SchedulerConfig

    engine = LLMEngine(model, None, cache_config=CacheConfig(BLOCK, batch * 16 + 16),
                       scheduler_config=SchedulerConfig(max_batch_size=batch, max_tokens_per_step=max(chunk, batch)),
                       prefill_chunk_size=chunk)
    engine.warmup()
    generator = torch.Generator().manual_seed(5)
    rates = []
    for _ in range(repeats + 1):     # the first run meets every size class for the first time
        prompts = [torch.randint(0, model.vocab_size, (prompt,), generator=generator).tolist() for _ in range(batch)]
        torch.cuda.synchronize()
        started = time.perf_counter()
        outputs = engine.generate_many(prompts, GenerationConfig(max_new_tokens=new_tokens))
        torch.cuda.synchronize()
        rates.append(sum(len(output) for output in outputs) / (time.perf_counter() - started))
    del engine
    torch.cuda.empty_cache()
    return sorted(rates[1:])[repeats // 2]


def time_chunks_beside_decoding(model, decoding: int = 8, prompt: int = 8192, chunk: int = 2048):
    """A ``prompt``-token prompt fed in ``chunk``-token portions beside ``decoding`` requests that decode (each
    holds ``chunk`` tokens): device milliseconds of each mixed step."""
    import torch

    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements

    context = model.spec.max_position_embeddings
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, (decoding + 1) * (context // BLOCK)), model.dtype,
                         model.device, context, num_state_slots=decoding + 1)
    runner = StepRunner(model, cache, max_tokens_per_step=chunk + decoding, max_segments=decoding + 1)
    generator = torch.Generator().manual_seed(4)
    times = []
    with torch.inference_mode():
        for index in range(decoding):
            cache.create(f"d{index}")
            runner.run([StepEntry(f"d{index}", torch.randint(0, model.vocab_size, (chunk,), generator=generator).tolist(), [])])
        for repeat in range(3):          # the first pass launches kernel by kernel, the second captures, the third replays
            cache.create("long")
            tokens = torch.randint(0, model.vocab_size, (prompt,), generator=generator).tolist()
            times = []
            for lo in range(0, prompt, chunk):
                entries = [StepEntry("long", tokens[lo:lo + chunk], [chunk - 1] if lo + chunk == prompt else [])]
                entries += [StepEntry(f"d{index}", [7], [0]) for index in range(decoding)]
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                runner.run(entries)
                end.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(end))
            cache.free("long")
    cache.free_all()
    del runner, cache
    torch.cuda.empty_cache()
    return times


def kernel_table(batch: int, layers: int) -> dict | None:
    """Per kind of kernel, what one decode step spends in it: a child process loads the tuning variant of the
    library (its kernels stamp the device's clock) and prints the sums as JSON.  None when that fails."""
    try:
        done = subprocess.run([sys.executable, os.path.abspath(__file__), "--timeline", "1", "--timeline-json", "--batch", str(batch),
                               "--layers", str(layers)], capture_output=True, text=True, timeout=600)
        for line in reversed(done.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
    except Exception:
        pass
    return None


def other_points(args, peak: dict) -> tuple[dict, dict]:
    """The workloads beyond the headline: the float32 path, contexts of 30,000 keys, the Qwen2.5-7B sizes under mixed
    traffic, the Qwen2.5-14B sizes at context 8,192 (fewer layers than the model has: both numbers are in the point's
    name or note)."""
    import torch

    points, notes = {}, {}
    steps = max(args.steps // 4, 8)

    def attempt(name, work):
        try:
            work()
        except Exception as error:    # a point that fails is reported as missing, the headline stands
            points[name] = None
            notes[name] = f"{type(error).__name__}: {str(error)[:120]}"
        torch.cuda.empty_cache()

    def float32():
        model, _ = build_model(FULL_LAYERS, dtype="float32")
        ms, kv_bytes, _, _ = time_decode(model, 8, steps, 3)
        points["fp32_decode_b8"] = round(8 / (ms / 1e3), 1)
        notes["fp32_decode_b8"] = (f"true float32 path, 28 layers, {ms:.3f} ms a step, "
                                   f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth")

    def sizes_7b():
        model, _ = build_model(LAYERS_7B, QWEN25_7B_SIZES)
        rate, generated, prompts, seconds = time_mixed_traffic(model)
        points["7b_mixed32_output_tok_s"] = round(rate, 1)
        notes["7b_mixed32_output_tok_s"] = (f"Qwen2.5-7B sizes, 28 of 28 layers, 32 requests at once, {prompts} prompt and {generated} "
                                            f"generated tokens in {seconds:.2f} s through LLMEngine.generate_many")
        ms, kv_bytes, _, _ = time_decode(model, 8, steps, 3)
        points["7b_decode_b8"] = round(8 / (ms / 1e3), 1)
        notes["7b_decode_b8"] = f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth"

    def sizes_14b():
        model, _ = build_model(LAYERS_14B_RUN, QWEN25_14B_SIZES)
        for batch in (1, 8, 64):
            ms, kv_bytes, _, _ = time_decode(model, batch, steps, 3, prompt=8192 - 64)
            name = f"14b_{LAYERS_14B_RUN}of{LAYERS_14B}_layers_ctx8192_decode_b{batch}"
            points[name] = round(batch / (ms / 1e3), 1)
            notes[name] = f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth"
        times = time_chunks_beside_decoding(model)
        name = f"14b_{LAYERS_14B_RUN}of{LAYERS_14B}_layers_prefill8192_in_2048_chunks_beside_8_decoding_tok_s"
        points[name] = round(8192 / (sum(times) / 1e3), 1)
        notes[name] = "ms of the four mixed steps: " + ", ".join(f"{value:.2f}" for value in times)

    def long_contexts():
        model, _ = build_model(FULL_LAYERS, {"max_position_embeddings": 32768})
        for batch in (1, 8):
            ms, kv_bytes, _, _ = time_decode(model, batch, steps, 3, prompt=30000)
            name = f"ctx30000_decode_b{batch}"
            points[name] = round(batch / (ms / 1e3), 1)
            notes[name] = (f"the headline's model, {ms:.3f} ms a step, "
                           f"{(model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9 / peak['hbm_gbs']:.3f} of the copy bandwidth")

    def short_requests():
        model, _ = build_model(FULL_LAYERS)
        published = {1: 18.84, 8: 128.61}    # the reference's own Tesla T4 results for this workload (the real Qwen2.5-1.5B, float16)
        for batch in (1, 8):
            rate = time_short_requests(model, batch)
            name = f"128x32_chunk32_b{batch}_output_tok_s"
            points[name] = round(rate, 1)
            notes[name] = (f"{batch} prompts of 128 tokens, 32 generated tokens each, portions of 32, through generate_many; the "
                           f"reference publishes {published[batch]} on a Tesla T4 for this workload (no B200 figure exists)")

    attempt("fp32_decode_b8", float32)
    attempt("128x32_chunk32", short_requests)
    attempt("ctx30000_decode", long_contexts)
    attempt("7b_mixed32_output_tok_s", sizes_7b)
    attempt("14b", sizes_14b)
    return points, notes


def run_ours(args) -> dict:
    import torch

    import __graft_entry__
    __graft_entry__.build()
    torch.cuda.set_device(0)
    layers = args.layers or FULL_LAYERS
    sizes = {"7b": QWEN25_7B_SIZES, "14b": QWEN25_14B_SIZES}.get(args.sizes)
    model, config = build_model(layers, sizes, dtype=args.dtype if args.only != "all" else "bfloat16")
    peak = peaks()
    weight_bytes = model.weight_bytes_per_step()
    batch = args.batch

    if args.only == "decode":     # a short run of one part, for profilers; prints no bench line
        ms, kv_bytes, _, _ = time_decode(model, batch, args.steps, args.warmup)
        return {"only": "decode", "batch": batch, "layers": layers, "ms_per_step": round(ms, 4),
                "gb_per_s": round((weight_bytes + kv_bytes) / (ms / 1000) / 1e9, 1)}
    if args.only == "prefill":
        ms = time_prefill(model, repeats=max(1, args.steps))
        return {"only": "prefill", "layers": layers, "ms": round(ms, 4),
                "tflops": round(prefill_flops(config, layers, PROMPT) / (ms / 1000) / 1e12, 1)}
    with ClockSampler() as clocks:
        ms, kv_bytes, launches, runs = time_decode(model, batch, args.steps, args.warmup, repeats=REPEATS)
    value = batch / (ms / 1e3)
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9

    prefill_ms = time_prefill(model)
    flops = prefill_flops(config, layers, PROMPT)
    points, fractions = {}, {}
    for point_batch in (1, 64):
        point_ms, point_kv, _, _ = time_decode(model, point_batch, max(args.steps // 2, 8), args.warmup, repeats=3)
        points[f"decode_b{point_batch}"] = round(point_batch / (point_ms / 1e3), 1)
        fractions[f"decode_b{point_batch}"] = round((weight_bytes + point_kv) / (point_ms / 1e3) / 1e9 / peak["hbm_gbs"], 4)
    e2e_value, h2d, d2h, _ = time_e2e(model, batch, max(args.steps, 16))
    del model
    torch.cuda.empty_cache()
    more, notes = ({}, {}) if args.quick else other_points(args, peak)
    points.update(more)
    kernels = None if args.quick else kernel_table(batch, layers)

    return {
        "metric": "decode tok/s at batch 8 (Qwen2.5-1.5B shape, 2,048-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)", "impl": "ours",
        "config": bench_config(config, layers, batch),
        "repeats": {"count": REPEATS, "ms_per_step": [round(run, 4) for run in runs], "reported": "median",
                    "spread": round((max(runs) - min(runs)) / ms, 4)},
        "prefill": {"value": round(PROMPT / (prefill_ms / 1e3), 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]},
        "points": points, "points_roofline_frac": fractions, "points_notes": notes,
        "kernels": kernels,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "pipeline": "one decode step in flight: every step copies its metadata from pinned host memory and its "
                            "tokens to the host; the tokens feed the next step on the device"},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
    }


def bench_config(config: dict, layers: int, batch: int) -> dict:
    """The ``config`` of the bench line: every size, flat; the same dict in both arms."""
    return {
        "model": "Qwen2.5-1.5B shape", "layers": layers, "layers_full": FULL_LAYERS, "hidden": config["hidden_size"],
        "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"],
        "head_dim": config["hidden_size"] // config["num_attention_heads"],
        "intermediate": config["intermediate_size"], "vocab": config["vocab_size"], "tied": True,
        "global_batch": batch, "seq_len": PROMPT, "context": config["max_position_embeddings"],
        "kv_block": BLOCK, "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 3 GB per step)",
    }


# -- the reference arm -----------------------------------------------------------------------
REFERENCE_DIR = os.path.join(ROOT, "baseline", "_ref")


def install_reference() -> str:
    """Put the unmodified reference into ``baseline/_ref`` (once, where its source tree is at hand) and
    return how.  The offline ``pip install`` is tried first; the reference's build backend (hatchling) is
    not in the wheelhouse, and its wheel is nothing but the pure-Python package ``src/llmserve``
    (``pyproject.toml``: ``packages = ["src/llmserve"]``), so a plain copy of that folder is the install."""
    import shutil

    if os.path.exists(os.path.join(REFERENCE_DIR, "llmserve", "engine.py")):
        return "present"
    source = os.environ.get("LLMSERVE_REFERENCE", "/root/reference")
    if not os.path.isdir(os.path.join(source, "src", "llmserve")):
        return ""
    os.makedirs(REFERENCE_DIR, exist_ok=True)
    pip = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                          "--find-links", "/opt/wheelhouse", "--target", REFERENCE_DIR, source],
                         capture_output=True, text=True)
    if pip.returncode == 0 and os.path.exists(os.path.join(REFERENCE_DIR, "llmserve", "engine.py")):
        return "pip"
    shutil.copytree(os.path.join(source, "src", "llmserve"), os.path.join(REFERENCE_DIR, "llmserve"),
                    ignore=shutil.ignore_patterns("__pycache__"), dirs_exist_ok=True)
    return "copy of src/llmserve (pip: no hatchling in the wheelhouse)"


def run_reference(args) -> dict:
    """The same metric and configuration through the UNMODIFIED reference: ``llmserve`` imported from
    ``baseline/_ref`` and nowhere else, its ``Transformer(ModelConfig(...))`` with its own random
    initialisation (``src/llmserve/cli.py:39-41``), its stock CUDA path (float16, ``cli.py:34``; Triton paged
    attention, ``engine.py:140-155``) and its public API (``LLMEngine.generate`` with per-token callbacks,
    ``engine.py:188-221``).  Nothing of this repository's package is imported.

    Device time per step comes from the CUDA event pairs that the reference records around every
    iteration when ``collect_iteration_metrics`` is on (the list behind its ``iteration_stats``,
    ``engine.py:246-254,358-370,438-458``): the decode iterations in which all requests decode together,
    the first ``--warmup`` of them left out, the next ``--steps`` taken.  ``e2e`` is measured from the
    callbacks' time stamps over the same iterations, as in this repository's own arm."""
    how = install_reference()
    if not how:
        return {"impl": "reference", "unavailable": "baseline/_ref holds no install of the reference and its source tree is not at hand"}
    sys.path.insert(0, REFERENCE_DIR)
    try:
        import asyncio

        import torch
        import llmserve
        from llmserve.config import CacheConfig, ModelConfig, SchedulerConfig
        from llmserve.engine import GenerationConfig, LLMEngine
        from llmserve.model import Transformer
        from llmserve.tokenizer import ByteTokenizer
        from llmserve.triton_kernels import is_triton_paged_attention_available
    except Exception as error:   # a missing dependency of the reference
        return {"impl": "reference", "unavailable": f"the reference does not import: {type(error).__name__}: {error}"}
    if not os.path.abspath(llmserve.__file__).startswith(REFERENCE_DIR):
        return {"impl": "reference", "unavailable": f"llmserve was imported from {llmserve.__file__}, not from baseline/_ref"}
    if "llm_serving_engine_b200" in sys.modules:
        raise RuntimeError("the reference arm must not load this repository's package")
    torch.cuda.set_device(0)
    device = torch.device("cuda")
    layers = args.layers or FULL_LAYERS
    config = dict(QWEN25_1P5B, num_hidden_layers=layers)
    peak = peaks()
    torch.manual_seed(0)
    model = Transformer(ModelConfig.from_dict(config))
    model = model.to(device=device, dtype=torch.float16).eval()
    backend = "triton" if is_triton_paged_attention_available(device) else "pytorch"
    if backend == "pytorch":
        return {"impl": "reference", "unavailable": "the reference's Triton paged attention reports itself unavailable on this GPU; "
                "its PyTorch block loop walks every (row, block) pair in Python: hours for 2,048-token prompts"}
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())   # tied head counted once
    kv_bytes_per_token = 2 * layers * config["num_key_value_heads"] * (config["hidden_size"] // config["num_attention_heads"]) * 2

    def make_engine(batch: int):
        return LLMEngine(model, ByteTokenizer(), cache_config=CacheConfig(BLOCK, batch * (config["max_position_embeddings"] // BLOCK)),
                         scheduler_config=SchedulerConfig(max_batch_size=batch, max_tokens_per_step=max(PROMPT, batch)),
                         paged_attention_backend=backend, prefill_chunk_size=PROMPT, collect_iteration_metrics=True,
                         device=device, dtype=torch.float16)

    def decode_run(batch: int, steps: int, warmup: int, inference_mode: bool = False):
        """(device ms per full-batch decode step, its median, end-to-end tokens/s over the same steps, the
        engine's stats).  ``inference_mode``: the driver wraps the run in ``torch.inference_mode()``."""
        with torch.inference_mode(inference_mode):
            return _decode_run(batch, steps, warmup)

    def _decode_run(batch: int, steps: int, warmup: int):
        engine = make_engine(batch)
        generator = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, config["vocab_size"], (PROMPT,), generator=generator).tolist() for _ in range(batch)]
        new_tokens = warmup + steps + 2 * batch + 2
        stamps: list[tuple[float, int]] = []

        def make_callback(index: int):
            def callback(_token: int) -> None:
                stamps.append((time.perf_counter(), index))
            return callback

        async def drive():
            try:
                await asyncio.gather(*[engine.generate(prompt, GenerationConfig(max_new_tokens=new_tokens, temperature=0.0),
                                                       make_callback(index)) for index, prompt in enumerate(prompts)])
                return engine.iteration_stats
            finally:
                await engine.close()

        stats = asyncio.run(drive())
        # iterations in which all requests decode together: from the one after the last request got its first
        # token to the one in which the first request got its last token; one stamp per request and iteration
        counts = [0] * batch
        first_full = last_full = None
        for position, (_, index) in enumerate(stamps):
            counts[index] += 1
            if first_full is None and min(counts) >= 1:
                first_full = position + 1
            if last_full is None and max(counts) >= new_tokens:
                last_full = position        # the first request's last token opens an iteration: that one is left out
        full = stamps[first_full:last_full]
        iterations = len(full) // batch
        if len(full) != iterations * batch or iterations < warmup + steps:
            raise RuntimeError(f"reference arm: {len(full)} stamps in the all-decoding window do not make {warmup + steps} steps of {batch}")
        events = engine._iteration_cuda_events["decode"][:iterations]    # the list behind iteration_stats
        times = sorted(a.elapsed_time(b) for a, b in events[warmup:warmup + steps])
        ms = sum(times) / len(times)
        begin = full[warmup * batch - 1][0] if warmup else stamps[first_full - 1][0]
        end = full[(warmup + steps) * batch - 1][0]
        e2e = steps * batch / max(end - begin, 1e-9)
        del engine, drive, make_callback
        gc.collect()
        torch.cuda.empty_cache()
        return ms, times[len(times) // 2], e2e, stats

    def prefill_run(repeats: int = 5):
        engine = make_engine(1)
        generator = torch.Generator().manual_seed(2)
        prompt = torch.randint(0, config["vocab_size"], (PROMPT,), generator=generator).tolist()

        async def drive():
            try:
                for _ in range(repeats + 2):
                    await engine.generate(prompt, GenerationConfig(max_new_tokens=1, temperature=0.0))
                return engine.iteration_stats
            finally:
                await engine.close()

        asyncio.run(drive())
        times = sorted(a.elapsed_time(b) for a, b in engine._iteration_cuda_events["prefill"][2:])
        del engine, drive
        gc.collect()
        torch.cuda.empty_cache()
        return times[len(times) // 2]

    # The reference decorates its async ``_step`` with ``@torch.inference_mode()`` (``engine.py:244``); on a
    # coroutine function that only covers the creation of the coroutine, so its stock path runs with autograd on:
    # the in-place cache write (``kv_cache.py:265-266``) chains every step's graph to the cache tensor and the
    # activations of all earlier steps stay allocated (about 3 GB per 2,048-token step here).  ``value`` and ``e2e``
    # are that stock path; the same run under the driver's ``torch.inference_mode()`` is given beside it.  Batch 64
    # (65 prompt steps) runs out of 180 GB on the stock path and is measured under inference mode only.
    batch = args.batch
    stock = batch <= 16
    with ClockSampler() as clocks:
        ms, median_ms, e2e_value, stats = decode_run(batch, args.steps, args.warmup, inference_mode=not stock)
    guarded = None
    if stock:
        guarded_ms, _, guarded_e2e, _ = decode_run(batch, args.steps, args.warmup, inference_mode=True)
        guarded = {"value": round(batch / (guarded_ms / 1e3), 1), "ms_per_step": round(guarded_ms, 4), "e2e": round(guarded_e2e, 1)}
    kv_bytes = batch * (PROMPT + args.warmup + args.steps // 2 + batch) * kv_bytes_per_token
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    prefill_ms = prefill_run()
    flops = prefill_flops(config, layers, PROMPT)
    points, notes = {}, {}
    for point_batch in (1, 64):
        try:
            point_ms, _, _, _ = decode_run(point_batch, max(args.steps // 2, 8), args.warmup, inference_mode=point_batch > 16)
            points[f"decode_b{point_batch}"] = round(point_batch / (point_ms / 1e3), 1)
            if point_batch > 16:
                notes[f"decode_b{point_batch}"] = "under the driver's torch.inference_mode()"
        except Exception as error:
            points[f"decode_b{point_batch}"] = None
            notes[f"decode_b{point_batch}"] = f"{type(error).__name__}: {str(error)[:160]}"
            torch.cuda.empty_cache()
    return {
        "metric": "decode tok/s at batch 8 (Qwen2.5-1.5B shape, 2,048-token prompts)",
        "value": round(batch / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "ms_per_step_median": round(median_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "reference", "install": how, "attention_backend": backend,
        "config": bench_config(config, layers, batch),
        "prefill": {"value": round(PROMPT / (prefill_ms / 1e3), 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]},
        "points": points, "points_notes": notes,
        "autograd": "on (stock: the reference's inference_mode decorator sits on an async function and has no effect)" if stock
                    else "off (driver's torch.inference_mode())",
        "under_inference_mode": guarded,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": batch * (8 + 8 + 4 * 4), "d2h_bytes_per_step": batch * 8,
                "pipeline": "the reference's own loop: token ids, positions (int64) and four int32 metadata arrays from pinned "
                            "host memory every step, sampled ids back through .tolist()"},
        "iteration_stats": {key: (round(value, 3) if isinstance(value, float) else value) for key, value in stats.items()},
        "clocks": clocks.summary(),
    }


def timeline(args) -> int:
    """One decode step seen from the device: the tuning variant of the kernel library (built with
    ``-DLSE_TRACE``) lets block 0 of every kernel record when it started, when its wait for the kernels
    before returned and when it ended (nanoseconds of the global timer).  Prints the kernels of the first
    layers in order and the sums per kind of kernel."""
    import ctypes

    import torch

    os.environ["LSE_TRACE"] = "1"   # before the library is loaded
    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config.runtime_config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.kernels import library
    from llm_serving_engine_b200.models import cache_requirements

    torch.cuda.set_device(0)
    lib = library.load()
    model, _ = build_model(args.layers or FULL_LAYERS, {"7b": QWEN25_7B_SIZES, "14b": QWEN25_14B_SIZES}.get(args.sizes))
    batch = args.batch
    context = model.spec.max_position_embeddings
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(BLOCK, batch * (context // BLOCK)), model.dtype,
                         model.device, context, num_state_slots=batch)
    runner = StepRunner(model, cache, max(PROMPT, batch), batch, use_graphs=USE_GRAPHS)
    generator = torch.Generator().manual_seed(1)
    names = {1: "embedding", 2: "add+norm", 3: "rope+cache", 4: "silu", 5: "product", 6: "attention"}

    def read_all(reset: int):
        rows = []
        for reader in ("lse_timeline_elementwise", "lse_timeline_gemm", "lse_timeline_attention"):
            function = getattr(lib, reader)
            function.argtypes = [ctypes.c_void_p, ctypes.c_int]
            function.restype = ctypes.c_int
            buffer = (ctypes.c_ulonglong * (4096 * 8))()
            count = function(buffer, reset)
            rows += [tuple(int(buffer[i * 8 + k]) for k in range(4)) for i in range(count)]
        return sorted(rows, key=lambda row: row[1])

    ids = [f"r{index}" for index in range(batch)]
    with torch.inference_mode():
        for rid in ids:
            cache.create(rid)
            runner.run([StepEntry(rid, torch.randint(0, model.vocab_size, (PROMPT,), generator=generator).tolist(), [])])
        for _ in range(max(args.warmup, 3)):
            runner.run([StepEntry(rid, [5], [0]) for rid in ids])
        torch.cuda.synchronize()
        read_all(1)
        runner.run([StepEntry(rid, [5], [0]) for rid in ids])
        torch.cuda.synchronize()
    rows = read_all(1)
    origin = rows[0][1]
    print(f"decode step, batch {batch}, {len(rows)} kernels, {(max(row[3] for row in rows) - origin) / 1000:.1f} us "
          f"from the first kernel's start to the last kernel's end (block 0 of each; microseconds)")
    print(f"{'#':>3} {'kernel':10} {'started':>9} {'wait over':>10} {'ended':>9} {'after wait':>11} {'since the kernel before ended':>30}")
    before = origin
    for index, (kind, started, waited, ended) in enumerate(rows[:2 + 9 * args.timeline]):
        print(f"{index:3d} {names.get(kind, str(kind)):10} {(started - origin) / 1000:9.2f} {(waited - origin) / 1000:10.2f} "
              f"{(ended - origin) / 1000:9.2f} {(ended - waited) / 1000:11.2f} {(waited - before) / 1000:30.2f}")
        before = ended
    totals: dict[str, list] = {}
    before = origin
    for kind, started, waited, ended in rows:
        entry = totals.setdefault(names.get(kind, str(kind)), [0, 0.0, 0.0])
        entry[0] += 1
        entry[1] += (ended - waited) / 1000
        entry[2] += max(0.0, (waited - before) / 1000)
        before = ended
    for name, (count, active, gaps) in totals.items():
        print(f"{name:10} x{count:4d}: {active:8.1f} us after the wait in total, {active / count:6.2f} us each; "
              f"{gaps:8.1f} us between the kernel before and the wait's return")
    if args.timeline_json:
        # bytes a kind of kernel has to read in a step over the time its block 0 spends after its wait: a lower
        # bound of the kind's rate (other blocks end later; the first tiles were fetched before the wait)
        kv_bytes = batch * (PROMPT + max(args.warmup, 3) + 1) * cache.kv_bytes_per_token()
        moved = {"product": model.weight_bytes_per_step(), "attention": kv_bytes}
        table = {"step_us": round((max(row[3] for row in rows) - origin) / 1000, 1), "kernels_in_step": len(rows),
                 "how": "block 0 of every kernel stamps the global timer at its start, when its wait for the kernels "
                        "before returns and at its end (tuning variant of the library, one decode step from a CUDA graph)"}
        for name, (count, active, gaps) in totals.items():
            table[name] = {"launches": count, "us_after_wait": round(active, 1), "us_handover": round(gaps, 1)}
            if name in moved:
                table[name]["gb_per_s_after_wait"] = round(moved[name] / (active * 1e-6) / 1e9, 1)
        print(json.dumps(table))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the full model (0 = all)")
    parser.add_argument("--only", choices=("all", "decode", "prefill"), default="all",
                        help="run one part only (a small case for ncu; no bench line)")
    parser.add_argument("--no-graphs", action="store_true", help="decode launch by launch instead of from CUDA graphs")
    parser.add_argument("--sizes", choices=("1.5b", "7b", "14b"), default="1.5b",
                        help="layer sizes (7b, 14b: those of Qwen2.5-7B / 14B; only with --only, give --layers to fit the time)")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                        help="with --only: the true float32 path instead of the serving precision")
    parser.add_argument("--quick", action="store_true", help="the headline, its points and the end-to-end number only "
                                                             "(no other model sizes, no float32 point, no kernel table)")
    parser.add_argument("--timeline-json", action="store_true", help="with --timeline: also one JSON line of sums per kind of kernel")
    parser.add_argument("--timeline", type=int, default=0, metavar="LAYERS",
                        help="print the device-side timeline of one decode step (the first LAYERS layers kernel by "
                             "kernel) from the tuning variant of the kernel library; no bench line")
    args = parser.parse_args()
    global USE_GRAPHS
    USE_GRAPHS = not args.no_graphs
    if args.sizes != "1.5b" and args.only == "all" and not args.timeline:
        print(f"--sizes {args.sizes} measures one part only: add --only decode or --only prefill")
        return 2
    if args.timeline:
        return timeline(args)
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        args.warmup = max(args.warmup, 3)
        print(json.dumps(run_reference(args)))
        return 0
    if args.only == "all":
        args.warmup = max(args.warmup, 3)
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
