"""Shared helpers of the GPU tests: model folders, traces in the four ways of
cutting, running them through the engine's trace replay, and the comparison."""
from __future__ import annotations

import json
import random
import tempfile
from pathlib import Path

import numpy as np
import torch

from plain import qwen2_plain

import os

# Tolerances, stated once.  float32: 256 units of float32 rounding of the largest
# logit; bfloat16: 8 units of bfloat16 rounding (2^-8) of the largest logit.
F32_UNITS = 256 * 2.0 ** -24
BF16_UNITS = 8 * 2.0 ** -8
# Beside the bound on the largest error, a bound on the error of a request as a whole: the root mean
# square of (engine - plain) over all its logits against the root mean square of the logits (each taken
# about its row's mean).  One wrong key among a hundred, a missing bias or a page of another request
# moves many logits a little: it may stay below the first bound, it does not stay below this one.  About twice
# the largest ratio measured over the whole suite on a B200 (LSE_TEST_PRINT_ERRORS=1 prints every ratio:
# 7.5e-7 in float32; 6.3e-3 in bfloat16 on the tiny configurations, 1.1e-2 at the benchmark's layer sizes).
RMS_RATIO = {"float32": 2.0e-6, "bfloat16": 1.3e-2}
RMS_RATIO_LARGE_LAYERS = 2.3e-2
_PRINT = os.environ.get("LSE_TEST_PRINT_ERRORS", "0") == "1"


def rms_ratio(got: torch.Tensor, reference: torch.Tensor) -> float:
    centred = reference - reference.mean(dim=-1, keepdim=True)
    return float((got - reference).double().pow(2).mean().sqrt() / centred.double().pow(2).mean().sqrt().clamp_min(1e-30))


def tolerance(dtype: str, reference: torch.Tensor) -> float:
    scale = max(1.0, float(reference.abs().max()))
    return (F32_UNITS if dtype == "float32" else BF16_UNITS) * scale


_FOLDERS: dict = {}


def model_folder(name: str) -> Path:
    """A temporary model folder for tiny configuration ``name`` (made once per process)."""
    from tiny_configs import ALL, EXTRA
    from llm_serving_engine_b200.weights import write_random_model

    if name not in _FOLDERS:
        config, _, seed = {**ALL, **EXTRA}[name]
        holder = tempfile.TemporaryDirectory(prefix=f"tiny_{name}_")
        write_random_model(holder.name, config, seed, "float32")
        _FOLDERS[name] = (holder, Path(holder.name))
    return _FOLDERS[name][1]


_PLAIN: dict = {}


def plain_logits(name: str, dtype: str, tokens: list[int]) -> torch.Tensor:
    """Whole-sequence logits of the plain implementation; for bfloat16 the matrices
    are first rounded to bfloat16 as the engine holds them, the arithmetic stays float32."""
    key = (name, dtype)
    if key not in _PLAIN:
        _PLAIN[key] = qwen2_plain.load_folder(model_folder(name),
                                              torch.bfloat16 if dtype == "bfloat16" else None)
    cfg, weights = _PLAIN[key]
    return qwen2_plain.forward_full(cfg, weights, tokens)


def random_tokens(rng: random.Random, vocab: int, count: int) -> list[int]:
    return [rng.randrange(vocab) for _ in range(count)]


# ------------------------------------------------------------------ traces
def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole: one step, every position wanted, then ended."""
    steps = []
    for number, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": number, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}],
                      "end": [rid]})
    return steps


def trace_tail_decode(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps = []
    number = 0
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": number, "entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}],
                      "end": []})
        number += 1
        for index in range(head, len(tokens)):
            steps.append({"step": number, "entries": [{"id": rid, "tokens": [tokens[index]], "want": [0]}],
                          "end": [rid] if index == len(tokens) - 1 else []})
            number += 1
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict[str, list[int]], sizes=(7, 2, 13, 3, 2, 31, 5, 16, 2, 64, 17)) -> list[dict]:
    """Each request in portions of changing size, down to two tokens."""
    steps = []
    number = 0
    for rid, tokens in requests.items():
        done = 0
        turn = 0
        while done < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - done)
            chunk = tokens[done:done + size]
            done += size
            steps.append({"step": number, "entries": [{"id": rid, "tokens": chunk, "want": list(range(size))}],
                          "end": [rid] if done == len(tokens) else []})
            number += 1
            turn += 1
    return steps


def trace_mixed(requests: dict[str, list[int]], seed: int, max_live: int = 4, page_round: int = 64):
    """Up to ``max_live`` requests live at a time: each first runs a prompt part in
    portions (random sizes, 2 and more), then its remaining tokens one by one, beside
    the portions of others; a request may sit a step out.  Returns (steps, max_tokens):
    the pool is sized to the most that live requests hold at any time (each rounded up
    to ``page_round``), so pages are used again when later requests start."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    number = 0
    peak = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, tokens = waiting.pop(0)
            decode_from = max(1, len(tokens) - rng.randrange(3, 20))
            live[rid] = {"tokens": tokens, "done": 0, "decode_from": decode_from}
        held = sum(-(-len(state["tokens"]) // page_round) * page_round for state in live.values())
        peak = max(peak, held)
        entries, ended = [], []
        for rid, state in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            tokens, done = state["tokens"], state["done"]
            if done < state["decode_from"]:
                size = min(rng.choice((2, 2, 3, 5, 8, 13, 21, 40)), state["decode_from"] - done)
            else:
                size = 1
            chunk = tokens[done:done + size]
            state["done"] = done + size
            entries.append({"id": rid, "tokens": chunk, "want": list(range(size))})
            if state["done"] == len(tokens):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": number, "entries": entries, "end": ended})
            number += 1
    return steps, peak


def trace_many_live(vocab: int, seed: int, prompt_range=(30, 52), page_round: int = 64):
    """Dozens of live requests: decode-only steps of 33, 64 and 65 rows (twice each, so that the second is a
    replay of the step captured at the first), prompt portions beside more than 32 decoding requests, and
    requests that end while others start, so that their pages are used again.  The schedule is laid out
    first, then every request gets as many tokens as it is asked for.  Returns (requests, steps, the pool in
    tokens: the most that live requests hold at any time, each rounded up to ``page_round``)."""
    rng = random.Random(seed)
    plan: list[dict] = []                 # per step: {request: tokens in this step}
    fed: dict[str, int] = {}
    live: list[str] = []
    ends: dict[int, list[str]] = {}

    def start(names, beside_decoders=True, per_step=4):
        for offset in range(0, len(names), per_step):
            step = {name: 1 for name in live} if beside_decoders else {}
            group = names[offset:offset + per_step]
            for name in group:
                step[name] = rng.randrange(*prompt_range)
            plan.append(step)
            live.extend(group)

    def decode(times):
        for _ in range(times):
            plan.append({name: 1 for name in live})

    def end(names):
        ends.setdefault(len(plan) - 1, []).extend(names)
        for name in names:
            live.remove(name)

    first = [f"q{index}" for index in range(33)]
    start(first, beside_decoders=True, per_step=8)       # the earliest decode beside the later prompts
    decode(2)                                            # 33 rows
    start([f"q{index}" for index in range(33, 64)])      # portions beside 33 .. 60 decoding requests
    decode(2)                                            # 64 rows
    start(["q64"])                                       # a portion beside 64 decoding requests
    decode(2)                                            # 65 rows
    end(first[:24])
    start([f"q{index}" for index in range(65, 85)])      # 20 new requests take the pages of the 24 that ended
    decode(2)
    for step in plan:
        for name, count in step.items():
            fed[name] = fed.get(name, 0) + count
    for name in list(live):
        end([name])
    requests = {name: random_tokens(rng, vocab, count) for name, count in fed.items()}
    steps, done = [], {name: 0 for name in fed}
    held, peak = set(), 0
    for number, step in enumerate(plan):
        entries = []
        for name, count in step.items():
            entries.append({"id": name, "tokens": requests[name][done[name]:done[name] + count], "want": list(range(count))})
            done[name] += count
            held.add(name)
        peak = max(peak, sum(-(-len(requests[name]) // page_round) * page_round for name in held))
        steps.append({"step": number, "entries": entries, "end": ends.get(number, [])})
        held -= set(ends.get(number, []))
    assert all(done[name] == len(requests[name]) for name in requests)
    return requests, steps, peak


# ------------------------------------------------------------------ running and comparing
def run_trace(name: str, dtype: str, steps: list[dict], max_tokens: int, page: int,
              max_requests: int = 8) -> dict[str, torch.Tensor]:
    """Replay ``steps`` through the engine (in this process) and return, per request,
    the logits of all its positions [S, V] collected from the step files."""
    from llm_serving_engine_b200.engine.trace_replay import replay

    with tempfile.TemporaryDirectory(prefix="trace_out_") as out:
        replay(model_folder(name), dtype, out, max_tokens, [json.dumps(step) for step in steps], block_size=page,
               max_requests=max_requests)
        return collect(steps, Path(out))


def collect(steps: list[dict], out: Path) -> dict[str, torch.Tensor]:
    rows: dict[str, list] = {}
    for step in steps:
        wanted = sum(len(entry["want"]) for entry in step["entries"])
        if not wanted:
            continue
        data = np.fromfile(out / f"{step['step']}.f32", dtype="<f4")
        assert data.size % wanted == 0, f"step {step['step']}: file size does not fit {wanted} rows"
        data = data.reshape(wanted, -1)
        cursor = 0
        for entry in step["entries"]:
            for _ in entry["want"]:
                rows.setdefault(entry["id"], []).append(torch.from_numpy(data[cursor].copy()))
                cursor += 1
    return {rid: torch.stack(values) for rid, values in rows.items()}


def max_tokens_for(requests: dict[str, list[int]], page_round: int = 64) -> int:
    """Pool size for traces that run one request at a time."""
    return max(-(-len(tokens) // page_round) * page_round for tokens in requests.values())


def assert_close(name: str, dtype: str, requests: dict[str, list[int]], got: dict[str, torch.Tensor], what: str):
    for rid, tokens in requests.items():
        reference = plain_logits(name, dtype, tokens)
        assert rid in got, f"{what}: no logits for request {rid}"
        assert got[rid].shape == reference.shape, f"{what}: {rid} shape {got[rid].shape} vs {reference.shape}"
        error = (got[rid] - reference).abs()
        limit = tolerance(dtype, reference)
        worst = float(error.max())
        ratio = rms_ratio(got[rid], reference)
        if _PRINT:
            print(f"[errors] {what} | {name} {dtype} {rid} ({len(tokens)} tokens): max {worst:.3e} of {limit:.3e}, "
                  f"rms ratio {ratio:.3e} of {RMS_RATIO[dtype]:.1e}", flush=True)
        if not ratio <= RMS_RATIO[dtype]:
            raise AssertionError(
                f"{what}: request {rid} ({len(tokens)} tokens, {dtype}) differs from the plain implementation as a whole: "
                f"rms error / rms logit {ratio:.3e} > {RMS_RATIO[dtype]:.1e} (largest error {worst:.3e})")
        if not worst <= limit:
            position = int(error.max(dim=1).values.argmax())
            first_bad = int((error.max(dim=1).values > limit).nonzero()[0])
            raise AssertionError(
                f"{what}: request {rid} ({len(tokens)} tokens, {dtype}) differs from the plain implementation: "
                f"max error {worst:.3e} > {limit:.3e} at position {position}; first wrong position {first_bad}")
