"""Trace replay on the GPU against the plain implementation: each request whole;
most of it in one step and the last 32 tokens one by one; portions of changing
size; and mixed batches with so few pages that they are used again.  In float32
and in bfloat16, for tiny configurations that differ in every size and option."""
import random

import pytest

import helpers
from tiny_configs import ALL

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
LENGTHS = {"A": (5, 17, 33, 150), "B": (1, 9, 24, 40, 131), "C": (3, 66, 97), "D": (7, 64, 65, 200),
           "E": (2, 129, 90)}


def _requests(name: str, seed: int = 0) -> dict[str, list[int]]:
    config, _, _ = ALL[name]
    rng = random.Random(1000 + seed)
    return {f"r{index}": helpers.random_tokens(rng, config["vocab_size"], length)
            for index, length in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALL))
def test_whole(name, dtype):
    requests = _requests(name)
    steps = helpers.trace_whole(requests)
    got = helpers.run_trace(name, dtype, steps, helpers.max_tokens_for(requests), ALL[name][1])
    helpers.assert_close(name, dtype, requests, got, "whole prompts")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALL))
def test_tail_decoded_one_by_one(name, dtype):
    requests = _requests(name)
    steps = helpers.trace_tail_decode(requests, tail=32)
    got = helpers.run_trace(name, dtype, steps, helpers.max_tokens_for(requests), ALL[name][1])
    helpers.assert_close(name, dtype, requests, got, "last 32 tokens one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALL))
def test_portions_of_changing_size(name, dtype):
    requests = _requests(name)
    steps = helpers.trace_portions(requests)
    got = helpers.run_trace(name, dtype, steps, helpers.max_tokens_for(requests), ALL[name][1])
    helpers.assert_close(name, dtype, requests, got, "portions of changing size")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALL))
def test_mixed_with_page_reuse(name, dtype):
    config, page, _ = ALL[name]
    rng = random.Random(77)
    lengths = [rng.randrange(20, 140) for _ in range(9)]
    requests = {f"m{index}": helpers.random_tokens(rng, config["vocab_size"], length)
                for index, length in enumerate(lengths)}
    steps, peak = helpers.trace_mixed(requests, seed=5)
    total_rounded = sum(-(-length // 64) * 64 for length in lengths)
    assert peak < total_rounded, "the pool must be smaller than all requests together, so pages are used again"
    got = helpers.run_trace(name, dtype, steps, peak, page)
    helpers.assert_close(name, dtype, requests, got, "mixed batches with page reuse")


@pytest.mark.parametrize("name, dtype", [("B", "float32"), ("D", "float32"), ("D", "bfloat16"), ("E", "bfloat16"), ("A", "bfloat16")])
def test_dozens_of_live_requests(name, dtype):
    """More than 32 rows of decoding and more than four live requests: decode-only steps of 33, 64 and 65 rows
    (other products, other graph buckets, other splits of the decode attention than a handful of rows take),
    prompt portions beside more than 32 decoding requests, and a pool so small that the pages of requests that
    ended serve the ones that start; every logit row against the plain implementation."""
    config, page, _ = ALL[name]
    requests, steps, peak = helpers.trace_many_live(config["vocab_size"], seed=31)
    assert max(len(step["entries"]) for step in steps) == 65
    assert {len(step["entries"]) for step in steps if all(len(e["tokens"]) == 1 for e in step["entries"])} >= {33, 64, 65}
    assert any(len(step["entries"]) > 40 and max(len(e["tokens"]) for e in step["entries"]) > 1 for step in steps)
    assert peak < sum(-(-len(tokens) // 64) * 64 for tokens in requests.values()), "pages must be used again"
    got = helpers.run_trace(name, dtype, steps, peak, page, max_requests=66)
    helpers.assert_close(name, dtype, requests, got, "dozens of live requests")


def test_float32_is_bitwise_the_same_however_it_is_cut():
    """In float32 every kernel sums in an order that depends on the row alone, so the
    logits of a position are the same bit for bit in every way of cutting and batching."""
    import torch

    name = "B"
    config, page, _ = ALL[name]
    requests = _requests(name, seed=3)
    whole = helpers.run_trace(name, "float32", helpers.trace_whole(requests), helpers.max_tokens_for(requests), page)
    portions = helpers.run_trace(name, "float32", helpers.trace_portions(requests),
                                 helpers.max_tokens_for(requests), page)
    steps, peak = helpers.trace_mixed(requests, seed=9)
    mixed = helpers.run_trace(name, "float32", steps, peak, page)
    for rid in requests:
        assert torch.equal(whole[rid], portions[rid]), f"{rid}: portions differ from whole"
        assert torch.equal(whole[rid], mixed[rid]), f"{rid}: mixed differs from whole"
    # and with dozens of live requests: steps of 33 to 65 rows, replayed from graphs of other sizes
    many, steps, peak = helpers.trace_many_live(config["vocab_size"], seed=32)
    crowded = helpers.run_trace(name, "float32", steps, peak, page, max_requests=66)
    some = {rid: many[rid] for rid in list(many)[::9]}
    alone = helpers.run_trace(name, "float32", helpers.trace_whole(some), helpers.max_tokens_for(some), page)
    for rid in some:
        assert torch.equal(alone[rid], crowded[rid]), f"{rid}: differs among dozens of live requests"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_long_decoding(name, dtype):
    """A short prompt, then hundreds of tokens one by one, across many pages."""
    config, page, _ = ALL[name]
    rng = random.Random(21)
    tokens = helpers.random_tokens(rng, config["vocab_size"], 8 + 400)
    requests = {"long": tokens}
    steps = helpers.trace_tail_decode(requests, tail=400)
    got = helpers.run_trace(name, dtype, steps, helpers.max_tokens_for(requests), page)
    helpers.assert_close(name, dtype, requests, got, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALL))
def test_first_tokens_of_a_sequence(name, dtype):
    """Positions 0, 1, 2, ... each in a step of its own, and prompts of one and two tokens."""
    config, page, _ = ALL[name]
    rng = random.Random(22)
    requests = {"one": helpers.random_tokens(rng, config["vocab_size"], 1),
                "two": helpers.random_tokens(rng, config["vocab_size"], 2),
                "steps": helpers.random_tokens(rng, config["vocab_size"], 6)}
    steps = helpers.trace_whole({"one": requests["one"], "two": requests["two"]})
    for index, token in enumerate(requests["steps"]):
        steps.append({"step": len(steps), "entries": [{"id": "steps", "tokens": [token], "want": [0]}],
                      "end": ["steps"] if index == 5 else []})
    got = helpers.run_trace(name, dtype, steps, 64, page)
    helpers.assert_close(name, dtype, requests, got, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_context_in_chunks_then_a_portion_then_decoding(dtype):
    """The long-context schedule of the largest benchmark shape in small: a prompt fed in 2,048-token chunks, a
    256-row portion on top of 6,144 earlier keys (512 pages a request), a long odd portion, and decoding at
    contexts 8,191 and 8,192, the position limit.  Five query heads on one key/value head of 128."""
    from tiny_configs import EXTRA

    config, page, _ = EXTRA["L"]
    rng = random.Random(41)
    tokens = helpers.random_tokens(rng, config["vocab_size"], 8192)
    cuts = [(0, 2048), (2048, 4096), (4096, 6144), (6144, 6400), (6400, 8190), (8190, 8191), (8191, 8192)]
    steps, wanted = [], []
    for number, (lo, hi) in enumerate(cuts):
        want = list(range(hi - lo)) if hi - lo <= 256 else [0, 1, (hi - lo) // 2, hi - lo - 1]
        wanted += [lo + index for index in want]
        steps.append({"step": number, "entries": [{"id": "long", "tokens": tokens[lo:hi], "want": want}],
                      "end": ["long"] if hi == 8192 else []})
    got = helpers.run_trace("L", dtype, steps, 8192, page)["long"]
    reference = helpers.plain_logits("L", dtype, tokens)[wanted]
    error = (got - reference).abs().max(dim=1).values
    limit = helpers.tolerance(dtype, reference)
    assert float(error.max()) <= limit, f"max error {float(error.max()):.3e} > {limit:.3e} at position {wanted[int(error.argmax())]}"
    assert helpers.rms_ratio(got, reference) <= helpers.RMS_RATIO[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_the_line_where_a_context_counts_as_long(dtype):
    """Decode steps over more than 8,192 keys are replayed from graphs of their own, in which a single request's keys
    are cut into more splits than one thread-block cluster adds up (the last-arriving block adds them).  One request
    decodes from 8,170 to 8,230 keys, a second one joins for a few steps at a short context."""
    from tiny_configs import EXTRA

    config, page, _ = EXTRA["L2"]
    rng = random.Random(43)
    long_tokens = helpers.random_tokens(rng, config["vocab_size"], 8230)
    short_tokens = helpers.random_tokens(rng, config["vocab_size"], 40)
    steps, wanted = [], {"long": [], "short": []}
    cuts = [(0, 2048), (2048, 4096), (4096, 6144), (6144, 8170)]
    for number, (lo, hi) in enumerate(cuts):
        steps.append({"step": number, "entries": [{"id": "long", "tokens": long_tokens[lo:hi], "want": [hi - lo - 1]}], "end": []})
        wanted["long"].append(hi - 1)
    for position in range(8170, 8230):
        entries = [{"id": "long", "tokens": [long_tokens[position]], "want": [0]}]
        wanted["long"].append(position)
        ends = ["long"] if position == 8229 else []
        if 8185 <= position < 8205:     # beside it, for twenty steps, a request at a short context
            index = position - 8185
            portion = short_tokens[:21] if index == 0 else [short_tokens[20 + index]]
            entries.append({"id": "short", "tokens": portion, "want": [len(portion) - 1]})
            wanted["short"].append(20 + index)
            if position == 8204:
                ends.append("short")
        steps.append({"step": len(steps), "entries": entries, "end": ends})
    got = helpers.run_trace("L2", dtype, steps, 8448, page)
    for name, tokens in (("long", long_tokens), ("short", short_tokens[:40])):
        reference = helpers.plain_logits("L2", dtype, tokens)[wanted[name]]
        rows = got[name]
        assert rows.shape[0] == len(wanted[name])
        error = (rows - reference).abs().max(dim=1).values
        limit = helpers.tolerance(dtype, reference)
        assert float(error.max()) <= limit, f"{name}: max error {float(error.max()):.3e} > {limit:.3e} at position {wanted[name][int(error.argmax())]}"
        assert helpers.rms_ratio(rows, reference) <= helpers.RMS_RATIO[dtype], name

