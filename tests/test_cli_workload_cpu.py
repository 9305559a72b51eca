"""The command line's options and the synthetic traffic (no GPU)."""
import asyncio

import pytest

from llm_serving_engine_b200.cli import parse, tiny_config
from llm_serving_engine_b200.tokenizer import ByteTokenizer
from llm_serving_engine_b200.workload import (ClippedLogNormal, TrafficProfile, TrafficResult, make_traffic,
                                              replay_traffic, summarise)


def test_benchmark_options_carry_the_reference_names_and_defaults():
    args = parse(["benchmark"])
    assert (args.config, args.policy, args.batch_size, args.block_size, args.num_blocks) == ("continuous", "fcfs", 16, 16, 1024)
    assert (args.max_tokens_per_step, args.seed, args.output) == (2048, 7, "artifacts/benchmark.json")
    assert args.profile == "configs/benchmark-sharegpt.yaml" and args.model is None and args.device == "auto"
    args = parse(["benchmark", "--config", "static", "--policy", "sjf", "--requests", "5",
                                      "--arrival-rate", "3.5", "--prefill-chunk-size", "64"])
    assert (args.config, args.policy, args.requests, args.arrival_rate, args.prefill_chunk_size) == ("static", "sjf", 5, 3.5, 64)
    with pytest.raises(SystemExit):
        parse(["benchmark", "--config", "speculative"])
    with pytest.raises(SystemExit):
        parse(["benchmark", "--linear-backend", "triton-int8"])     # a part this engine does not have
    args = parse(["generate", "--prompt-ids", "1 2 3", "--prompt-ids", "4,5", "--temperature", "0.8",
                                      "--dtype", "float32", "--random", "small"])
    assert args.prompt_ids == ["1 2 3", "4,5"] and args.temperature == 0.8 and args.dtype == "float32" and args.random == "small"
    args = parse(["replay", "--model", "m", "--out", "o", "--max-tokens", "64"])
    assert args.rest == ["--model", "m", "--out", "o", "--max-tokens", "64"]


def test_the_stand_in_model_is_a_configuration_of_the_architecture():
    from llm_serving_engine_b200.config import load_config

    _, config, spec = load_config(tiny_config())
    assert (config.hidden_size, config.num_hidden_layers, spec.vocab_size) == (128, 4, 260)
    text = "héllo"
    tokenizer = ByteTokenizer()
    ids = tokenizer.encode(text)
    assert min(ids) >= 4 and max(ids) < tokenizer.vocab_size and tokenizer.decode(ids) == text


def test_traffic_is_fixed_by_the_seed_and_keeps_its_ranges(tmp_path):
    profile = TrafficProfile(requests=200, arrival_rate=5.0, prompt=ClippedLogNormal(512, 1.0, 64, 4096),
                             output=ClippedLogNormal(200, 0.6, 128, 512), seed=3, vocabulary_size=1000)
    first, again = make_traffic(profile), make_traffic(profile)
    assert first == again and len(first) == 200
    lengths = sorted(len(item.prompt_token_ids) for item in first)
    assert lengths[0] >= 64 and lengths[-1] <= 4096 and 350 < lengths[100] < 750        # median near 512
    assert all(128 <= item.max_new_tokens <= 512 for item in first)
    assert all(4 <= token < 1000 for item in first for token in item.prompt_token_ids)
    arrivals = [item.arrives_at for item in first]
    assert arrivals[0] == 0.0 and arrivals == sorted(arrivals) and 20 < arrivals[-1] < 80   # 199 gaps of 0.2 s on average
    assert make_traffic(TrafficProfile(requests=3, seed=4)) != make_traffic(TrafficProfile(requests=3, seed=5))
    burst = make_traffic(TrafficProfile(requests=4, arrival_rate=0.0))
    assert [item.arrives_at for item in burst] == [0.0] * 4
    path = tmp_path / "profile.yaml"
    path.write_text("requests: 9\narrival_rate: 1.5\nseed: 11\nvocabulary_size: 300\n"
                    "prompt: {median: 20, sigma: 0.5, minimum: 2, maximum: 50}\noutput: {median: 6, sigma: 0.2, minimum: 1, maximum: 9}\n")
    loaded = TrafficProfile.from_file(path)
    assert (loaded.requests, loaded.arrival_rate, loaded.seed, loaded.prompt.maximum, loaded.output.median) == (9, 1.5, 11, 50, 6)
    fitted = loaded.fitted_to(260, 40)
    assert fitted.vocabulary_size == 260 and fitted.prompt.maximum == 31       # 40 positions less 9 output tokens


def test_replayed_traffic_is_timed_per_request_and_failures_keep_their_row():
    traffic = make_traffic(TrafficProfile(requests=4, arrival_rate=0.0, prompt=ClippedLogNormal(5, 0.1, 2, 9),
                                          output=ClippedLogNormal(3, 0.1, 2, 4), vocabulary_size=50))

    async def generate(item, on_token):
        if item.request_id.endswith("2"):
            raise RuntimeError("no room")
        for token in range(item.max_new_tokens):
            await asyncio.sleep(0.001)
            on_token(token)

    result = asyncio.run(replay_traffic("test", traffic, generate))
    assert [row.request_id for row in result.rows] == [item.request_id for item in traffic]
    assert result.rows[2].error == "RuntimeError: no room" and result.rows[2].output_tokens == 0
    good = [row for row in result.rows if row.error is None]
    assert all(row.output_tokens == item.max_new_tokens for row, item in zip(result.rows, traffic) if row.error is None)
    assert all(row.first_token >= row.arrived and row.ended >= row.first_token for row in good)
    summary = summarise(result)
    assert summary["requests"] == 4 and summary["successful_requests"] == 3 and summary["throughput_tokens_per_s"] > 0
    assert 0 < summary["ttft_ms_p50"] <= summary["e2e_ms_p99"] and summary["tpot_ms_p95"] > 0
    assert set(result.as_dict()) == {"summary", "metadata", "requests"}
    assert summarise(TrafficResult("empty", 1.0, []))["ttft_ms_p50"] == 0.0
