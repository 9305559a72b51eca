"""The ``llmserve`` command line.

``benchmark`` has the option names and meanings of the reference's subcommand
(``src/llmserve/cli.py:244-316``): ``--config {naive,paged,static,continuous}``, ``--policy``,
``--profile``, ``--model``, ``--device``, ``--requests``, ``--arrival-rate``, ``--batch-size``,
``--block-size``, ``--num-blocks``, ``--prefill-chunk-size``, ``--max-tokens-per-step``, ``--seed``,
``--output``.  Options of parts this engine does not have are absent (the HTTP service, quantized
linear layers, a choice of attention backend, rebuilt device metadata).  ``generate`` (token ids in,
token ids out) and ``replay`` (the trace replay program) are this engine's own.

Without ``--model`` a small random model stands in, as in the reference (``cli.py:39-41``);
``--random NAME`` picks which one (``tiny`` is the reference's bundled demo size).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import sys
from pathlib import Path

# Random stand-in models by name: config.json contents of the architecture, sizes only.
RANDOM_MODELS = {
    # the reference's ModelConfig.tiny (src/llmserve/config.py:34-44) over the byte tokenizer's vocabulary
    "tiny": dict(vocab_size=260, hidden_size=128, intermediate_size=352, num_hidden_layers=4, num_attention_heads=4,
                 num_key_value_heads=2, max_position_embeddings=1024, rope_theta=10000.0, rms_norm_eps=1e-6),
    "small": dict(vocab_size=4096, hidden_size=512, intermediate_size=1376, num_hidden_layers=8, num_attention_heads=8,
                  num_key_value_heads=2, max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-6),
}


def tiny_config(vocab_size: int = 260, name: str = "tiny") -> dict:
    """config.json of a random stand-in model."""
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "attention_bias": True,
            "tie_word_embeddings": True, **RANDOM_MODELS[name], "vocab_size": vocab_size}


class _Runtime:
    """What the subcommands share: the model, a tokenizer if text can be handled, engine settings."""

    def __init__(self, args) -> None:
        import torch

        from .models import load_model, random_model
        from .tokenizer import ByteTokenizer

        if args.device not in ("auto", "cuda") and not args.device.startswith("cuda:"):
            raise SystemExit(f"llmserve: device {args.device!r}: this engine runs on CUDA devices only")
        if not torch.cuda.is_available():
            raise SystemExit("llmserve: no CUDA device; this engine has no CPU path")
        device = "cuda" if args.device == "auto" else args.device
        self.args = args
        if args.model:
            self.model = load_model(args.model, dtype=args.dtype, device=device)
            self.tokenizer = None        # a model folder is served by token ids; text tokenizers are outside this engine
        else:
            self.tokenizer = ByteTokenizer()
            vocab = max(self.tokenizer.vocab_size, RANDOM_MODELS[args.random]["vocab_size"])
            self.model = random_model(tiny_config(vocab, args.random), args.seed, dtype=args.dtype, device=device)

    def engine(self, *, batch_size=None, mode="continuous", policy="fcfs", metrics=False):
        from .config.runtime_config import CacheConfig, SchedulerConfig
        from .engine.llm_engine import LLMEngine

        args = self.args
        return LLMEngine(self.model, self.tokenizer,
                         cache_config=CacheConfig(block_size=args.block_size, num_blocks=args.num_blocks),
                         scheduler_config=SchedulerConfig(max_batch_size=batch_size or args.batch_size,
                                                          max_tokens_per_step=args.max_tokens_per_step, policy=policy),
                         scheduler_mode=mode, prefill_chunk_size=args.prefill_chunk_size,
                         collect_iteration_metrics=metrics)


class NaiveDecoder:
    """The sequential baseline of ``--config naive``: every token recomputes its whole prefix
    (``src/llmserve/engine.py:75-105``), here as one whole-prompt step of the same step function."""

    def __init__(self, model) -> None:
        from .cache.manager import CacheManager
        from .config.runtime_config import CacheConfig
        from .engine.step import StepRunner
        from .models import cache_requirements
        from .sampling.sampler import Sampler

        limit = model.spec.max_position_embeddings
        self.cache = CacheManager(cache_requirements(model.spec), CacheConfig(16, -(-limit // 16)), model.dtype,
                                  model.device, limit, num_state_slots=1)
        self.runner = StepRunner(model, self.cache, limit, 1)
        self.sampler = Sampler(model.vocab_size, 1, model.device)
        self._turn = asyncio.Lock()

    async def generate(self, prompt_token_ids, config, callback=None) -> list[int]:
        from .engine.step import StepEntry

        produced: list[int] = []
        async with self._turn:
            while len(produced) < config.max_new_tokens:
                prefix = [*prompt_token_ids, *produced]
                self.cache.create("naive")
                try:
                    logits = self.runner.run([StepEntry("naive", prefix, [len(prefix) - 1])])
                    token = self.sampler.sample(logits, [config], [len(produced)])[0]
                finally:
                    self.cache.free("naive")
                produced.append(token)
                if callback is not None:
                    callback(token)
                if token in config.stop_token_ids:
                    break
                await asyncio.sleep(0)
        return produced


def run_benchmark(args) -> dict:
    """``llmserve benchmark``: synthetic traffic of the profile against one of four serving set-ups."""
    from .sampling.sampler import GenerationConfig
    from .workload import TrafficProfile, make_traffic, replay_traffic, summarise

    runtime = _Runtime(args)
    model = runtime.model
    profile = TrafficProfile.from_file(args.profile) if args.profile and Path(args.profile).exists() else TrafficProfile()
    overrides = {key: value for key, value in (("requests", args.requests), ("arrival_rate", args.arrival_rate)) if value}
    profile = TrafficProfile(**{**vars(profile), **overrides}).fitted_to(model.vocab_size, model.spec.max_position_embeddings)
    traffic = make_traffic(profile)

    def sampling(item):
        return GenerationConfig(max_new_tokens=item.max_new_tokens, temperature=0.0, seed=args.seed)

    async def drive():
        if args.config == "naive":
            decoder = NaiveDecoder(model)
            return await replay_traffic(f"naive-{args.policy}", traffic, lambda item, on_token: decoder.generate(
                item.prompt_token_ids, sampling(item), on_token)), None
        engine = runtime.engine(batch_size=1 if args.config == "paged" else None, policy=args.policy, metrics=True,
                                mode="static" if args.config == "static" else "continuous")
        async with engine:
            result = await replay_traffic(f"{args.config}-{args.policy}", traffic, lambda item, on_token: engine.generate(
                list(item.prompt_token_ids), sampling(item), on_token, request_id=item.request_id))
            result.cache = engine.cache_stats
            result.extra["engine"] = engine.iteration_stats
        return result, engine

    result, _ = asyncio.run(drive())
    result.extra["profile"] = {**{k: v for k, v in vars(profile).items() if k not in ("prompt", "output")},
                               "prompt": vars(profile.prompt), "output": vars(profile.output)}
    target = Path(args.output)
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_text(json.dumps(result.as_dict(), indent=2) + "\n")
    summary = summarise(result)
    print(json.dumps(summary, indent=2))
    return summary


def run_generate(args) -> list[dict]:
    """``llmserve generate``: one JSON line per prompt with its ids and the generated ids."""
    from .sampling.sampler import GenerationConfig

    runtime = _Runtime(args)
    prompts = [[int(item) for item in text.replace(",", " ").split()] for text in args.prompt_ids or []]
    for text in args.prompt or []:
        if runtime.tokenizer is None:
            raise SystemExit("llmserve generate: --prompt needs a tokenizer (the random model has one); give --prompt-ids")
        prompts.append(runtime.tokenizer.encode(text))
    if not prompts:
        raise SystemExit("llmserve generate: give --prompt-ids or --prompt")
    sampling = GenerationConfig(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_p=args.top_p,
                                seed=args.seed, stop_token_ids=tuple(args.stop_token_ids or ()))
    records = []
    for prompt, output in zip(prompts, runtime.engine().generate_many(prompts, sampling)):
        record = {"prompt_ids": prompt, "output_ids": output}
        if runtime.tokenizer is not None:
            record["text"] = runtime.tokenizer.decode(output)
        print(json.dumps(record))
        records.append(record)
    return records


def _engine_options(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--model", help="folder with config.json and safetensors (default: a random stand-in model)")
    parser.add_argument("--random", choices=sorted(RANDOM_MODELS), default="tiny", help="which random stand-in model")
    parser.add_argument("--device", default="auto")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--batch-size", type=int, default=16)
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-blocks", type=int, default=1024)
    parser.add_argument("--prefill-chunk-size", type=int, default=2048)
    parser.add_argument("--max-tokens-per-step", type=int, default=2048)
    parser.add_argument("--seed", type=int, default=7)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="llmserve")
    commands = parser.add_subparsers(dest="command", required=True)
    benchmark = commands.add_parser("benchmark", help="synthetic traffic against the engine; latency and throughput report")
    benchmark.add_argument("--config", choices=("naive", "paged", "static", "continuous"), default="continuous")
    benchmark.add_argument("--policy", choices=("fcfs", "sjf", "priority"), default="fcfs")
    benchmark.add_argument("--profile", default="configs/benchmark-sharegpt.yaml")
    benchmark.add_argument("--requests", type=int)
    benchmark.add_argument("--arrival-rate", type=float)
    benchmark.add_argument("--output", default="artifacts/benchmark.json")
    _engine_options(benchmark)
    generate = commands.add_parser("generate", help="generate token ids for given prompts")
    generate.add_argument("--prompt-ids", action="append", help="token ids, separated by spaces or commas")
    generate.add_argument("--prompt", action="append", help="text (needs a tokenizer)")
    generate.add_argument("--max-new-tokens", type=int, default=32)
    generate.add_argument("--temperature", type=float, default=0.0)
    generate.add_argument("--top-p", type=float, default=1.0)
    generate.add_argument("--stop-token-ids", type=int, nargs="*")
    _engine_options(generate)
    replay = commands.add_parser("replay", help="trace replay: steps of token ids from standard input, logits to files "
                                                "(the same program as bin/trace_run)")
    replay.description = "every option after `replay` goes to trace_run: --model --dtype --out --max-tokens"
    return parser


def parse(argv=None):
    """Arguments of the command line; ``rest`` holds what follows ``replay`` (trace_run's own options)."""
    parser = build_parser()
    args, rest = parser.parse_known_args(argv)
    if rest and args.command != "replay":
        parser.error("unrecognized arguments: " + " ".join(rest))
    args.rest = rest
    return args


def main(argv=None) -> int:
    args = parse(argv)
    if args.command == "benchmark":
        run_benchmark(args)
    elif args.command == "generate":
        run_generate(args)
    else:
        from .engine.trace_replay import main as replay_main
        return replay_main(args.rest)
    return 0


if __name__ == "__main__":
    sys.exit(main())
