"""The ``llmserve`` command line, in the reference's manner (``src/llmserve/cli.py``).

``benchmark`` keeps the reference's option names and meanings (``cli.py:248-275``);
options of parts this engine does not have (the HTTP service, quantized linear
layers, the choice of an attention backend, rebuilt device metadata) are left
out.  ``generate`` is this engine's own: ids in, ids out.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import sys
from dataclasses import replace
from pathlib import Path


def tiny_config(vocab_size: int = 260) -> dict:
    """The bundled demo model of the reference (``ModelConfig.tiny``, ``src/llmserve/config.py:34-44``)."""
    return {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab_size,
        "hidden_size": 128, "intermediate_size": 352, "num_hidden_layers": 4, "num_attention_heads": 4,
        "num_key_value_heads": 2, "max_position_embeddings": 1024, "rope_theta": 10000.0,
        "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": True,
    }


def _device(name: str) -> str:
    import torch

    if name in ("auto", "cuda") or name.startswith("cuda:"):
        if not torch.cuda.is_available():
            raise SystemExit("llmserve: no CUDA device; this engine has no CPU path")
        return "cuda" if name == "auto" else name
    raise SystemExit(f"llmserve: device {name!r} is not supported; this engine runs on CUDA only")


def _load_runtime(args):
    from .models import load_model, random_model
    from .tokenizer import ByteTokenizer, HuggingFaceTokenizer

    device = _device(args.device)
    if args.model:
        model = load_model(args.model, dtype=args.dtype, device=device)
        try:
            tokenizer = HuggingFaceTokenizer(args.model)
        except Exception:
            tokenizer = None  # a folder without tokenizer files still serves token ids
    else:
        tokenizer = ByteTokenizer()
        model = random_model(tiny_config(tokenizer.vocab_size), args.seed, dtype=args.dtype, device=device)
    return model, tokenizer


class NaiveDecoder:
    """Sequential baseline: recompute the whole prefix for every token
    (``src/llmserve/engine.py:75-105``), through the same step function."""

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
        self._lock = asyncio.Lock()

    async def generate(self, prompt_token_ids, config, callback=None) -> list[int]:
        from .engine.step import StepEntry

        async with self._lock:
            output: list[int] = []
            for _ in range(config.max_new_tokens):
                tokens = list(prompt_token_ids) + output
                self.cache.create("naive")
                try:
                    logits = self.runner.run([StepEntry("naive", tokens, [len(tokens) - 1])])
                    token = self.sampler.sample(logits, [config], [len(output)])[0]
                finally:
                    self.cache.free("naive")
                output.append(token)
                if callback:
                    callback(token)
                if token in config.stop_token_ids:
                    break
                await asyncio.sleep(0)
            return output


async def _benchmark(args) -> None:
    from .config.runtime_config import CacheConfig, SchedulerConfig
    from .engine.llm_engine import LLMEngine
    from .sampling.sampler import GenerationConfig
    from .workload import LoadProfile, run_open_loop

    model, tokenizer = _load_runtime(args)
    profile = LoadProfile.from_yaml(args.profile) if args.profile and Path(args.profile).exists() else LoadProfile()
    limit = model.spec.max_position_embeddings
    profile = replace(
        profile,
        requests=args.requests or profile.requests,
        arrival_rate=args.arrival_rate or profile.arrival_rate,
        vocabulary_size=model.vocab_size,
        prompt=replace(profile.prompt, maximum=min(profile.prompt.maximum, limit - profile.output.maximum)),
    )

    def generation_for(spec):
        return GenerationConfig(max_new_tokens=spec.max_new_tokens, temperature=0.0, seed=args.seed)

    engine = None
    if args.config == "naive":
        decoder = NaiveDecoder(model)

        async def generate(spec, callback):
            return await decoder.generate(list(spec.prompt_token_ids), generation_for(spec), callback)
    else:
        engine = LLMEngine(
            model, tokenizer,
            cache_config=CacheConfig(block_size=args.block_size, num_blocks=args.num_blocks),
            scheduler_config=SchedulerConfig(max_batch_size=1 if args.config == "paged" else args.batch_size,
                                             max_tokens_per_step=args.max_tokens_per_step, policy=args.policy),
            scheduler_mode="static" if args.config == "static" else "continuous",
            prefill_chunk_size=args.prefill_chunk_size, collect_iteration_metrics=True)

        async def generate(spec, callback):
            return await engine.generate(list(spec.prompt_token_ids), generation_for(spec), callback,
                                         request_id=spec.request_id)

    report = await run_open_loop(f"{args.config}-{args.policy}", profile, generate)
    if engine:
        report.cache = engine.cache_stats
        report.metadata["engine"] = engine.iteration_stats
        await engine.close()
    output = Path(args.output)
    output.parent.mkdir(parents=True, exist_ok=True)
    output.write_text(json.dumps(report.to_dict(), indent=2) + "\n")
    print(json.dumps(report.summary, indent=2))


def _generate(args) -> None:
    from .config.runtime_config import CacheConfig, SchedulerConfig
    from .engine.llm_engine import LLMEngine
    from .sampling.sampler import GenerationConfig

    model, tokenizer = _load_runtime(args)
    prompts = []
    for text in args.prompt_ids or []:
        prompts.append([int(item) for item in text.replace(",", " ").split()])
    for text in args.prompt or []:
        if tokenizer is None:
            raise SystemExit("llmserve: --prompt needs a tokenizer; pass --prompt-ids")
        prompts.append(tokenizer.encode(text))
    if not prompts:
        raise SystemExit("llmserve generate: give --prompt-ids or --prompt")
    engine = LLMEngine(model, tokenizer,
                       cache_config=CacheConfig(block_size=args.block_size, num_blocks=args.num_blocks),
                       scheduler_config=SchedulerConfig(max_batch_size=args.batch_size,
                                                        max_tokens_per_step=args.max_tokens_per_step),
                       prefill_chunk_size=args.prefill_chunk_size)
    config = GenerationConfig(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_p=args.top_p,
                              seed=args.seed, stop_token_ids=tuple(args.stop_token_ids or ()))
    for prompt, output in zip(prompts, engine.generate_many(prompts, config)):
        record = {"prompt_ids": prompt, "output_ids": output}
        if tokenizer is not None:
            record["text"] = tokenizer.decode(output)
        print(json.dumps(record))


def _engine_options(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--model", help="folder with config.json and safetensors (default: a random tiny model)")
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
    benchmark = commands.add_parser("benchmark", help="run the open-loop workload harness")
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
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "benchmark":
        asyncio.run(_benchmark(args))
    else:
        _generate(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
