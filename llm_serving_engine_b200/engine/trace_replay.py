"""Trace replay: feeds given token ids through the model step by step and writes
logits.  It samples nothing and has no forward pass, cache or loader of its
own: it drives ``load_model``, ``CacheManager`` and ``StepRunner``, the ones
that generation uses.

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: for a step in which something is wanted, ``OUT/<step>.f32`` holds the
logits at the wanted places (order of the entries, then of ``want``) as
little-endian float32 [wanted, vocab]; after every step a line ``done <step>``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--out", required=True, help="folder the logits are written to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    parser.add_argument("--max-requests", type=int, default=8, help="most requests live at a time")
    return parser


def replay(model_dir, dtype: str, out_dir, max_tokens: int, lines, block_size: int = 16,
           max_requests: int = 8, report=None) -> None:
    import numpy as np
    import torch

    from ..cache.manager import CacheManager
    from ..config.runtime_config import CacheConfig
    from ..models import cache_requirements, load_model
    from .step import StepEntry, StepRunner

    if not torch.cuda.is_available():
        raise RuntimeError("trace_run needs a CUDA device: the engine has no CPU path")
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = load_model(model_dir, dtype=dtype, device="cuda")
    pages = max(1, math.ceil(max_tokens / block_size))
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(block_size=block_size, num_blocks=pages),
                         model.dtype, model.device, model.spec.max_position_embeddings,
                         num_state_slots=max_requests)
    runner = StepRunner(model, cache, max_tokens_per_step=max(max_tokens, 64), max_segments=max_requests)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        number = record["step"]
        entries = []
        for item in record.get("entries", []):
            request_id = str(item["id"])
            if request_id not in cache.requests:
                cache.create(request_id)
            entries.append(StepEntry(request_id, list(item["tokens"]), list(item.get("want", []))))
        if entries:
            logits = runner.run(entries)
            if logits.shape[0]:
                array = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                np.ascontiguousarray(array).tofile(out_dir / f"{number}.f32")
            else:
                torch.cuda.synchronize()
        for request_id in record.get("end", []):
            request_id = str(request_id)
            if request_id in cache.requests:
                cache.free(request_id)
        if report is not None:
            report(number)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)

    def report(number) -> None:
        sys.stdout.write(f"done {number}\n")
        sys.stdout.flush()

    replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, block_size=args.block_size,
           max_requests=args.max_requests, report=report)
    return 0


if __name__ == "__main__":
    sys.exit(main())
