"""Anchors the plain implementation on the reference's own model code.

Run once, on the CPU, where the reference project is readable:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

It writes the tiny configurations' random weights (the engine's random-weights
mode), loads the same tensors into the reference's ``llmserve.model.Transformer``
(``load_state_dict``; names match after the ``model.`` prefix is stripped, and a
tied head shares the embedding), runs ``Transformer.forward`` in float32,
checks that ``tests/plain/qwen2_plain.py`` gives the same logits and stores
tokens and logits in ``tests/golden/tiny_<name>.npz``.  ``test_plain_cpu.py``
then checks the plain implementation against these files without needing the
reference.  Configuration C is left out: the reference has neither a free head
size nor half-split rotary pairs.
"""
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from plain import qwen2_plain  # noqa: E402
from tiny_configs import ALL  # noqa: E402

from llm_serving_engine_b200.weights import write_random_model  # noqa: E402


def main() -> None:
    from llmserve.config import ModelConfig
    from llmserve.model import Transformer

    for name in ("A", "B"):
        config, _, seed = ALL[name]
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(folder, config, seed, "float32")
            cfg, weights = qwen2_plain.load_folder(folder)
        model = Transformer(ModelConfig.from_dict(config)).eval()
        state = {key.removeprefix("model."): value for key, value in weights.items()}
        if config["tie_word_embeddings"]:
            state["lm_head.weight"] = state["embed_tokens.weight"]
        model.load_state_dict(state, strict=True)
        generator = torch.Generator().manual_seed(100 + seed)
        tokens = torch.randint(0, config["vocab_size"], (24,), generator=generator)
        with torch.no_grad():
            reference = model(tokens[None])[0]
        plain = qwen2_plain.forward_full(cfg, weights, tokens)
        error = float((plain - reference).abs().max())
        print(f"tiny {name}: max |plain - reference| = {error:.3e}")
        assert error < 1e-5, error
        np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), tokens=tokens.numpy(),
                            logits=reference.numpy().astype(np.float32))


if __name__ == "__main__":
    main()
