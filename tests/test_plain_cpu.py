"""The plain implementation itself (no GPU): against the logits of the reference's
own model code stored under tests/golden, and against simple identities."""
import math
import os

import numpy as np
import pytest
import torch

from plain import qwen2_plain
from tiny_configs import ALL

from llm_serving_engine_b200.weights import write_random_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_model_code(name, tmp_path):
    config, _, seed = ALL[name]
    write_random_model(tmp_path, config, seed, "float32")
    cfg, weights = qwen2_plain.load_folder(tmp_path)
    golden = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    logits = qwen2_plain.forward_full(cfg, weights, golden["tokens"])
    assert float((logits - torch.from_numpy(golden["logits"])).abs().max()) < 1e-5


def test_rms_norm_and_rope_identities():
    x = torch.randn(5, 24)
    y = qwen2_plain.rms_norm(x, torch.ones(24), 0.0)
    assert torch.allclose(y.pow(2).mean(-1), torch.ones(5), atol=1e-5)
    q = torch.randn(7, 3, 16)
    positions = torch.arange(7)
    for pairing in ("interleaved", "half"):
        rotated = qwen2_plain.rope(q, positions, 10000.0, pairing)
        assert torch.allclose(rotated.norm(dim=-1), q.norm(dim=-1), atol=1e-5)   # a rotation keeps lengths
        assert torch.allclose(rotated[0], q[0], atol=1e-6)                       # position 0 turns nothing
    # the score of two rotated vectors depends on their distance only
    a, b = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    def score(pa, pb):
        ra = qwen2_plain.rope(a, torch.tensor([pa]), 10000.0)
        rb = qwen2_plain.rope(b, torch.tensor([pb]), 10000.0)
        return float((ra * rb).sum())
    assert math.isclose(score(3, 10), score(20, 27), rel_tol=1e-4, abs_tol=1e-5)


def test_causal_attention_reads_no_later_key_and_groups_heads():
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = qwen2_plain.causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0
    assert torch.allclose(out[:4], qwen2_plain.causal_attention(q, k2, v2)[:4])
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])  # heads 0,1 -> group 0; 2,3 -> 1
