"""Weight loading errors and the random-weights mode (no GPU)."""
import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from llm_serving_engine_b200.config import load_config
from llm_serving_engine_b200.models import expected_tensors
from llm_serving_engine_b200.weights import WeightError, load_weights, write_random_model
from tiny_configs import TINY_A, TINY_B


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    write_random_model(tmp_path, TINY_A, seed=3, dtype="float32")
    assert json.loads((tmp_path / "config.json").read_text())["hidden_size"] == 64
    tensors = load_file(str(tmp_path / "model.safetensors"))
    _, _, spec = load_config(tmp_path)
    assert set(tensors) == set(expected_tensors(spec))
    norm = tensors["model.layers.0.input_layernorm.weight"]
    assert 0.9 <= float(norm.min()) and float(norm.max()) <= 1.1 and float(norm.std()) > 0.01
    assert 0.015 < float(tensors["model.embed_tokens.weight"].std()) < 0.025
    assert float(tensors["model.layers.1.self_attn.k_proj.bias"].abs().max()) > 0  # biases are not zero


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    write_random_model(tmp_path / "a", TINY_B, seed=5, dtype="float32")
    write_random_model(tmp_path / "b", TINY_B, seed=5, dtype="float32")
    write_random_model(tmp_path / "c", TINY_B, seed=6, dtype="float32")
    a, b, c = (load_file(str(tmp_path / name / "model.safetensors")) for name in "abc")
    assert all(torch.equal(a[name], b[name]) for name in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    # the same tensor in a model with fewer layers has the same values
    write_random_model(tmp_path / "d", {**TINY_B, "num_hidden_layers": 1}, seed=5, dtype="float32")
    d = load_file(str(tmp_path / "d" / "model.safetensors"))
    assert torch.equal(a["model.layers.0.mlp.up_proj.weight"], d["model.layers.0.mlp.up_proj.weight"])


def test_how_tensors_are_held(tmp_path):
    write_random_model(tmp_path, TINY_A, seed=0, dtype="bfloat16")
    stored = load_file(str(tmp_path / "model.safetensors"))
    assert stored["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert stored["model.norm.weight"].dtype == torch.float32      # stored in 32-bit
    _, _, spec = load_config(tmp_path)
    held = load_weights(tmp_path, expected_tensors(spec), torch.bfloat16, "cpu")
    assert held["model.layers.0.mlp.gate_proj.weight"].dtype == torch.bfloat16
    assert held["model.norm.weight"].dtype == torch.float32        # and stays so
    assert held["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    wide = load_weights(tmp_path, expected_tensors(spec), torch.float32, "cpu")
    assert wide["model.embed_tokens.weight"].dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    write_random_model(tmp_path, TINY_A, seed=0, dtype="float32")
    path = str(tmp_path / "model.safetensors")
    tensors = load_file(path)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    save_file(tensors, path)
    _, _, spec = load_config(tmp_path)
    with pytest.raises(WeightError) as info:
        load_weights(tmp_path, expected_tensors(spec), torch.float32, "cpu")
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.0.extra.weight"]
    assert error.wrong_shapes == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    text = str(error)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[16, 64]", "[32, 64]"):
        assert piece in text


def test_no_safetensors_and_a_repeated_tied_head(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    _, _, spec = load_config(tmp_path)
    with pytest.raises(FileNotFoundError):
        load_weights(tmp_path, expected_tensors(spec), torch.float32, "cpu")
    write_random_model(tmp_path, TINY_A, seed=0, dtype="float32")
    path = str(tmp_path / "model.safetensors")
    tensors = load_file(path)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, path)
    with pytest.raises(WeightError):
        load_weights(tmp_path, expected_tensors(spec), torch.float32, "cpu")
    held = load_weights(tmp_path, expected_tensors(spec), torch.float32, "cpu", optional=frozenset({"lm_head.weight"}))
    assert "lm_head.weight" not in held
