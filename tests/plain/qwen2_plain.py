"""Plain, slow, whole-sequence implementation of the Qwen2-style dense decoder.

It is the oracle of the test suite: no cache, no batching, no kernels, one
function per part, float32 (or float64) torch ops on the CPU.  It shares no
code with the engine package: it reads ``config.json`` and the safetensors
file by itself and takes every constant from the configuration dictionary.

Each function restates a formula of the reference project
(Arnavsharma2/llm-serving-engine); the citation gives the file and the lines of
that project where the formula stands.  ``tests/golden/make_golden.py`` compares
this file once with the reference's own ``Transformer.forward`` on tiny random
models and commits the logits.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """h0 = embed_tokens.weight[token_ids]   (src/llmserve/model.py:243,265)."""
    return table[token_ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """variance = mean(x^2); y = (x * rsqrt(variance + eps)) * weight
    (src/llmserve/model.py:20-23)."""
    variance = x.pow(2).mean(-1, keepdim=True)
    return (x * torch.rsqrt(variance + eps)) * weight


def rope_inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
    """inv_i = 1 / theta^(2i / D), i in [0, D/2), in float32
    (src/llmserve/model.py:29)."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, pairing: str = "interleaved") -> torch.Tensor:
    """Rotate ``x`` [S, heads, D] by the angle position * inv_i.

    ``interleaved`` pairs (2i, 2i+1), as the reference does
    (src/llmserve/model.py:35-43):
        out[2i]   = x[2i]   * cos_i - x[2i+1] * sin_i
        out[2i+1] = x[2i+1] * cos_i + x[2i]   * sin_i
    ``half`` pairs (i, i + D/2) with the same angles; the reference has no
    such mode, it is the engine's own option and is written here likewise.
    """
    head_dim = x.shape[-1]
    inverse = rope_inverse_frequencies(head_dim, theta)
    angles = torch.outer(positions.float(), inverse)  # model.py:30-31
    cos = angles.cos().to(x.dtype)[:, None, :]
    sin = angles.sin().to(x.dtype)[:, None, :]
    out = torch.empty_like(x)
    if pairing == "interleaved":
        even, odd = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = even * cos - odd * sin
        out[..., 1::2] = odd * cos + even * sin
    elif pairing == "half":
        half = head_dim // 2
        first, second = x[..., :half], x[..., half:]
        out[..., :half] = first * cos - second * sin
        out[..., half:] = second * cos + first * sin
    else:
        raise ValueError(pairing)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ W^T (+ b); W is [out, in] as nn.Linear keeps it
    (src/llmserve/model.py:51-66,183-185)."""
    y = x @ weight.t()
    if bias is not None:
        y = y + bias
    return y


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Causal softmax attention with grouped key/value heads.

    q [S, Hq, D], k and v [S, Hkv, D].  Query head h reads key/value head
    h // (Hq / Hkv) (``repeat_interleave``, src/llmserve/model.py:84-86);
    scores = q.k / sqrt(D) for keys j <= i, softmax over j, out = sum p_j v_j
    (src/llmserve/model.py:88-95; the paged form, model.py:143-176, is the same
    sum computed block by block).
    """
    seq, n_q, head_dim = q.shape
    n_kv = k.shape[1]
    group = n_q // n_kv
    scale = 1.0 / math.sqrt(head_dim)
    out = torch.empty_like(q)
    mask = torch.ones(seq, seq, dtype=torch.bool).tril()
    for head in range(n_q):
        kv_head = head // group
        scores = (q[:, head, :] @ k[:, kv_head, :].t()) * scale
        scores = scores.masked_fill(~mask, float("-inf"))
        probabilities = torch.softmax(scores, dim=-1)
        out[:, head, :] = probabilities @ v[:, kv_head, :]
    return out


def attention_block(x, positions, w, prefix, cfg):
    """q/k/v projections with bias, RoPE on q and k, causal attention, o_proj
    without bias (src/llmserve/model.py:71-95)."""
    n_q = cfg["num_attention_heads"]
    n_kv = cfg["num_key_value_heads"]
    head_dim = cfg.get("head_dim") or cfg["hidden_size"] // n_q
    seq = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).view(seq, n_q, head_dim)
    k = linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).view(seq, n_kv, head_dim)
    v = linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).view(seq, n_kv, head_dim)
    theta = float(cfg.get("rope_theta", 10000.0))
    pairing = cfg.get("rope_pairing", "interleaved")
    q = rope(q, positions, theta, pairing)
    k = rope(k, positions, theta, pairing)
    out = causal_attention(q, k, v).reshape(seq, n_q * head_dim)
    return linear(out, w[prefix + "o_proj.weight"])


def swiglu(x, w, prefix):
    """down(silu(gate(x)) * up(x)), no biases (src/llmserve/model.py:180-188)."""
    gate = linear(x, w[prefix + "gate_proj.weight"])
    up = linear(x, w[prefix + "up_proj.weight"])
    return linear(torch.nn.functional.silu(gate) * up, w[prefix + "down_proj.weight"])


def decoder_layer(h, positions, w, index, cfg):
    """h = h + attn(norm1(h)); h = h + mlp(norm2(h))   (src/llmserve/model.py:199-201)."""
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    base = f"model.layers.{index}."
    h = h + attention_block(rms_norm(h, w[base + "input_layernorm.weight"], eps), positions, w,
                            base + "self_attn.", cfg)
    h = h + swiglu(rms_norm(h, w[base + "post_attention_layernorm.weight"], eps), w, base + "mlp.")
    return h


def forward_full(cfg: dict, w: dict, token_ids) -> torch.Tensor:
    """Logits [S, V] of one whole sequence: embed, layers in order, final norm,
    LM head that is the embedding matrix when ``tie_word_embeddings``
    (src/llmserve/model.py:249-250,260-268)."""
    token_ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(token_ids.shape[0])
    h = embedding(w["model.embed_tokens.weight"], token_ids)
    for index in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, positions, w, index, cfg)
    h = rms_norm(h, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-6)))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", True) else w["lm_head.weight"]
    return linear(h, head)


# --------------------------------------------------------------------------- loading
def load_folder(folder, weight_dtype: torch.dtype | None = None, compute_dtype=torch.float32):
    """Read config.json and every safetensors file of ``folder``.

    ``weight_dtype`` rounds the matrices first (for instance to bfloat16, the
    way a bfloat16 engine holds them) before they are widened to
    ``compute_dtype``; vectors (norm weights, biases) are widened only.
    """
    from safetensors import safe_open

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights: dict[str, torch.Tensor] = {}
    for filename in sorted(folder.glob("*.safetensors")):
        with safe_open(str(filename), framework="pt", device="cpu") as source:
            for name in source.keys():
                tensor = source.get_tensor(name)
                if weight_dtype is not None and tensor.ndim >= 2:
                    tensor = tensor.to(weight_dtype)
                weights[name] = tensor.to(compute_dtype)
    return cfg, weights


def greedy_generate(cfg: dict, w: dict, prompt, max_new_tokens: int) -> list[int]:
    """Recompute the whole prefix for every new token and take the argmax
    (NaiveDecoder, src/llmserve/engine.py:83-105)."""
    tokens = list(prompt)
    out: list[int] = []
    for _ in range(max_new_tokens):
        logits = forward_full(cfg, w, tokens)[-1]
        token = int(logits.argmax())
        out.append(token)
        tokens.append(token)
    return out
