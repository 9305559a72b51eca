"""Tokenizers in the reference's manner (``src/llmserve/tokenizer.py``): the engine
works on token ids; these turn text into ids for the command line."""
from __future__ import annotations


class ByteTokenizer:
    """ids = byte + 4; 0/1/2 are pad/bos/eos; vocabulary 260."""

    pad_token_id = 0
    bos_token_id = 1
    eos_token_id = 2
    vocab_size = 260

    def encode(self, text: str) -> list[int]:
        return [byte + 4 for byte in text.encode("utf-8")]

    def decode(self, token_ids: list[int]) -> str:
        return bytes(token - 4 for token in token_ids if 4 <= token < 260).decode("utf-8", errors="replace")


class HuggingFaceTokenizer:
    """The tokenizer files of a model folder, through ``transformers.AutoTokenizer``
    (tokenization only; no model code of that package is used)."""

    def __init__(self, model_path: str) -> None:
        from transformers import AutoTokenizer

        self.inner = AutoTokenizer.from_pretrained(model_path, trust_remote_code=False)
        self.eos_token_id = int(self.inner.eos_token_id)
        self.vocab_size = int(self.inner.vocab_size)

    def encode(self, text: str) -> list[int]:
        return list(self.inner.encode(text, add_special_tokens=False))

    def decode(self, token_ids: list[int]) -> str:
        return self.inner.decode(token_ids, skip_special_tokens=True)
