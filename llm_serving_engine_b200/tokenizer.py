"""The byte tokenizer of the reference (``src/llmserve/tokenizer.py:15-28``): the engine
works on token ids; this turns text into ids for the command line's demo model.
Text tokenizers of real checkpoints are outside this engine: it takes token ids."""
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
