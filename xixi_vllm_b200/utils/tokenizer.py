"""Tokenizer loading. A directory with Hugging Face tokenizer files gets ``AutoTokenizer``
(reference: src/control/engine.py:86-93); a synthetic model directory without them gets a
reversible byte-level stand-in so token-id workloads and tests need no tokenizer assets.
"""

from __future__ import annotations

import os

__all__ = ["ByteTokenizer", "load_tokenizer"]


class ByteTokenizer:
    """UTF-8 bytes shifted past a few reserved ids; ids outside that range decode to ``<id>``."""

    OFFSET = 3

    def __init__(self, vocab_size: int, eos_token_id: int | None = None) -> None:
        self.vocab_size = vocab_size
        self.eos_token_id = eos_token_id if eos_token_id is not None else min(2, vocab_size - 1)
        self.pad_token_id = self.eos_token_id
        self.pad_token = self.eos_token = "<eos>"

    def encode(self, text: str) -> list[int]:
        return [(b + self.OFFSET) % self.vocab_size for b in text.encode("utf-8")]

    def decode(self, ids) -> str:
        out, buf = [], bytearray()
        for i in ids:
            b = int(i) - self.OFFSET
            if 0 <= b < 256:
                buf.append(b)
            else:
                if buf:
                    out.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                out.append(f"<{int(i)}>")
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)


_TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "tokenizer.model")


def load_tokenizer(model_dir: str, vocab_size: int):
    if any(os.path.isfile(os.path.join(model_dir, f)) for f in _TOKENIZER_FILES):
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(model_dir, trust_remote_code=True)
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        return tok
    return ByteTokenizer(vocab_size)
