"""Tokenizer: HuggingFace `tokenizers` from the artifact's tokenizer.json when present, else the
byte-mod-vocab fallback (each UTF-8 byte b becomes token b mod vocab), which is enough to drive a
random-weight model. Same two paths as the reference (crates/skein_runtime/src/tokenizer.rs:14-56;
fallback in crates/skein_parity/src/verify.rs:19 and server/forward.rs:592).
"""
from __future__ import annotations

from pathlib import Path


class Tokenizer:
    def __init__(self, vocab_size: int, tokenizer_json: str | Path | None = None):
        self.vocab_size = vocab_size
        self._tok = None
        if tokenizer_json is not None and Path(tokenizer_json).exists():
            from tokenizers import Tokenizer as HFTokenizer

            self._tok = HFTokenizer.from_file(str(tokenizer_json))

    @property
    def is_fallback(self) -> bool:
        return self._tok is None

    def encode(self, text: str) -> list[int]:
        if self._tok is not None:
            return list(self._tok.encode(text).ids)
        return [b % self.vocab_size for b in text.encode("utf-8")]

    def decode(self, ids) -> str:
        if self._tok is not None:
            return self._tok.decode(list(ids))
        return bytes(i % 256 for i in ids).decode("utf-8", errors="replace")
