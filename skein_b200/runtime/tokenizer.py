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


class IncrementalDecoder:
    """Text of a token stream, piece by piece. Decoding tokens one at a time loses what only shows between tokens (the
    space a sentencepiece token carries in front, a character whose bytes are spread over several tokens), so each piece
    is the difference between two decodes of a short window: the tokens since the last emitted piece with and without
    the new ones. A piece that would end in the middle of a character is held back until the character is complete."""

    def __init__(self, tokenizer: Tokenizer):
        self.tok = tokenizer
        self.ids: list[int] = []
        self.prefix_off = 0      # start of the decode window
        self.read_off = 0        # tokens before this index have been emitted

    def push(self, token: int) -> str:
        self.ids.append(int(token))
        before = self.tok.decode(self.ids[self.prefix_off:self.read_off])
        now = self.tok.decode(self.ids[self.prefix_off:])
        if len(now) > len(before) and not now.endswith("\ufffd"):
            self.prefix_off, self.read_off = self.read_off, len(self.ids)
            return now[len(before):]
        return ""
