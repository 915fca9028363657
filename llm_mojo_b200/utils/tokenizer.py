"""Decode-only GPT-2 tokenizer read from ``gpt2_tokenizer.bin`` (``llmm/tokenizer.mojo:70-157``).

File: 256×int32 header (magic 20240328 or 20240520, version 1|2, vocab size, [3]=EOT for v2)
followed by one length byte + raw bytes per token.  ``write_tokenizer`` emits the same file
(``train_gpt2.py:1633-1650``).
"""
from __future__ import annotations

import struct
from typing import List, Sequence

TOKENIZER_MAGIC = 20240520
TOKENIZER_MAGIC_LEGACY = 20240328
GPT2_VOCAB_SIZE = 50257
GPT2_EOT_TOKEN = 50256


class Tokenizer:
    def __init__(self, path: str | None = None):
        self.vocab_size = 0
        self.eot_token = GPT2_EOT_TOKEN
        self.token_table: List[bytes] = []
        self.has_initialized = False
        if path is not None:
            try:
                with open(path, "rb") as f:
                    self._load(f)
                self.has_initialized = True
            except FileNotFoundError:
                print("---\nWARNING: Failed to open the tokenizer file " + path)
                print("The Tokenizer is a new feature added April 14 2024.")
                print("Re-run `python train_gpt2.py` to write it\n---")

    def _load(self, f) -> None:
        raw = f.read(1024)
        if len(raw) < 1024:
            raise ValueError("Tokenizer error: header is too short")
        header = struct.unpack("<256i", raw)
        if header[0] not in (TOKENIZER_MAGIC, TOKENIZER_MAGIC_LEGACY):
            raise ValueError(f"Tokenizer error: bad magic number in header: {header[0]}")
        version = header[1]
        self.vocab_size = header[2]
        if version == 1:
            if self.vocab_size != GPT2_VOCAB_SIZE:
                raise ValueError(f"Tokenizer error: unexpected vocab size for version 1: {self.vocab_size}")
            self.eot_token = GPT2_EOT_TOKEN
        elif version == 2:
            self.eot_token = header[3]
        else:
            raise ValueError(f"Tokenizer error: bad version in header: {version}")
        table = []
        for _ in range(self.vocab_size):
            lb = f.read(1)
            if len(lb) < 1:
                raise ValueError("Tokenizer error: truncated token length byte")
            n = lb[0]
            if n <= 0:
                raise ValueError("Tokenizer error: token length must be positive")
            tok = f.read(n)
            if len(tok) < n:
                raise ValueError("Tokenizer error: truncated token bytes")
            table.append(tok)
        self.token_table = table

    def decode_bytes(self, token_id: int) -> bytes:
        if not self.has_initialized or token_id < 0 or token_id >= self.vocab_size:
            return b""
        return self.token_table[token_id]

    def decode(self, token_id: int) -> str:
        return self.decode_bytes(token_id).decode("utf-8", errors="replace")

    def decode_sequence(self, ids: Sequence[int]) -> str:
        return b"".join(self.decode_bytes(int(i)) for i in ids).decode("utf-8", errors="replace")


def write_tokenizer(path: str, tokens: Sequence[bytes], eot_token: int = GPT2_EOT_TOKEN) -> None:
    header = [0] * 256
    header[0], header[1], header[2], header[3] = TOKENIZER_MAGIC_LEGACY, 2, len(tokens), eot_token
    with open(path, "wb") as f:
        f.write(struct.pack("<256i", *header))
        for t in tokens:
            assert 0 < len(t) < 256
            f.write(bytes([len(t)]))
            f.write(t)
