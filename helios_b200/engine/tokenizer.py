"""Tokenizers: the byte-level one that random model folders carry, or the
folder's own tokenizer files through ``transformers.AutoTokenizer`` (tokenizer
only; python/helios/engine.py:242-250).  Token-id APIs work without any."""
from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional


class ByteTokenizer:
    """Ids 0..2 are <pad>, <s>, </s>; byte b is id ``first_byte_id + b`` while it is
    inside the vocabulary, else <pad>."""

    def __init__(self, spec: dict) -> None:
        self.vocab_size = int(spec["vocab_size"])
        self.pad, self.bos, self.eos = int(spec["pad"]), int(spec["bos"]), int(spec["eos"])
        self.first = int(spec["first_byte_id"])
        self.eos_token_id = self.eos if self.eos < self.vocab_size else None

    def encode(self, text: str) -> List[int]:
        ids = []
        for b in text.encode("utf-8"):
            i = self.first + b
            ids.append(i if i < self.vocab_size else self.pad)
        return ids

    def decode(self, ids: List[int]) -> str:
        data = bytes(i - self.first for i in ids if self.first <= i < self.first + 256)
        return data.decode("utf-8", errors="replace")


def load_tokenizer(folder) -> Optional[object]:
    folder = Path(folder)
    spec = folder / "byte_tokenizer.json"
    if spec.exists():
        with open(spec, "r", encoding="utf-8") as f:
            return ByteTokenizer(json.load(f))
    if (folder / "tokenizer.json").exists() or (folder / "tokenizer_config.json").exists():
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(str(folder))
    return None
