"""Whitespace word-level tokenizer built from a corpus or a vocabulary list; used by tests and offline fixtures."""
from __future__ import annotations

import hashlib
import json

from .base import BaseTokenizer


class WhitespaceTokenizer(BaseTokenizer):
    SPECIALS = ["<pad>", "<unk>", "<bos>", "<eos>", "<|im_start|>", "<|im_end|>"]

    def __init__(self, vocab: list[str]):
        self.itos = list(dict.fromkeys(self.SPECIALS + list(vocab)))
        self.stoi = {w: i for i, w in enumerate(self.itos)}
        self.pad_id, self.unk_id, self.bos_id, self.eos_id = 0, 1, 2, 3

    @classmethod
    def from_texts(cls, texts, max_vocab: int = 50000) -> "WhitespaceTokenizer":
        freq: dict[str, int] = {}
        for t in texts:
            for w in t.split():
                freq[w] = freq.get(w, 0) + 1
        words = [w for w, _ in sorted(freq.items(), key=lambda kv: (-kv[1], kv[0]))][:max_vocab]
        return cls(words)

    @classmethod
    def from_file(cls, path: str) -> "WhitespaceTokenizer":
        with open(path) as f:
            return cls(json.load(f)["vocab"])

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"vocab": [w for w in self.itos if w not in self.SPECIALS]}, f)

    def encode(self, text, add_bos=False, add_eos=False):
        ids = [self.stoi.get(w, self.unk_id) for w in text.replace("<|im_start|>", " <|im_start|> ").replace("<|im_end|>", " <|im_end|> ").split()]
        return ([self.bos_id] if add_bos else []) + ids + ([self.eos_id] if add_eos else [])

    def decode(self, ids):
        return " ".join(self.itos[i] for i in ids if 0 <= i < len(self.itos))

    @property
    def vocab_size(self):
        return len(self.itos)

    def identity(self):
        return "ws:" + hashlib.sha256("\n".join(self.itos).encode()).hexdigest()[:16]
