"""Vocabulary shard bounds (reference: llmtuner/utils/vocabulary.py:4-40):
chunk = ceil(V/tp); rank r owns [min(V, r*chunk), min(V, start+chunk))."""
from __future__ import annotations


def vocab_shard_bounds(vocab_size: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    if tp_size < 1 or not 0 <= tp_rank < tp_size:
        raise ValueError(f"bad tp coordinates rank={tp_rank} size={tp_size}")
    chunk = -(-vocab_size // tp_size)
    start = min(vocab_size, tp_rank * chunk)
    return start, min(vocab_size, start + chunk)
