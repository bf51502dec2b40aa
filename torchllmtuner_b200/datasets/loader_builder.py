"""`build_dataloader`: synthetic path, or recipe + tokenizer + packing + collator + prefetching loader
(reference: llmtuner/datasets/loader_builder.py:154-317)."""
from __future__ import annotations

from ..errors import ConfigError
from .synthetic import RandomPackedSource, RandomTokenDataLoader, RandomTokenSource


def build_dataloader(data_cfg, *, vocab_size: int, global_batch: int, seq_len: int, seed: int, dp_rank: int, dp_degree: int,
                     rows_per_rank: int, pin_memory: bool = False, split: str = "train"):
    name = data_cfg.dataset
    if name == "random":
        return RandomTokenDataLoader(RandomTokenSource(vocab_size, global_batch, seq_len, seed), dp_rank, dp_degree,
                                     rows_per_rank, pin_memory)
    if name == "random_packed":
        src = RandomPackedSource(vocab_size, global_batch, seq_len, seed, data_cfg.packed_min_doc_len, data_cfg.packed_max_doc_len)
        return RandomTokenDataLoader(src, dp_rank, dp_degree, rows_per_rank, pin_memory)
    try:
        from .text import build_text_dataloader
    except ImportError as e:  # pragma: no cover
        raise ConfigError(f"dataset {name!r} needs the text pipeline: {e}") from e
    return build_text_dataloader(data_cfg, vocab_size=vocab_size, seq_len=seq_len, seed=seed, dp_rank=dp_rank,
                                 dp_degree=dp_degree, rows_per_rank=rows_per_rank, pin_memory=pin_memory, split=split)
