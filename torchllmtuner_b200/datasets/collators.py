"""Collators: packed rows -> trainer batches (reference: llmtuner/datasets/collators.py:44-186)."""
from __future__ import annotations

import torch

from .contracts import IGNORE_INDEX


class TextCollator:
    """Stacks `rows_per_rank` packed rows into `input` / `labels` / `positions` [B, S] (pinned when asked) and the global
    document cut points `cu_seqlens` of the flattened [B*S] rows."""

    def __init__(self, seq_len: int, pin_memory: bool = False):
        self.seq_len, self.pin = seq_len, pin_memory

    def __call__(self, rows) -> dict:
        B, S = len(rows), self.seq_len
        mk = lambda: torch.empty(B, S, dtype=torch.int64, pin_memory=self.pin)  # noqa: E731
        inp, lab, pos = mk(), mk(), mk()
        cu = [0]
        for i, r in enumerate(rows):
            inp[i] = torch.tensor(r.tokens, dtype=torch.int64)
            lab[i] = torch.tensor(r.labels, dtype=torch.int64)
            pos[i] = torch.tensor(r.positions, dtype=torch.int64)
            cu += [i * S + c for c in r.cuts[1:]]
        return {"input": inp, "labels": lab, "positions": pos, "cu_seqlens": torch.tensor(cu, dtype=torch.int32),
                "num_valid_tokens": int((lab != IGNORE_INDEX).sum())}
