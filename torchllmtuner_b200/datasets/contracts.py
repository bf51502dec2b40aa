"""Data contracts (reference: llmtuner/datasets/contracts.py:44-268).

`Batch(input_ids, labels)` carries UNSHIFTED labels (synthetic source); `TrainerBatch` is the dict the trainer
consumes: `input` [B,S], `labels` [B,S] already shifted targets with IGNORE_INDEX, optional `positions`,
`cu_seqlens` (document cuts of the packed rows, int32 host), `num_valid_tokens`.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..errors import ConfigError

IGNORE_INDEX = -100


class DataloaderExhaustedError(RuntimeError):
    pass


class Stateful:
    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, sd: dict) -> None:
        pass


class BaseDataLoader(Stateful):
    def __iter__(self):
        return self

    def __next__(self) -> dict:
        raise NotImplementedError

    def close(self) -> None:
        """Ends background work (prefetch threads); the trainer calls it on shutdown."""


@dataclass
class Batch:
    input_ids: torch.Tensor
    labels: torch.Tensor


@dataclass
class TextSequence:
    tokens: list[int]
    labels: list[int]          # already shifted; IGNORE_INDEX where no loss
    positions: list[int]
    document_ids: list[int]


@dataclass
class DatasetBuildContext:
    dp_rank: int
    dp_degree: int
    seq_len: int
    batch_size: int
    seed: int
    vocab_size: int


def require_positive_integer(name: str, v) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v < 1:
        raise ConfigError(f"{name} must be a positive integer, got {v!r}")
    return v


def require_same_dp_degree(saved: int, current: int) -> None:
    if saved != current:
        raise ConfigError(f"the data cursor was saved with dp degree {saved} and cannot resume at {current}")


def validate_dp_coordinates(dp_rank: int, dp_degree: int) -> None:
    require_positive_integer("dp_degree", dp_degree)
    if not 0 <= dp_rank < dp_degree:
        raise ConfigError(f"dp_rank {dp_rank} outside [0, {dp_degree})")


def to_trainer_batch(batch: Batch) -> dict:
    """Shift unshifted labels at loss time: position t predicts token t+1; count valid targets."""
    labels = torch.full_like(batch.labels, IGNORE_INDEX)
    labels[:, :-1] = batch.labels[:, 1:]
    return {"input": batch.input_ids, "labels": labels, "num_valid_tokens": int((labels != IGNORE_INDEX).sum())}
