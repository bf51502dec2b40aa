"""Rank-aware logging (reference: llmtuner/utils/logging.py:76-257).

Rank 0 (or the ranks in `set_log_ranks`) prints below ERROR; every rank prints ERROR.
An optional file handler is attached on rank 0 only.
"""
from __future__ import annotations

import logging
import os
import sys

_LOG_RANKS: set[int] = {0}
_ROOT = "torchllmtuner_b200"


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


class _RankFilter(logging.Filter):
    def filter(self, record: logging.LogRecord) -> bool:
        return record.levelno >= logging.ERROR or _rank() in _LOG_RANKS


def set_log_ranks(ranks) -> None:
    global _LOG_RANKS
    _LOG_RANKS = {int(r) for r in ranks}


def get_logger(name: str | None = None, log_file: str | None = None, level: int = logging.INFO) -> logging.Logger:
    root = logging.getLogger(_ROOT)
    if not root.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(f"[%(asctime)s][rank{_rank()}][%(levelname)s] %(message)s", "%H:%M:%S"))
        h.addFilter(_RankFilter())
        root.addHandler(h)
        root.setLevel(level)
        root.propagate = False
    if log_file and _rank() == 0 and not any(isinstance(h, logging.FileHandler) for h in root.handlers):
        os.makedirs(os.path.dirname(os.path.abspath(log_file)), exist_ok=True)
        fh = logging.FileHandler(log_file)
        fh.setFormatter(logging.Formatter("[%(asctime)s][%(levelname)s] %(message)s"))
        root.addHandler(fh)
    return root if not name else root.getChild(name.replace(_ROOT + ".", ""))
