"""Random-access data sources (reference: llmtuner/datasets/sources.py:44-391): an indexed JSONL reader (byte offsets
scanned once, rows parsed on demand) and an optional Hugging Face `datasets` adapter."""
from __future__ import annotations

import glob
import json
import os

from ..errors import ConfigError


def file_patterns_to_paths(pattern: str) -> list[str]:
    if os.path.isdir(pattern):
        paths = sorted(glob.glob(os.path.join(pattern, "*.jsonl")) + glob.glob(os.path.join(pattern, "*.json")))
    else:
        paths = sorted(glob.glob(pattern)) or ([pattern] if os.path.exists(pattern) else [])
    if not paths:
        raise ConfigError(f"no data files match {pattern!r}")
    return paths


class IndexedJsonlSource:
    """len() rows over one or more JSONL files; `__getitem__` parses one row."""

    def __init__(self, pattern: str):
        self.paths = file_patterns_to_paths(pattern)
        self.index: list[tuple[int, int]] = []
        for fi, p in enumerate(self.paths):
            off = 0
            with open(p, "rb") as f:
                for line in f:
                    if line.strip():
                        self.index.append((fi, off))
                    off += len(line)
        self._fh: dict[int, object] = {}

    def __len__(self) -> int:
        return len(self.index)

    def __getitem__(self, i: int) -> dict:
        fi, off = self.index[i]
        fh = self._fh.get(fi)
        if fh is None:
            fh = self._fh[fi] = open(self.paths[fi], "rb")
        fh.seek(off)
        return json.loads(fh.readline())


class HuggingFaceRandomAccessSource:
    def __init__(self, name: str, split: str = "train", **kw):
        try:
            import datasets
        except ImportError as e:
            raise ConfigError("Hugging Face `datasets` is not installed; use dataset=local_jsonl") from e
        self.ds = datasets.load_dataset(name, split=split, **kw)

    def __len__(self):
        return len(self.ds)

    def __getitem__(self, i):
        return self.ds[int(i)]


def build_source(data_cfg, split: str = "train"):
    if data_cfg.dataset in ("local_jsonl", "local_jsonl_sft", "local_jsonl_sft_multiturn"):
        if not data_cfg.dataset_path:
            raise ConfigError(f"dataset {data_cfg.dataset!r} needs dataset_path")
        return IndexedJsonlSource(data_cfg.dataset_path)
    if data_cfg.dataset in ("c4", "c4_test", "c4_validation"):
        return HuggingFaceRandomAccessSource("allenai/c4", split={"c4": "train", "c4_test": "train[:1000]", "c4_validation": "validation"}[data_cfg.dataset], name="en")
    raise ConfigError(f"unknown dataset {data_cfg.dataset!r}")
