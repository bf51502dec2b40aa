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


class HuggingFaceDiskSource(HuggingFaceRandomAccessSource):
    """A dataset saved with `Dataset.save_to_disk` (works offline)."""

    def __init__(self, path: str):
        try:
            import datasets
        except ImportError as e:
            raise ConfigError("Hugging Face `datasets` is not installed; use dataset=local_jsonl") from e
        ds = datasets.load_from_disk(path)
        self.ds = ds["train"] if isinstance(ds, dict) else ds


class StreamingSource:
    """Forward-only iteration over a (possibly unbounded) iterable of rows with a checkpointable cursor and an optional
    shuffle buffer (reference: llmtuner/datasets/sources.py:250-391). `state_dict()` holds the number of rows consumed
    and the shuffle RNG state; `load_state_dict` replays the iterable to that point, so a resumed run sees the same rows
    in the same order. `make_iterable` is called once per (re)start and must return rows in a reproducible order."""

    def __init__(self, make_iterable, shuffle_buffer_size: int = 0, seed: int = 0):
        import random
        self.make_iterable, self.buffer_size, self.seed = make_iterable, int(shuffle_buffer_size), seed
        self.consumed = 0
        self._rng = random.Random(seed)
        self._it = None
        self._buf: list = []

    def _start(self, skip: int) -> None:
        import random
        self._rng = random.Random(self.seed)
        self._it = iter(self.make_iterable())
        self._buf = []
        self.consumed = 0
        for _ in range(skip):
            next(self)

    def __iter__(self):
        if self._it is None:
            self._start(0)
        return self

    def __next__(self):
        if self._it is None:
            self._start(0)
        if self.buffer_size <= 1:
            row = next(self._it)
        else:
            while len(self._buf) < self.buffer_size:
                try:
                    self._buf.append(next(self._it))
                except StopIteration:
                    break
            if not self._buf:
                raise StopIteration
            row = self._buf.pop(self._rng.randrange(len(self._buf)))
        self.consumed += 1
        return row

    def state_dict(self) -> dict:
        return {"consumed": self.consumed, "seed": self.seed, "buffer_size": self.buffer_size}

    def load_state_dict(self, sd: dict) -> None:
        if sd.get("seed", self.seed) != self.seed or sd.get("buffer_size", self.buffer_size) != self.buffer_size:
            raise ConfigError("streaming source: seed or shuffle buffer differs from the checkpointed run")
        self._start(int(sd["consumed"]))


def build_source(data_cfg, split: str = "train"):
    if data_cfg.dataset == "hf_disk":
        if not data_cfg.dataset_path:
            raise ConfigError("dataset 'hf_disk' needs dataset_path")
        return HuggingFaceDiskSource(data_cfg.dataset_path)
    if data_cfg.dataset in ("local_jsonl", "local_jsonl_sft", "local_jsonl_sft_multiturn"):
        if not data_cfg.dataset_path:
            raise ConfigError(f"dataset {data_cfg.dataset!r} needs dataset_path")
        return IndexedJsonlSource(data_cfg.dataset_path)
    if data_cfg.dataset in ("c4", "c4_test", "c4_validation"):
        return HuggingFaceRandomAccessSource("allenai/c4", split={"c4": "train", "c4_test": "train[:1000]", "c4_validation": "validation"}[data_cfg.dataset], name="en")
    raise ConfigError(f"unknown dataset {data_cfg.dataset!r}")
