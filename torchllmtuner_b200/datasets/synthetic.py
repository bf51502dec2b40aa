"""Deterministic synthetic token data (reference: llmtuner/datasets/synthetic.py:29-200).

Global batch `step` = randint(0, vocab, (B, S)) from a CPU generator seeded (seed*100000 + step) mod 2^64; each
data-parallel rank takes a contiguous row slice; the state is the absolute step cursor plus the batch layout.
`RandomPackedSource` additionally cuts every row into documents whose lengths are log-uniform in [lo, hi].
"""
from __future__ import annotations

import math

import torch

from .contracts import (BaseDataLoader, Batch, IGNORE_INDEX, require_same_dp_degree, to_trainer_batch,
                        validate_dp_coordinates)


class RandomTokenSource:
    def __init__(self, vocab_size: int, global_batch: int, seq_len: int, seed: int):
        self.vocab_size, self.global_batch, self.seq_len, self.seed = vocab_size, global_batch, seq_len, seed

    def generator(self, step: int) -> torch.Generator:
        return torch.Generator(device="cpu").manual_seed((self.seed * 100000 + step) % (2 ** 64))

    def global_batch_at(self, step: int) -> Batch:
        ids = torch.randint(0, self.vocab_size, (self.global_batch, self.seq_len), generator=self.generator(step), dtype=torch.int64)
        return Batch(ids, ids.clone())


class RandomPackedSource(RandomTokenSource):
    def __init__(self, vocab_size, global_batch, seq_len, seed, min_doc: int = 512, max_doc: int = 32768):
        super().__init__(vocab_size, global_batch, seq_len, seed)
        self.min_doc, self.max_doc = min(min_doc, seq_len), min(max_doc, seq_len)

    def document_cuts(self, step: int, row: int) -> list[int]:
        g = torch.Generator(device="cpu").manual_seed((self.seed * 100000 + step) * 1009 + row + 17)
        cuts, pos = [0], 0
        lo, hi = math.log(self.min_doc), math.log(self.max_doc)
        while pos < self.seq_len:
            n = int(round(math.exp(lo + (hi - lo) * torch.rand((), generator=g).item())))
            pos = min(self.seq_len, pos + max(1, n))
            cuts.append(pos)
        return cuts


class RandomTokenDataLoader(BaseDataLoader):
    """Yields trainer batches for one data-parallel rank; resumable through `state_dict`."""

    def __init__(self, source: RandomTokenSource, dp_rank: int, dp_degree: int, rows_per_rank: int, pin_memory: bool = False):
        validate_dp_coordinates(dp_rank, dp_degree)
        if rows_per_rank * dp_degree > source.global_batch:
            raise ValueError(f"{rows_per_rank} rows x {dp_degree} ranks exceed the global batch {source.global_batch}")
        self.source, self.dp_rank, self.dp_degree, self.rows = source, dp_rank, dp_degree, rows_per_rank
        self.pin_memory = pin_memory
        self.cursor = 0          # micro-batches consumed so far (absolute)
        self.mb_per_step = source.global_batch // (rows_per_rank * dp_degree)

    def __next__(self) -> dict:
        step, mb = divmod(self.cursor, self.mb_per_step)
        g = self.source.global_batch_at(step)
        r0 = mb * self.rows * self.dp_degree + self.dp_rank * self.rows
        b = to_trainer_batch(Batch(g.input_ids[r0:r0 + self.rows], g.labels[r0:r0 + self.rows]))
        if isinstance(self.source, RandomPackedSource):
            S = self.source.seq_len
            cu, pos = [0], []
            for i in range(self.rows):
                cuts = self.source.document_cuts(step, r0 + i)
                for a, e in zip(cuts[:-1], cuts[1:]):
                    cu.append(i * S + e)
                    pos.append(torch.arange(e - a))
                    b["labels"][i, e - 1] = IGNORE_INDEX     # the last token of a document predicts nothing
            b["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32)
            b["positions"] = torch.cat(pos).view(self.rows, S)
            b["num_valid_tokens"] = int((b["labels"] != IGNORE_INDEX).sum())
        if self.pin_memory:
            for k, v in list(b.items()):
                if isinstance(v, torch.Tensor) and k != "cu_seqlens":
                    b[k] = v.pin_memory()
        self.cursor += 1
        return b

    def state_dict(self) -> dict:
        return {"cursor": self.cursor, "dp_degree": self.dp_degree, "rows": self.rows, "global_batch": self.source.global_batch,
                "seq_len": self.source.seq_len, "seed": self.source.seed}

    def load_state_dict(self, sd: dict) -> None:
        require_same_dp_degree(int(sd["dp_degree"]), self.dp_degree)
        for k, cur in (("rows", self.rows), ("global_batch", self.source.global_batch), ("seq_len", self.source.seq_len)):
            if int(sd[k]) != cur:
                raise ValueError(f"data layout changed: saved {k}={sd[k]}, now {cur}")
        self.cursor = int(sd["cursor"])
