"""Dataset composition (reference: llmtuner/datasets/composition.py:51-337): a single source, a weighted mix, or a
concatenation, each with a map-side policy: epoch-seeded shuffle -> data-parallel shard -> repeat."""
from __future__ import annotations

import random
from dataclasses import dataclass


@dataclass
class DatasetIterationPolicy:
    shuffle: bool = True
    seed: int = 0
    repeat: bool = True


class SingleDataset:
    def __init__(self, source, processor):
        self.source, self.processor = source, processor

    def __len__(self):
        return len(self.source)

    def get(self, i: int):
        return self.processor(self.source[i])


class DatasetConcat:
    def __init__(self, parts):
        self.parts = list(parts)
        self.offsets = [0]
        for p in self.parts:
            self.offsets.append(self.offsets[-1] + len(p))

    def __len__(self):
        return self.offsets[-1]

    def get(self, i: int):
        for k, p in enumerate(self.parts):
            if i < self.offsets[k + 1]:
                return p.get(i - self.offsets[k])
        raise IndexError(i)


class DatasetMix:
    """Weighted interleave: sample index i deterministically picks a member by its weight and that member's next row."""

    def __init__(self, parts, weights, seed: int = 0):
        self.parts, self.weights, self.seed = list(parts), list(weights), seed

    def __len__(self):
        return sum(len(p) for p in self.parts)

    def get(self, i: int):
        rng = random.Random(self.seed * 1_000_003 + i)
        k = rng.choices(range(len(self.parts)), weights=self.weights)[0]
        return self.parts[k].get(rng.randrange(len(self.parts[k])))


def epoch_order(n: int, epoch: int, policy: DatasetIterationPolicy, dp_rank: int, dp_degree: int) -> list[int]:
    idx = list(range(n))
    if policy.shuffle:
        random.Random(policy.seed * 7919 + epoch).shuffle(idx)
    return idx[dp_rank::dp_degree]
