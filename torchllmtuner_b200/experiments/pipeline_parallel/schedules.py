"""Pipeline schedules as explicit action lists (reference: torch.distributed.pipelining schedules selected in
experiments/pipeline_parallel/pipeline_parallel.py:262-423): GPipe and 1F1B with one stage per rank, interleaved 1F1B with
`chunks` looped stages per rank (global stage `c * pp + rank` lives on `rank` as chunk `c`)."""
from __future__ import annotations

from ...errors import ConfigError


def stages_per_rank(name: str) -> int:
    """1 for GPipe / 1F1B, 2 for the looped schedules (reference: pipeline_parallel.py:134-186)."""
    return 2 if name.lower() in ("interleaved1f1b", "interleaved_1f1b") else 1


def build_schedule(name: str, rank: int, num_ranks: int, num_microbatches: int) -> list[tuple[str, int, int]]:
    """[("F" | "B", chunk, microbatch)] for this pipeline rank."""
    n = name.lower()
    M = num_microbatches
    if n == "gpipe":
        return [("F", 0, m) for m in range(M)] + [("B", 0, m) for m in range(M)]
    if n == "1f1b":
        warm = min(M, num_ranks - rank - 1)
        acts = [("F", 0, m) for m in range(warm)]
        f, b = warm, 0
        while f < M:
            acts.append(("F", 0, f)); f += 1
            acts.append(("B", 0, b)); b += 1
        while b < M:
            acts.append(("B", 0, b)); b += 1
        return acts
    if n in ("interleaved1f1b", "interleaved_1f1b"):
        V, pp = stages_per_rank(n), num_ranks
        if M % pp:
            raise ConfigError(f"interleaved 1F1B needs num_pp_microbatches ({M}) divisible by pipeline_parallel_size ({pp})")
        total = M * V

        def item(k: int, backward: bool) -> tuple[int, int]:
            chunk = (k // pp) % V
            if backward:
                chunk = V - 1 - chunk
            return chunk, (k // (pp * V)) * pp + k % pp

        warm = min(total, (pp - rank - 1) * 2 + (V - 1) * pp)
        acts = [("F", *item(k, False)) for k in range(warm)]
        for i in range(total - warm):
            acts.append(("F", *item(warm + i, False)))
            acts.append(("B", *item(i, True)))
        acts += [("B", *item(i, True)) for i in range(total - warm, total)]
        return acts
    if n in ("zbv", "dualpipev") or n.endswith(".csv"):
        raise ConfigError(f"pipeline schedule {name!r} is recognised but not implemented")
    raise ConfigError(f"unknown pipeline schedule {name!r}")
