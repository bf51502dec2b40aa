"""Pipeline schedules as explicit action lists (reference: torch.distributed.pipelining schedules selected in
experiments/pipeline_parallel/pipeline_parallel.py:262-423; GPipe and 1F1B with one stage per rank)."""
from __future__ import annotations

from ...errors import ConfigError


def build_schedule(name: str, stage: int, num_stages: int, num_microbatches: int) -> list[tuple[str, int]]:
    """[("F", mb) | ("B", mb)] for this stage."""
    n = name.lower()
    if n == "gpipe":
        return [("F", m) for m in range(num_microbatches)] + [("B", m) for m in range(num_microbatches)]
    if n == "1f1b":
        warm = min(num_microbatches, num_stages - stage - 1)
        acts = [("F", m) for m in range(warm)]
        f, b = warm, 0
        while f < num_microbatches:
            acts.append(("F", f)); f += 1
            acts.append(("B", b)); b += 1
        while b < num_microbatches:
            acts.append(("B", b)); b += 1
        return acts
    if n in ("interleaved1f1b", "zbv", "dualpipev") or n.endswith(".csv"):
        raise ConfigError(f"pipeline schedule {name!r} is recognised but not implemented (one stage per rank only)")
    raise ConfigError(f"unknown pipeline schedule {name!r}")
