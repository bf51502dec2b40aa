"""Process groups that the per-step reductions run on (reference: llmtuner/trainer/runtime/reductions.py:1-74):
`dp` for the valid-token count (batch axes), `loss` for the reported loss (batch x cp x tp), `sequence` for the axes that
split one row (cp x tp)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TrainingReductionMeshes:
    dp_group: object | None
    loss_group: object | None
    sequence_degree: int
    dp_degree: int

    @classmethod
    def from_topology(cls, topo) -> "TrainingReductionMeshes":
        return cls(dp_group=topo.get_group("dp") if topo.dp > 1 else None, loss_group=topo.get_group("loss"),
                   sequence_degree=topo.cp * topo.tp, dp_degree=topo.dp)
