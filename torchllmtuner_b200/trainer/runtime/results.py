"""Step results and progress state (reference: llmtuner/trainer/runtime/results.py:15-117)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class TrainingProgress:
    step: int = 0
    ntokens_seen: int = 0

    def state_dict(self) -> dict:
        return {"step": self.step, "ntokens_seen": self.ntokens_seen}

    def load_state_dict(self, sd: dict) -> None:
        self.step, self.ntokens_seen = int(sd["step"]), int(sd["ntokens_seen"])


@dataclass
class StepResult:
    step: int
    loss: float
    grad_norm: float
    lr: float
    global_tokens: int
    step_seconds: float
    max_loss: float | None = None
    extra: dict = field(default_factory=dict)
