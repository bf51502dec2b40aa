"""Warm-up / stable / decay schedule (reference: llmtuner/components/optimizer/lr_scheduler.py:36-307).

factor(step), step counted from 0:
  step < warmup                 -> (step + 1) / warmup                  (not blended with the minimum factor)
  step < warmup + stable        -> 1
  otherwise                     -> min + (1 - min) * shape(p),  p = (step + 1 - warmup - stable) / decay
with shape linear 1-p, sqrt 1-sqrt(p), cosine (1+cos(pi p))/2. Phase lengths come from `resolve_phases`:
decay = round(total * decay_ratio); warm-up longer than the schedule is clamped to it; warm-up + decay longer than the
schedule shortens the decay; stable = total + 1 - warmup - decay (the extra step keeps the last real step off the end
of the decay, where a linear factor would be exactly the minimum)."""
from __future__ import annotations

import math

from ...utils.logging import get_logger

logger = get_logger(__name__)

_SHAPES = {
    "linear": lambda p: 1.0 - p,
    "sqrt": lambda p: 1.0 - math.sqrt(p),
    "cosine": lambda p: 0.5 * (1.0 + math.cos(math.pi * p)),
}


def resolve_phases(total: int, warmup: int, decay_ratio: float, warn: bool = False) -> tuple[int, int, int]:
    """(warmup, stable, decay) step counts of a schedule of `total` steps; `warn` logs the two clamps."""
    log = logger.warning if warn else (lambda *a: None)
    if warmup > total:
        log("lr warmup_steps (%d) exceeds the schedule (%d steps); the warm-up covers the whole schedule", warmup, total)
        warmup = total
    decay = round(total * decay_ratio)
    if warmup + decay > total:
        log("lr warm-up (%d) + decay (%d) exceed the schedule (%d steps); the decay is shortened to %d",
                       warmup, decay, total, total - warmup)
        decay = total - warmup
    return warmup, total + 1 - warmup - decay, decay


def wsd_factor(step: int, *, warmup: int, total: int, decay_ratio: float, decay_type: str = "linear", min_lr_factor: float = 0.0) -> float:
    if decay_type not in _SHAPES:
        raise ValueError(f"unknown decay_type {decay_type!r}")
    warmup, stable, decay = resolve_phases(total, warmup, decay_ratio)
    if step < warmup:
        return (step + 1) / warmup
    if step < warmup + stable or decay <= 0:
        return 1.0
    p = (step + 1 - warmup - stable) / decay
    return min_lr_factor + (1.0 - min_lr_factor) * _SHAPES[decay_type](p)


class LRSchedulersContainer:
    """One schedule shared by every optimizer of the container; state is the single `last_epoch` counter."""

    def __init__(self, optimizers, cfg, total_steps: int):
        self.optimizers = optimizers
        self.cfg = cfg
        self.total = cfg.total_steps if cfg.total_steps is not None else total_steps
        if self.total < total_steps:
            raise ValueError(f"lr_scheduler.total_steps ({self.total}) is shorter than the run ({total_steps} steps): the decay "
                             "would run past its end and the learning rate would turn negative")
        resolve_phases(max(1, self.total), cfg.warmup_steps, cfg.decay_ratio, warn=True)
        self.last_epoch = 0
        self.base_lrs = [[g["lr"] for g in o.param_groups] for o in optimizers.optimizers]
        self._apply()

    def factor(self, step: int | None = None) -> float:
        c = self.cfg
        return wsd_factor(self.last_epoch if step is None else step, warmup=c.warmup_steps, total=max(1, self.total),
                          decay_ratio=c.decay_ratio, decay_type=c.decay_type, min_lr_factor=c.min_lr_factor)

    def _apply(self) -> None:
        f = self.factor()
        for o, bases in zip(self.optimizers.optimizers, self.base_lrs):
            for g, b in zip(o.param_groups, bases):
                g["lr"] = b * f

    def step(self) -> None:
        self.last_epoch += 1
        self._apply()

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for o in self.optimizers.optimizers for g in o.param_groups]

    def state_dict(self) -> dict:
        return {"last_epoch": self.last_epoch}

    def load_state_dict(self, sd: dict) -> None:
        self.last_epoch = int(sd["last_epoch"])
        self._apply()


def build_lr_scheduler(optimizers, cfg, total_steps: int) -> LRSchedulersContainer:
    return LRSchedulersContainer(optimizers, cfg, total_steps)
