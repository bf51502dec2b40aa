"""Warm-up / stable / decay schedule (reference: llmtuner/components/optimizer/lr_scheduler.py:36-307).

factor(step): warm-up (step+1)/warmup; stable 1.0; decay progress p = (step+1-warmup-stable)/decay with
linear 1-p, sqrt 1-sqrt(p), cosine (1+cos(pi p))/2; result min + (1-min)*factor; stable = total+1-warmup-decay."""
from __future__ import annotations

import math


def wsd_factor(step: int, *, warmup: int, total: int, decay_ratio: float, decay_type: str = "linear", min_lr_factor: float = 0.0) -> float:
    decay = int(total * decay_ratio)
    stable = total + 1 - warmup - decay
    s = step + 1
    if warmup > 0 and s <= warmup:
        f = s / warmup
    elif s <= warmup + stable or decay <= 0:
        f = 1.0
    else:
        p = min(1.0, max(0.0, (s - warmup - stable) / decay))
        f = {"linear": 1.0 - p, "sqrt": 1.0 - math.sqrt(p), "cosine": 0.5 * (1.0 + math.cos(math.pi * p))}[decay_type]
    return min_lr_factor + (1.0 - min_lr_factor) * f


class LRSchedulersContainer:
    """One schedule shared by every optimizer of the container; state is the single `last_epoch` counter."""

    def __init__(self, optimizers, cfg, total_steps: int):
        self.optimizers = optimizers
        self.cfg = cfg
        self.total = cfg.total_steps if cfg.total_steps is not None else total_steps
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
