"""Optimizer and LR-schedule config groups (reference: llmtuner/config/optimizer_config.py:15-232,
lr_scheduler_config.py)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..errors import ConfigError
from .utils import require_choice, require_integer_at_least


@dataclass
class LRSchedulerConfig:
    warmup_steps: int = 0
    total_steps: int | None = None
    decay_ratio: float = 0.0
    decay_type: str = "linear"       # linear | sqrt | cosine
    min_lr_factor: float = 0.0

    def __post_init__(self):
        require_integer_at_least("warmup_steps", self.warmup_steps, 0)
        require_choice("decay_type", self.decay_type, ("linear", "sqrt", "cosine"))
        if not 0.0 <= self.decay_ratio <= 1.0:
            raise ConfigError("decay_ratio must be in [0, 1]")
        if not 0.0 <= self.min_lr_factor <= 1.0:
            raise ConfigError("min_lr_factor must be in [0, 1]")


@dataclass
class ParamGroupConfig:
    """First-match regex group: parameters whose FQN matches `pattern` use these overrides."""
    pattern: str = ".*"
    optimizer_type: str | None = None
    optimizer_kwargs: dict[str, Any] = field(default_factory=dict)


def validated_betas(betas) -> tuple[float, float]:
    if len(betas) != 2 or not all(0.0 <= float(b) < 1.0 for b in betas):
        raise ConfigError(f"betas must be two values in [0, 1), got {betas!r}")
    return float(betas[0]), float(betas[1])


@dataclass
class OptimizerConfig:
    optimizer_type: str = "AdamW"            # Adam | AdamW | AdamWSwap | DistMuon
    learning_rate: float = 3e-4
    weight_decay: float = 0.0
    betas: list[float] = field(default_factory=lambda: [0.9, 0.999])
    eps: float = 1e-8
    implementation: str = "fused"            # fused | foreach | for-loop
    state_residency: str = "device"          # device | host (pinned host moments)
    swap_max_device_bytes: int = 0
    swap_prefetch: bool = True
    swap_memory_fraction: float | None = None
    swap_max_host_bytes: int = 0
    param_groups: list[ParamGroupConfig] = field(default_factory=list)
    compute_sharding_by_fqn: dict[str, Any] = field(default_factory=dict)
    bucket_configs: list[Any] = field(default_factory=list)
    lr_scheduler_config: LRSchedulerConfig = field(default_factory=LRSchedulerConfig)

    def __post_init__(self):
        require_choice("optimizer_type", self.optimizer_type, ("Adam", "AdamW", "AdamWSwap", "DistMuon"))
        require_choice("implementation", self.implementation, ("fused", "foreach", "for-loop"))
        require_choice("state_residency", self.state_residency, ("device", "host", "npu_virtual"))
        if self.state_residency == "npu_virtual":
            raise ConfigError("state_residency='npu_virtual' is an Ascend feature; use 'host' for pinned-host moments")
        if not self.learning_rate >= 0 or not self.weight_decay >= 0 or not self.eps > 0:
            raise ConfigError("learning_rate and weight_decay must be >= 0 and eps > 0")
        self.betas = list(validated_betas(self.betas))
        self.param_groups = [g if isinstance(g, ParamGroupConfig) else ParamGroupConfig(**g) for g in self.param_groups]
        if isinstance(self.lr_scheduler_config, dict):
            self.lr_scheduler_config = LRSchedulerConfig(**self.lr_scheduler_config)
