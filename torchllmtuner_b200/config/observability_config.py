"""Metrics and profiler config groups (reference: llmtuner/config/observability_config.py:1-163)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import ConfigError
from .utils import require_integer_at_least


@dataclass
class MetricsConfig:
    log_freq: int = 1
    metrics_warmup_steps: int = 2
    steady_window_steps: int = 1024
    measure_moe_dispatch: bool = False
    enable_tensorboard: bool = False
    disable_color_printing: bool = False
    save_tb_folder: str = "tb"
    save_for_all_ranks: bool = False
    log_ranks: list[int] = field(default_factory=lambda: [0])
    enable_wandb: bool = False
    tag: str | None = None

    def __post_init__(self):
        require_integer_at_least("log_freq", self.log_freq, 1)
        require_integer_at_least("metrics_warmup_steps", self.metrics_warmup_steps, 0)
        require_integer_at_least("steady_window_steps", self.steady_window_steps, 1)
        self.log_ranks = [int(r) for r in self.log_ranks]


@dataclass
class ProfilerConfig:
    enable_profiling: bool = False
    npu_profiler_level: str | None = None
    save_traces_folder: str = "profiling/traces"
    profile_freq: int = 10
    profiler_repeat: int | None = None
    profiler_skip_first: int | None = None
    profiler_skip_first_wait: int | None = None
    profiler_active: int = 1
    profiler_warmup: int = 3
    enable_memory_snapshot: bool = False
    memory_snapshot_freq: int | None = None
    save_memory_snapshot_folder: str = "profiling/memory_snapshot"
    memory_snapshot_max_entries: int = 1_000_000

    def __post_init__(self):
        require_integer_at_least("profile_freq", self.profile_freq, 1)
        require_integer_at_least("profiler_active", self.profiler_active, 1)
        require_integer_at_least("profiler_warmup", self.profiler_warmup, 0)
        if self.enable_profiling and self.profile_freq < self.profiler_active + self.profiler_warmup:
            raise ConfigError("profile_freq must be >= profiler_active + profiler_warmup")
        if self.npu_profiler_level is not None:
            raise ConfigError("npu_profiler_level is an Ascend option; leave it unset on CUDA")
