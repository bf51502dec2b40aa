"""Checkpoint config group (reference: llmtuner/config/checkpoint_config.py:24-241)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

from ..errors import ConfigError
from .utils import require_choice, require_integer_at_least


@dataclass
class CheckpointConfig:
    enable: bool = False
    folder: str = "checkpoint"
    backend: str = "dcp"                         # dcp | torch_checkpointing
    interval: int = 500
    sharded_expert_parallel: bool = False
    sharded_tensor_parallel: bool = False
    initial_load_path: str | None = None
    initial_load_model_only: bool = True
    initial_load_in_hf: bool = False
    last_save_model_only: bool = True
    last_save_in_hf: bool = False
    export_dtype: str = "float32"
    keep_latest_k: int = 10
    purge_exempt: Callable[[int], bool] | None = None
    load_step: int = -1
    exclude_from_loading: list[str] = field(default_factory=list)
    enable_first_step_checkpoint: bool = False
    create_seed_checkpoint: bool = False
    load_only: bool = False
    async_mode: str = "disabled"                 # disabled | async | async_with_pinned_mem

    def __post_init__(self):
        require_choice("backend", self.backend, ("dcp", "torch_checkpointing"))
        require_integer_at_least("interval", self.interval, 1)
        require_choice("export_dtype", self.export_dtype, ("float16", "bfloat16", "float32"))
        require_choice("async_mode", self.async_mode, ("disabled", "async", "async_with_pinned_mem"))
        require_integer_at_least("keep_latest_k", self.keep_latest_k, 0)
        if self.keep_latest_k == 1:
            raise ConfigError("keep_latest_k=1 is unsafe (a save in flight would leave no complete checkpoint); use 0 or >= 2")
        if self.last_save_in_hf and not self.last_save_model_only:
            raise ConfigError("last_save_in_hf requires last_save_model_only")
        if self.initial_load_in_hf and not self.initial_load_model_only:
            raise ConfigError("initial_load_in_hf requires initial_load_model_only")
        if self.backend == "torch_checkpointing":
            raise ConfigError("checkpoint backend 'torch_checkpointing' needs an optional third-party package that is "
                              "not part of this build; use 'dcp'")
