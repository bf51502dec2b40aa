"""Aggregate run configuration with cross-group checks
(reference: llmtuner/config/llmtuner_config.py:37-382).

`LLMTunerConfig(model, parallel, optimizer, training)`; `from_groups` accepts the thirteen flat
parser groups and nests them; `from_dict`/`from_file` read a nested or flat YAML/JSON mapping.
A read-only flat view (`cfg.max_seq_len`, `cfg.tensor_parallel_size`, ...) resolves any field name
that is unique across the groups.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any

from ..errors import ConfigError, UnsupportedCombinationError
from .checkpoint_config import CheckpointConfig
from .data_config import DataloaderConfig
from .model_config import ModelConfig
from .observability_config import MetricsConfig, ProfilerConfig
from .optimizer_config import LRSchedulerConfig, OptimizerConfig
from .parallel_config import (ContextParallelConfig, ExpertParallelConfig, FSDPConfig, ParallelConfig,
                              TensorParallelConfig)
from .training_config import TrainingConfig

_NESTED = {
    ParallelConfig: {"fsdp_config": FSDPConfig, "tp_config": TensorParallelConfig, "cp_config": ContextParallelConfig,
                     "ep_config": ExpertParallelConfig},
    OptimizerConfig: {"lr_scheduler_config": LRSchedulerConfig},
    TrainingConfig: {"checkpoint_config": CheckpointConfig, "dataloader_config": DataloaderConfig,
                     "metrics_config": MetricsConfig, "profiler_config": ProfilerConfig},
}


def _flat_index(obj, out: dict[str, list], seen=None):
    for f in dataclasses.fields(obj):
        v = getattr(obj, f.name)
        if dataclasses.is_dataclass(v):
            _flat_index(v, out)
        else:
            out.setdefault(f.name, []).append((obj, f.name))


@dataclass
class LLMTunerConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_groups(cls, groups) -> "LLMTunerConfig":
        """Nest flat parser groups: FSDP/TP/CP/EP into parallel, LR into optimizer,
        checkpoint/data/metrics/profiler into training."""
        by_type = {type(g): g for g in groups}
        tops = {}
        for top in (ModelConfig, ParallelConfig, OptimizerConfig, TrainingConfig):
            inst = by_type.get(top) or top()
            for attr, sub in _NESTED.get(top, {}).items():
                if sub in by_type:
                    setattr(inst, attr, by_type[sub])
            if hasattr(inst, "__post_init__"):
                inst.__post_init__()
            tops[top] = inst
        return cls(tops[ModelConfig], tops[ParallelConfig], tops[OptimizerConfig], tops[TrainingConfig])

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "LLMTunerConfig":
        """Accepts {"model": {...}, "parallel": {...}, ...} with nested groups, or one flat mapping of
        field names (each must be unique across groups)."""
        data = dict(data or {})
        tops = {"model": ModelConfig, "parallel": ParallelConfig, "optimizer": OptimizerConfig, "training": TrainingConfig}
        if set(data) <= set(tops):
            built = {}
            for key, tcls in tops.items():
                sub = dict(data.get(key) or {})
                for attr, scls in _NESTED.get(tcls, {}).items():
                    if isinstance(sub.get(attr), dict):
                        sub[attr] = scls(**sub[attr])
                names = {f.name for f in dataclasses.fields(tcls)}
                unknown = set(sub) - names
                if unknown:
                    raise ConfigError(f"{key}: unknown fields {sorted(unknown)}")
                built[key] = tcls(**sub)
            return cls(**built)
        cfg = cls()
        cfg.apply_flat(data)
        return cfg

    @classmethod
    def from_file(cls, path: str) -> "LLMTunerConfig":
        with open(path) as f:
            if path.endswith((".yaml", ".yml")):
                import yaml
                data = yaml.safe_load(f)
            elif path.endswith(".json"):
                data = json.load(f)
            else:
                raise ConfigError(f"config file must end in .yaml, .yml or .json: {path}")
        if not isinstance(data, dict):
            raise ConfigError(f"config file {path} must hold a mapping at top level")
        return cls.from_dict(data)

    def apply_flat(self, values: dict[str, Any]) -> "LLMTunerConfig":
        """Set fields by flat name and re-validate every group."""
        index: dict[str, list] = {}
        _flat_index(self, index)
        for k, v in values.items():
            if k not in index:
                raise ConfigError(f"unknown configuration field {k!r}")
            if len(index[k]) > 1:
                raise ConfigError(f"configuration field {k!r} is ambiguous; use the nested form")
            obj, name = index[k][0]
            setattr(obj, name, v)
        self.revalidate()
        return self

    def revalidate(self) -> None:
        def visit(o):
            for f in dataclasses.fields(o):
                v = getattr(o, f.name)
                if dataclasses.is_dataclass(v):
                    visit(v)
            if hasattr(o, "__post_init__"):
                o.__post_init__()
        visit(self)

    def to_dict(self) -> dict[str, Any]:
        def conv(o):
            if dataclasses.is_dataclass(o):
                return {f.name: conv(getattr(o, f.name)) for f in dataclasses.fields(o) if not callable(getattr(o, f.name))
                        or dataclasses.is_dataclass(getattr(o, f.name))}
            if isinstance(o, (list, tuple)):
                return [conv(x) for x in o]
            if isinstance(o, dict):
                return {k: conv(v) for k, v in o.items()}
            return o
        return conv(self)

    # ------------------------------------------------------------------ flat read-only view
    def __getattr__(self, name: str):
        if name.startswith("_") or name in ("model", "parallel", "optimizer", "training"):
            raise AttributeError(name)
        index: dict[str, list] = {}
        try:
            _flat_index(self, index)
        except AttributeError:
            raise AttributeError(name) from None
        hits = index.get(name)
        if not hits:
            for top in (self.model, self.parallel, self.optimizer, self.training):
                if hasattr(type(top), name) or name in {f.name for f in dataclasses.fields(top)}:
                    return getattr(top, name)
            raise AttributeError(f"LLMTunerConfig has no field {name!r}")
        if len(hits) > 1:
            raise AttributeError(f"field {name!r} is ambiguous across groups")
        obj, n = hits[0]
        return getattr(obj, n)

    # ------------------------------------------------------------------ cross-group validation
    def __post_init__(self):
        m, p, o, t = self.model, self.parallel, self.optimizer, self.training
        cc = t.compile_config
        if cc.enable_async_tensor_parallel and not (t.compile and p.tensor_parallel_size > 1):
            raise ConfigError("enable_async_tensor_parallel requires compile=True and tensor_parallel_size > 1")
        if t.metrics_config.measure_moe_dispatch and t.compile:
            raise ConfigError("measure_moe_dispatch places device events inside the MoE block and cannot be used with compile")
        if t.metrics_config.measure_moe_dispatch and p.ep_config.ep_token_dispatcher == "domino":
            raise ConfigError("measure_moe_dispatch cannot time the overlapped domino dispatcher")
        if o.optimizer_type == "AdamWSwap" and t.checkpoint_config.enable and t.checkpoint_config.backend != "dcp":
            raise ConfigError("AdamWSwap keeps moments in pinned host memory and needs the sharded dcp checkpoint backend")
        if o.state_residency == "host" and p.fsdp_config.fsdp_cpu_offload:
            raise ConfigError("state_residency='host' cannot be combined with fsdp_cpu_offload")
        if m.qkv_projection == "fused" and p.tensor_parallel_size > 1:
            raise UnsupportedCombinationError("qkv_projection='fused' packs q/k/v rows in one matrix and cannot be "
                                              "column-sharded per projection; use 'separate' with tensor parallelism")
        span = p.cp_size * p.tensor_parallel_size
        if t.max_seq_len % span:
            raise ConfigError(f"max_seq_len {t.max_seq_len} must be divisible by cp*tp = {span}")
        if p.cp_config.context_parallel_load_balancer == "headtail" and t.max_seq_len % (2 * p.cp_size):
            raise ConfigError("headtail load balancing needs max_seq_len divisible by 2*cp")
        if t.activation_swap and t.activation_checkpoint_mode not in ("none", "selective"):
            raise ConfigError("activation_swap works on saved activations: use activation_checkpoint_mode none or selective")
        if t.validation_config is not None and t.validation_config.steps == -1 and t.dataloader_config.dataset in ("random", "random_packed"):
            t.validation_config.steps = 1   # an infinite synthetic stream needs a bound

    def auto_fill_model(self, **sizes) -> "LLMTunerConfig":
        """Fill toy model sizes (used by examples and tests)."""
        for k, v in sizes.items():
            if not hasattr(self.model, k):
                raise ConfigError(f"ModelConfig has no field {k!r}")
            setattr(self.model, k, v)
        self.model.__post_init__()
        return self
