"""CLI view of the config groups: which groups become flat flags and which fields stay
programmatic-only (reference: llmtuner/config/cli_config.py:27-80)."""
from __future__ import annotations

import argparse
import dataclasses
import json
import typing

from ..errors import ConfigError
from .checkpoint_config import CheckpointConfig
from .data_config import DataloaderConfig
from .model_config import ModelConfig
from .observability_config import MetricsConfig, ProfilerConfig
from .optimizer_config import LRSchedulerConfig, OptimizerConfig
from .parallel_config import (ContextParallelConfig, ExpertParallelConfig, FSDPConfig, ParallelConfig,
                              TensorParallelConfig)
from .training_config import TrainingConfig

PARSER_GROUPS: tuple[type, ...] = (
    ModelConfig, ParallelConfig, FSDPConfig, TensorParallelConfig, ContextParallelConfig, ExpertParallelConfig,
    OptimizerConfig, LRSchedulerConfig, TrainingConfig, CheckpointConfig, DataloaderConfig, MetricsConfig,
    ProfilerConfig,
)

PROGRAMMATIC_ONLY: dict[type, frozenset[str]] = {
    ModelConfig: frozenset({"arch_overrides"}),
    OptimizerConfig: frozenset({"param_groups", "lr_scheduler_config", "compute_sharding_by_fqn", "bucket_configs"}),
    CheckpointConfig: frozenset({"purge_exempt"}),
    ParallelConfig: frozenset({"fsdp_config", "tp_config", "cp_config", "ep_config"}),
    FSDPConfig: frozenset({"fsdp_apply_modules"}),
    DataloaderConfig: frozenset({"chat_template_kwargs"}),
    TrainingConfig: frozenset({"ema_config", "validation_config", "checkpoint_config", "dataloader_config",
                               "metrics_config", "profiler_config", "compile_config", "selective_ac",
                               "memory_budget_ac", "region_ac"}),
}


def cli_view(cls: type) -> list[dataclasses.Field]:
    """Fields of `cls` that the command line can carry."""
    hidden = PROGRAMMATIC_ONLY.get(cls, frozenset())
    names = {f.name for f in dataclasses.fields(cls)}
    stale = hidden - names
    if stale:
        raise ConfigError(f"PROGRAMMATIC_ONLY names stale fields of {cls.__name__}: {sorted(stale)}")
    return [f for f in dataclasses.fields(cls) if f.name not in hidden]


def _str2bool(v: str) -> bool:
    if v.lower() in ("1", "true", "yes", "y", "on"):
        return True
    if v.lower() in ("0", "false", "no", "n", "off"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


def _add_flag(parser: argparse.ArgumentParser, f: dataclasses.Field, hints: dict) -> None:
    tp = hints.get(f.name, str)
    origin, args = typing.get_origin(tp), typing.get_args(tp)
    kw: dict = {"dest": f.name, "default": argparse.SUPPRESS}
    if origin is typing.Union or (origin is not None and origin.__name__ == "UnionType"):
        non_none = [a for a in args if a is not type(None)]
        tp = non_none[0] if non_none else str
        origin, args = typing.get_origin(tp), typing.get_args(tp)
    if tp is bool:
        kw.update(type=_str2bool, nargs="?", const=True)
    elif origin in (list, tuple):
        inner = args[0] if args else str
        kw.update(type=inner if inner in (int, float, str) else str, nargs="*")
    elif origin is dict or tp is dict:
        kw.update(type=json.loads)
    elif tp in (int, float, str):
        kw.update(type=tp)
    else:
        kw.update(type=str)
    parser.add_argument(f"--{f.name}", **kw)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="llmtuner", description="B200-native hybrid-parallel LLM trainer",
                                     allow_abbrev=False)
    parser.add_argument("--config", dest="config", default=None,
                        help="YAML or JSON file; flags given on the command line override file values")
    seen: dict[str, type] = {}
    for cls in PARSER_GROUPS:
        hints = typing.get_type_hints(cls)
        grp = parser.add_argument_group(cls.__name__)
        for f in cli_view(cls):
            if f.name in seen:
                raise ConfigError(f"flag --{f.name} defined by both {seen[f.name].__name__} and {cls.__name__}")
            seen[f.name] = cls
            _add_flag(grp, f, hints)
    return parser
