"""Training config group and its small nested groups (reference: llmtuner/config/training_config.py:31-315,
compile_config.py, activation_checkpoint_config.py, ema_config.py, validation_config.py)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import ConfigError
from .checkpoint_config import CheckpointConfig
from .data_config import DataloaderConfig
from .observability_config import MetricsConfig, ProfilerConfig
from .utils import require_choice, require_integer_at_least

AC_MODES = ("none", "full", "selective", "memory_budget", "region")


@dataclass
class CompileConfig:
    """`compile` here means CUDA-graph capture of the per-block launch sequence; no tracing compiler is used."""
    per_block: bool = True
    backend: str = "cudagraph"
    enable_async_tensor_parallel: bool = False
    enable_sdc: bool = False      # silent-data-corruption guard: non-finite check on block outputs


@dataclass
class SelectiveACConfig:
    force_recompute_mm_shapes_by_fqns: list[str] = field(default_factory=list)
    preserve_rng_state: bool = True
    determinism_check: str = "default"
    debug: bool = False
    # "op": every block is checkpointed with the per-op policy (attention and every other linear keep their outputs, the
    # rest is recomputed; linears named by force_recompute_mm_shapes_by_fqns are always recomputed). "block": every
    # `save_every_nth_block`-th block keeps all its activations and the others recompute everything.
    selective_ac_policy: str = "op"
    save_every_nth_block: int = 2

    def __post_init__(self):
        require_choice("selective_ac_policy", self.selective_ac_policy, ("op", "block"))


@dataclass
class MemoryBudgetACConfig:
    memory_budget: float = 0.5

    def __post_init__(self):
        if not 0.0 <= self.memory_budget <= 1.0:
            raise ConfigError("memory_budget must be in [0, 1]")


@dataclass
class RegionACConfig:
    save_regions: list[str] = field(default_factory=list)
    recompute_regions: list[str] = field(default_factory=list)
    determinism_check: str = "default"
    preserve_rng_state: bool = True


@dataclass
class EMAConfig:
    decay: float | None = None
    half_life_fraction: float = 0.05
    start_step: int = 0
    step_bias: int = 0
    update_every_n_steps: int = 1
    buffer_patterns: list[str] = field(default_factory=list)

    def __post_init__(self):
        if self.decay is not None and not 0.0 <= self.decay < 1.0:
            raise ConfigError("ema decay must be in [0, 1)")
        if not 0.0 < self.half_life_fraction <= 1.0:
            raise ConfigError("half_life_fraction must be in (0, 1]")
        require_integer_at_least("update_every_n_steps", self.update_every_n_steps, 1)


@dataclass
class ValidationConfig:
    freq: int = 10
    steps: int = -1
    dataset: str | None = None

    def __post_init__(self):
        require_integer_at_least("freq", self.freq, 1)


def resolve_batch_size_per_rank(global_batch_size: int, dp_degree: int, accumulation: int = 1) -> int:
    """Rows per DP rank per microbatch; the global batch must divide evenly."""
    denom = dp_degree * accumulation
    if global_batch_size % denom:
        raise ConfigError(f"global_batch_size {global_batch_size} is not divisible by dp*accumulation = {denom}")
    return global_batch_size // denom


@dataclass
class TrainingConfig:
    global_batch_size: int = 8
    max_seq_len: int = 64
    steps: int = 20
    seed: int = 42
    compile: bool = False
    compile_config: CompileConfig = field(default_factory=CompileConfig)
    activation_checkpoint_mode: str = "none"
    activation_swap: bool = False
    activation_swap_sync_release: bool = False
    activation_swap_max_host_bytes: int = 0
    selective_ac: SelectiveACConfig = field(default_factory=SelectiveACConfig)
    memory_budget_ac: MemoryBudgetACConfig = field(default_factory=MemoryBudgetACConfig)
    region_ac: RegionACConfig = field(default_factory=RegionACConfig)
    deterministic: bool = True
    detect_anomaly: bool = False
    max_norm: float = 1.0
    grad_norm_precision: str = "float32"
    gc_freq: int = 50
    gradient_accumulation_steps: int = 1
    overlap_optimizer_step: bool = True          # the training loop lets the parameter update run under the next forward (one shard rank)
    chunked_loss_num_chunks: int = 0
    dump_folder: str = "./outputs"
    checkpoint_config: CheckpointConfig = field(default_factory=CheckpointConfig)
    dataloader_config: DataloaderConfig = field(default_factory=DataloaderConfig)
    metrics_config: MetricsConfig = field(default_factory=MetricsConfig)
    profiler_config: ProfilerConfig = field(default_factory=ProfilerConfig)
    ema_config: EMAConfig | None = None
    validation_config: ValidationConfig | None = None

    def __post_init__(self):
        for n, lo in (("global_batch_size", 1), ("max_seq_len", 2), ("steps", 0), ("gc_freq", 1),
                      ("gradient_accumulation_steps", 1), ("chunked_loss_num_chunks", 0)):
            require_integer_at_least(n, getattr(self, n), lo)
        require_choice("activation_checkpoint_mode", self.activation_checkpoint_mode, AC_MODES)
        require_choice("grad_norm_precision", self.grad_norm_precision, ("float32", "parameter"))
        if not self.max_norm > 0:
            raise ConfigError("max_norm must be > 0")
        if self.activation_swap and self.activation_checkpoint_mode == "full":
            raise ConfigError("activation_swap offloads saved activations; with full recompute there are none to offload")
        for name, cls in (("compile_config", CompileConfig), ("selective_ac", SelectiveACConfig),
                          ("memory_budget_ac", MemoryBudgetACConfig), ("region_ac", RegionACConfig),
                          ("checkpoint_config", CheckpointConfig), ("dataloader_config", DataloaderConfig),
                          ("metrics_config", MetricsConfig), ("profiler_config", ProfilerConfig),
                          ("ema_config", EMAConfig), ("validation_config", ValidationConfig)):
            v = getattr(self, name)
            if isinstance(v, dict):
                setattr(self, name, cls(**v))
