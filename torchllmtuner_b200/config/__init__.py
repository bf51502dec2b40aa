"""L3 configuration: thirteen dataclass groups, the `LLMTunerConfig` aggregate and the CLI view."""
from .checkpoint_config import CheckpointConfig  # noqa: F401
from .cli_config import PARSER_GROUPS, PROGRAMMATIC_ONLY, build_parser, cli_view  # noqa: F401
from .data_config import DataloaderConfig  # noqa: F401
from .llmtuner_config import LLMTunerConfig  # noqa: F401
from .model_config import ModelConfig  # noqa: F401
from .observability_config import MetricsConfig, ProfilerConfig  # noqa: F401
from .optimizer_config import LRSchedulerConfig, OptimizerConfig, ParamGroupConfig  # noqa: F401
from .parallel_config import (ContextParallelConfig, ExpertParallelConfig, FSDPConfig, ParallelConfig,  # noqa: F401
                              TensorParallelConfig)
from .training_config import (CompileConfig, EMAConfig, MemoryBudgetACConfig, RegionACConfig, SelectiveACConfig,  # noqa: F401
                              TrainingConfig, ValidationConfig, resolve_batch_size_per_rank)
from .utils import rebuild_config_group, require_bool, require_integer_at_least, require_string_patterns  # noqa: F401
