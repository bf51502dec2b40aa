"""Pipeline parallelism (experiment; own CLI: `python -m torchllmtuner_b200.experiments.pipeline_parallel.cli`)."""
from .partition import split_layers  # noqa: F401
from .runtime import PipelineTrainer  # noqa: F401
from .schedules import build_schedule  # noqa: F401
