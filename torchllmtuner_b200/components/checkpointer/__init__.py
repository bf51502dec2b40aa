"""Checkpoint managers (reference: llmtuner/components/checkpointer/*)."""
from .manager import CheckpointManager, build_checkpointer  # noqa: F401
