"""Checkpoint manager placeholder wired into the trainer; the full implementation lives in `dcp_manager.py`."""
from __future__ import annotations


class CheckpointManager:
    enabled = False

    def load(self, step: int = -1) -> bool:
        return False

    def save(self, step: int, last_step: bool = False, force: bool = False) -> None:
        pass

    def maybe_wait_for_staging(self) -> None:
        pass

    def wait(self) -> None:
        pass

    def close(self) -> None:
        pass


def build_checkpointer(config, trainer) -> CheckpointManager:
    if not config.training.checkpoint_config.enable:
        return CheckpointManager()
    from .dcp_manager import DistributedCheckpointManager
    return DistributedCheckpointManager(config, trainer)
