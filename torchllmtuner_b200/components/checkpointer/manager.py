"""The checkpoint manager interface and its disabled form: the object a trainer holds when `checkpoint.enable` is off.
Every call is a no-op; `dcp_manager.DistributedCheckpointManager` overrides them when checkpointing is on."""
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
