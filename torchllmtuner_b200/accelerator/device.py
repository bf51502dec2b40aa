"""Device selection (reference: llmtuner/accelerator/device.py:49-178). This build targets CUDA (sm_100a) with a CPU
path for tests: cuda -> nccl, cpu -> gloo."""
from __future__ import annotations

import os

import torch

_BACKENDS = {"cuda": "nccl", "cpu": "gloo"}


def get_device_type() -> str:
    forced = os.environ.get("LLMTUNER_DEVICE")
    if forced in _BACKENDS:
        return forced
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_distributed_backend(device_type: str | None = None) -> str:
    return _BACKENDS[device_type or get_device_type()]


def get_env_dist_info() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)))


def get_current_device() -> torch.device:
    if get_device_type() == "cuda":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def set_device(local_rank: int) -> torch.device:
    if get_device_type() == "cuda":
        torch.cuda.set_device(local_rank % max(1, torch.cuda.device_count()))
    return get_current_device()


def should_use_pin_memory() -> bool:
    return get_device_type() == "cuda"


def is_cuda_available() -> bool:
    return torch.cuda.is_available()


def get_max_cuda_memory(device=None) -> int:
    if not torch.cuda.is_available():
        return 0
    return torch.cuda.get_device_properties(device or torch.cuda.current_device()).total_memory
