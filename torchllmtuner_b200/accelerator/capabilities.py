"""Named capability probes (reference: llmtuner/accelerator/capabilities.py:83-253)."""
from __future__ import annotations

import functools

import torch

from ..errors import EnvironmentUnsupportedError


@functools.lru_cache(maxsize=None)
def _probe(name: str) -> bool:
    if name == "cuda":
        return torch.cuda.is_available()
    if name == "sm100":
        return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10
    if name == "kernel_library":
        from ..ops.cuda_ext import available
        return available()
    if name == "symm_mem":
        import importlib                       # an `import torch.x` statement here would make `torch` local to the function
        try:
            importlib.import_module("torch.distributed._symmetric_memory")
            return torch.cuda.is_available()
        except ImportError:
            return False
    if name == "peer_access":
        if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
            return False
        return all(torch.cuda.can_device_access_peer(0, i) for i in range(1, torch.cuda.device_count()))
    if name == "dcp":
        import importlib
        try:
            importlib.import_module("torch.distributed.checkpoint")
            return True
        except ImportError:
            return False
    if name in ("tensorboard", "wandb", "safetensors", "tokenizers", "yaml"):
        import importlib.util
        return importlib.util.find_spec({"tensorboard": "tensorboard", "yaml": "yaml"}.get(name, name)) is not None
    raise KeyError(f"unknown capability {name!r}")


CAPABILITIES = ("cuda", "sm100", "kernel_library", "symm_mem", "peer_access", "dcp", "tensorboard", "wandb", "safetensors",
                "tokenizers", "yaml")


def has(name: str) -> bool:
    return _probe(name)


def require(name: str, why: str = "") -> None:
    if not has(name):
        raise EnvironmentUnsupportedError(f"capability {name!r} is required{': ' + why if why else ''}")


def report() -> dict[str, bool]:
    return {n: has(n) for n in CAPABILITIES}
