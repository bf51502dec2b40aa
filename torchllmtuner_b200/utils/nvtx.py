"""NVTX ranges around the phases of a step (forward/backward of a micro-batch, optimizer, checkpoint), visible in
Nsight Systems / torch.profiler timelines. Off by default: `enable(True)` is called when profiling is configured."""
from __future__ import annotations

import contextlib

import torch

_ENABLED = False


def enable(flag: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(flag) and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _ENABLED:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
