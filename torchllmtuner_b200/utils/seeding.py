"""Seeding and determinism (reference: llmtuner/utils/seeding.py:24-240)."""
from __future__ import annotations

import contextlib
import hashlib
import os
import random

import numpy as np
import torch


def derive_distinct_seed(base_seed: int, *coords: int) -> int:
    """A per-rank seed that differs for every coordinate tuple and is stable across runs."""
    h = hashlib.sha256(("/".join(str(int(c)) for c in (base_seed, *coords))).encode()).digest()
    return int.from_bytes(h[:8], "little") % (2**63 - 1)


def seed_everything(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def set_deterministic_algorithms(enabled: bool, detect_anomaly: bool = False) -> None:
    """Deterministic mode: deterministic torch algorithms, cuDNN deterministic and the cuBLAS
    workspace setting; uninitialised-memory filling is switched off because it races with side
    streams (reference: utils/seeding.py:145-164)."""
    if enabled:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    torch.use_deterministic_algorithms(bool(enabled), warn_only=True)
    torch.backends.cudnn.deterministic = bool(enabled)
    torch.backends.cudnn.benchmark = not enabled
    if hasattr(torch.utils, "deterministic"):
        torch.utils.deterministic.fill_uninitialized_memory = False
    torch.autograd.set_detect_anomaly(bool(detect_anomaly))


@contextlib.contextmanager
def preserve_rng_state(devices=None):
    cpu = torch.get_rng_state()
    cuda = torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None
    py, npst = random.getstate(), np.random.get_state()
    try:
        yield
    finally:
        torch.set_rng_state(cpu)
        if cuda is not None:
            torch.cuda.set_rng_state_all(cuda)
        random.setstate(py)
        np.random.set_state(npst)
