"""Loader of the in-tree sm_100a kernel library (`torchllmtuner_b200/_C.so`).

On a machine with a GPU the CUDA path is the only path for CUDA tensors: a missing or unloadable extension raises
`EnvironmentUnsupportedError` instead of falling back to library kernels.
"""
from __future__ import annotations

import importlib.util
import os
import threading

from ..errors import EnvironmentUnsupportedError, KernelStatusError

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_PKG, "_C.so")
_lock = threading.Lock()
_mod = None
_err: Exception | None = None

STATUS_NAMES = {1: "bounded mbarrier wait expired", 2: "bounded flag wait expired", 3: "capacity overflow",
                4: "bad argument detected on the device"}


def load(build_if_missing: bool = True):
    """Import the extension module, building it first when the `.so` is absent."""
    global _mod, _err
    if _mod is not None:
        return _mod
    with _lock:
        if _mod is not None:
            return _mod
        try:
            if not os.path.exists(_SO) and build_if_missing:
                from ..csrc.build import build
                build()
            import torch  # noqa: F401  (libtorch symbols must be loaded first)
            spec = importlib.util.spec_from_file_location("torchllmtuner_b200._C", _SO)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _mod = mod
        except Exception as e:  # noqa: BLE001
            _err = e
            raise EnvironmentUnsupportedError(f"sm_100a kernel library could not be loaded from {_SO}: {e}") from e
    return _mod


def available() -> bool:
    try:
        load(build_if_missing=False)
        return True
    except EnvironmentUnsupportedError:
        return False


def status_word(device):
    """The kernels' status word as a device tensor, or None when `device` is not CUDA (nothing can have written one)."""
    import torch
    if torch.device(device).type != "cuda":
        return None
    return load().status_tensor()


def so_path() -> str:
    return _SO


def check_status(where: str = "") -> None:
    """Read the device status word (synchronises) and raise `KernelStatusError` when a kernel reported a failure."""
    code, site, block, extra = load().read_status(True)
    if code != 0:
        raise KernelStatusError(where or "sm_100a kernel", int(code),
                                f"{STATUS_NAMES.get(int(code), 'unknown')} at site {site}, block {block}, extra {extra}")
