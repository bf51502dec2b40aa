"""Named kernel registry keyed by (name, device_type) with an explicit CPU fallback
(reference: llmtuner/kernel/registry.py:1-103). The built-in ops register themselves at import."""
from __future__ import annotations

from typing import Callable

_REGISTRY: dict[tuple[str, str], Callable] = {}


def register_kernel(name: str, device_type: str, fn: Callable | None = None):
    def deco(f):
        _REGISTRY[(name, device_type)] = f
        return f
    return deco(fn) if fn is not None else deco


def get_kernel(name: str, device_type: str, allow_cpu_fallback: bool = False) -> Callable:
    key = (name, device_type)
    if key in _REGISTRY:
        return _REGISTRY[key]
    if allow_cpu_fallback and (name, "cpu") in _REGISTRY:
        return _REGISTRY[(name, "cpu")]
    raise KeyError(f"no kernel {name!r} registered for device {device_type!r}")


def dispatch_kernel(name: str, tensor, *args, **kwargs):
    return get_kernel(name, tensor.device.type)(tensor, *args, **kwargs)


def _register_builtins():
    from . import functional as F
    from . import reference as R
    for n in ("linear", "rms_norm", "add_rms_norm", "qk_norm_rope", "swiglu", "attention", "cross_entropy_sum",
              "linear_cross_entropy_sum"):
        register_kernel(n, "cuda", getattr(F, n))
        register_kernel(n, "cpu", getattr(R, n) if hasattr(R, n) else getattr(F, n))


_register_builtins()
