"""Argument contracts of the kernel facade (reference: llmtuner/kernel/validation.py:1-133): shape, dtype, device and
alignment checks that turn a bad call into a `ConfigError` with the operand's name instead of a failed launch."""
from __future__ import annotations

import torch

from ..errors import ConfigError


def require_tensor(x, name: str, *, dims: int | None = None, dtype=None, device_type: str | None = None) -> torch.Tensor:
    if not isinstance(x, torch.Tensor):
        raise ConfigError(f"{name} must be a tensor, got {type(x).__name__}")
    if dims is not None and x.dim() != dims:
        raise ConfigError(f"{name} must have {dims} dimensions, got shape {tuple(x.shape)}")
    if dtype is not None and x.dtype not in (dtype if isinstance(dtype, (tuple, list)) else (dtype,)):
        raise ConfigError(f"{name} must have dtype {dtype}, got {x.dtype}")
    if device_type is not None and x.device.type != device_type:
        raise ConfigError(f"{name} must live on {device_type}, got {x.device}")
    return x


def require_same_device(*named) -> None:
    devs = {t.device for _, t in named}
    if len(devs) > 1:
        raise ConfigError("operands on different devices: " + ", ".join(f"{n}={t.device}" for n, t in named))


def require_last_dim_contiguous(x: torch.Tensor, name: str, multiple: int = 8) -> None:
    """The tcgen05 / TMA paths need a unit inner stride, 16-byte aligned rows and a 16-byte aligned base."""
    if x.stride(-1) != 1:
        raise ConfigError(f"{name} must be contiguous in its last dimension")
    if x.dim() >= 2 and x.stride(-2) % multiple:
        raise ConfigError(f"{name}: row stride {x.stride(-2)} is not a multiple of {multiple} elements")
    if x.data_ptr() % 16:
        raise ConfigError(f"{name}: base address is not 16-byte aligned")


def validate_attention_inputs(q, k, v) -> None:
    """q [T, Hq, d], k [S, Hkv, d], v [S, Hkv, dv]; Hq a multiple of Hkv; on the device d and dv at most 256."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        require_tensor(t, n, dims=3)
    require_same_device(("q", q), ("k", k), ("v", v))
    if k.shape[:2] != v.shape[:2]:
        raise ConfigError(f"k {tuple(k.shape)} and v {tuple(v.shape)} must agree in rows and heads")
    if q.shape[2] != k.shape[2] or q.shape[1] % k.shape[1]:
        raise ConfigError(f"q {tuple(q.shape)} is not compatible with k {tuple(k.shape)} (head_dim equal, Hq % Hkv == 0)")


def validate_rms_norm_inputs(x, weight) -> None:
    require_tensor(x, "x")
    require_tensor(weight, "weight", dims=1)
    if x.shape[-1] != weight.shape[0]:
        raise ConfigError(f"weight has {weight.shape[0]} elements, the normalised dimension has {x.shape[-1]}")


def validate_router_inputs(logits, k: int) -> None:
    require_tensor(logits, "logits", dims=2)
    if not (1 <= k <= logits.shape[1]):
        raise ConfigError(f"top-k {k} must be in [1, {logits.shape[1]}]")
