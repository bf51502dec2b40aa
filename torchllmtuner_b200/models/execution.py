"""Execution contracts between a model and the trainer (reference: llmtuner/models/execution.py:10-108).

A model's `prepare_inputs` returns a dict here (`tokens`, `targets`, `positions`, `attn_meta`, optional multimodal fields),
its forward returns hidden states `[T, D]` (with `skip_lm_head=True`) or logits `[T, V]`. The engine checks both
boundaries on geometry only (shapes, dtypes, devices; never tensor contents), so that a model that shards or packs its
tokens wrongly fails at the boundary with a message instead of deep inside a kernel. `ModelExecutionCapabilities` is
what a model class declares it can produce; the execution layout may only ask for a declared output kind.
"""
from __future__ import annotations

from dataclasses import dataclass
from math import prod

import torch

REQUIRED_INPUT_KEYS = ("tokens", "targets", "positions", "attn_meta")
_INDEX_DTYPES = (torch.int32, torch.int64)


def validate_prepared_model_inputs(prepared) -> dict:
    """One target and one position per local token, all on one device; returns the dict."""
    if not isinstance(prepared, dict):
        raise TypeError(f"prepare_inputs must return a dict, got {type(prepared).__name__}")
    for k in REQUIRED_INPUT_KEYS:
        if k not in prepared:
            raise KeyError(f"prepared model inputs lack {k!r}")
    tokens, targets, positions = prepared["tokens"], prepared["targets"], prepared["positions"]
    for name, t in (("tokens", tokens), ("targets", targets), ("positions", positions)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"prepared {name} must be a tensor")
        if t.dtype not in _INDEX_DTYPES:
            raise TypeError(f"prepared {name} must hold integer indices, got {t.dtype}")
        if t.dim() not in (1, 2):
            raise ValueError(f"prepared {name} must have one or two dimensions, got {t.dim()}")
    if tokens.numel() != targets.numel():
        raise ValueError(f"prepared tokens ({tokens.numel()}) and targets ({targets.numel()}) must have equal token counts")
    if tokens.dim() == targets.dim() == 2 and tokens.shape != targets.shape:
        raise ValueError("prepared tokens and targets disagree on the token axis order")
    if positions.numel() % max(1, tokens.numel()) and tokens.numel() % max(1, positions.numel()):
        raise ValueError(f"prepared positions ({positions.numel()}) do not tile the tokens ({tokens.numel()})")
    if tokens.device != targets.device:
        raise ValueError("prepared tokens and targets must be on the same device")
    return prepared


def validate_training_output(output: torch.Tensor, targets: torch.Tensor, *, output_width: int | None = None) -> None:
    """The forward result has one floating-point row per target token (flat or [B, S] rows), on the targets' device."""
    if not isinstance(output, torch.Tensor) or not isinstance(targets, torch.Tensor):
        raise TypeError("training output and targets must be tensors")
    if output.dim() < 2 or output.shape[-1] <= 0:
        raise ValueError(f"training output must be [tokens..., width], got {tuple(output.shape)}")
    if not output.is_floating_point():
        raise TypeError(f"training output must be floating point, got {output.dtype}")
    if targets.dim() not in (1, 2) or targets.dtype not in _INDEX_DTYPES:
        raise TypeError("training targets must hold one or two integer token axes")
    if output.device != targets.device:
        raise ValueError(f"training output on {output.device}, targets on {targets.device}")
    if prod(output.shape[:-1]) != targets.numel():
        raise ValueError(f"training output has {prod(output.shape[:-1])} rows for {targets.numel()} targets")
    if output.dim() > 2 and targets.dim() > 1 and tuple(output.shape[:-1]) != tuple(targets.shape):
        raise ValueError("training output and targets disagree on the token axis order")
    if output_width is not None and output.shape[-1] != output_width:
        raise ValueError(f"training output width {output.shape[-1]} differs from the declared width {output_width}")


@dataclass(frozen=True)
class ModelExecutionCapabilities:
    """Output kinds a model supports. Hidden output is the `skip_lm_head=True` call."""
    logits: bool = True
    hidden_states: bool = False
    hidden_size: int | None = None
    vocab_size: int | None = None
    packed_documents: bool = True          # accepts rows packed from several documents (cu_seqlens / attention metadata)

    def __post_init__(self):
        if type(self.logits) is not bool or type(self.hidden_states) is not bool:
            raise TypeError("execution capabilities must be booleans")
        if self.hidden_size is not None and (type(self.hidden_size) is not int or self.hidden_size <= 0):
            raise ValueError("declared hidden size must be a positive integer")
        if self.hidden_size is not None and not self.hidden_states:
            raise ValueError("a declared hidden size needs hidden-state output support")

    def require(self, kind: str) -> None:
        ok = self.hidden_states if kind == "hidden" else self.logits
        if not ok:
            raise ValueError(f"the model does not produce {kind} output")

    def width(self, kind: str) -> int | None:
        return self.hidden_size if kind == "hidden" else self.vocab_size


def capabilities_of(model) -> ModelExecutionCapabilities:
    """A model may declare `execution_capabilities`; decoders of this package that take `skip_lm_head` support both kinds."""
    cap = getattr(model, "execution_capabilities", None)
    if isinstance(cap, ModelExecutionCapabilities):
        return cap
    cfg = getattr(model, "config", None)
    return ModelExecutionCapabilities(True, True, getattr(cfg, "hidden_size", None), getattr(cfg, "vocab_size", None))
