"""Gradient services between backward and the optimizer (reference: llmtuner/trainer/runtime/gradients.py:70-372).
The sums themselves live with the sharding runtime, which owns the flat gradient buffers: tensor-parallel-replicated
parameters in `parallel/fsdp.py::reduce_grads`, parameters excluded from sharding in `wait_reductions`, the clip coefficient
in `components/optimizer/container.py::GradientClipper`. What is left here is the finite verdict that raises on every rank."""
from __future__ import annotations

from ...components.optimizer import check_finite


def check_step_condition(clipper, loss_value: float | None = None) -> None:
    """Raises `LLMTunerError` on every rank when the global gradient norm or the loss is not finite; the update kernels
    have skipped the step in that case (the clip coefficient they read is NaN)."""
    check_finite(clipper, loss_value)
