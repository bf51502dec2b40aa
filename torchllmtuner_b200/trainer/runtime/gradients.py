"""Gradient services between backward and the optimizer (reference: llmtuner/trainer/runtime/gradients.py:70-372):
summing the gradients of parameters that tensor-parallel ranks hold in full, the clip coefficient, and the finite
verdict that raises on every rank before any parameter changes."""
from __future__ import annotations

from ...components.optimizer import check_finite
from ...parallel.tensor_parallel import allreduce_replicated_tp_grads


def reduce_replicated_gradients(params, topo) -> None:
    """Norm weights, q/k norms, routers and a replicated head see only their rank's tokens under TP + SP."""
    if topo.tp > 1:
        allreduce_replicated_tp_grads(params, topo.get_group("tp"))


def check_step_condition(clipper, loss_value: float | None = None) -> None:
    """Raises `LLMTunerError` on every rank when the global gradient norm or the loss is not finite; the update kernels
    have skipped the step in that case (the clip coefficient they read is NaN)."""
    check_finite(clipper, loss_value)
