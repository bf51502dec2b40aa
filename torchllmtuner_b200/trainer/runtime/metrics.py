"""Step metrics (reference: llmtuner/trainer/runtime/metrics.py:44-96): one device->host read per step of
[loss sum, gradient norm, valid tokens]; the loss sum is all-reduced over the loss mesh (batch x cp x tp) and divided by
the global valid-token count."""
from __future__ import annotations

import torch
import torch.distributed as dist


def build_step_metrics(step_loss: torch.Tensor, grad_norm: torch.Tensor, global_valid: torch.Tensor, reductions):
    """Returns (loss, grad_norm, global_tokens) as Python floats."""
    stats = torch.stack([step_loss, grad_norm.reshape(()).to(torch.float32), global_valid])
    if reductions.loss_group is not None:
        red = stats[:1].clone()
        dist.all_reduce(red, group=reductions.loss_group)     # sequence shards and batch shards both add up
        stats[0] = red[0]
    loss_sum, gnorm, gtok = (float(x) for x in stats.tolist())
    return loss_sum / max(1.0, gtok), gnorm, gtok
