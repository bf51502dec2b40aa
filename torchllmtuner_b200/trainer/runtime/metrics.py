"""Step metrics (reference: llmtuner/trainer/runtime/metrics.py:44-96): one device->host read per step of
[loss sum, gradient norm, valid tokens]; the loss sum is all-reduced over the loss mesh (batch x cp x tp) and divided by
the global valid-token count."""
from __future__ import annotations

import torch
import torch.distributed as dist


def build_step_metrics(step_loss: torch.Tensor, grad_norm: torch.Tensor, global_valid: torch.Tensor, reductions, status=None):
    """Returns (loss, grad_norm, global_tokens) as Python floats. With `status` (the kernels' device status word) its
    code rides in the same read and is returned as a fourth value: non-zero means that some kernel of this step gave up
    a bounded wait or refused its arguments."""
    parts = [step_loss, grad_norm.reshape(()).to(torch.float32), global_valid]
    if status is not None:
        parts.append(status.reshape(-1)[0].to(torch.float32))
    stats = torch.stack(parts)
    if reductions.loss_group is not None:
        red = stats[:1].clone()
        dist.all_reduce(red, group=reductions.loss_group)     # sequence shards and batch shards both add up
        stats[0] = red[0]
    loss_sum, gnorm, gtok, *code = (float(x) for x in stats.tolist())
    if status is not None:
        return loss_sum / max(1.0, gtok), gnorm, gtok, int(code[0])
    return loss_sum / max(1.0, gtok), gnorm, gtok
