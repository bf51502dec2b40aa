"""Loss services (reference: llmtuner/components/loss.py:35-421).

All losses are SUMS in fp32 over local tokens; the trainer divides by the global valid-token count.
  cross_entropy_loss                full logits (picks the vocab-parallel form when logits are a vocab shard)
  chunked_lm_head_cross_entropy     head projection + CE chunk by chunk, logits never materialised
  LossParallelCrossEntropy          vocab-sharded logits: one fused exchange of (max, sum-exp, target logit)
  vocab_parallel_entropy, compute_logprobs, mse_loss
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..ops import IGNORE_INDEX


def cross_entropy_loss(logits: torch.Tensor, targets: torch.Tensor, vocab_group=None, vocab_start: int = 0) -> torch.Tensor:
    if vocab_group is not None and dist.is_initialized() and dist.get_world_size(vocab_group) > 1:
        return LossParallelCrossEntropy.apply(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), vocab_group, vocab_start)
    return ops.cross_entropy_sum(logits, targets)


def chunked_lm_head_cross_entropy(hidden: torch.Tensor, head_weight: torch.Tensor, targets: torch.Tensor, num_chunks: int = 8):
    return ops.linear_cross_entropy_sum(hidden, head_weight, targets, num_chunks)


class LossParallelCrossEntropy(torch.autograd.Function):
    """Cross-entropy over vocab-sharded logits [T, V/tp]. Forward exchanges three per-token scalars (running max,
    sum of exponentials, target logit) in ONE all-reduce pass pair (max, then a packed sum) instead of the three
    separate all-reduces of the reference (loss.py:176-196); backward needs no communication."""

    @staticmethod
    def forward(ctx, logits, targets, group, vocab_start):
        lf = logits.float()
        V = lf.shape[-1]
        local_max = lf.max(dim=-1).values
        gmax = local_max.clone()
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        ex = torch.exp(lf - gmax[:, None])
        local = targets - vocab_start
        mine = (local >= 0) & (local < V) & (targets != IGNORE_INDEX)
        tl = torch.where(mine, lf.gather(-1, local.clamp(0, V - 1)[:, None]).squeeze(-1), torch.zeros_like(gmax))
        packed = torch.stack([ex.sum(-1), tl], dim=0)
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        sumexp, tlogit = packed[0], packed[1]
        valid = targets != IGNORE_INDEX
        loss = torch.where(valid, torch.log(sumexp) + gmax - tlogit, torch.zeros_like(gmax)).sum()
        ctx.save_for_backward(ex / sumexp[:, None], local, mine, valid)
        ctx.in_dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        p, local, mine, valid = ctx.saved_tensors
        grad = p.clone()
        idx = local.clamp(0, p.shape[-1] - 1)[:, None]
        grad.scatter_add_(-1, idx, -mine.to(grad.dtype)[:, None])
        grad = grad * valid.to(grad.dtype)[:, None] * g
        return grad.to(ctx.in_dtype), None, None, None


def vocab_parallel_entropy(logits: torch.Tensor, group=None) -> torch.Tensor:
    """Per-token entropy of the softmax over (possibly vocab-sharded) logits."""
    lf = logits.float()
    m = lf.max(-1).values
    if group is not None and dist.is_initialized():
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
    ex = torch.exp(lf - m[:, None])
    s, sx = ex.sum(-1), (ex * lf).sum(-1)
    if group is not None and dist.is_initialized():
        pk = torch.stack([s, sx])
        dist.all_reduce(pk, group=group)
        s, sx = pk[0], pk[1]
    return torch.log(s) + m - sx / s


def compute_logprobs(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    lp = torch.log_softmax(logits.float(), dim=-1)
    t = targets.clamp_min(0)
    out = lp.gather(-1, t[..., None]).squeeze(-1)
    return torch.where(targets == IGNORE_INDEX, torch.zeros_like(out), out)


def mse_loss(pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    return (pred.float() - target.float()).pow(2).sum()


class LossFunctions:
    """The pair the engine needs: a logits loss and a chunked head loss, both returning sums. With a vocabulary-parallel
    head (`head` is then the `VocabParallelHead` module of the model) the loss always takes the hidden-state path."""

    def __init__(self, num_chunks: int = 0, vocab_group=None, vocab_start: int = 0, head=None):
        self.num_chunks, self.vocab_group, self.vocab_start = num_chunks, vocab_group, vocab_start
        self.head = head

    @property
    def chunked(self) -> bool:
        return self.num_chunks > 0 or self.head is not None

    def from_logits(self, logits, targets):
        return cross_entropy_loss(logits, targets, self.vocab_group, self.vocab_start)

    def from_hidden(self, hidden, head_weight, targets):
        if self.head is not None:
            from ..parallel.vocab_parallel import vocab_parallel_head_loss
            return vocab_parallel_head_loss(hidden, self.head, targets, max(1, self.num_chunks))
        return chunked_lm_head_cross_entropy(hidden, head_weight, targets, max(1, self.num_chunks))


def validate_loss_sum(loss: torch.Tensor) -> None:
    if loss.dim() != 0 or loss.dtype != torch.float32:
        raise ValueError(f"loss functions must return an fp32 scalar sum, got {tuple(loss.shape)} {loss.dtype}")
