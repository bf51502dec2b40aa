"""Forward, backward, gradient reduction, clipping and the optimizer step. The training loop above it never asks which
parallelism is on: the reductions follow from each parameter's `kind`."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .parallel import Mesh, all_reduce_

IGNORE = -100


def token_loss_sum(logits, targets):
    """Sum (not mean) of the token losses and the number of valid targets: the engine divides by the count of the whole
    accumulation window over all data ranks, so micro-batches with different numbers of valid tokens weigh correctly."""
    loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1), ignore_index=IGNORE, reduction="sum")
    return loss, (targets != IGNORE).sum()


class SyntheticData:
    """Uniform random tokens, a pure function of (seed, step, micro-batch): the cursor of a resume is the step number.
    The global micro-batch is generated whole and every data rank takes its rows, so a run on one rank with
    `batch_size x data_ranks` sequences sees the same tokens as the parallel run."""

    def __init__(self, cfg, mesh: Mesh):
        self.cfg, self.mesh = cfg, mesh

    def batch(self, step: int, micro: int):
        c, m = self.cfg, self.mesh
        g = torch.Generator().manual_seed(c.seed * 1_000_003 + step * 1009 + micro)
        ids = torch.randint(0, c.vocab_size, (c.batch_size * m.data_ranks, c.seq_len + 1), generator=g)
        mine = ids[m.data_rank * c.batch_size:(m.data_rank + 1) * c.batch_size]
        targets = mine[:, 1:].clone()
        targets[:, : (step + micro) % 3] = IGNORE                       # unequal numbers of valid tokens per micro-batch
        return mine[:, :-1].contiguous(), targets


class Engine:
    def __init__(self, cfg, mesh: Mesh, model, optimizer, scheduler):
        self.cfg, self.mesh, self.model, self.opt, self.sched = cfg, mesh, model, optimizer, scheduler
        self.device = torch.device(cfg.device)

    def reduce_gradients(self) -> None:
        m = self.mesh
        for p in self.model.parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)                            # an expert that got no token still joins the reduction
            all_reduce_(p.grad, m.dp_group if p.kind == "expert" else m.data_group)

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm with every element counted once: replicated tensors as they are, shards summed over the axes
        they are cut along."""
        m = self.mesh
        sq = {"dense": torch.zeros((), device=self.device), "tp": torch.zeros((), device=self.device),
              "expert": torch.zeros((), device=self.device)}
        for p in self.model.parameters():
            sq[p.kind] += p.grad.float().pow(2).sum()
        all_reduce_(sq["tp"], m.tp_group)
        all_reduce_(sq["expert"], m.tp_group)
        all_reduce_(sq["expert"], m.ep_group)
        return (sq["dense"] + sq["tp"] + sq["expert"]).sqrt()

    def train_step(self, data: SyntheticData, step: int) -> dict:
        cfg, m = self.cfg, self.mesh
        self.opt.zero_grad(set_to_none=True)
        loss_total = torch.zeros((), device=self.device)
        valid_total = torch.zeros((), device=self.device)
        for micro in range(cfg.gradient_accumulation_steps):
            tokens, targets = (t.to(self.device) for t in data.batch(step, micro))
            loss, valid = token_loss_sum(self.model(tokens), targets)
            loss.backward()                                            # gradients of the SUM; normalised once below
            loss_total += loss.detach()
            valid_total += valid
        all_reduce_(loss_total, m.data_group)
        all_reduce_(valid_total, m.data_group)
        self.reduce_gradients()
        for p in self.model.parameters():
            p.grad.div_(valid_total)
        norm = self.grad_norm()
        if cfg.max_grad_norm > 0:
            coef = torch.clamp(cfg.max_grad_norm / (norm + 1e-6), max=1.0)
            for p in self.model.parameters():
                p.grad.mul_(coef)
        self.opt.step()
        self.sched.step()
        return {"loss": (loss_total / valid_total).item(), "grad_norm": norm.item(), "lr": self.sched.get_last_lr()[0]}


def warmup_constant(cfg):
    """Linear warm-up, then constant: the curve does not depend on the target step count, so a resume may raise it."""
    def f(step):
        return (step + 1) / cfg.warmup_steps if step < cfg.warmup_steps else 1.0
    return f
