"""Validation loop (reference: llmtuner/trainer/runtime/validation.py:54-415): eval mode, RNG preserved, training
mode restored; runs at step 1 and every `freq` steps for `steps` batches of the validation stream."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...datasets import build_dataloader
from ...utils.seeding import preserve_rng_state


class Validator:
    def __init__(self, config, trainer):
        self.cfg = config.training.validation_config
        self.trainer = trainer
        t = config.training
        dc = t.dataloader_config
        if self.cfg.dataset is not None:
            import copy
            dc = copy.copy(dc)
            dc.dataset = self.cfg.dataset
        arch = trainer.model.config
        self.make_loader = lambda: build_dataloader(dc, vocab_size=arch.vocab_size, global_batch=t.global_batch_size,
                                                    seq_len=t.max_seq_len, seed=t.seed + 1, dp_rank=trainer.dp_rank,
                                                    dp_degree=trainer.dp_degree, rows_per_rank=trainer.rows_per_rank,
                                                    pin_memory=False, split="validation")
        self.history: list[tuple[int, float]] = []

    def should_validate(self, step: int) -> bool:
        return step == 1 or step % self.cfg.freq == 0

    def validate(self, step: int) -> float:
        tr = self.trainer
        n = self.cfg.steps if self.cfg.steps > 0 else 1
        tot = torch.zeros(2, dtype=torch.float64, device=tr.env.device)
        with preserve_rng_state():
            it = iter(self.make_loader())
            for _ in range(n):
                try:
                    b = next(it)
                except StopIteration:
                    break
                loss, valid = tr.engine.evaluate(b)
                tot[0] += loss.double()
                tot[1] += valid
        g = tr.env.topo.get_group("loss")
        if g is not None:
            dist.all_reduce(tot, group=g)
        val = float(tot[0] / tot[1].clamp_min(1))
        self.history.append((step, val))
        tr.logger.info(f"validation step {step}: loss {val:.4f}")
        return val
