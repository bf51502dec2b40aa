"""Life cycle: build mesh, model, optimizer, data; run steps; save and resume."""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import checkpoint
from .config import MiniConfig
from .engine import Engine, SyntheticData, warmup_constant
from .model import MiniQwen3Moe
from .parallel import Mesh


class MiniTrainer:
    def __init__(self, cfg: MiniConfig):
        world = dist.get_world_size() if dist.is_initialized() else 1
        cfg.validate(world)
        self.cfg = cfg
        self.mesh = Mesh(cfg.dp, cfg.ep, cfg.tp)
        self.model = MiniQwen3Moe(cfg, self.mesh).to(cfg.device)
        # the optimizer is created after every parameter has been cut to its final shard
        self.opt = torch.optim.AdamW(self.model.parameters(), lr=cfg.learning_rate, weight_decay=cfg.weight_decay)
        self.sched = torch.optim.lr_scheduler.LambdaLR(self.opt, warmup_constant(cfg))
        self.data = SyntheticData(cfg, self.mesh)
        self.engine = Engine(cfg, self.mesh, self.model, self.opt, self.sched)
        self.step = 0
        self.history: list[dict] = []

    def resume(self, folder: str) -> None:
        self.step = checkpoint.load(folder, self.mesh.rank, self.cfg, self.model, self.opt, self.sched)

    def save(self, folder: str) -> None:
        checkpoint.save(folder, self.mesh.rank, self.cfg, self.model, self.opt, self.sched, self.step)
        if dist.is_initialized():
            dist.barrier()

    def train(self, log=None) -> list[dict]:
        while self.step < self.cfg.steps:
            m = self.engine.train_step(self.data, self.step)
            self.step += 1
            m["step"] = self.step
            self.history.append(m)
            if log is not None and self.mesh.rank == 0:
                log(f"step {self.step}  loss {m['loss']:.4f}  grad_norm {m['grad_norm']:.4f}  lr {m['lr']:.2e}")
        return self.history
