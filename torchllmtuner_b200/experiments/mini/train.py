"""`python -m torchllmtuner_b200.experiments.mini.train --device cpu --steps 3 [--tp 2 --ep 2 --dp 2] [--checkpoint DIR]
[--resume DIR]`; under torchrun the process group is created from the launcher's environment (gloo on CPU, NCCL on
CUDA)."""
from __future__ import annotations

import argparse
import os
from dataclasses import fields

import torch
import torch.distributed as dist

from .config import MiniConfig
from .trainer import MiniTrainer


def main(argv=None) -> list[dict]:
    ap = argparse.ArgumentParser(prog="mini")
    for f in fields(MiniConfig):
        if f.name.isupper():
            continue
        ap.add_argument("--" + f.name.replace("_", "-"), type=type(f.default), default=f.default)
    ap.add_argument("--checkpoint", default=None, help="folder to save the final state to")
    ap.add_argument("--resume", default=None, help="folder to resume from")
    a = vars(ap.parse_args(argv))
    ckpt, resume = a.pop("checkpoint"), a.pop("resume")
    cfg = MiniConfig(**a)
    if cfg.device.startswith("cuda") and not torch.cuda.is_available():
        raise SystemExit("--device cuda was asked for but no CUDA device is visible; pass --device cpu to run on the host")
    started = False
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and not dist.is_initialized():
        if cfg.device.startswith("cuda"):
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            cfg.device = f"cuda:{os.environ.get('LOCAL_RANK', '0')}"
        dist.init_process_group("nccl" if cfg.device.startswith("cuda") else "gloo")
        started = True
    try:
        tr = MiniTrainer(cfg)
        if resume:
            tr.resume(resume)
        hist = tr.train(log=print)
        if ckpt:
            tr.save(ckpt)
        return hist
    finally:
        if started:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
