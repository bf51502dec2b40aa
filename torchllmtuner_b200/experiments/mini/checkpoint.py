"""Per-rank `state-<rank>.pt`, replaced atomically: model shard, optimizer, scheduler, step, RNG state and the
configuration signature. A resume may raise the target number of steps; any other change of the configuration (model,
mesh, batch, schedule, seed) is refused."""
from __future__ import annotations

import os

import torch


def save(folder: str, rank: int, cfg, model, opt, sched, step: int) -> None:
    os.makedirs(folder, exist_ok=True)
    state = {"version": 1, "signature": cfg.signature(), "step": step, "model": model.state_dict(), "optimizer": opt.state_dict(),
             "scheduler": sched.state_dict(), "rng": torch.get_rng_state()}
    path = os.path.join(folder, f"state-{rank}.pt")
    tmp = path + ".tmp"
    torch.save(state, tmp)
    os.replace(tmp, path)


def load(folder: str, rank: int, cfg, model, opt, sched) -> int:
    path = os.path.join(folder, f"state-{rank}.pt")
    state = torch.load(path, map_location="cpu", weights_only=False)   # local, trusted file
    if state.get("version") != 1:
        raise ValueError(f"{path}: unknown checkpoint version {state.get('version')}")
    if state["signature"] != cfg.signature():
        raise ValueError(f"{path} was written with another configuration; only `steps` and `device` may change on resume")
    model.load_state_dict(state["model"])
    opt.load_state_dict(state["optimizer"])
    sched.load_state_dict(state["scheduler"])
    torch.set_rng_state(state["rng"])
    return int(state["step"])
