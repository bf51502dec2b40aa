"""The self-contained teaching framework: every mesh shape reproduces the single-rank loss curve; resume is exact."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torchllmtuner_b200.experiments.mini import MiniConfig, MiniTrainer
from torchllmtuner_b200.experiments.mini.train import main as mini_main


def _worker(rank, world, store_path, kw, out_path):
    store = dist.FileStore(store_path, world)
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        tr = MiniTrainer(MiniConfig(**kw))
        hist = tr.train()
        if rank == 0:
            torch.save(hist, out_path)
    finally:
        dist.destroy_process_group()


def _run(world, tmp_path, **kw):
    if world == 1:
        return MiniTrainer(MiniConfig(**kw)).train()
    store, out = str(tmp_path / f"store{world}{kw.get('tp', 1)}{kw.get('ep', 1)}"), str(tmp_path / "hist.pt")
    mp.spawn(_worker, args=(world, store, kw, out), nprocs=world, join=True)
    return torch.load(out, weights_only=False)


BASE = dict(steps=3, gradient_accumulation_steps=2, seq_len=16)


@pytest.mark.parametrize("mesh", [dict(tp=2), dict(ep=2), dict(dp=2), dict(ep=2, tp=2), dict(dp=2, ep=2)])
def test_mesh_matches_single_rank(tmp_path, mesh):
    world = mesh.get("tp", 1) * mesh.get("ep", 1) * mesh.get("dp", 1)
    data_ranks = mesh.get("ep", 1) * mesh.get("dp", 1)
    ref = _run(1, tmp_path, batch_size=2 * data_ranks, **BASE)
    got = _run(world, tmp_path, batch_size=2, **BASE, **mesh)
    for a, b in zip(ref, got):
        assert abs(a["loss"] - b["loss"]) < 2e-5 and abs(a["grad_norm"] - b["grad_norm"]) < 2e-4, (ref, got)


def test_resume_continues_exactly_and_refuses_another_configuration(tmp_path):
    full = MiniTrainer(MiniConfig(steps=4)).train()
    first = MiniTrainer(MiniConfig(steps=2))
    first.train()
    first.save(str(tmp_path))
    second = MiniTrainer(MiniConfig(steps=4))
    second.resume(str(tmp_path))
    assert second.step == 2
    rest = second.train()
    assert [m["loss"] for m in rest] == [m["loss"] for m in full[2:]]
    other = MiniTrainer(MiniConfig(steps=4, learning_rate=1e-3))
    with pytest.raises(ValueError):
        other.resume(str(tmp_path))
    assert not [f for f in os.listdir(tmp_path) if f.endswith(".tmp")]


def test_cli_runs_and_saves(tmp_path, capsys):
    import math
    hist = mini_main(["--device", "cpu", "--steps", "4", "--checkpoint", str(tmp_path)])
    # fresh uniform random tokens every step: the loss stays at ln(vocab)
    assert all(abs(m["loss"] - math.log(128)) < 0.2 for m in hist) and "step 4" in capsys.readouterr().out
    assert os.path.exists(tmp_path / "state-0.pt")
    with pytest.raises(ValueError):
        MiniConfig(tp=3).validate(3)
    with pytest.raises(ValueError):
        MiniConfig(tp=2).validate(4)


def test_it_does_not_import_the_production_package():
    import re
    folder = os.path.dirname(__import__("torchllmtuner_b200.experiments.mini", fromlist=["x"]).__file__)
    for f in os.listdir(folder):
        if f.endswith(".py"):
            src = open(os.path.join(folder, f)).read()
            assert not re.search(r"^\s*from \.\.|^\s*(from|import) torchllmtuner_b200", src, re.M), f
