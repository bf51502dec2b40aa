"""The recipe files parse into valid configurations and their topologies are consistent for 8 ranks."""
import glob
import os

import pytest

from torchllmtuner_b200 import LLMTunerConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples", "*.yaml"))))
def test_recipe_parses_and_fits_eight_ranks(path):
    from torchllmtuner_b200.parallel.topology import resolve_parallel_topology
    cfg = LLMTunerConfig.from_file(path)
    for rank in range(8):
        topo = resolve_parallel_topology(cfg.parallel, 8, rank)
        assert topo.world_size == 8
        assert sorted(r for g in topo.all_groups("tp") for r in g) == list(range(8))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples", "*.yaml"))))
def test_recipe_builds_its_model_without_memory(path):
    """Every recipe names a registered family and sizes that the family accepts (built on the meta device)."""
    import torch
    from torchllmtuner_b200.models.registry import build_registered_model
    cfg = LLMTunerConfig.from_file(path)
    m = build_registered_model(cfg.model, dtype=torch.bfloat16, device="meta")
    n = sum(p.numel() for p in m.parameters())
    assert n > 1e9 and all(p.is_meta for p in m.parameters())
    expect = {"qwen3_8b": 8.19e9, "qwen3_30b_a3b": 30.53e9}.get(cfg.model.model_name_or_path)
    if expect:
        assert abs(n - expect) / expect < 0.01
