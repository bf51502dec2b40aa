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
