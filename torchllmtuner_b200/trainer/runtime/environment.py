"""Runtime environment: determinism flags, process group, topology, seeding, device
(reference: llmtuner/trainer/runtime/environment.py:58-117)."""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ...accelerator import get_current_device, get_device_type, get_env_dist_info, init_dist, set_device
from ...parallel.topology import ParallelTopology, build_device_mesh, resolve_parallel_topology
from ...utils.seeding import derive_distinct_seed, seed_everything, set_deterministic_algorithms


@dataclass
class RuntimeEnvironment:
    rank: int
    local_rank: int
    world_size: int
    device: torch.device
    topo: ParallelTopology
    param_dtype: torch.dtype


def build_runtime_environment(config) -> RuntimeEnvironment:
    t = config.training
    set_deterministic_algorithms(t.deterministic and get_device_type() == "cpu", t.detect_anomaly)
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        init_dist()
    rank, local_rank, world = get_env_dist_info()
    device = set_device(local_rank) if get_device_type() == "cuda" else get_current_device()
    topo = resolve_parallel_topology(config.parallel, world, rank)
    build_device_mesh(topo)
    # every rank of one model replica must draw the same initial weights; data-parallel ranks differ only in data
    seed_everything(t.seed)
    cd = config.model.compute_dtype
    if cd is None:
        dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    else:
        dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[cd]
    return RuntimeEnvironment(rank, local_rank, world, device, topo, dtype)


def rank_seed(base: int, topo: ParallelTopology) -> int:
    return derive_distinct_seed(base, topo.coord("dp"), topo.coord("cp"), topo.coord("tp"))
