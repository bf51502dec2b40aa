"""Parallel topology: degrees, rank coordinates, named mesh views and their process groups
(reference: llmtuner/parallel/topology.py:36-645).

World layout, outer to inner: [pp,] dp_replicate, dp_shard, cp_kv, cp_ulysses, kcp, tp. So TP ranks are adjacent.
The sparse (expert) view re-factors the inner dp_shard*cp*tp ranks as (efsdp, ep) with ep innermost:
`efsdp = dp_shard*cp*tp / ep`. The topology itself is pure arithmetic (usable for any rank without communication);
`build_device_mesh` creates the process groups, collectively and in a fixed order.

Named views:
  dense      (dp_replicate, dp_shard, cp, tp)      loss   = flatten(dp_replicate, dp_shard, cp, tp)
  batch      = flatten(dp_replicate, dp_shard)      dp_shard_cp = flatten(dp_shard, cp)  (FSDP shard axis)
  sparse     (dp_replicate, efsdp, ep)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from itertools import product

import torch.distributed as dist

from ..errors import ConfigError

DENSE_DIMS = ("pp", "dp_replicate", "dp_shard", "cp_kv", "cp_ulysses", "kcp", "tp")
FLATTENED = {
    "dp": ("dp_replicate", "dp_shard"),
    "batch": ("dp_replicate", "dp_shard"),
    "cp": ("cp_kv", "cp_ulysses", "kcp"),
    "dp_shard_cp": ("dp_shard", "cp_kv", "cp_ulysses", "kcp"),
    "dp_cp": ("dp_replicate", "dp_shard", "cp_kv", "cp_ulysses", "kcp"),
    "loss": ("dp_replicate", "dp_shard", "cp_kv", "cp_ulysses", "kcp", "tp"),
    "world": DENSE_DIMS,
}
SPARSE_DIMS = ("pp", "dp_replicate", "efsdp", "ep")


@dataclass
class ParallelTopology:
    world_size: int
    rank: int = 0
    dp_replicate: int = 1
    dp_shard: int = -1
    cp_kv: int = 1
    cp_ulysses: int = 1
    kcp: int = 1
    tp: int = 1
    ep: int = 1
    pp: int = 1
    _groups: dict = field(default_factory=dict, repr=False)

    def __post_init__(self):
        self._validate()

    # ------------------------------------------------------------------ validation
    def _validate(self) -> None:
        for n in ("dp_replicate", "cp_kv", "cp_ulysses", "kcp", "tp", "ep", "pp"):
            if getattr(self, n) < 1:
                raise ConfigError(f"{n} must be >= 1")
        fixed = self.dp_replicate * self.cp * self.tp * self.pp
        if self.dp_shard == -1:
            if self.world_size % fixed:
                raise ConfigError(f"world size {self.world_size} is not divisible by dp_replicate*cp*tp*pp = {fixed}")
            self.dp_shard = self.world_size // fixed
        if self.dp_shard < 1:
            raise ConfigError("dp_shard must be >= 1 or -1")
        if fixed * self.dp_shard != self.world_size:
            raise ConfigError(f"dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * cp({self.cp}) * tp({self.tp})"
                              f" * pp({self.pp}) = {fixed * self.dp_shard} != world size {self.world_size}")
        inner = self.dp_shard * self.cp * self.tp
        if inner % self.ep:
            raise ConfigError(f"dp_shard*cp*tp = {inner} must be divisible by expert_parallel_size {self.ep}")
        if not 0 <= self.rank < self.world_size:
            raise ConfigError(f"rank {self.rank} outside world of {self.world_size}")

    # ------------------------------------------------------------------ sizes
    @property
    def cp(self) -> int:
        return self.cp_kv * self.cp_ulysses * self.kcp

    @property
    def dp(self) -> int:
        return self.dp_replicate * self.dp_shard

    @property
    def efsdp(self) -> int:
        return self.dp_shard * self.cp * self.tp // self.ep

    @property
    def fsdp_shard_size(self) -> int:
        return self.dp_shard * self.cp

    def size(self, name: str) -> int:
        if name in FLATTENED:
            n = 1
            for d in FLATTENED[name]:
                n *= getattr(self, d)
            return n
        return getattr(self, name)

    @property
    def dp_enabled(self): return self.dp > 1
    @property
    def tp_enabled(self): return self.tp > 1
    @property
    def cp_enabled(self): return self.cp > 1
    @property
    def ep_enabled(self): return self.ep > 1
    @property
    def pp_enabled(self): return self.pp > 1
    @property
    def fsdp_enabled(self): return self.dp_shard * self.cp > 1

    # ------------------------------------------------------------------ coordinates
    def _shape(self, dims) -> list[int]:
        return [getattr(self, d) for d in dims]

    def coords(self, rank: int | None = None, sparse: bool = False) -> dict[str, int]:
        r = self.rank if rank is None else rank
        dims = SPARSE_DIMS if sparse else DENSE_DIMS
        out = {}
        for d, n in reversed(list(zip(dims, self._shape(dims)))):
            out[d] = r % n
            r //= n
        return out

    def coord(self, name: str, rank: int | None = None) -> int:
        """Coordinate along a dim or a flattened view (row-major over its members)."""
        if name in ("efsdp", "ep"):
            return self.coords(rank, sparse=True)[name]
        c = self.coords(rank)
        if name in FLATTENED:
            v = 0
            for d in FLATTENED[name]:
                v = v * getattr(self, d) + c[d]
            return v
        return c[name]

    def group_ranks(self, name: str, rank: int | None = None) -> list[int]:
        """World ranks of the group along `name` that contains `rank`, ordered by coordinate."""
        sparse = name in ("efsdp", "ep")
        dims = SPARSE_DIMS if sparse else DENSE_DIMS
        members = (name,) if (sparse or name not in FLATTENED) else FLATTENED[name]
        me = self.coords(rank, sparse)
        shape = self._shape(dims)
        out = []
        for combo in product(*[range(getattr(self, d)) for d in members]):
            c = dict(me)
            c.update(dict(zip(members, combo)))
            r = 0
            for d, n in zip(dims, shape):
                r = r * n + c[d]
            out.append(r)
        return out

    def all_groups(self, name: str) -> list[list[int]]:
        seen, out = set(), []
        for r in range(self.world_size):
            g = tuple(self.group_ranks(name, r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out

    # ------------------------------------------------------------------ process groups
    def get_group(self, name: str):
        """Process group along `name` (None when its size is 1 or torch.distributed is not initialised)."""
        if self.size(name) == 1 or not dist.is_initialized():
            return None
        if name not in self._groups:
            raise ConfigError(f"process group {name!r} was not built; call build_device_mesh first")
        return self._groups[name]

    def get_optional_mesh(self, name: str):
        return self.get_group(name)

    def snapshot(self) -> dict:
        """Degrees as stored in checkpoints (reference: topology.py snapshots)."""
        return {k: getattr(self, k) for k in ("world_size", "dp_replicate", "dp_shard", "cp_kv", "cp_ulysses", "kcp", "tp", "ep", "pp")}

    def describe(self) -> str:
        return ", ".join(f"{k}={v}" for k, v in self.snapshot().items() if k == "world_size" or v != 1)


MESH_VIEWS = ("pp", "dp_replicate", "dp_shard", "cp_kv", "cp_ulysses", "kcp", "tp", "dp", "cp", "dp_shard_cp", "dp_cp", "loss",
              "efsdp", "ep")


def build_device_mesh(topo: ParallelTopology, timeout=None) -> ParallelTopology:
    """Create every process group with more than one member. Every rank creates every group, in one fixed order,
    so the call is collective. Publishes nothing when any creation fails (no partially built cache)."""
    if not dist.is_initialized() or topo.world_size == 1:
        return topo
    built = {}
    for name in MESH_VIEWS:
        if topo.size(name) == 1:
            continue
        if topo.size(name) == topo.world_size:
            built[name] = dist.group.WORLD
            continue
        mine = None
        for ranks in topo.all_groups(name):
            g = dist.new_group(ranks=ranks, timeout=timeout) if timeout is not None else dist.new_group(ranks=ranks)
            if topo.rank in ranks:
                mine = g
        built[name] = mine
    topo._groups.update(built)
    return topo


def resolve_parallel_topology(parallel_config, world_size: int, rank: int = 0) -> ParallelTopology:
    p = parallel_config
    return ParallelTopology(world_size=world_size, rank=rank, dp_replicate=p.data_parallel_replicate_size,
                            dp_shard=p.data_parallel_shard_size, cp_kv=p.context_parallel_kv_allgather_size,
                            cp_ulysses=p.context_parallel_ulysses_size, kcp=p.context_parallel_kcp_size,
                            tp=p.tensor_parallel_size, ep=p.expert_parallel_size,
                            pp=getattr(p, "pipeline_parallel_size", 1))
