"""L5 parallel layer: topology, stage order, compatibility matrix and the parallelism stages."""
from .stages import STAGE_ORDER, STAGES  # noqa: F401
from .topology import ParallelTopology, build_device_mesh, resolve_parallel_topology  # noqa: F401
