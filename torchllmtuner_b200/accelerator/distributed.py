"""Process-group bring-up for torchrun / MPI / SLURM launches and small world/rank helpers
(reference: llmtuner/accelerator/distributed.py:94-517)."""
from __future__ import annotations

import datetime
import functools
import os
import subprocess

import torch.distributed as dist

from ..errors import EnvironmentUnsupportedError
from .device import get_device_type, get_distributed_backend, set_device


def infer_launcher() -> str:
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return "pytorch"
    if "OMPI_COMM_WORLD_RANK" in os.environ:
        return "mpi"
    if "SLURM_PROCID" in os.environ and "SLURM_NTASKS" in os.environ:
        return "slurm"
    return "none"


def init_dist(launcher: str | None = None, backend: str | None = None, timeout_s: int = 1800) -> bool:
    """Initialise torch.distributed when the environment describes a multi-process job. Returns True when a
    process group exists afterwards."""
    if dist.is_initialized():
        return True
    launcher = launcher or infer_launcher()
    if launcher == "none":
        return False
    if launcher == "mpi":
        os.environ["RANK"] = os.environ["OMPI_COMM_WORLD_RANK"]
        os.environ["WORLD_SIZE"] = os.environ["OMPI_COMM_WORLD_SIZE"]
        os.environ["LOCAL_RANK"] = os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", "0")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
    elif launcher == "slurm":
        os.environ["RANK"] = os.environ["SLURM_PROCID"]
        os.environ["WORLD_SIZE"] = os.environ["SLURM_NTASKS"]
        os.environ["LOCAL_RANK"] = os.environ.get("SLURM_LOCALID", "0")
        if "MASTER_ADDR" not in os.environ:
            nodes = os.environ.get("SLURM_NODELIST", "127.0.0.1")
            try:
                host = subprocess.check_output(["scontrol", "show", "hostname", nodes], text=True).split()[0]
            except (OSError, subprocess.CalledProcessError):
                host = "127.0.0.1"
            os.environ["MASTER_ADDR"] = host
        os.environ.setdefault("MASTER_PORT", "29500")
    elif launcher != "pytorch":
        raise EnvironmentUnsupportedError(f"unknown launcher {launcher!r}")
    return init_dist_pytorch(backend, timeout_s)


def init_dist_pytorch(backend: str | None = None, timeout_s: int = 1800) -> bool:
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ["WORLD_SIZE"])
    device = set_device(local_rank)
    backend = backend or get_distributed_backend()
    kwargs = {}
    if get_device_type() == "cuda":
        kwargs["device_id"] = device
    dist.init_process_group(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return True


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size(group=None) -> int:
    return dist.get_world_size(group) if is_distributed() else 1


def get_rank(group=None) -> int:
    return dist.get_rank(group) if is_distributed() else 0


def get_dist_info(group=None) -> tuple[int, int]:
    return get_rank(group), get_world_size(group)


def is_main_process(group=None) -> bool:
    return get_rank(group) == 0


def master_only(fn):
    @functools.wraps(fn)
    def wrapper(*a, **kw):
        if is_main_process():
            return fn(*a, **kw)
        return None
    return wrapper


def barrier(group=None) -> None:
    if is_distributed():
        dist.barrier(group)


def get_comm_device(group=None):
    import torch
    if not is_distributed():
        return torch.device("cpu")
    b = dist.get_backend(group)
    return torch.device("cuda", torch.cuda.current_device()) if "nccl" in b else torch.device("cpu")


def destroy() -> None:
    if is_distributed():
        dist.destroy_process_group()
