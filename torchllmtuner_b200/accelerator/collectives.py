"""Collective services (reference: llmtuner/accelerator/collectives.py:61-686): process-group timeouts, in-place
all-reduce with mean emulation, the framework-wide error-coordination primitive `synchronize_local_errors`
(int32 status, MIN all-reduce: one rank raising becomes every rank raising), and an all-reduce whose backward is
the identity (`PartialToInvariantAllReduce`)."""
from __future__ import annotations

import contextlib
import datetime

import torch
import torch.distributed as dist

from ..errors import LLMTunerError
from .distributed import get_comm_device, is_distributed


class CoordinatedError(LLMTunerError, RuntimeError):
    """Raised on ranks whose own work succeeded when a peer rank failed in the same phase."""


def set_pg_timeouts(timeout_s: int, groups) -> None:
    """Barrier, then shorten the timeout of every given group (called after the first step, when lazy
    initialisation is over)."""
    if not is_distributed():
        return
    dist.barrier()
    td = datetime.timedelta(seconds=timeout_s)
    for g in [None, *[g for g in groups if g is not None]]:
        try:
            torch.distributed.distributed_c10d._set_pg_timeout(td, g)
        except Exception:  # noqa: BLE001  (backend without runtime timeout support)
            pass


def all_reduce(t: torch.Tensor, op: str = "sum", group=None) -> torch.Tensor:
    """In-place all-reduce; `mean` is emulated as sum / size so it works on every backend."""
    if not is_distributed() or dist.get_world_size(group) == 1:
        return t
    ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "mean": dist.ReduceOp.SUM}
    dist.all_reduce(t, op=ops[op], group=group)
    if op == "mean":
        t.div_(dist.get_world_size(group))
    return t


def agree_status(ok: bool, group=None) -> bool:
    """MIN all-reduce of a local ok flag: True only if every rank of the group is ok."""
    if not is_distributed() or dist.get_world_size(group) == 1:
        return ok
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=get_comm_device(group))
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())


@contextlib.contextmanager
def synchronize_local_errors(phase: str, group=None):
    """Run rank-local work; afterwards all ranks agree on success. A rank that raised re-raises its own error;
    the others raise `CoordinatedError` naming the phase, so nobody is left waiting in the next collective."""
    err: BaseException | None = None
    try:
        yield
    except Exception as e:  # noqa: BLE001
        err = e
    ok = agree_status(err is None, group)
    if err is not None:
        raise err
    if not ok:
        raise CoordinatedError(f"a peer rank failed during {phase!r}")


def synchronize_after_wait(work, phase: str, group=None):
    """Wait for an async work handle inside an error-coordination boundary."""
    with synchronize_local_errors(phase, group):
        if work is not None:
            work.wait()


class PartialToInvariantAllReduce(torch.autograd.Function):
    """Forward: sum over the group. Backward: identity (every rank already holds the full upstream gradient)."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        all_reduce(y, "sum", group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None
