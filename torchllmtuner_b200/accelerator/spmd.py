"""Thread-local record of the meshes the current computation runs on (reference: llmtuner/accelerator/spmd.py:46-199).

The reference needs it because DTensor ops look their mesh up implicitly; here every collective receives its group
explicitly from `ParallelTopology`, so the context only serves code that wants to ask "which dense / sparse mesh am I
under" without threading the topology through (model-side helpers, activation-checkpoint replay, tests)."""
from __future__ import annotations

import contextlib
import threading

_state = threading.local()


def _stack() -> list:
    if not hasattr(_state, "stack"):
        _state.stack = []
    return _state.stack


def set_spmd_meshes(dense, sparse=None) -> None:
    """Install the process-wide default meshes (dense = (dp_replicate, dp_shard, cp, tp); sparse = (dp_replicate, efsdp, ep))."""
    _state.default = (dense, sparse)


def spmd_dense_mesh():
    return getattr(_state, "default", (None, None))[0]


def spmd_sparse_mesh():
    return getattr(_state, "default", (None, None))[1]


def current_spmd_mesh():
    """Innermost mesh entered with `spmd_context`, else the dense default."""
    st = _stack()
    return st[-1] if st else spmd_dense_mesh()


def spmd_mesh_size(name: str) -> int:
    m = current_spmd_mesh()
    return 1 if m is None else int(m.size(name))


def spmd_mesh_group(name: str):
    m = current_spmd_mesh()
    return None if m is None else m.get_group(name)


def capture_spmd_context():
    """Snapshot for a later replay (activation checkpointing re-enters the forward outside the original `with`)."""
    return (getattr(_state, "default", (None, None)), list(_stack()))


@contextlib.contextmanager
def restore_spmd_context(snapshot):
    old_default, old_stack = getattr(_state, "default", (None, None)), list(_stack())
    _state.default, _state.stack = snapshot[0], list(snapshot[1])
    try:
        yield
    finally:
        _state.default, _state.stack = old_default, old_stack


@contextlib.contextmanager
def spmd_context(mesh):
    """Run a region under `mesh` (a `ParallelTopology` or anything with `size(name)` / `get_group(name)`)."""
    _stack().append(mesh)
    try:
        yield mesh
    finally:
        _stack().pop()
