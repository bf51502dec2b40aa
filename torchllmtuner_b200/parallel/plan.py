"""Resolve-then-execute plans (reference: llmtuner/parallel/plan.py:29-365).

`parallelize_model` resolves every stage's plan against the untouched model first: which modules a stage will replace or
wrap and in what role, at which degree, with which implementation. Resolution is metadata only and raises configuration
errors before anything has been mutated, so a bad expert-parallel setting cannot leave a half tensor-parallel model
behind. Each plan carries a snapshot of what it was resolved against; right before a stage runs, `validate_binding`
compares the live model with that snapshot and refuses a stale plan (a module swapped, a parameter re-created, a forward
re-bound, a buffer's persistence changed, an alias group broken) instead of applying it to the wrong objects.

The snapshot's scope is the stage's targets and everything under them: earlier stages may legitimately change other
parts of the model (tensor parallelism replaces the projections inside a block before expert parallelism converts that
block's experts), which is why a plan declares which aspects it binds:
  "modules"     the target objects must still be registered in the model, as the same objects of the same class
  "parameters"  additionally, the parameters under the targets must be the same objects with the same geometry
  "forwards"    additionally, the targets' `forward` must be bound as it was (nobody patched or compiled them since)
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from ..errors import LLMTunerError

TARGET_KINDS = ("dense", "moe", "vocab", "attention", "decoder", "fsdp_unit", "head")
BIND_ASPECTS = ("modules", "parameters", "forwards")


class StalePlanError(LLMTunerError):
    """A plan was resolved against a model that has changed since."""


@dataclass(frozen=True)
class PlanTarget:
    """One concrete module path and its role in the stage; never a pattern."""
    path: str
    kind: str
    layout: str = ""                                   # e.g. "colwise" / "rowwise" / "vocab" / "ep"
    module: nn.Module | None = field(default=None, repr=False, compare=False)

    def __post_init__(self):
        if self.kind not in TARGET_KINDS:
            raise ValueError(f"plan target kind {self.kind!r} is not one of {TARGET_KINDS}")
        if self.path and any(not part.strip() for part in self.path.split(".")):
            raise ValueError(f"plan target path {self.path!r} is not a concrete module path")
        if self.module is not None and not isinstance(self.module, nn.Module):
            raise ValueError("plan target binding must be a module")


def _tensor_meta(t: torch.Tensor) -> tuple:
    shape = tuple(getattr(t, "_meta_shape", t.shape))
    return shape, t.dtype, t.device.type, bool(t.requires_grad)


@dataclass(frozen=True)
class TargetSnapshot:
    """What `validate_binding` compares for one target."""
    path: str
    module_id: int
    module_class: type
    params: tuple            # ((relative name, id, meta), ...) of the whole subtree, duplicates kept
    buffers: tuple           # ((relative name, id, meta, persistent), ...)
    forward: tuple           # (function object, receiver id) of the target's own forward
    alias_groups: tuple      # groups of relative names that share one Parameter object

    @classmethod
    def capture(cls, path: str, module: nn.Module) -> "TargetSnapshot":
        params = tuple((n, id(p), _tensor_meta(p)) for n, p in module.named_parameters(remove_duplicate=False))
        nonpersistent = {id(m): m._non_persistent_buffers_set for m in module.modules()}
        owners = {}
        for mn, m in module.named_modules(remove_duplicate=False):
            for bn in m._buffers:
                owners[f"{mn}.{bn}" if mn else bn] = (m, bn)
        buffers = tuple((n, id(b), _tensor_meta(b), n in owners and owners[n][1] not in nonpersistent[id(owners[n][0])])
                        for n, b in module.named_buffers(remove_duplicate=False))
        fwd = module.forward
        groups: dict[int, list[str]] = {}
        for n, pid, _ in params:
            groups.setdefault(pid, []).append(n)
        aliases = tuple(tuple(v) for v in groups.values() if len(v) > 1)
        return cls(path, id(module), type(module), params, buffers, (getattr(fwd, "__func__", fwd), id(getattr(fwd, "__self__", None))), aliases)


@dataclass(frozen=True)
class ParallelPlan:
    stage: str
    degree: int
    implementation: str
    targets: tuple[PlanTarget, ...]
    binds: tuple[str, ...] = ("modules",)
    snapshots: tuple[TargetSnapshot, ...] = field(default=(), repr=False, compare=False)
    notes: tuple[str, ...] = ()

    def __post_init__(self):
        object.__setattr__(self, "targets", tuple(self.targets))
        object.__setattr__(self, "binds", tuple(self.binds))
        if not isinstance(self.stage, str) or not self.stage.strip():
            raise ValueError("plan stage must not be empty")
        if type(self.degree) is not int or self.degree < 1:
            raise ValueError("plan degree must be a positive integer")
        if not isinstance(self.implementation, str) or not self.implementation.strip():
            raise ValueError("plan implementation must not be empty")
        for b in self.binds:
            if b not in BIND_ASPECTS:
                raise ValueError(f"plan binds {b!r}; expected a subset of {BIND_ASPECTS}")
        seen = set()
        for t in self.targets:
            if (t.path, t.kind) in seen:
                raise ValueError(f"plan names {t.path!r} twice as {t.kind}")
            seen.add((t.path, t.kind))
        if not self.snapshots:
            object.__setattr__(self, "snapshots", tuple(TargetSnapshot.capture(t.path, t.module) for t in self.targets
                                                         if t.module is not None))

    # ------------------------------------------------------------------ queries
    def count(self, kind: str) -> int:
        return sum(t.kind == kind for t in self.targets)

    def paths(self, kind: str | None = None) -> list[str]:
        return [t.path for t in self.targets if kind is None or t.kind == kind]

    def describe(self) -> dict:
        by_kind: dict[str, int] = {}
        for t in self.targets:
            by_kind[t.kind] = by_kind.get(t.kind, 0) + 1
        return {"stage": self.stage, "degree": self.degree, "implementation": self.implementation, "targets": by_kind,
                "binds": list(self.binds), "notes": list(self.notes)}

    # ------------------------------------------------------------------ validation
    def validate_binding(self, model: nn.Module) -> None:
        """Raises `StalePlanError` when the live model no longer matches what the plan was resolved against."""
        live = {id(m): n for n, m in model.named_modules(remove_duplicate=False)}
        by_id = {id(m): m for m in model.modules()}
        for snap in self.snapshots:
            if snap.module_id not in live:
                raise StalePlanError(f"{self.stage} plan is stale: the module resolved at {snap.path!r} is no longer part of the model")
            mod = by_id[snap.module_id]
            if type(mod) is not snap.module_class:
                raise StalePlanError(f"{self.stage} plan is stale: {snap.path!r} changed class from {snap.module_class.__name__} "
                                     f"to {type(mod).__name__}")
            if "parameters" in self.binds:
                now = tuple((n, id(p), _tensor_meta(p)) for n, p in mod.named_parameters(remove_duplicate=False))
                if len(now) != len(snap.params):
                    raise StalePlanError(f"{self.stage} plan is stale: {snap.path!r} owns {len(now)} parameters, resolved with {len(snap.params)}")
                for (n, pid, meta), (n0, pid0, meta0) in zip(now, snap.params):
                    if n != n0 or pid != pid0:
                        raise StalePlanError(f"{self.stage} plan is stale: parameter {snap.path}.{n0} was replaced")
                    if meta != meta0:
                        raise StalePlanError(f"{self.stage} plan is stale: parameter {snap.path}.{n0} changed geometry {meta0} -> {meta}")
                groups: dict[int, list[str]] = {}
                for n, pid, _ in now:
                    groups.setdefault(pid, []).append(n)
                if tuple(tuple(v) for v in groups.values() if len(v) > 1) != snap.alias_groups:
                    raise StalePlanError(f"{self.stage} plan is stale: parameter sharing under {snap.path!r} changed")
                nonpersistent = {id(m): m._non_persistent_buffers_set for m in mod.modules()}
                owners = {}
                for mn, m in mod.named_modules(remove_duplicate=False):
                    for bn in m._buffers:
                        owners[f"{mn}.{bn}" if mn else bn] = (m, bn)
                nowb = tuple((n, id(b), _tensor_meta(b), n in owners and owners[n][1] not in nonpersistent[id(owners[n][0])])
                             for n, b in mod.named_buffers(remove_duplicate=False))
                if nowb != snap.buffers:
                    raise StalePlanError(f"{self.stage} plan is stale: buffers under {snap.path!r} changed (identity, geometry or persistence)")
            if "forwards" in self.binds:
                fwd = mod.forward
                if (getattr(fwd, "__func__", fwd), id(getattr(fwd, "__self__", None))) != snap.forward:
                    raise StalePlanError(f"{self.stage} plan is stale: forward of {snap.path!r} was re-bound")
