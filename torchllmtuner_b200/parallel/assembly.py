"""Final layout of one local model part: who owns which parameter under which name
(reference: llmtuner/parallel/assembly.py:18-231).

After the parallel stages have run, three consumers need to agree on parameter identity: the optimizer (state keyed by
parameter name), the exponential moving average, and the checkpointer (one on-disk name per parameter, wrappers
invisible). `ModelPartLayout` is the single record they bind to:

  * `bindings`         every registered path -> parameter object, in registration order, aliases kept
  * `aliases`          parameter -> all paths it is registered under (tied embeddings: two paths, one parameter)
  * `state_names`      path -> wrapper-free checkpoint name; two different parameters may not collapse to one name
  * `owner_names`      parameter -> the one name that keys its optimizer / EMA / checkpoint state: its first registration
  * `execution`, `topology`   the resolved execution layout and degree snapshot the model was assembled for

`refresh` re-reads the model after materialisation (meta -> device swaps every parameter object) and checks that paths,
order and sharing survived: an alias that was split, or two parameters merged into one, is an error rather than a silent
change of what the optimizer trains. A consumer keeps the `LayoutSnapshot` it was built from and calls
`snapshot.validate(layout, consumer=...)` before it touches state: a model that was re-parallelised, or a parameter
that was swapped after the optimizer was built, is refused with the consumer's name in the message.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Mapping, Sequence

import torch.nn as nn

from ..errors import LLMTunerError
from .replacements import ReplacementMap


class LayoutError(LLMTunerError):
    """Parameter ownership, naming or sharing no longer matches the recorded layout."""


def wrapper_free_name(path: str) -> str:
    """Parallelism and checkpoint wrappers register the wrapped module as `inner`; state names never show them."""
    parts = [p for p in path.split(".") if p not in ("inner", "_checkpoint_wrapped_module", "_orig_mod")]
    return ".".join(parts)


@dataclass(frozen=True, eq=False)
class LayoutSnapshot:
    parameters: Mapping[str, nn.Parameter]
    topology: Mapping | None
    execution: object | None

    def validate(self, layout: "ModelPartLayout", *, consumer: str) -> None:
        now = layout.bindings
        if tuple(now) != tuple(self.parameters) or any(now[k] is not p for k, p in self.parameters.items()):
            raise LayoutError(f"{consumer}: parameter ownership changed since it was built; rebuild it against the final model layout")
        if layout.topology != self.topology or layout.execution != self.execution:
            raise LayoutError(f"{consumer}: topology or execution layout changed since it was built; rebuild it")


@dataclass
class ModelPartLayout:
    execution: object | None = None
    topology: Mapping | None = None
    bindings: dict[str, nn.Parameter] = field(default_factory=dict)
    replaced: dict[int, nn.Parameter] = field(default_factory=dict)     # id(old parameter) -> its replacement
    replacements: ReplacementMap = field(default_factory=ReplacementMap)   # composed over every refresh
    _captured: bool = field(default=False, repr=False)

    # ------------------------------------------------------------------ capture / refresh
    def refresh(self, model: nn.Module) -> None:
        current = dict(model.named_parameters(remove_duplicate=False))
        if self._captured:
            if tuple(current) != tuple(self.bindings):
                gone = [k for k in self.bindings if k not in current][:3]
                new = [k for k in current if k not in self.bindings][:3]
                raise LayoutError(f"layout refresh: registered parameter paths or their order changed (gone {gone}, new {new})")
            forward: dict[int, nn.Parameter] = {}
            backward: dict[int, nn.Parameter] = {}
            for path, old in self.bindings.items():
                new = current[path]
                if forward.setdefault(id(old), new) is not new:
                    raise LayoutError(f"layout refresh: the parameter shared at {path!r} was split into two objects")
                if backward.setdefault(id(new), old) is not old:
                    raise LayoutError(f"layout refresh: two distinct parameters were merged at {path!r}")
                if new is not old:
                    self.replaced[id(old)] = new
            self.replacements.record(parameters={old: (new,) for old, new in ((o, forward[id(o)]) for o in dict.fromkeys(self.bindings.values()))
                                                 if new is not old})
        self.bindings = current
        self._captured = True

    # ------------------------------------------------------------------ views
    @property
    def aliases(self) -> Mapping[nn.Parameter, tuple[str, ...]]:
        out: dict[nn.Parameter, list[str]] = {}
        for path, p in self.bindings.items():
            out.setdefault(p, []).append(path)
        return MappingProxyType({p: tuple(v) for p, v in out.items()})

    def _named(self):
        owners: dict[str, nn.Parameter] = {}
        for path, p in self.bindings.items():
            name = wrapper_free_name(path)
            if owners.setdefault(name, p) is not p:
                raise LayoutError(f"two parameters collapse to the checkpoint name {name!r} once wrappers are removed")
            yield path, name, p

    @property
    def state_names(self) -> Mapping[str, str]:
        return MappingProxyType({path: name for path, name, _ in self._named()})

    @property
    def owner_names(self) -> Mapping[nn.Parameter, str]:
        out: dict[nn.Parameter, str] = {}
        for _, name, p in self._named():
            out.setdefault(p, name)
        return MappingProxyType(out)

    # ------------------------------------------------------------------ validation
    def validate(self, model: nn.Module) -> Mapping[str, str]:
        if self.execution is not None and hasattr(self.execution, "validate_model"):
            self.execution.validate_model(model)
        if self.execution is not None and self.topology is not None:
            degree = {"cp": int(self.topology.get("cp_kv", 1)) * int(self.topology.get("cp_ulysses", 1)) * int(self.topology.get("kcp", 1)),
                      "tp": int(self.topology.get("tp", 1))}
            axes = tuple(a for a in ("cp", "tp") if degree[a] > 1)
            declared = tuple(getattr(self.execution, "sequence_shard_axes", axes))
            if declared != axes:
                raise LayoutError(f"execution layout shards the sequence over {declared}, the topology over {axes}")
        current = dict(model.named_parameters(remove_duplicate=False))
        if tuple(current) != tuple(self.bindings) or any(current[k] is not p for k, p in self.bindings.items()):
            raise LayoutError("model layout is stale: parameters were registered, removed, reordered or replaced since the last refresh")
        live = {id(p) for p in current.values()}
        for new in self.replaced.values():
            if id(new) not in live:
                raise LayoutError("model layout is stale: a recorded replacement parameter is no longer registered")
        for _src, targets in self.replacements.parameter_targets():
            if any(id(t) not in live for t in targets):
                raise LayoutError("model layout is stale: a parameter that replaced an earlier one is no longer registered")
        return self.state_names

    def snapshot(self) -> LayoutSnapshot:
        return LayoutSnapshot(MappingProxyType(dict(self.bindings)), self.topology, self.execution)


def capture_layouts(model_parts: Sequence[nn.Module], *, execution=None, topology=None) -> tuple[ModelPartLayout, ...]:
    out = []
    for m in model_parts:
        lay = ModelPartLayout(execution=execution, topology=topology)
        lay.refresh(m)
        out.append(lay)
    return tuple(out)


def validate_layouts(model_parts: Sequence[nn.Module], layouts: Sequence[ModelPartLayout]) -> None:
    """Across the local model parts (pipeline stages held by this rank): every part valid, no parameter and no
    checkpoint name owned by two parts, one topology."""
    if len(model_parts) != len(layouts):
        raise LayoutError(f"{len(layouts)} layouts for {len(model_parts)} model parts")
    topologies = {tuple(sorted(l.topology.items())) if l.topology is not None else None for l in layouts}
    if len(topologies) > 1:
        raise LayoutError("model parts were assembled under different topologies")
    param_owner: dict[int, int] = {}
    name_owner: dict[str, int] = {}
    for i, (m, lay) in enumerate(zip(model_parts, layouts)):
        names = lay.validate(m)
        for p in lay.aliases:
            j = param_owner.setdefault(id(p), i)
            if j != i:
                raise LayoutError(f"a parameter is registered in model parts {j} and {i}; sharing across parts is not supported")
        for name in names.values():
            j = name_owner.setdefault(name, i)
            if j != i:
                raise LayoutError(f"checkpoint name {name!r} is claimed by model parts {j} and {i}")
