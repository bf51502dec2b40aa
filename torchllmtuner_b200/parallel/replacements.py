"""Which object took the place of which, across successive conversions
(reference: llmtuner/parallel/replacements.py:25-124).

Parallel stages and materialisation replace modules (a linear by its column-parallel form) and parameters (a meta
parameter by a device one, one fused projection by three). A consumer that captured an object before a conversion asks
this map what it has become. Events COMPOSE: if a -> b was recorded and then b -> (c, d), the map answers a -> (c, d).
An empty target tuple means the parameter was removed. Sources are held weakly and compared by identity (tensor
equality is element-wise and must never be used as a dictionary test)."""
from __future__ import annotations

import weakref

import torch.nn as nn


class _IdentityTable:
    """id(source) -> (weak reference to source, target); an entry whose source died, or whose id was reused by another
    object, never answers."""

    def __init__(self):
        self._rows: dict[int, tuple[weakref.ref, object]] = {}

    def set(self, source, target) -> None:
        key = id(source)

        def gone(ref, key=key, table=weakref.ref(self)):
            t = table()
            if t is not None and key in t._rows and t._rows[key][0] is ref:
                del t._rows[key]
        self._rows[key] = (weakref.ref(source, gone), target)

    def get(self, source, default=None):
        row = self._rows.get(id(source))
        return row[1] if row is not None and row[0]() is source else default

    def items(self):
        for ref, target in list(self._rows.values()):
            src = ref()
            if src is not None:
                yield src, target

    def __len__(self) -> int:
        return len(self._rows)


class ReplacementMap:
    def __init__(self):
        self._modules = _IdentityTable()
        self._params = _IdentityTable()

    def record(self, modules: dict | None = None, parameters: dict | None = None) -> None:
        """One simultaneous event: `modules` {old module: new module}, `parameters` {old parameter: tuple of new
        parameters}. Both tables are rebuilt before either is replaced, so a bad event leaves the map as it was."""
        modules, parameters = modules or {}, parameters or {}
        for k, v in parameters.items():
            if not isinstance(k, nn.Parameter) or not isinstance(v, tuple) or any(not isinstance(p, nn.Parameter) for p in v):
                raise TypeError("parameter replacements map a Parameter to a tuple of Parameters")
        for k, v in modules.items():
            if not isinstance(k, nn.Module) or not isinstance(v, nn.Module):
                raise TypeError("module replacements map a Module to a Module")
        new_modules, new_params = _IdentityTable(), _IdentityTable()
        by_id_m = {id(k): v for k, v in modules.items()}
        by_id_p = {id(k): v for k, v in parameters.items()}
        for src, tgt in self._modules.items():
            new_modules.set(src, by_id_m.get(id(tgt), tgt))
        for src, tgts in self._params.items():
            out: list[nn.Parameter] = []
            for t in tgts:
                for r in by_id_p.get(id(t), (t,)):
                    if all(r is not o for o in out):
                        out.append(r)
            new_params.set(src, tuple(out))
        for k, v in modules.items():
            new_modules.set(k, v)
        for k, v in parameters.items():
            new_params.set(k, v)
        self._modules, self._params = new_modules, new_params

    def module(self, source: nn.Module) -> nn.Module:
        """What `source` has become (itself when it was never replaced)."""
        return self._modules.get(source, source)

    def parameters(self, source: nn.Parameter) -> tuple:
        """What `source` has become: a tuple of parameters (itself when never replaced, empty when removed)."""
        return self._params.get(source, (source,))

    def parameter_targets(self):
        return list(self._params.items())
