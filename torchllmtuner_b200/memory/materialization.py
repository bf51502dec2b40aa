"""Materialise a model that was built on the meta device (reference: llmtuner/memory/materialization.py:23-154).
Under FSDP the flat units allocate storage and bind parameter views themselves; this helper covers buffers and any
parameter left outside every unit. A tensor registered under several names (a tied embedding and head, a buffer shared
by two modules) stays ONE tensor: every alias is rebound to the same new object, and buffer persistence is untouched."""
from __future__ import annotations

import torch


def materialize_meta_model(model: torch.nn.Module, device) -> int:
    """Returns how many distinct tensors were given storage (their contents are unspecified; buffers are zeroed)."""
    made: dict[int, torch.Tensor] = {}
    for mod in model.modules():
        for name, buf in list(mod._buffers.items()):
            if buf is not None and buf.is_meta:
                if id(buf) not in made:
                    made[id(buf)] = torch.zeros(buf.shape, dtype=buf.dtype, device=device)
                mod._buffers[name] = made[id(buf)]
        for name, p in list(mod._parameters.items()):
            if p is not None and p.is_meta:
                if id(p) not in made:
                    new = torch.nn.Parameter(torch.empty(p.shape, dtype=p.dtype, device=device), requires_grad=p.requires_grad)
                    for k, v in p.__dict__.items():          # marks such as the tensor-parallel cut travel with the parameter
                        setattr(new, k, v)
                    made[id(p)] = new
                mod._parameters[name] = made[id(p)]
    return len(made)
