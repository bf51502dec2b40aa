"""Materialise a model that was built on the meta device (reference: llmtuner/memory/materialization.py:23-154).
Under FSDP the flat units allocate storage and bind parameter views themselves; this helper covers buffers and any
parameter left outside every unit."""
from __future__ import annotations

import torch


def materialize_meta_model(model: torch.nn.Module, device) -> None:
    for mod in model.modules():
        for name, buf in list(mod._buffers.items()):
            if buf is not None and buf.is_meta:
                mod._buffers[name] = torch.zeros(buf.shape, dtype=buf.dtype, device=device)
        for name, p in list(mod._parameters.items()):
            if p is not None and p.is_meta:
                mod._parameters[name] = torch.nn.Parameter(torch.empty(p.shape, dtype=p.dtype, device=device), requires_grad=p.requires_grad)
