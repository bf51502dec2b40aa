"""Stage split (reference: experiments/pipeline_parallel/partition.py:141-243, pipeline_parallel.py:134-186): the model is
`input_weight` pseudo-layers + L decoder layers + `output_weight` pseudo-layers, spread evenly over the stages with the
remainder going to the first stages. The first stage owns the embedding, the last owns the final norm and the head."""
from __future__ import annotations

import torch.nn as nn

from ...errors import ConfigError


def split_layers(num_layers: int, num_stages: int, input_weight: int = 1, output_weight: int = 1) -> list[tuple[int, int]]:
    """[(first_layer, end_layer)] per stage."""
    total = num_layers + input_weight + output_weight
    if num_stages > total or num_stages < 1:
        raise ConfigError(f"cannot cut {num_layers} layers into {num_stages} stages")
    base, rem = divmod(total, num_stages)
    sizes = [base + (1 if s < rem else 0) for s in range(num_stages)]
    out, pos = [], 0
    for s, n in enumerate(sizes):
        a, b = pos, pos + n
        la = max(0, a - input_weight)
        lb = min(num_layers, b - input_weight)
        out.append((min(la, num_layers), max(min(lb, num_layers), min(la, num_layers))))
        pos = b
    if any(b <= a for a, b in out) and num_layers >= num_stages:
        # degenerate weights: fall back to an even split of the real layers
        base, rem = divmod(num_layers, num_stages)
        out, pos = [], 0
        for s in range(num_stages):
            n = base + (1 if s < rem else 0)
            out.append((pos, pos + n))
            pos += n
    return out


class _Empty(nn.Module):
    """Parameter-free stand-in for a part another stage owns."""

    def forward(self, x, *a, **k):
        return x


def prune_to_stage(model, stage: int, num_stages: int, input_weight: int = 1, output_weight: int = 1):
    """Keep only this stage's layers; returns the (first, end) layer range."""
    layers = model.model.layers
    a, b = split_layers(len(layers), num_stages, input_weight, output_weight)[stage]
    for i, l in enumerate(layers):
        l.layer_idx = i
    model.model.layers = nn.ModuleDict({str(i): l for i, l in enumerate(layers) if a <= i < b})   # global indices stay in the names
    model.pp_first, model.pp_last = stage == 0, stage == num_stages - 1
    if not model.pp_first:
        model.model.embed_tokens = _Empty()
    if not model.pp_last:
        model.model.norm = _Empty()
        model.lm_head = _Empty()
    return a, b


def partition_signature(model, stage: int) -> dict:
    return {"stage": stage, "params": sorted(n for n, _ in model.named_parameters())}
