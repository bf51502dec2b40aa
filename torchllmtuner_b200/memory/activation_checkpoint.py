"""Activation checkpointing modes (reference: llmtuner/memory/activation_checkpoint.py:80-656).

  none           keep every activation
  full           keep only each block's input; the block forward is replayed in backward
  selective      policy "op" (default): every block is checkpointed, but attention and every other linear keep their
                 outputs and are not recomputed in the replay (`ops.functional.SelectiveReplay`);
                 policy "block": every `save_every_nth_block`-th block keeps its activations, the others recompute
  memory_budget  the fraction of blocks that recompute is chosen from `memory_budget` (0 = all recompute, 1 = none)
  region         per-block choice from module-name patterns: blocks matching `recompute_regions` recompute
Expert-parallel token exchanges are replayed with the block (the reference keeps all_to_all results under a MUST_SAVE
policy, activation_checkpoint.py:278-300; here the exchange is a pair of peer-memory kernels and cheap to repeat).
"""
from __future__ import annotations

import re


def recompute_mm_shapes(model, fqn_parts) -> set[tuple[int, int]]:
    """Weight shapes of the linears whose name contains one of `fqn_parts`: the per-op policy always recomputes a linear
    of such a shape (reference: `force_recompute_mm_shapes_by_fqns`, activation_checkpoint.py:140-200). A part that names
    no two-dimensional weight raises, so that a typo does not silently keep everything."""
    shapes: set[tuple[int, int]] = set()
    for part in fqn_parts:
        hit = [tuple(getattr(p, "_meta_shape", p.shape)) for n, p in model.named_parameters() if part in n and p.dim() == 2]
        if not hit:
            raise ValueError(f"force_recompute_mm_shapes_by_fqns: {part!r} names no linear weight")
        shapes.update(hit)
    return shapes


def apply_ac(model, training_config) -> None:
    mode = training_config.activation_checkpoint_mode
    n_layers = len(model.model.layers) if hasattr(model, "model") and hasattr(model.model, "layers") else 0
    if mode in ("none", "full"):
        model.activation_checkpoint = mode
        return
    if mode == "selective":
        sc = training_config.selective_ac
        model.activation_checkpoint = "selective"
        model.ac_save_every = max(1, sc.save_every_nth_block)
        model.ac_per_op = sc.selective_ac_policy == "op"
        if model.ac_per_op:
            model.ac_recompute_mm_shapes = recompute_mm_shapes(model, sc.force_recompute_mm_shapes_by_fqns)
        return
    if mode == "memory_budget":
        b = training_config.memory_budget_ac.memory_budget
        if b >= 1.0:
            model.activation_checkpoint = "none"
        elif b <= 0.0:
            model.activation_checkpoint = "full"
        else:
            model.activation_checkpoint = "selective"
            model.ac_save_every = max(2, round(1.0 / b))
        return
    if mode == "region":
        rc = training_config.region_ac
        save = [re.compile(p) for p in rc.save_regions]
        rec = [re.compile(p) for p in rc.recompute_regions]
        recompute_all = not save
        sel = []
        for i in range(n_layers):
            name = f"model.layers.{i}"
            r = any(p.search(name) for p in rec) or (recompute_all and not rec)
            if any(p.search(name) for p in save):
                r = False
            sel.append(r)
        model.activation_checkpoint = "full" if all(sel) else ("none" if not any(sel) else "selective")
        model.ac_block_mask = sel
        return
    raise ValueError(mode)
