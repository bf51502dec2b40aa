"""Moves over nested containers of tensors (reference: llmtuner/accelerator/tensor_tree.py:18-128)."""
from __future__ import annotations

import torch


def _children(obj):
    if isinstance(obj, dict):
        return list(obj.values())
    if isinstance(obj, (list, tuple)):
        return list(obj)
    return []


def get_tensor_tree_device(tree):
    if isinstance(tree, torch.Tensor):
        return tree.device
    for c in _children(tree):
        d = get_tensor_tree_device(c)
        if d is not None:
            return d
    return None


def move_tensor_tree(tree, device, non_blocking: bool = True):
    if isinstance(tree, torch.Tensor):
        return tree.to(device, non_blocking=non_blocking)
    if isinstance(tree, dict):
        return {k: move_tensor_tree(v, device, non_blocking) for k, v in tree.items()}
    if isinstance(tree, tuple):
        return tuple(move_tensor_tree(v, device, non_blocking) for v in tree)
    if isinstance(tree, list):
        return [move_tensor_tree(v, device, non_blocking) for v in tree]
    return tree


def clone_local_tensor(t: torch.Tensor) -> torch.Tensor:
    return t.detach().clone()
