"""Activation swap: tensors saved for backward are moved to pinned host memory on a side stream during forward and
brought back on demand in backward, bounded by a host byte budget
(reference: llmtuner/memory/activation_swap.py:1-565; there an Ascend-only feature, here a CUDA host-offload option)."""
from __future__ import annotations

import torch


class ActivationSwap:
    def __init__(self, max_host_bytes: int = 0, min_bytes: int = 1 << 20, sync_release: bool = False):
        self.max_host_bytes, self.min_bytes, self.sync_release = max_host_bytes, min_bytes, sync_release
        self.host_bytes = 0
        self.d2h = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.stats = {"swapped": 0, "kept": 0}

    def _pack(self, t: torch.Tensor):
        nbytes = t.numel() * t.element_size()
        if (not t.is_cuda or nbytes < self.min_bytes or isinstance(t, torch.nn.Parameter) or
                (self.max_host_bytes and self.host_bytes + nbytes > self.max_host_bytes)):
            self.stats["kept"] += 1
            return ("keep", t)
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        self.d2h.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.d2h):
            host.copy_(t, non_blocking=True)
            ev = self.d2h.record_event()
        t.record_stream(self.d2h)
        self.host_bytes += nbytes
        self.stats["swapped"] += 1
        if self.sync_release:
            ev.synchronize()
        return ("host", host, ev, t.device, nbytes)

    def _unpack(self, packed):
        if packed[0] == "keep":
            return packed[1]
        _, host, ev, dev, nbytes = packed
        torch.cuda.current_stream().wait_event(ev)
        out = host.to(dev, non_blocking=True)
        self.host_bytes -= nbytes
        return out

    def hooks(self):
        return torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)


def apply_activation_swap(model, training_config) -> ActivationSwap:
    """Wraps every decoder block's forward in the saved-tensor hooks."""
    swap = ActivationSwap(training_config.activation_swap_max_host_bytes, sync_release=training_config.activation_swap_sync_release)
    layers = model.model.layers
    for layer in (layers.values() if isinstance(layers, torch.nn.ModuleDict) else layers):
        inner = layer.forward

        def fwd(*a, _inner=inner, **k):
            if torch.is_grad_enabled() and any(isinstance(x, torch.Tensor) and x.is_cuda for x in a):
                with swap.hooks():
                    return _inner(*a, **k)
            return _inner(*a, **k)
        layer.forward = fwd
    model.activation_swap = swap
    return swap
