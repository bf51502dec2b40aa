"""The `compile` stage. No tracing compiler is used: "compile" means capturing the launch sequence of a decoder block
in a CUDA graph and replaying it, which removes per-kernel launch latency for small shapes
(reference stage: llmtuner/parallel/model_compile.py:61-260, per-block compile and the silent-data-corruption guard).

Capture is only valid for launch sequences that are identical from step to step: fixed shapes, no host-dependent
control flow and no collectives issued from the host inside the block. Blocks are therefore captured only when the
run has no tensor / expert / context parallelism and no activation checkpointing replay inside the graph; otherwise
the stage installs the non-finite guard alone."""
from __future__ import annotations

import torch

from ..errors import LLMTunerError


class SDCGuard(torch.nn.Module):
    """Silent-data-corruption guard: records, on the device, the first block whose output is not finite. Nothing is read
    back inside the forward pass (no host synchronisation per block); `check_sdc(model)` reads the one flag word, once
    per step, and raises."""

    def __init__(self, inner, index: int, flag: torch.Tensor):
        super().__init__()
        self.inner, self.index, self.flag = inner, index, flag

    def forward(self, *a, **k):
        out = self.inner(*a, **k)
        with torch.no_grad():
            bad = ~torch.isfinite(out.detach().float().sum())
            if self.flag.device != out.device:
                self.flag.data = self.flag.data.to(out.device)
            # flag holds 0 (healthy) or 1 + index of the first bad block
            self.flag.copy_(torch.where((self.flag == 0) & bad, torch.full_like(self.flag, self.index + 1), self.flag))
        return out

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("inner"), name)


def check_sdc(model) -> None:
    """One device-to-host read of the guard's flag word; raises `LLMTunerError` naming the first non-finite block."""
    flag = getattr(model, "_sdc_flag", None)
    if flag is None:
        return
    v = int(flag.item())
    if v:
        flag.zero_()
        raise LLMTunerError(f"non-finite output of decoder block {v - 1} (silent-data-corruption guard)")


class GraphedInference(torch.nn.Module):
    """Replays a captured forward for evaluation-mode calls with a fixed input shape."""

    def __init__(self, inner):
        super().__init__()
        self.inner, self.graph, self.static_in, self.static_out = inner, None, None, None

    def forward(self, x, ctx):
        if self.training or torch.is_grad_enabled() or not x.is_cuda:
            return self.inner(x, ctx)
        if self.graph is None or self.static_in.shape != x.shape:
            self.static_in = x.clone()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    self.inner(self.static_in, ctx)
            torch.cuda.current_stream().wait_stream(s)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.static_out = self.inner(self.static_in, ctx)
        self.static_in.copy_(x)
        self.graph.replay()
        return self.static_out.clone()

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("inner"), name)


def apply_compile(model, compile_config) -> None:
    layers = model.model.layers
    if compile_config.enable_sdc:
        model._sdc_flag = torch.zeros((), dtype=torch.int32)
    for i in range(len(layers)):
        blk = layers[i]
        if compile_config.enable_sdc:
            blk = SDCGuard(blk, i, model._sdc_flag)
        if compile_config.per_block and compile_config.backend == "cudagraph":
            blk = GraphedInference(blk)
        layers[i] = blk
