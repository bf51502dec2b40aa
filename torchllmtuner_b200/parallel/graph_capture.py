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
    """Silent-data-corruption guard: raises when a block returns non-finite values."""

    def __init__(self, inner):
        super().__init__()
        self.inner = inner

    def forward(self, *a, **k):
        out = self.inner(*a, **k)
        if not torch.isfinite(out.float().sum()):
            raise LLMTunerError(f"non-finite output of {type(self.inner).__name__}")
        return out

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("inner"), name)


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
    for i in range(len(layers)):
        blk = layers[i]
        if compile_config.enable_sdc:
            blk = SDCGuard(blk)
        if compile_config.per_block and compile_config.backend == "cudagraph":
            blk = GraphedInference(blk)
        layers[i] = blk
