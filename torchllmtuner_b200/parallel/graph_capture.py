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


def context_leaves(obj, max_depth: int = 6):
    """(tensors, constants) reachable from a forward context, in a fixed order. A captured graph reads the tensors by
    address and has the constants (document pieces, flags, sizes) baked into its launch parameters, so a later call may
    replay the graph only if its constants are equal and its tensors fit the captured ones."""
    tensors, consts = [], []

    def rec(o, depth):
        if isinstance(o, torch.Tensor):
            tensors.append(o)
        elif depth >= max_depth:
            consts.append(("deep", id(o)))
        elif isinstance(o, (list, tuple)):
            consts.append((type(o).__name__, len(o)))
            for x in o:
                rec(x, depth + 1)
        elif isinstance(o, dict):
            consts.append(("dict", tuple(o)))
            for k in o:
                rec(o[k], depth + 1)
        elif isinstance(o, (int, float, str, bool, type(None))):
            consts.append(o)
        elif hasattr(o, "__dict__") and type(o).__module__.startswith(__name__.split(".")[0]):
            consts.append(type(o).__qualname__)
            for k in sorted(vars(o)):
                consts.append(k)
                rec(vars(o)[k], depth + 1)
        else:
            consts.append(("object", id(o)))          # anything else must be the very same object
    rec(obj, 0)
    return tensors, consts


def _cuda_graph_capture(fn):
    """Warm up on a side stream, capture `fn()` in a CUDA graph; returns (its output, a replay function)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fn()
    return out, graph.replay


class GraphedInference(torch.nn.Module):
    """Replays a captured forward for evaluation-mode calls. The graph is tied to the input's shape AND to the forward
    context it was captured with: a call whose context has the same constants (same documents, same flags) and tensors of
    the same shapes copies them into the captured ones and replays; any other context is captured anew (a packed
    validation set with a different document layout per batch therefore gains nothing, and loses nothing but the
    capture). `capture` is the backend, replaceable for tests without a device."""

    def __init__(self, inner, capture=_cuda_graph_capture):
        super().__init__()
        self.inner, self.capture = inner, capture
        self.replay, self.static_in, self.static_out, self.static_tensors, self.static_consts = None, None, None, [], []
        self.captures = 0

    def _fits(self, x, tensors, consts) -> bool:
        return (self.replay is not None and self.static_in.shape == x.shape and consts == self.static_consts
                and len(tensors) == len(self.static_tensors)
                and all(a.shape == b.shape and a.dtype == b.dtype and a.device == b.device for a, b in zip(tensors, self.static_tensors)))

    def forward(self, x, ctx):
        if self.training or torch.is_grad_enabled() or (self.capture is _cuda_graph_capture and not x.is_cuda):
            return self.inner(x, ctx)
        tensors, consts = context_leaves(ctx)
        if not self._fits(x, tensors, consts):
            self.static_in = x.clone()
            self.static_tensors, self.static_consts = tensors, consts      # the captured context stays alive with the graph
            static_ctx = ctx
            self.static_out, self.replay = self.capture(lambda: self.inner(self.static_in, static_ctx))
            self.captures += 1
        else:
            for mine, new in zip(self.static_tensors, tensors):
                if mine is not new:
                    mine.copy_(new)
        self.static_in.copy_(x)
        self.replay()
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
