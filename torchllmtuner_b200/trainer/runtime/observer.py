"""Device-timed step observer (reference: llmtuner/trainer/runtime/training_observer.py:29-300): CUDA events
around the step, MAX over ranks of the step time, SUM of tokens, rolling steady-state percentiles after warm-up."""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


class TrainingObserver:
    def __init__(self, metrics_cfg, device, world_size: int):
        self.cfg, self.device, self.world = metrics_cfg, torch.device(device), world_size
        self.cuda = self.device.type == "cuda"
        self.window: list[float] = []
        self._t0 = None
        self._e0 = self._e1 = None
        self.steps_seen = 0

    def begin_step(self) -> None:
        if self.cuda:
            self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._e0.record()
        self._t0 = time.perf_counter()

    def end_step(self, tokens: int) -> tuple[float, int]:
        """Returns (slowest-rank step seconds, global tokens)."""
        if self.cuda:
            self._e1.record()
            self._e1.synchronize()
            sec = self._e0.elapsed_time(self._e1) / 1e3
        else:
            sec = time.perf_counter() - self._t0
        if dist.is_initialized() and self.world > 1:
            dev = self.device if self.cuda else torch.device("cpu")
            t = torch.tensor([sec], dtype=torch.float64, device=dev)
            n = torch.tensor([tokens], dtype=torch.int64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(n, op=dist.ReduceOp.SUM)
            sec, tokens = float(t.item()), int(n.item())
        self.steps_seen += 1
        if self.steps_seen > self.cfg.metrics_warmup_steps:
            self.window.append(sec)
            self.window = self.window[-self.cfg.steady_window_steps:]
        return sec, tokens

    def steady_state(self) -> dict[str, float]:
        if not self.window:
            return {}
        s = sorted(self.window)
        pick = lambda q: s[min(len(s) - 1, int(q * (len(s) - 1) + 0.5))]  # noqa: E731
        return {"steady/step_time_p50(s)": pick(0.5), "steady/step_time_p90(s)": pick(0.9)}


class DispatchTimer:
    """Device events around MoE token dispatch and combine (reference: llmtuner/trainer/runtime/training_observer.py:41-181).
    The MoE blocks call `span(kind)`; `collect()` turns the finished pairs of a step into p50 / p90 milliseconds."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.pending: dict[str, list] = {"dispatch": [], "combine": []}

    class _Span:
        def __init__(self, timer, kind):
            self.timer, self.kind = timer, kind

        def __enter__(self):
            if self.timer.cuda:
                self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self.a.record()
            else:
                self.t0 = time.perf_counter()
            return self

        def __exit__(self, *exc):
            if self.timer.cuda:
                self.b.record()
                self.timer.pending[self.kind].append((self.a, self.b))
            else:
                self.timer.pending[self.kind].append((time.perf_counter() - self.t0) * 1e3)
            return False

    def span(self, kind: str):
        return DispatchTimer._Span(self, kind)

    def collect(self) -> dict[str, float]:
        """Call after the step's device work has been synchronised (the observer's end_step does that)."""
        out = {}
        for kind, items in self.pending.items():
            ms = sorted((a.elapsed_time(b) if self.cuda else a) for a, b in items) if self.cuda else sorted(items)
            if ms:
                pick = lambda q: ms[min(len(ms) - 1, int(q * (len(ms) - 1) + 0.5))]  # noqa: E731
                out[f"moe/{kind}_p50(ms)"] = pick(0.5)
                out[f"moe/{kind}_p90(ms)"] = pick(0.9)
                out[f"moe/{kind}_total(ms)"] = float(sum(ms))
            items.clear()
        return out
