"""Profiler wrappers (reference: llmtuner/components/profiler.py:60-507).

`Profiler` drives `torch.profiler.profile` on a wait/warmup/active schedule and writes
`<dump>/<traces>/iteration_{step}/rank{rank}_trace.json.gz`. `MemoryProfiler` records allocator history and dumps
`step_{step:012d}/{rank:06d}_step_{step}.pickle` snapshots, plus one on an out-of-memory exit."""
from __future__ import annotations

import contextlib
import os
import pickle

import torch


def caused_by_oom(exc: BaseException) -> bool:
    return isinstance(exc, torch.cuda.OutOfMemoryError) or "out of memory" in str(exc).lower()


class MemoryProfiler:
    def __init__(self, cfg, dump_folder: str, rank: int):
        self.enabled = cfg.enable_memory_snapshot and torch.cuda.is_available()
        self.freq = cfg.memory_snapshot_freq or cfg.profile_freq
        self.folder = os.path.join(dump_folder, cfg.save_memory_snapshot_folder)
        self.rank, self.step_num = rank, 0
        if self.enabled:
            torch.cuda.memory._record_memory_history(max_entries=cfg.memory_snapshot_max_entries, stacks="python")

    def dump(self, tag: str | None = None) -> str | None:
        if not self.enabled:
            return None
        d = os.path.join(self.folder, f"step_{self.step_num:012d}" if tag is None else tag)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, f"{self.rank:06d}_step_{self.step_num}.pickle")
        with open(path, "wb") as f:
            pickle.dump(torch.cuda.memory._snapshot(), f)
        return path

    def step(self, exit_ctx: bool = False) -> None:
        self.step_num += 1
        if self.enabled and (exit_ctx or self.step_num % self.freq == 0):
            self.dump("oom" if exit_ctx else None)

    def close(self) -> None:
        if self.enabled:
            torch.cuda.memory._record_memory_history(enabled=None)


class Profiler(contextlib.AbstractContextManager):
    def __init__(self, cfg, dump_folder: str, rank: int):
        self.cfg, self.rank = cfg, rank
        self.folder = os.path.join(dump_folder, cfg.save_traces_folder)
        self.memory = MemoryProfiler(cfg, dump_folder, rank)
        self.prof = None
        self.step_num = 0
        if cfg.enable_profiling:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            wait = cfg.profile_freq - (cfg.profiler_active + cfg.profiler_warmup)
            sched = torch.profiler.schedule(wait=wait, warmup=cfg.profiler_warmup, active=cfg.profiler_active,
                                            repeat=cfg.profiler_repeat or 0,
                                            skip_first=cfg.profiler_skip_first or 0)
            self.prof = torch.profiler.profile(activities=acts, schedule=sched, on_trace_ready=self._on_trace, record_shapes=True)

    def _on_trace(self, prof) -> None:
        d = os.path.join(self.folder, f"iteration_{self.step_num}")
        os.makedirs(d, exist_ok=True)
        prof.export_chrome_trace(os.path.join(d, f"rank{self.rank}_trace.json.gz"))

    def __enter__(self):
        if self.prof is not None:
            self.prof.__enter__()
        return self

    def __exit__(self, et, ev, tb):
        if ev is not None and caused_by_oom(ev):
            self.memory.step(exit_ctx=True)
        if self.prof is not None:
            self.prof.__exit__(et, ev, tb)
        return False

    def step(self) -> None:
        self.step_num += 1
        if self.prof is not None:
            self.prof.step()
        self.memory.step()

    def close(self) -> None:
        self.memory.close()


def build_profiler(config, env) -> Profiler:
    return Profiler(config.training.profiler_config, config.training.dump_folder, env.rank)
