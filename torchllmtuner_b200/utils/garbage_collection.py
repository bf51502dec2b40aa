"""Manual GC every `gc_freq` steps so collection pauses are aligned across ranks
(reference: llmtuner/utils/garbage_collection.py:29-104)."""
from __future__ import annotations

import gc
import time


class GarbageCollection:
    def __init__(self, gc_freq: int = 50, disable_automatic: bool = True):
        if gc_freq < 1:
            raise ValueError("gc_freq must be >= 1")
        self.gc_freq = gc_freq
        self._was_enabled = gc.isenabled()
        self.last_pause_s = 0.0
        if disable_automatic:
            gc.disable()
        self.collect()

    def collect(self, generation: int = 1) -> None:
        t = time.perf_counter()
        gc.collect(generation)
        self.last_pause_s = time.perf_counter() - t

    def run(self, step: int) -> None:
        if step > 1 and step % self.gc_freq == 0:
            self.collect()

    def close(self) -> None:
        if self._was_enabled:
            gc.enable()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
