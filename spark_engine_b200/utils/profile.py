"""Section timers, NVTX ranges and the profiler window.

`Profiler.section(name)` accumulates wall/device milliseconds per named section (CUDA events on the current
stream, read lazily, no device-wide synchronisation per section); with `nvtx=True` every section is also an NVTX
range; `profiler_window()` brackets steady-state work with cudaProfilerStart/Stop so `ncu --profile-from-start
off` captures only that.  Reference: engine-rs/src/ds41/model.rs:3045-3075 (prof sections), profile.rs:23-26,
shim.cpp:1274-1276 (NVTX push/pop).
"""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict

import torch


class Profiler:
    def __init__(self, enabled: bool = False, nvtx: bool = False):
        self.enabled, self.nvtx = enabled, nvtx
        self.ms = defaultdict(float)
        self.calls = defaultdict(int)
        self._pending = []

    @contextlib.contextmanager
    def section(self, name: str):
        if not (self.enabled or self.nvtx):
            yield
            return
        cuda = torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing()
        if self.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
        t0 = time.perf_counter()
        ev = None
        if cuda and self.enabled:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        try:
            yield
        finally:
            if ev is not None:
                ev[1].record()
                self._pending.append((name, ev))
            elif self.enabled:
                self.ms[name] += (time.perf_counter() - t0) * 1e3
            self.calls[name] += 1
            if self.nvtx and torch.cuda.is_available():
                torch.cuda.nvtx.range_pop()

    def table(self) -> dict:
        still = []
        for name, ev in self._pending:
            if ev[1].query():
                self.ms[name] += ev[0].elapsed_time(ev[1])
            else:
                still.append((name, ev))
        self._pending = still
        return {k: round(v, 3) for k, v in self.ms.items()}


@contextlib.contextmanager
def profiler_window():
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStart()
    try:
        yield
    finally:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStop()
