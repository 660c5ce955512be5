"""Per-phase timing of a training step (the reference reports host time per phase of
``Parallel.Backward`` and, with MIMIR_DP_WAITS=1, device time by forcing synchronisation:
train/parallel.go:288-315).  Here a phase is bracketed by CUDA events on the launching stream (no
synchronisation inside the step), optionally wrapped in an NVTX range for timeline tools, and the
report takes the maximum over the ranks of a process group.  On a machine without CUDA the same
calls measure host time."""
from __future__ import annotations

import contextlib
import time

import torch


class PhaseTimer:
    def __init__(self, nvtx: bool = False, enabled: bool = True):
        self.cuda = torch.cuda.is_available()
        self.nvtx = nvtx and self.cuda
        self.enabled = enabled
        self._open = []     # (name, start event or host time, stop event or host time)
        self.totals, self.counts = {}, {}

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        else:
            a = time.perf_counter()
        try:
            yield
        finally:
            if self.cuda:
                b.record()
            else:
                b = time.perf_counter()
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
            self._open.append((name, a, b))

    def collect(self) -> dict:
        """Folds the finished phases into the totals (synchronises once) and returns milliseconds per phase."""
        if self.cuda and self._open:
            torch.cuda.synchronize()
        for name, a, b in self._open:
            ms = a.elapsed_time(b) if self.cuda else (b - a) * 1e3
            self.totals[name] = self.totals.get(name, 0.0) + ms
            self.counts[name] = self.counts.get(name, 0) + 1
        self._open = []
        return dict(self.totals)

    def report(self, group=None) -> dict:
        """``{phase: {"ms": total, "calls": n, "ms_per_call": ...}}``; with a process group the slowest rank counts."""
        totals = self.collect()
        names = sorted(totals)
        vals = torch.tensor([totals[n] for n in names], dtype=torch.float64)
        if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
            dev = "cuda" if self.cuda and torch.distributed.get_backend(group) == "nccl" else "cpu"
            v = vals.to(dev)
            torch.distributed.all_reduce(v, op=torch.distributed.ReduceOp.MAX, group=group)
            vals = v.cpu()
        return {n: {"ms": float(v), "calls": self.counts[n], "ms_per_call": float(v) / self.counts[n]}
                for n, v in zip(names, vals)}

    def reset(self) -> None:
        self._open, self.totals, self.counts = [], {}, {}
