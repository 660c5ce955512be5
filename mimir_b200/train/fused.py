"""Fused training step for the kernel-sequence engines (``models/gpt2.py``).

``FusedTrainer.step(tokens, targets)`` is the call a user makes: it copies the
batch from pinned host memory, replays the captured CUDA graph of forward +
loss + backward + AdamW, and returns the loss read back from the device.  The
capture plays the role of the reference's plan cache and step replay
(internal/sched/replay.go:63-204, tensor/record.go:70-184): structure is frozen,
the learning rate and bias corrections stay run-time values read from device
memory, so replays follow any schedule.
"""
from __future__ import annotations

import os

import torch

from .. import _native


class FusedTrainer:
    def __init__(self, engine, lr: float = 6e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, use_graph: bool = True, schedule=None, dp=None, phases=None):
        """``phases``: a ``utils.phases.PhaseTimer``; forward / loss / backward / optimizer of every step
        are then bracketed by CUDA events on the launching stream (and NVTX ranges when the timer was
        made with ``nvtx=True`` or ``MIMIR_NVTX=1`` is set), and ``phases.report()`` gives device time
        per phase, the slowest rank counting.  Phase timing needs plain launches: it switches the
        CUDA-graph replay off."""
        self.engine = engine
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        # MIMIR_CUDA_GRAPHS=0 runs every step as plain launches (reference: backend/cuda/batch_linux.go:63)
        if phases is None and os.environ.get("MIMIR_NVTX", "") == "1":
            from ..utils.phases import PhaseTimer
            phases = PhaseTimer(nvtx=True)
        self.phases = phases
        self.use_graph = use_graph and os.environ.get("MIMIR_CUDA_GRAPHS", "1") != "0" and phases is None
        self.schedule = schedule
        self.dp = dp  # optional parallel.dp.FusedDataParallel
        self.graph = None
        self.launches_per_step = 0
        self._warm = 0
        dev = engine.device
        self._tok_host = torch.zeros(engine.M, dtype=torch.int64).pin_memory()
        self._tgt_host = torch.zeros(engine.M, dtype=torch.int64).pin_memory()
        self._loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.h2d_bytes_per_step = 2 * engine.M * 8 + 16
        self.d2h_bytes_per_step = 4
        self._stream = torch.cuda.current_stream(dev)

    # The device work of one step, launched on the current stream.
    def _device_step(self) -> None:
        e = self.engine
        import contextlib
        ph = self.phases.phase if self.phases is not None else (lambda name: contextlib.nullcontext())
        if self.dp is not None:
            self.dp.begin_step()
        with ph("forward"):
            e.forward()
        with ph("loss"):
            e.loss_and_dlogits()
        if self.dp is not None:
            with ph("backward+reduce+update"):
                self.dp.run_backward_and_update(self)
        else:
            with ph("backward"):
                e.backward()
            with ph("optimizer"):
                e.adamw(self.betas[0], self.betas[1], self.eps, self.wd)

    def _current_lr(self) -> float:
        if self.schedule is None:
            return self.lr
        return float(self.schedule(self.engine.step_count))

    def stage_hyper(self) -> None:
        world = 1 if self.dp is None else self.dp.world
        self.engine.set_hyper(self._current_lr(), self.betas[0], self.betas[1], 1.0 / world)

    def run_device_step(self) -> None:
        """Stages hyperparameters and runs (or replays) the step; no host sync."""
        lib = _native.lib()
        self.stage_hyper()
        if not self.use_graph:
            before = lib.mimir_launch_count()
            self._device_step()
            self.launches_per_step = lib.mimir_launch_count() - before
            return
        if self.graph is None:
            if self._warm < 2:  # eager warm-up: first launches configure kernels and scratch
                self._warm += 1
                before = lib.mimir_launch_count()
                self._device_step()
                self.launches_per_step = lib.mimir_launch_count() - before
                return
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = lib.mimir_launch_count()
            with torch.cuda.graph(g):
                self._device_step()
            self.launches_per_step = lib.mimir_launch_count() - before
            self.graph = g
        self.graph.replay()
        lib.mimir_launch_count_add(self.launches_per_step)

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> float:
        """One optimizer step on a host batch ``[B, T]`` of token ids; returns the loss."""
        e = self.engine
        if tokens.is_cuda:
            e.tokens.copy_(tokens.reshape(-1), non_blocking=True)
            e.targets.copy_(targets.reshape(-1), non_blocking=True)
        else:
            if not tokens.is_pinned():
                self._tok_host.copy_(tokens.reshape(-1))
                self._tgt_host.copy_(targets.reshape(-1))
                tokens, targets = self._tok_host, self._tgt_host
            e.tokens.copy_(tokens.reshape(-1), non_blocking=True)
            e.targets.copy_(targets.reshape(-1), non_blocking=True)
        self.run_device_step()
        self._loss_host.copy_(e.loss, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        # the error word lives in host-mapped memory: reading it costs a memory load.  A wait on a peer
        # that ran out means this rank skipped its slice of the update, so the step must not pass
        # silently (the word is cleared: the caller decides whether to resume from a checkpoint).
        word = int(_native.lib().mimir_error_word(0))
        if word:
            from ..parallel.health import DeviceFault
            _native.lib().mimir_error_word(1)
            raise DeviceFault(word)
        return float(self._loss_host[0])
