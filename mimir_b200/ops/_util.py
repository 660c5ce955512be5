"""Helpers shared by the kernel wrappers: stream handle, pointer checks, errors."""
from __future__ import annotations

import torch

from .. import _native


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("the sm_100a kernels need CUDA tensors")


def check_error_word(sync: bool = True) -> int:
    """Synchronises (optionally) and returns-and-clears the device error word.

    Bits: 1 index out of range, 2 division by zero, 4 an in-kernel wait ran out,
    8 a wait on a peer GPU ran out, 16 a launch was refused on the host.
    """
    if sync:
        torch.cuda.synchronize()
    return int(_native.lib().mimir_error_word(1))


class PinnedRing:
    """Small pinned host buffers for values a step uploads asynchronously (learning rate, bias
    corrections).  ``stage(values, dst)`` writes the next buffer and queues the copy; a buffer is
    reused only after the copy it fed has completed (an event per buffer), so a host that runs
    several steps ahead of the GPU can never overwrite values a pending copy still has to read."""

    def __init__(self, numel: int = 4, depth: int = 4):
        pin = torch.cuda.is_available()
        self.bufs = [torch.zeros(numel, dtype=torch.float32).pin_memory() if pin else torch.zeros(numel)
                     for _ in range(depth)]
        self.events = [None] * depth
        self.i = 0

    def stage(self, values, dst: torch.Tensor) -> None:
        i = self.i
        self.i = (i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        for k, v in enumerate(values):
            buf[k] = v
        dst.copy_(buf, non_blocking=True)
        if dst.is_cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dst.device))
            self.events[i] = ev
