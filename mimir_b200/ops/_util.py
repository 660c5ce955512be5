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
