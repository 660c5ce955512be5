"""ctypes wrapper over ``csrc/sampling.cu``: temperature / top-k / top-p / min-p sampling on the device."""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import ptr, stream_ptr

_done = False


def _L():
    global _done
    lib = _native.lib()
    if not _done:
        P, I, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_ulonglong
        lib.mimir_sample.restype = I
        lib.mimir_sample.argtypes = [P, I, I, I, I, F, I, F, F, U, U, P, P, P, P]
        _done = True
    return lib


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
           seed: int = 0, draw: int = 0, return_prob: bool = False, draw_dev: torch.Tensor | None = None,
           out: torch.Tensor | None = None):
    """One token per row of ``logits`` ``[rows, V]`` (fp32 or bf16, on the GPU), as int32 ``[rows]``.

    ``draw`` numbers the call: with one seed, every (draw, row) pair gets its own uniform, element
    ``draw * 4 * ceil(rows / 4) + row`` of the Philox stream of ``seed`` (``tensor.random.philox_uniform``
    gives the same stream on the host).  ``draw_dev`` (an int32 tensor on the device) replaces ``draw``
    with a number read by the kernel, for decode steps replayed from a CUDA graph; ``out`` is an optional
    int32 ``[rows]`` result buffer.  ``temperature <= 0`` or ``top_k == 1`` is the arg-max."""
    if logits.dim() == 1:
        logits = logits[None]
    if logits.dtype not in (torch.float32, torch.bfloat16):
        logits = logits.float()
    if logits.stride(-1) != 1:
        logits = logits.contiguous()
    rows, V = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    prob = torch.empty(rows, dtype=torch.float32, device=logits.device) if return_prob else None
    _native.check(_L().mimir_sample(ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), rows, V,
                                    float(temperature), int(top_k), float(top_p), float(min_p),
                                    int(seed) & (2**64 - 1), int(draw),
                                    ptr(draw_dev) if draw_dev is not None else None, ptr(out),
                                    ptr(prob) if prob is not None else None, stream_ptr()), "sample")
    return (out, prob) if return_prob else out
