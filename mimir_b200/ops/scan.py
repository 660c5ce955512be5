"""ctypes wrapper over ``csrc/scan.cu``: running sum / maximum / log-sum-exp along one axis."""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import ptr, stream_ptr

_MODES = {"sum": 0, "max": 1, "logsumexp": 2}
_done = False


def _L():
    global _done
    lib = _native.lib()
    if not _done:
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.mimir_scan_rows.restype = I
        lib.mimir_scan_rows.argtypes = [P, P, I, I, I, L, L, I, I, P]
        _done = True
    return lib


def supported(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.numel() > 0 and x.dim() >= 1


def scan(x: torch.Tensor, mode: str, dim: int = -1, reverse: bool = False) -> torch.Tensor:
    """Inclusive scan of ``x`` (fp32 or bf16, on the GPU) along ``dim``."""
    dim %= x.dim()
    moved = dim != x.dim() - 1
    src = (x.transpose(dim, -1) if moved else x).contiguous()
    n = src.shape[-1]
    out = torch.empty_like(src)
    _native.check(_L().mimir_scan_rows(ptr(src), ptr(out), int(src.dtype == torch.float32), src.numel() // n, n, n, n,
                                       _MODES[mode], int(reverse), stream_ptr()), "scan_rows")
    return out.transpose(dim, -1) if moved else out
