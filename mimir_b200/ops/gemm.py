"""tcgen05 bf16 GEMM with fused epilogues (``csrc/gemm_sm100.cu``).

Reference behaviour covered: ``OpMatMul`` with transposed operands and the
bias / activation / residual epilogue program (internal/sched/fuse.go:293-325).
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, require_cuda, stream_ptr

GEMM_FLAGS = {
    "out_f32": 1,
    "accumulate": 2,
    "gelu": 4,
    "residual": 8,
    "mul_dgelu": 16,
    "write_pre": 32,
}

_workspaces: dict = {}
_retired: list = []


def workspace(device, nbytes: int = 128 << 20) -> torch.Tensor:
    """Per-device split-K scratch buffer (grown on demand, never shrunk)."""
    key = (device.index if device.index is not None else torch.cuda.current_device())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)       # a captured CUDA graph may still point at it: never freed
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
         aux: torch.Tensor | None = None, aux_out: torch.Tensor | None = None,
         gelu: bool = False, residual: bool = False, mul_dgelu: bool = False,
         accumulate: bool = False, out_dtype: torch.dtype = torch.bfloat16, alpha: float = 1.0,
         splits: int = 0, bn: int = 0, use_workspace: bool = True) -> torch.Tensor:
    """``out[M,N] = epilogue(alpha * A @ B^T)`` with bf16 operands, fp32 accumulation.

    ``a`` is ``[M,K]`` (``a_mn=False``) or stored transposed ``[K,M]`` (``a_mn=True``);
    ``b`` is ``[N,K]`` (weight layout) or stored ``[K,N]`` (``b_mn=True``).
    Epilogue: ``+bias[N]``, then one of ``gelu`` (optionally writing the
    pre-activation to ``aux_out``), ``residual`` (``+aux``), ``mul_dgelu``
    (``* gelu'(aux)``); ``accumulate`` adds into ``out``.
    """
    require_cuda(a, b, out, bias, aux, aux_out)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm operands must be bfloat16")
    if a.dim() != 2 or b.dim() != 2 or a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("gemm operands must be 2-D with unit inner stride")
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm: contraction sizes differ ({K} vs {Kb})")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    flags = 0
    if out.dtype == torch.float32:
        flags |= 1
    elif out.dtype != torch.bfloat16:
        raise TypeError("gemm output must be bfloat16 or float32")
    if accumulate:
        flags |= 2
    if gelu:
        flags |= 4
        if aux_out is not None:
            flags |= 32
    if residual:
        flags |= 8
    if mul_dgelu:
        flags |= 16
    ldaux = 0
    if aux is not None:
        ldaux = aux.stride(0)
    if aux_out is not None:
        if aux is not None and aux.stride(0) != aux_out.stride(0):
            raise ValueError("aux and aux_out must share a row pitch")
        ldaux = aux_out.stride(0)
    ws = workspace(a.device) if use_workspace else None
    rc = _native.lib().mimir_gemm_bf16(
        ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), ptr(bias), ptr(aux), ldaux, ptr(aux_out), flags, float(alpha),
        ptr(ws), 0 if ws is None else ws.numel(), int(splits), int(bn), stream_ptr())
    _native.check(rc, "gemm")
    return out
