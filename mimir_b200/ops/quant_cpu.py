"""CPU products with block-quantized weights read in place (``csrc/cpu_quant.cc``): the host path of
decoding, where the reference keeps its weights quantized too (backend/cpu/quant.go,
llm/decode.go:79-160).  ``mode``: ``"exact"`` multiplies float activations with weights decoded value
by value (exactly ``x @ dequant(W)^T`` up to float summation order); ``"int8"`` rounds the
activation rows to 32-value int8 blocks and uses VNNI dot products (the CPU must have AVX-512 VNNI);
``"auto"`` takes int8 where the CPU has it."""
from __future__ import annotations

import ctypes

import torch

from .. import _native

_MODES = {"exact": 0, "int8": 1, "auto": -1}
MAX_ROWS = 8


def _lib():
    lib = _native.lib()
    if not getattr(lib, "_cpuq_bound", False):
        c = ctypes
        lib.mimir_cpu_qgemv.argtypes = [c.c_int, c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_void_p]
        lib.mimir_cpu_qgemv_has_int8.restype = c.c_int
        lib.mimir_cpu_set_threads.argtypes = [c.c_int]
        lib._cpuq_bound = True
    return lib


def has_int8() -> bool:
    return bool(_lib().mimir_cpu_qgemv_has_int8())


def set_threads(n: int) -> int:
    """Threads of the next products (0 = one per hardware thread); returns the previous setting."""
    return _lib().mimir_cpu_set_threads(int(n))


def qgemv(code: int, raw: torch.Tensor, n: int, k: int, x: torch.Tensor, mode: str = "auto") -> torch.Tensor:
    """``x [B, K] @ W^T`` -> fp32 ``[B, N]`` for a weight of ``n`` rows of ``k`` values stored as ggml
    blocks of ``code`` in the uint8 tensor ``raw``; up to 8 rows per call (more are chunked)."""
    if raw.device.type != "cpu" or raw.dtype != torch.uint8 or not raw.is_contiguous():
        raise ValueError("qgemv: the weight must be a contiguous uint8 CPU tensor")
    rows = x.reshape(-1, x.shape[-1]).float().contiguous()
    if rows.shape[1] != k:
        raise ValueError(f"qgemv: activations of {rows.shape[1]} columns for a weight of {k}")
    out = torch.empty(rows.shape[0], n, dtype=torch.float32)
    lib = _lib()
    for b0 in range(0, rows.shape[0], MAX_ROWS):
        xb = rows[b0:b0 + MAX_ROWS]
        yb = out[b0:b0 + MAX_ROWS]
        rc = lib.mimir_cpu_qgemv(code, raw.data_ptr(), n, k, xb.data_ptr(), xb.shape[0], yb.data_ptr(), _MODES[mode], None)
        if rc:
            raise ValueError(f"qgemv: unsupported arguments (code {code}, N {n}, K {k}, mode {mode})")
    return out


def dequant_bf16(code: int, raw: torch.Tensor, n: int, k: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """The weight's values as a bfloat16 ``[n, k]`` tensor (written into ``out`` when given: one scratch
    buffer serves every matrix of a model), expanded by the worker pool."""
    if raw.device.type != "cpu" or raw.dtype != torch.uint8 or not raw.is_contiguous():
        raise ValueError("dequant_bf16: the weight must be a contiguous uint8 CPU tensor")
    if out is None:
        out = torch.empty(n, k, dtype=torch.bfloat16)
    elif out.dtype != torch.bfloat16 or out.numel() < n * k or not out.is_contiguous():
        raise ValueError("dequant_bf16: the scratch buffer must be contiguous bfloat16 of at least n * k values")
    lib = _lib()
    if not getattr(lib, "_dequant_bound", False):
        import ctypes
        lib.mimir_cpu_dequant_bf16.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.mimir_cpu_dequant_bf16.restype = ctypes.c_int
        lib._dequant_bound = True
    view = out.reshape(-1)[: n * k].view(n, k)
    if lib.mimir_cpu_dequant_bf16(int(code), raw.data_ptr(), n, k, view.data_ptr()) != 0:
        raise ValueError(f"dequant_bf16: bad arguments (code {code}, {n} x {k})")
    return view


class DecodeLayer(ctypes.Structure):
    """The argument block of ``mimir_cpu_decode_layer`` (``csrc/cpu_decode.cc``): one decoder layer for one
    new token per sequence.  The caller keeps every tensor whose address it holds alive."""

    _fields_ = [(n, ctypes.c_int32) for n in (
        "B", "E", "H", "Hk", "D", "hidden", "rope_dim", "interleaved", "pos", "cap", "mode", "qkv_code", "o_code",
        "gate_up_code", "down_code", "pad_")] + [("eps", ctypes.c_float), ("pad2_", ctypes.c_float)] + [
        (n, ctypes.c_void_p) for n in ("attn_norm", "ffn_norm", "qkv_bias", "inv_freq", "qkv", "o", "gate_up", "down",
                                       "k_cache", "v_cache", "x", "scratch")]


def decode_scratch(B: int, E: int, H: int, Hk: int, D: int, hidden: int, cap: int) -> int:
    """Floats of scratch one ``decode_layer`` call needs."""
    lib = _lib()
    lib.mimir_cpu_decode_scratch.restype = ctypes.c_longlong
    lib.mimir_cpu_decode_scratch.argtypes = [ctypes.c_int] * 7
    return int(lib.mimir_cpu_decode_scratch(B, E, H, Hk, D, hidden, cap))


def decode_layer(args: DecodeLayer) -> None:
    """Runs one layer in place on ``args.x`` and appends the new key and value rows at ``args.pos``."""
    lib = _lib()
    if not getattr(lib, "_decode_bound", False):
        lib.mimir_cpu_decode_layer.argtypes = [ctypes.POINTER(DecodeLayer)]
        lib.mimir_cpu_decode_layer.restype = ctypes.c_int
        lib._decode_bound = True
    if lib.mimir_cpu_decode_layer(ctypes.byref(args)) != 0:
        raise ValueError("decode_layer: bad arguments")
