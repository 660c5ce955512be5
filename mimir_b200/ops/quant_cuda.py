"""ctypes wrappers over ``csrc/quant_sm100.cu``."""
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
        P, I, F, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
        PP = ctypes.POINTER(ctypes.c_void_p)
        for name, args in {
            "mimir_dequant": [I, P, P, L, P],
            "mimir_qgemv_ggml": [I, P, P, I, I, P, P, I, I, I, I, P],
            "mimir_q4_0_to_planar": [P, P, P, L, P],
            "mimir_quantize_act": [P, I, P, P, P, P, I, I, I, F, P],
            "mimir_q4_gemv": [P, P, P, P, P, I, I, I, I, I, P],
            "mimir_q4_gemv_allreduce": [P, P, P, P, PP, PP, P, P, P, P, I, I, I, I, I, I, P],
            "mimir_oneshot_allreduce": [PP, PP, P, P, P, P, I, I, I, I, I, P],
            "mimir_attn_decode": [P, P, P, P, I, I, I, I, I, P, F, I, P, P, I, P],
            "mimir_kv_cache_write": [P, I, I, I, P, P, I, I, I, I, P, P],
            "mimir_f32_to_bf16": [P, P, L, P],
            "mimir_rope_kv_write": [P, I, P, P, P, P, I, I, I, I, I, P, P],
            "mimir_q4_planar_to_bf16": [P, P, P, L, P],
            "mimir_peer_allgather": [P, PP, PP, P, P, L, I, I, I, P],
            "mimir_q4_planar_to_tiled": [P, P, P, I, I, P],
            "mimir_round_act_q8": [P, P, P, I, P, P, I, I, I, F, P],
            "mimir_q4_tc": [P, P, I, PP, PP, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P],
        }.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = I, args
        lib.mimir_q4_tiled_bytes.argtypes, lib.mimir_q4_tiled_bytes.restype = [I, I], L
        lib.mimir_q_set_peer_wait_ms.argtypes = [L]
        lib.mimir_q_set_peer_wait_ms.restype = None
        _done = True
    return lib


def dequantize(code: int, raw: torch.Tensor, n: int) -> torch.Tensor:
    out = torch.empty(n, dtype=torch.float32, device=raw.device)
    _native.check(_L().mimir_dequant(code, ptr(raw), ptr(out), n, stream_ptr()), "dequant")
    return out


def qgemv_ggml(code: int, raw: torch.Tensor, N: int, K: int, x: torch.Tensor, bias=None) -> torch.Tensor:
    """``x [B, K] @ dequant(W [N, K])^T`` with ``W`` read in its ggml block encoding (Q8_0, Q4_0, Q4_K,
    Q6_K); fp32 result ``[B, N]``.  ``x`` is fp32 or bf16, rows contiguous."""
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    x = x.contiguous()
    if K % 8:
        raise ValueError("qgemv: K must be a multiple of 8")
    out = torch.empty(x.shape[0], N, dtype=torch.float32, device=x.device)
    b = None if bias is None else bias.float().contiguous()
    _native.check(_L().mimir_qgemv_ggml(code, ptr(raw), ptr(x), int(x.dtype == torch.float32), K,
                                        ptr(b) if b is not None else None, ptr(out), N, N, K, x.shape[0],
                                        stream_ptr()), "qgemv_ggml")
    return out


class PlanarQ4:
    """Q4_0 weight matrix [N, K] in the GPU layout: fp16 scales [N, K/32] + 16-byte quants."""

    def __init__(self, scales: torch.Tensor, quants: torch.Tensor, N: int, K: int):
        self.scales, self.quants, self.N, self.K = scales, quants, N, K

    @staticmethod
    def from_ggml(raw: torch.Tensor, N: int, K: int) -> "PlanarQ4":
        nb = N * K // 32
        raw = raw.contiguous()
        scales = torch.empty(nb, dtype=torch.float16, device=raw.device)
        quants = torch.empty(nb * 16, dtype=torch.uint8, device=raw.device)
        _native.check(_L().mimir_q4_0_to_planar(ptr(raw), ptr(scales), ptr(quants), nb, stream_ptr()), "to_planar")
        return PlanarQ4(scales, quants, N, K)

    @staticmethod
    def quantize(w: torch.Tensor) -> "PlanarQ4":
        from .quant import quantize_q4_0
        N, K = w.shape
        return PlanarQ4.from_ggml(quantize_q4_0(w).reshape(-1), N, K)

    def to_bf16(self, out: torch.Tensor | None = None) -> torch.Tensor:
        out = torch.empty(self.N, self.K, dtype=torch.bfloat16, device=self.scales.device) if out is None else out
        _native.check(_L().mimir_q4_planar_to_bf16(ptr(self.scales), ptr(self.quants), ptr(out),
                                                   self.N * self.K // 32, stream_ptr()), "planar_to_bf16")
        return out

    def nbytes(self) -> int:
        return self.scales.numel() * 2 + self.quants.numel()


def quantize_act(x, xq, xs, K, mode=0, gamma=None, y=None, eps=1e-5):
    """Planar Q8_0 of the activation rows (int8 ``xq`` with row pitch K, scales ``xs``); bf16 inputs take
    the kernel that spreads a row over many blocks, fp32 inputs the warp-per-row one."""
    if x.dtype == torch.bfloat16 and y is None:
        round_act_q8(x, None, K, mode, gamma, eps, xq, xs)
        return
    rows = xq.shape[0]
    _native.check(_L().mimir_quantize_act(ptr(x), int(x.dtype == torch.float32), ptr(gamma), ptr(y), ptr(xq), ptr(xs),
                                          rows, K, mode, eps, stream_ptr()), "quantize_act")


def q4_gemv(w: PlanarQ4, xq, xs, out):
    B = xq.shape[0]
    _native.check(_L().mimir_q4_gemv(ptr(w.scales), ptr(w.quants), ptr(xq), ptr(xs), ptr(out),
                                     int(out.dtype == torch.bfloat16), w.N, w.K, B, out.stride(0), stream_ptr()), "q4_gemv")
    return out


def attn_decode(q, kc, vc, length, scale=None, splits=0, out=None):
    """Single-query attention of ``q`` [B, Hq, D] bf16 over the fp16 cache ``kc``/``vc``
    [B, Hkv, cap, D]; ``length`` is a 1-element int32 device tensor with the number of valid keys.
    ``splits`` = 0 picks enough key ranges to fill the GPU."""
    B, Hq, D = q.shape
    Hkv, cap = kc.shape[1], kc.shape[2]
    if splits <= 0:
        sms = torch.cuda.get_device_properties(q.device).multi_processor_count
        splits = max(1, min((cap + 63) // 64, (4 * sms) // max(1, B * Hkv), 64))
    ws = torch.empty(B * Hq * splits * (D + 2), dtype=torch.float32, device=q.device)
    cnt = torch.zeros(B * Hkv, dtype=torch.int32, device=q.device)
    out = torch.empty(B, Hq, D, dtype=torch.bfloat16, device=q.device) if out is None else out
    _native.check(_L().mimir_attn_decode(ptr(q), ptr(kc), ptr(vc), ptr(out), B, Hq, Hkv, D, cap, ptr(length),
                                         float(scale if scale is not None else D ** -0.5), q.stride(0), ptr(ws),
                                         ptr(cnt), splits, stream_ptr()), "attn_decode")
    return out


class TiledQ4:
    """Q4_0 weight matrix [N, K] in the tensor-core kernel's layout: per (128-row tile, 64-column
    k-block) 4608 contiguous bytes (quants [2][128][16], then fp16 scales [2][128])."""

    def __init__(self, blob: torch.Tensor, N: int, K: int):
        self.blob, self.N, self.K = blob, N, K

    @staticmethod
    def from_planar(w: PlanarQ4) -> "TiledQ4":
        if w.K % 64:
            raise ValueError("tiled Q4_0 needs K % 64 == 0")
        blob = torch.empty(_L().mimir_q4_tiled_bytes(w.N, w.K), dtype=torch.uint8, device=w.scales.device)
        _native.check(_L().mimir_q4_planar_to_tiled(ptr(w.scales), ptr(w.quants), ptr(blob), w.N, w.K, stream_ptr()),
                      "planar_to_tiled")
        return TiledQ4(blob, w.N, w.K)

    @staticmethod
    def quantize(w: torch.Tensor) -> "TiledQ4":
        return TiledQ4.from_planar(PlanarQ4.quantize(w))

    def nbytes(self) -> int:
        return self.blob.numel()


def round_act_q8(x, y, K, mode=0, gamma=None, eps=1e-5, xq=None, xs=None):
    """y [rows, K] bf16 = the Q8_0 rounding (32-value blocks) of x (mode 0), of RMSNorm(x) * gamma
    (mode 1) or of silu(gate) * up for x = [rows, 2K] (mode 2).  With ``xq`` / ``xs`` the planar
    Q8_0 form (int8 values, fp32 scale per 32) is written too; ``y`` may then be None."""
    _native.check(_L().mimir_round_act_q8(ptr(x), ptr(gamma), ptr(y), y.stride(0) if y is not None else 0, ptr(xq),
                                          ptr(xs), x.shape[0], K, mode, eps, stream_ptr()), "round_act_q8")
    return y


class TcScratch:
    """Single-GPU scratch of ``q4_tc``: split-K partials, flag pad, epoch and arrival counter."""

    def __init__(self, max_elems: int, device, max_splits: int = 8):
        self.max_splits = max_splits
        self.partial = torch.zeros(max_splits * max_elems, dtype=torch.float32, device=device)
        self.sig = torch.zeros(64, dtype=torch.int32, device=device)
        self.words = torch.zeros(2, dtype=torch.int32, device=device)
        self.partial_arr = (ctypes.c_void_p * 1)(self.partial.data_ptr())
        self.sig_arr = (ctypes.c_void_p * 1)(self.sig.data_ptr())


def q4_tc(w: TiledQ4, x, out, scratch: TcScratch, residual=None, splits=0):
    """out[b, n] = residual[b, n] + sum_k W[n, k] x[b, k] on the tensor cores (one GPU); x bf16 [B, K]."""
    B = x.shape[0]
    _native.check(_L().mimir_q4_tc(ptr(w.blob), ptr(x), x.stride(0), scratch.partial_arr, scratch.sig_arr,
                                   scratch.words.data_ptr(), scratch.words[1:].data_ptr(), ptr(residual), ptr(out),
                                   int(out.dtype == torch.float32), out.stride(0), w.N, w.K, B, splits,
                                   scratch.max_splits, 0, 1, 0, stream_ptr()), "q4_tc")
    return out
