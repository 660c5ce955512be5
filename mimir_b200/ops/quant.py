"""Block-quantized tensors (ggml layouts): Q8_0, Q4_0, Q4_K, Q6_K.

Dequantisation follows the reference bit for bit (backend/internal/gen/quant.go:41-131,
backend/cpu/quant.go); Q4_0 (32 values, fp16 scale, 16 bytes of nibbles: low
nibbles are values 0..15, high nibbles values 16..31, each minus 8) is the
format the reference's file layer knows but never computes in.  The torch code
here is the oracle and the CPU path; ``csrc/quant_sm100.cu`` holds the CUDA
kernels (dequantise, quantise activations to Q8_0, int8 dot-product GEMV).
"""
from __future__ import annotations

import torch

Q8_0, Q4_0, Q4_K, Q6_K = 64, 65, 66, 67
BLOCK = {Q8_0: (32, 34), Q4_0: (32, 18), Q4_K: (256, 144), Q6_K: (256, 210)}


def _f16(raw: torch.Tensor) -> torch.Tensor:
    """Little-endian fp16 from a [..., 2] uint8 tensor."""
    return raw.contiguous().view(torch.float16).squeeze(-1).float()


def dequantize_raw(code: int, raw: torch.Tensor, numel: int) -> torch.Tensor:
    """fp32 values of ``numel`` elements stored as blocks in the uint8 tensor ``raw``."""
    vals, nbytes = BLOCK[code]
    b = raw.reshape(-1, nbytes)
    if code == Q8_0:
        d = _f16(b[:, :2])
        q = b[:, 2:].view(torch.int8).float()
        out = q * d[:, None]
    elif code == Q4_0:
        d = _f16(b[:, :2])
        qs = b[:, 2:]
        lo = (qs & 0xF).float() - 8
        hi = (qs >> 4).float() - 8
        out = torch.cat([lo, hi], 1) * d[:, None]
    elif code == Q4_K:
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc_raw = b[:, 4:16].int()
        qs = b[:, 16:144]
        sc = torch.empty(b.shape[0], 8, dtype=torch.int32, device=b.device)
        mn = torch.empty_like(sc)
        for j in range(8):
            if j < 4:
                sc[:, j] = sc_raw[:, j] & 63
                mn[:, j] = sc_raw[:, j + 4] & 63
            else:
                sc[:, j] = (sc_raw[:, j + 4] & 0xF) | ((sc_raw[:, j - 4] >> 6) << 4)
                mn[:, j] = (sc_raw[:, j + 4] >> 4) | ((sc_raw[:, j] >> 6) << 4)
        parts = []
        for pair in range(4):
            q = qs[:, 32 * pair: 32 * pair + 32]
            d1 = (d * sc[:, 2 * pair].float())[:, None]
            m1 = (dmin * mn[:, 2 * pair].float())[:, None]
            d2 = (d * sc[:, 2 * pair + 1].float())[:, None]
            m2 = (dmin * mn[:, 2 * pair + 1].float())[:, None]
            parts += [d1 * (q & 0xF).float() - m1, d2 * (q >> 4).float() - m2]
        out = torch.cat(parts, 1)
    elif code == Q6_K:
        ql, qh = b[:, :128].int(), b[:, 128:192].int()
        sc = b[:, 192:208].view(torch.int8).float()
        d = _f16(b[:, 208:210])
        halves = []
        for h in range(2):
            l_, h_ = ql[:, 64 * h: 64 * h + 64], qh[:, 32 * h: 32 * h + 32]
            s = sc[:, 8 * h: 8 * h + 8]
            q1 = ((l_[:, :32] & 0xF) | (((h_ >> 0) & 3) << 4)) - 32
            q2 = ((l_[:, 32:] & 0xF) | (((h_ >> 2) & 3) << 4)) - 32
            q3 = ((l_[:, :32] >> 4) | (((h_ >> 4) & 3) << 4)) - 32
            q4 = ((l_[:, 32:] >> 4) | (((h_ >> 6) & 3) << 4)) - 32
            idx = torch.arange(32, device=b.device) // 16
            halves += [q1.float() * s[:, idx + 0], q2.float() * s[:, idx + 2], q3.float() * s[:, idx + 4],
                       q4.float() * s[:, idx + 6]]
        out = torch.cat(halves, 1) * d[:, None]
    else:
        raise ValueError(f"unknown quantized dtype code {code}")
    return out.reshape(-1)[:numel]


def dequantize(qt, dtype=torch.float32) -> torch.Tensor:
    """``QuantizedTensor`` -> dense tensor of its logical shape."""
    n = 1
    for s in qt.shape:
        n *= s
    if qt.raw.is_cuda and qt.code in (Q8_0, Q4_0, Q4_K, Q6_K):
        from . import quant_cuda
        return quant_cuda.dequantize(qt.code, qt.raw, n).view(qt.shape).to(dtype)
    return dequantize_raw(qt.code, qt.raw, n).view(qt.shape).to(dtype)


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    """Rows of ``x`` (last dim a multiple of 32) -> uint8 blocks [..., K/32 * 34] (ggml reference rounding)."""
    xb = x.float().reshape(-1, 32)
    amax = xb.abs().amax(1)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(xb * inv[:, None]).clamp(-127, 127).to(torch.int8)
    out = torch.empty(xb.shape[0], 34, dtype=torch.uint8, device=x.device)
    out[:, :2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(torch.uint8)
    return out.reshape(*x.shape[:-1], x.shape[-1] // 32 * 34)


def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    """ggml reference Q4_0: d = (value of largest magnitude) / -8, q = min(15, floor(x/d + 8.5))."""
    xb = x.float().reshape(-1, 32)
    idx = xb.abs().argmax(1, keepdim=True)
    mx = xb.gather(1, idx).squeeze(1)
    d = mx / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (xb * inv[:, None] + 8.5).floor().clamp(0, 15).to(torch.uint8)
    out = torch.empty(xb.shape[0], 18, dtype=torch.uint8, device=x.device)
    out[:, :2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(*x.shape[:-1], x.shape[-1] // 32 * 18)


def qmatmul_t(x: torch.Tensor, w) -> torch.Tensor:
    """``x @ dequant(w)^T`` for a ``QuantizedTensor`` weight [N, K] (OpQMatMul, tensor/quant.go:35)."""
    if x.is_cuda and w.code in (Q8_0, Q4_0, Q4_K, Q6_K) and len(w.shape) == 2:
        from . import quant_cuda
        raw = w.raw if w.raw.is_cuda and w.raw.device == x.device else w.raw.to(x.device)
        rows = x.reshape(-1, x.shape[-1])
        if rows.shape[0] <= _QGEMV_MAX_ROWS:
            # few rows (decode): the weight is read once in its block encoding
            y = quant_cuda.qgemv_ggml(w.code, raw, w.shape[0], w.shape[1], rows)
            return y.reshape(*x.shape[:-1], w.shape[0]).to(x.dtype)
        n = w.shape[0] * w.shape[1]
        wd = quant_cuda.dequantize(w.code, raw, n).view(w.shape)       # many rows (prefill): dequantise on the GPU
        return (x.float() @ wd.t()).to(x.dtype)
    if x.device.type == "cpu" and w.raw.device.type == "cpu" and w.code in (Q8_0, Q4_0, Q4_K, Q6_K) and len(w.shape) == 2 \
            and not torch.is_grad_enabled() and x.numel() // max(x.shape[-1], 1) <= _QGEMV_MAX_ROWS \
            and w.shape[1] % BLOCK[w.code][0] == 0:
        # few rows on the host (decode): the native kernel reads the weight once in its block
        # encoding; CPU_MODE picks float activations ("exact") or int8 blocks with VNNI ("int8" / "auto")
        from . import quant_cpu
        raw = w.raw if w.raw.is_contiguous() else w.raw.contiguous()
        y = quant_cpu.qgemv(w.code, raw.reshape(-1), w.shape[0], w.shape[1], x, CPU_MODE)
        return y.reshape(*x.shape[:-1], w.shape[0]).to(x.dtype)
    wd = dequantize(w, torch.float32).to(x.device)
    return (x.float() @ wd.t()).to(x.dtype)


_QGEMV_MAX_ROWS = 16
CPU_MODE = "exact"      # the lazy layer's product keeps the meaning x @ dequant(W)^T; decoders ask for "auto"
