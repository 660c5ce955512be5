"""Convolution and pooling on the native sm_100a kernels (``csrc/conv_sm100.cu``).

Activations are bf16 NHWC with the channel count padded to a multiple of 64
(``to_nhwc`` / ``from_nhwc`` convert at the edges of a network); filters are
packed once per step into ``[Co, KH*KW*Cp]`` rows ordered (kh, kw, ci).
Stride-1 convolutions (any padding, dilation) run as implicit GEMMs; other
strides gather the windows explicitly and call the GEMM kernel.
Reference semantics: OpConv / OpConvInput / OpConvWeight and OpMaxPool
(backend/op.go:140-151, :227-233).
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, stream_ptr

_declared = False


def _L():
    global _declared
    lib = _native.lib()
    if not _declared:
        import ctypes as C
        P, I, L = C.c_void_p, C.c_int, C.c_longlong
        for name, args in {
            "mimir_conv2d_fwd": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P],
            "mimir_conv2d_wgrad": [P, P, P, P, L, I, I, I, I, I, I, I, I, I, I, I, I, I, P],
            "mimir_maxpool2d_fwd": [P, P, P, I, I, I, I, I, I, P],
            "mimir_maxpool2d_bwd": [P, P, P, I, I, I, I, I, I, P],
            "mimir_relu_bwd": [P, P, P, L, P],
        }.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, C.c_int
        _declared = True
    return lib


def pad64(c: int) -> int:
    return (c + 63) // 64 * 64


def to_nhwc(x: torch.Tensor) -> torch.Tensor:
    """[N, C, H, W] (any float dtype) -> bf16 [N, H, W, pad64(C)] with zero padding channels."""
    N, C, H, W = x.shape
    out = torch.zeros(N, H, W, pad64(C), dtype=torch.bfloat16, device=x.device)
    out[..., :C] = x.permute(0, 2, 3, 1)
    return out


def from_nhwc(x: torch.Tensor, C: int) -> torch.Tensor:
    return x[..., :C].permute(0, 3, 1, 2).contiguous()


def pack_filter(w: torch.Tensor) -> torch.Tensor:
    """[Co, Ci, KH, KW] -> bf16 [Co, KH*KW*pad64(Ci)] ordered (kh, kw, ci)."""
    Co, Ci, KH, KW = w.shape
    out = torch.zeros(Co, KH, KW, pad64(Ci), dtype=torch.bfloat16, device=w.device)
    out[..., :Ci] = w.permute(0, 2, 3, 1)
    return out.view(Co, -1)


def pack_filter_dgrad(w: torch.Tensor) -> torch.Tensor:
    """Filter of the input-gradient convolution: [Ci, KH*KW*pad64(Co)], taps flipped."""
    return pack_filter(w.flip(2, 3).transpose(0, 1).contiguous())


def unpack_filter_grad(dw: torch.Tensor, shape) -> torch.Tensor:
    """fp32 [Co, KH*KW*Cp] -> [Co, Ci, KH, KW]."""
    Co, Ci, KH, KW = shape
    return dw.view(Co, KH, KW, -1)[..., :Ci].permute(0, 3, 1, 2).contiguous()


def conv2d_fwd(x, w_packed, KH, KW, padding=0, dilation=1, bias=None, relu=False, out=None):
    """x bf16 [N,H,W,Cp]; w_packed [Co, KH*KW*Cp]; bias fp32 [pad64(Co)] or None -> [N,Ho,Wo,pad64(Co)]."""
    N, H, W, Cp = x.shape
    Co = w_packed.shape[0]
    Cop = pad64(Co)
    ph, pw = (padding, padding) if isinstance(padding, int) else padding
    Ho, Wo = H + 2 * ph - dilation * (KH - 1), W + 2 * pw - dilation * (KW - 1)
    if out is None:
        out = torch.empty(N, Ho, Wo, Cop, dtype=torch.bfloat16, device=x.device)
    _native.check(_L().mimir_conv2d_fwd(ptr(x), ptr(w_packed), ptr(bias), ptr(out), N, H, W, Cp, Cop, Co, KH, KW,
                                        ph, pw, dilation, int(relu), stream_ptr()), "conv2d_fwd")
    return out


def conv2d_dgrad(dy, w_dgrad_packed, KH, KW, padding=0, dilation=1, out=None):
    """dy bf16 [N,Ho,Wo,Cop] -> dx [N,H,W,pad64(Ci)] for a stride-1 convolution."""
    ph, pw = (padding, padding) if isinstance(padding, int) else padding
    return conv2d_fwd(dy, w_dgrad_packed, KH, KW, (dilation * (KH - 1) - ph, dilation * (KW - 1) - pw), dilation, out=out)


_scratch: dict = {}


def conv2d_wgrad(dy, x, Co, KH, KW, padding=0, dilation=1, out=None, accumulate=False, splits=0):
    """fp32 [Co, KH*KW*Cp] filter gradient of a stride-1 convolution."""
    N, H, W, Cp = x.shape
    Cop = dy.shape[-1]
    ph, pw = (padding, padding) if isinstance(padding, int) else padding
    n = Co * KH * KW * Cp
    if out is None:
        out = torch.empty(Co, KH * KW * Cp, dtype=torch.float32, device=x.device)
    key = (x.device, torch.cuda.current_stream().cuda_stream)
    part = _scratch.get(key)
    need = n * 64
    if part is None or part.numel() < min(need, 64 << 20):
        part = _scratch[key] = torch.empty(max(min(need, 64 << 20), n), dtype=torch.float32, device=x.device)
    _native.check(_L().mimir_conv2d_wgrad(ptr(dy), ptr(x), ptr(out), ptr(part), part.numel(), N, H, W, Cp, Cop, Co, KH,
                                          KW, ph, pw, dilation, splits, int(accumulate), stream_ptr()), "conv2d_wgrad")
    return out


def maxpool2d_fwd(x, k, s=None):
    s = s or k
    N, H, W, C = x.shape
    Ho, Wo = (H - k) // s + 1, (W - k) // s + 1
    y = torch.empty(N, Ho, Wo, C, dtype=torch.bfloat16, device=x.device)
    arg = torch.empty(N, Ho, Wo, C, dtype=torch.uint8, device=x.device)
    _native.check(_L().mimir_maxpool2d_fwd(ptr(x), ptr(y), ptr(arg), N, H, W, C, k, s, stream_ptr()), "maxpool_fwd")
    return y, arg


def maxpool2d_bwd(dy, arg, in_shape, k, s=None):
    s = s or k
    N, H, W, C = in_shape
    dx = torch.empty(N, H, W, C, dtype=torch.bfloat16, device=dy.device)
    _native.check(_L().mimir_maxpool2d_bwd(ptr(dy), ptr(arg), ptr(dx), N, H, W, C, k, s, stream_ptr()), "maxpool_bwd")
    return dx


def relu_bwd(y, dy, out=None):
    out = torch.empty_like(dy) if out is None else out
    _native.check(_L().mimir_relu_bwd(ptr(y), ptr(dy), ptr(out), y.numel(), stream_ptr()), "relu_bwd")
    return out
