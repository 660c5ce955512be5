"""Thin wrappers over the row / elementwise kernels (``csrc/rowops.cu``,
``csrc/elementwise.cu``).  Every function launches on the current torch
stream and raises if the native launcher refuses the arguments.
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, stream_ptr

ACT_MODES = {"gelu": 0, "silu": 1, "relu": 2}


def _L():
    return _native.lib()


def norm_bwd_scratch(C: int, device) -> torch.Tensor:
    return torch.empty(_L().mimir_norm_bwd_blocks() * 2 * C, dtype=torch.float32, device=device)


def layernorm_fwd(x, gamma, beta, out, mean, rstd, eps=1e-5):
    rows, C = x.numel() // x.shape[-1], x.shape[-1]
    _native.check(_L().mimir_layernorm_fwd(ptr(x), ptr(gamma), ptr(beta), ptr(out), ptr(mean),
                                           ptr(rstd), rows, C, eps, stream_ptr()), "layernorm_fwd")
    return out


def layernorm_bwd(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, accumulate=False):
    rows, C = x.numel() // x.shape[-1], x.shape[-1]
    _native.check(_L().mimir_layernorm_bwd(ptr(dy), ptr(x), ptr(gamma), ptr(mean), ptr(rstd),
                                           ptr(dres), ptr(dx), ptr(dgamma), ptr(dbeta),
                                           ptr(scratch), rows, C, int(accumulate), stream_ptr()),
                  "layernorm_bwd")
    return dx


def rmsnorm_fwd(x, gamma, out, rstd, eps=1e-5):
    rows, C = x.numel() // x.shape[-1], x.shape[-1]
    _native.check(_L().mimir_rmsnorm_fwd(ptr(x), ptr(gamma), ptr(out), ptr(rstd), rows, C, eps,
                                         stream_ptr()), "rmsnorm_fwd")
    return out


def rmsnorm_bwd(dy, x, gamma, rstd, dres, dx, dgamma, scratch, accumulate=False):
    rows, C = x.numel() // x.shape[-1], x.shape[-1]
    _native.check(_L().mimir_rmsnorm_bwd(ptr(dy), ptr(x), ptr(gamma), ptr(rstd), ptr(dres), ptr(dx),
                                         ptr(dgamma), ptr(scratch), rows, C, int(accumulate),
                                         stream_ptr()), "rmsnorm_bwd")
    return dx


def colsum(x, out, scratch, accumulate=False):
    rows, N = x.shape
    _native.check(_L().mimir_colsum(ptr(x), rows, N, x.stride(0), ptr(out), ptr(scratch),
                                    int(accumulate), stream_ptr()), "colsum")
    return out


def cross_entropy(logits, target, loss_rows, dlogits, mean_loss, V, gscale, loss_scale):
    rows = logits.shape[0]
    _native.check(_L().mimir_cross_entropy(ptr(logits), ptr(target), ptr(loss_rows), ptr(dlogits),
                                           ptr(mean_loss), rows, V, logits.stride(0), gscale,
                                           loss_scale, stream_ptr()), "cross_entropy")


def softmax_rows(x, out, log=False):
    rows, C = x.numel() // x.shape[-1], x.shape[-1]
    _native.check(_L().mimir_softmax_rows(ptr(x), ptr(out), rows, C, int(log), stream_ptr()),
                  "softmax")
    return out


def embedding_fwd(tok, wte, wpe, out, T):
    rows = tok.numel()
    V, C = wte.shape
    _native.check(_L().mimir_embedding_fwd(ptr(tok), ptr(wte), ptr(wpe), ptr(out), rows, T, C, V,
                                           stream_ptr()), "embedding_fwd")
    return out


def embedding_bwd(tok, dx, dwte, dwpe, B, T, accumulate_wpe=False):
    V, C = dwte.shape
    _native.check(_L().mimir_embedding_bwd(ptr(tok), ptr(dx), ptr(dwte), ptr(dwpe), B, T, C, V,
                                           int(accumulate_wpe), stream_ptr()), "embedding_bwd")


def act_fwd(x, out, mode="gelu"):
    _native.check(_L().mimir_act_fwd(ptr(x), ptr(out), x.numel(), ACT_MODES[mode], stream_ptr()),
                  "act_fwd")
    return out


def act_bwd(x, dy, dx, mode="gelu"):
    _native.check(_L().mimir_act_bwd(ptr(x), ptr(dy), ptr(dx), x.numel(), ACT_MODES[mode],
                                     stream_ptr()), "act_bwd")
    return dx


def swiglu_fwd(gu, out):
    rows, F2 = gu.shape
    _native.check(_L().mimir_swiglu_fwd(ptr(gu), ptr(out), rows, F2 // 2, stream_ptr()), "swiglu_fwd")
    return out


def swiglu_bwd(gu, dy, dgu):
    rows, F2 = gu.shape
    _native.check(_L().mimir_swiglu_bwd(ptr(gu), ptr(dy), ptr(dgu), rows, F2 // 2, stream_ptr()),
                  "swiglu_bwd")
    return dgu


def swiglu2_fwd(gate, up, out):
    """``silu(gate) * up`` with gate and up in separate contiguous buffers."""
    _native.check(_L().mimir_swiglu2_fwd(ptr(gate), ptr(up), ptr(out), gate.numel(), stream_ptr()), "swiglu2_fwd")
    return out


def swiglu2_bwd(gate, up, dy, dgate, dup):
    _native.check(_L().mimir_swiglu2_bwd(ptr(gate), ptr(up), ptr(dy), ptr(dgate), ptr(dup), gate.numel(),
                                         stream_ptr()), "swiglu2_bwd")


def rope_(x2d, pos, freqs, col0, nheads, D, interleaved, inverse=False):
    rows = x2d.shape[0]
    _native.check(_L().mimir_rope(ptr(x2d), ptr(pos), ptr(freqs), rows, x2d.stride(0), col0, nheads,
                                  D, int(interleaved), int(inverse), stream_ptr()), "rope")
    return x2d


def cast_f32_bf16(x, out, scale=1.0):
    _native.check(_L().mimir_cast_f32_bf16(ptr(x), ptr(out), x.numel(), scale, stream_ptr()), "cast")
    return out


def cast_bf16_f32(x, out, scale=1.0):
    _native.check(_L().mimir_cast_bf16_f32(ptr(x), ptr(out), x.numel(), scale, stream_ptr()), "cast")
    return out


def axpby(a, b, out, alpha=1.0, beta=1.0):
    _native.check(_L().mimir_axpby(ptr(a), ptr(b), ptr(out), a.numel(), alpha, beta, stream_ptr()),
                  "axpby")
    return out


def sumsq(g, out):
    _native.check(_L().mimir_sumsq(ptr(g), g.numel(), int(g.dtype == torch.float32), ptr(out),
                                   stream_ptr()), "sumsq")
    return out


def adamw_flat(master, param, grad, m, v, *, decay_n=None, lr, beta1=0.9, beta2=0.999, eps=1e-8,
               wd=0.01, step=1, gscale=1.0, gnorm_sq=None, clip=0.0, hyper=None):
    n = master.numel()
    if decay_n is None:
        decay_n = n
    _native.check(_L().mimir_adamw_flat(ptr(master), ptr(param), ptr(grad),
                                        int(grad.dtype == torch.float32), ptr(m), ptr(v), n, decay_n,
                                        lr, beta1, beta2, eps, wd, step, gscale, ptr(gnorm_sq), clip,
                                        ptr(hyper), stream_ptr()), "adamw")


def philox_uniform(n: int, seed: int, device="cuda") -> torch.Tensor:
    """``n`` uniforms in [0, 1) of the Philox stream ``seed``; bit-identical to ``tensor.random.philox_uniform``."""
    out = torch.empty(n, dtype=torch.float32, device=device)
    _native.check(_L().mimir_philox_uniform(ptr(out), n, seed & 0xFFFFFFFFFFFFFFFF, stream_ptr()), "philox_uniform")
    return out


def dropout(x, p: float, seed: int, out=None):
    """Inverted dropout of a bf16 tensor with the Philox mask of ``seed`` (same seed = same mask)."""
    out = torch.empty_like(x) if out is None else out
    _native.check(_L().mimir_philox_dropout(ptr(x), ptr(out), x.numel(), seed & 0xFFFFFFFFFFFFFFFF, p, stream_ptr()),
                  "dropout")
    return out
