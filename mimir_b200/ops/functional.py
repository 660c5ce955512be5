"""Differentiable forms of the native sm_100a kernels.

Each class is a ``torch.autograd.Function`` whose forward and backward both run the
hand-written kernels (tcgen05 GEMM in its three operand layouts, fused attention,
row kernels, embedding, SwiGLU, implicit-GEMM convolution), so that the lazy tensor
layer and the ``nn`` modules train through them: the reference gets the same effect from
its vector-Jacobian rules over fused schedule nodes (tensor/autograd.go:585,
internal/sched/fuse.go:293-325).  All of them take bf16 CUDA tensors; the callers in
``tensor/core.py`` decide when an operation qualifies and fall back to PyTorch otherwise.

Shapes: the product functions take 2-D operands (callers flatten leading axes);
attention takes ``[B, H, T, D]`` tensors in any layout whose head axis is contiguous
inside a token (what ``split -> reshape -> permute`` of a fused QKV product gives).
"""
from __future__ import annotations

import math

import torch

from . import kernels as K
from .gemm import gemm

_BF = torch.bfloat16


def _scratch(key: str, numel: int, device, dtype=torch.float32) -> torch.Tensor:
    """Per-(device, stream) scratch that grows and is reused: the kernels that take it run on
    the launching stream in program order, so one buffer per stream is enough."""
    k = (key, device.index, torch.cuda.current_stream(device).cuda_stream, dtype)
    buf = _SCRATCH.get(k)
    if buf is None or buf.numel() < numel:
        if buf is not None:
            _RETIRED.append(buf)      # a captured CUDA graph may still point at it: never freed
        buf = _SCRATCH[k] = torch.empty(numel, dtype=dtype, device=device)
    return buf


_SCRATCH: dict = {}
_RETIRED: list = []


def _rows(t: torch.Tensor) -> torch.Tensor:
    """The tensor as contiguous 2-D [rows, last]."""
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.is_contiguous() else t2.contiguous()


def _colsum_bf16(dy: torch.Tensor) -> torch.Tensor:
    out = torch.empty(dy.shape[1], dtype=_BF, device=dy.device)
    K.colsum(dy, out, _scratch("colsum", 64 * dy.shape[1], dy.device))
    return out


# --------------------------------------------------------------------------- products
class LinearFn(torch.autograd.Function):
    """``y = act(x @ w^T + bias) (+ residual)``: one GEMM with the epilogue fused.

    ``act`` is 0 (none) or 1 (GELU-tanh; the pre-activation is kept for backward).
    Backward: input gradient = NN product (with GELU' folded into the epilogue of the
    product above it), weight gradient = TN product, bias gradient = column sums."""

    @staticmethod
    def forward(ctx, x, w, bias, residual, act):
        pre = None
        if act == 1:
            pre = torch.empty(x.shape[0], w.shape[0], dtype=_BF, device=x.device)
            y = gemm(x, w, bias=bias, gelu=True, aux_out=pre)
        elif residual is not None:
            y = gemm(x, w, bias=bias, residual=True, aux=residual)
        else:
            y = gemm(x, w, bias=bias)
        ctx.save_for_backward(x, w, pre)
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, pre = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        if pre is not None:
            # d(pre) = dy * gelu'(pre): one pass of the activation-gradient kernel
            dpre = torch.empty_like(dy)
            K.act_bwd(pre, dy, dpre, "gelu")
            dy = dpre
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = gemm(dy, x, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        db = _colsum_bf16(dy) if ctx.has_bias and ctx.needs_input_grad[2] else None
        dres = dy if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, None


class MatmulFn(torch.autograd.Function):
    """``a[M,K] @ b[K,N]`` with ``b`` stored row-major (an MN-major B operand)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm(a, b, b_mn=True)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        da = gemm(dy, b) if ctx.needs_input_grad[0] else None                    # dy @ b^T: b rows are [K, N]
        db = gemm(a, dy, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None  # a^T @ dy
        return da, db


def linear_supported(x2d_rows: int, K_: int, N: int) -> bool:
    return K_ % 8 == 0 and N % 8 == 0 and x2d_rows > 0


def linear(x, w, bias=None, residual=None, act: int = 0):
    """``act(x @ w^T + bias) + residual`` over any leading axes of ``x``."""
    lead = x.shape[:-1]
    x2 = _rows(x)
    r2 = _rows(residual) if residual is not None else None
    y = LinearFn.apply(x2, w if w.is_contiguous() else w.contiguous(), bias, r2, act)
    return y.view(*lead, w.shape[0])


# --------------------------------------------------------------------------- attention
def _as_bthd(t: torch.Tensor) -> torch.Tensor:
    """``[B, H, T, D]`` -> ``[B, T, H, D]`` view the kernel can read: unit stride over D, heads
    D apart, batches T tokens apart; copied only when the layout is something else."""
    v = t.transpose(1, 2)
    B, T, H, D = v.shape
    if v.stride(3) == 1 and v.stride(2) == D and v.stride(0) == T * v.stride(1) and v.stride(1) % 8 == 0 \
            and v.data_ptr() % 16 == 0:
        return v
    return v.contiguous()


class AttentionFn(torch.autograd.Function):
    """Fused attention over ``[B, H, T, D]`` (grouped-query when k / v have fewer heads), causal with
    offset or unmasked; the forward keeps the log-sum-exp rows, the backward recomputes the
    probabilities from them in two kernels without atomics."""

    @staticmethod
    def forward(ctx, q, k, v, causal, offset, scale):
        from .attention import attention_fwd
        qb, kb, vb = _as_bthd(q), _as_bthd(k), _as_bthd(v)
        B, Tq, Hq, D = qb.shape
        out = torch.empty(B, Tq, Hq, D, dtype=_BF, device=q.device)
        lse = torch.empty(B * Hq * Tq, dtype=torch.float32, device=q.device)
        attention_fwd(qb, kb, vb, out, lse, causal=causal, offset=offset, scale=scale)
        ctx.save_for_backward(qb, kb, vb, out, lse)
        ctx.cfg = (causal, offset, scale)
        return out.transpose(1, 2)

    @staticmethod
    def backward(ctx, dout):
        from .attention import attention_bwd
        qb, kb, vb, out, lse = ctx.saved_tensors
        causal, offset, scale = ctx.cfg
        B, Tq, Hq, D = qb.shape
        Tk, Hk = kb.shape[1], kb.shape[2]
        do = dout.transpose(1, 2)
        do = do if do.is_contiguous() else do.contiguous()
        # one packed gradient buffer [B, T, (Hq + 2 Hk) D] when the lengths agree: the split that
        # produced q, k, v differentiates into a concatenation that finds the pieces adjacent
        if Tq == Tk:
            pack = torch.empty(B, Tq, (Hq + 2 * Hk) * D, dtype=_BF, device=do.device)
            dq = pack[:, :, : Hq * D].unflatten(2, (Hq, D))
            dk = pack[:, :, Hq * D: (Hq + Hk) * D].unflatten(2, (Hk, D))
            dv = pack[:, :, (Hq + Hk) * D:].unflatten(2, (Hk, D))
        else:
            dq = torch.empty(B, Tq, Hq, D, dtype=_BF, device=do.device)
            dk = torch.empty(B, Tk, Hk, D, dtype=_BF, device=do.device)
            dv = torch.empty(B, Tk, Hk, D, dtype=_BF, device=do.device)
        dsum = _scratch("attn_dsum", B * Hq * Tq, do.device)
        attention_bwd(qb, kb, vb, out, do, lse, dsum, dq, dk, dv, causal=causal, offset=offset, scale=scale)
        return dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2), None, None, None


def attention(q, k, v, causal=False, offset=None, scale=None):
    D = q.shape[-1]
    if offset is None:
        offset = k.shape[2] - q.shape[2]
    return AttentionFn.apply(q, k, v, bool(causal), int(offset), float(scale if scale is not None else 1.0 / math.sqrt(D)))


def attention_supported(q, k, v) -> bool:
    return q.shape[-1] in (64, 128) and q.shape[1] % k.shape[1] == 0 and k.shape == v.shape


# --------------------------------------------------------------------------- row kernels
class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        rows = x.shape[0]
        out = torch.empty_like(x)
        stats = torch.empty(2, rows, dtype=torch.float32, device=x.device)
        K.layernorm_fwd(x, gamma, beta, out, stats[0], stats[1], eps)
        ctx.save_for_backward(x, gamma, stats)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, gamma, stats = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        C = x.shape[1]
        dx = torch.empty_like(x)
        dg = torch.empty(C, dtype=_BF, device=x.device)
        db = torch.empty(C, dtype=_BF, device=x.device)
        K.layernorm_bwd(dy, x, gamma, stats[0], stats[1], None, dx, dg, db,
                        _scratch("norm_bwd", K._L().mimir_norm_bwd_blocks() * 2 * C, x.device))
        return dx, dg, db, None


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, eps):
        out = torch.empty_like(x)
        rstd = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
        K.rmsnorm_fwd(x, gamma, out, rstd, eps)
        ctx.save_for_backward(x, gamma, rstd)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, gamma, rstd = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        C = x.shape[1]
        dx = torch.empty_like(x)
        dg = torch.empty(C, dtype=_BF, device=x.device)
        K.rmsnorm_bwd(dy, x, gamma, rstd, None, dx, dg,
                      _scratch("norm_bwd", K._L().mimir_norm_bwd_blocks() * 2 * C, x.device))
        return dx, dg, None


def norm_supported(C: int) -> bool:
    return C % 8 == 0 and C <= 8192


def layer_norm(x, gamma, beta, eps):
    return LayerNormFn.apply(_rows(x), gamma, beta, float(eps)).view(x.shape)


def rms_norm(x, gamma, eps):
    return RMSNormFn.apply(_rows(x), gamma, float(eps)).view(x.shape)


class CrossEntropyFn(torch.autograd.Function):
    """Mean cross-entropy of bf16 logits ``[rows, V]`` against integer targets in one pass that also
    leaves d(loss)/d(logits); rows whose target is negative contribute nothing."""

    @staticmethod
    def forward(ctx, logits, target):
        rows, V = logits.shape
        dlogits = torch.empty_like(logits)
        loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
        loss = torch.empty(1, dtype=torch.float32, device=logits.device)
        K.cross_entropy(logits, target, loss_rows, dlogits, loss, V, 1.0 / rows, 1.0 / rows)
        ctx.save_for_backward(dlogits)
        return loss.view(())

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g.to(dlogits.dtype), None


def cross_entropy(logits, target):
    l2 = _rows(logits)
    t = target.reshape(-1)
    if t.dtype != torch.int64:
        t = t.long()
    return CrossEntropyFn.apply(l2, t.contiguous())


def cross_entropy_supported(logits) -> bool:
    return logits.shape[-1] % 8 == 0


class EmbeddingFn(torch.autograd.Function):
    """Row gather ``w[idx]``; the gradient scatters with bf16x2 atomics into a zeroed table."""

    @staticmethod
    def forward(ctx, w, idx):
        V, C = w.shape
        rows = idx.numel()
        out = torch.empty(rows, C, dtype=_BF, device=w.device)
        K.embedding_fwd(idx, w, None, out, max(rows, 1))
        ctx.save_for_backward(idx)
        ctx.shape = (V, C)
        return out

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        V, C = ctx.shape
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dw = torch.zeros(V, C, dtype=_BF, device=dy.device)
        K.embedding_bwd(idx, dy, dw, None, 1, idx.numel())
        return dw, None


def embedding(w, idx):
    i = idx.reshape(-1)
    if i.dtype != torch.int64:
        i = i.long()
    return EmbeddingFn.apply(w if w.is_contiguous() else w.contiguous(), i.contiguous()).view(*idx.shape, w.shape[1])


class SwiGLUFn(torch.autograd.Function):
    """``silu(gate) * up`` in one pass over two separate buffers; backward likewise."""

    @staticmethod
    def forward(ctx, gate, up):
        out = torch.empty_like(gate)
        K.swiglu2_fwd(gate, up, out)
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, dy):
        gate, up = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dg, du = torch.empty_like(gate), torch.empty_like(up)
        K.swiglu2_bwd(gate, up, dy, dg, du)
        return dg, du


def swiglu(gate, up):
    g = gate if gate.is_contiguous() else gate.contiguous()
    u = up if up.is_contiguous() else up.contiguous()
    return SwiGLUFn.apply(g, u)


class ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mode):
        out = torch.empty_like(x)
        K.act_fwd(x, out, mode)
        ctx.save_for_backward(x)
        ctx.mode = mode
        return out

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dx = torch.empty_like(x)
        K.act_bwd(x, dy, dx, ctx.mode)
        return dx, None


def activation(x, mode: str):
    xc = x if x.is_contiguous() else x.contiguous()
    return ActFn.apply(xc, mode)


# --------------------------------------------------------------------------- convolution
class Conv2dFn(torch.autograd.Function):
    """Stride-1 ``conv2d`` of an NCHW bf16 tensor on the implicit-GEMM kernels.  The kernels work
    on NHWC with channels padded to 64; the conversion happens at the edges of this function,
    and the output is returned as an NCHW *view* of the NHWC result (channels-last memory)."""

    @staticmethod
    def forward(ctx, x, w, bias, padding, dilation):
        from . import conv as CV
        Co, Ci, KH, KW = w.shape
        xn = CV.to_nhwc(x)
        wp = CV.pack_filter(w)
        b32 = None
        if bias is not None:
            b32 = torch.zeros(CV.pad64(Co), dtype=torch.float32, device=x.device)
            b32[:Co] = bias.float()
        y = CV.conv2d_fwd(xn, wp, KH, KW, padding, dilation, bias=b32)
        ctx.save_for_backward(xn, w)
        ctx.cfg = (padding, dilation, Ci, bias is not None)
        return y[..., :Co].permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        from . import conv as CV
        xn, w = ctx.saved_tensors
        padding, dilation, Ci, has_bias = ctx.cfg
        Co, _, KH, KW = w.shape
        dyn = CV.to_nhwc(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dxn = CV.conv2d_dgrad(dyn, CV.pack_filter_dgrad(w), KH, KW, padding, dilation)
            dx = dxn[..., :Ci].permute(0, 3, 1, 2)
        if ctx.needs_input_grad[1]:
            dwp = CV.conv2d_wgrad(dyn, xn, Co, KH, KW, padding, dilation)
            dw = CV.unpack_filter_grad(dwp, w.shape).to(_BF)
        if has_bias and ctx.needs_input_grad[2]:
            db = _colsum_bf16(dyn.view(-1, dyn.shape[-1]))[:Co]
        return dx, dw, db, None, None


def conv2d_supported(x, w, stride, padding, dilation, groups) -> bool:
    one = lambda v: v == 1 or v == (1, 1)  # noqa: E731
    return one(stride) and groups == 1 and isinstance(dilation, int) and x.dim() == 4 \
        and (isinstance(padding, int) or (isinstance(padding, tuple) and len(padding) == 2))


def conv2d(x, w, bias, padding, dilation):
    return Conv2dFn.apply(x, w, bias, padding, dilation)


class MaxPool2dFn(torch.autograd.Function):
    """Max pooling without padding on channels-last bf16 data (the layout ``Conv2dFn`` returns)."""

    @staticmethod
    def forward(ctx, x, k, s):
        from . import conv as CV
        xn = x.permute(0, 2, 3, 1)
        xn = xn if xn.is_contiguous() else xn.contiguous()
        y, arg = CV.maxpool2d_fwd(xn, k, s)
        ctx.save_for_backward(arg)
        ctx.cfg = (tuple(xn.shape), k, s)
        return y.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        from . import conv as CV
        (arg,) = ctx.saved_tensors
        shape, k, s = ctx.cfg
        dyn = dy.permute(0, 2, 3, 1)
        dyn = dyn if dyn.is_contiguous() else dyn.contiguous()
        return CV.maxpool2d_bwd(dyn, arg, shape, k, s).permute(0, 3, 1, 2), None, None


def max_pool2d_supported(x, kernel, stride, padding) -> bool:
    return x.dim() == 4 and isinstance(kernel, int) and padding in (0, (0, 0)) and (stride is None or isinstance(stride, int)) \
        and x.shape[1] % 8 == 0


def max_pool2d(x, kernel, stride):
    return MaxPool2dFn.apply(x, kernel, stride or kernel)
