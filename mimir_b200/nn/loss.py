"""Losses over lazy tensors (reference: nn/loss/loss.go:35-96, more.go:66-296).

Every loss is a composition of the tensor layer's own ops, so it is a piece of the lazy graph like
any other: the fusion planner, the partitioner's layout rules and the exporter see its parts.  Only
``cross_entropy`` is one node: on bf16 CUDA logits it is the fused native kernel (loss and
d(loss)/d(logits) in one pass over the logits).  Every loss returns the mean over the batch; class
targets are integer tensors.  Half-precision inputs are widened to float32 first; a shape mismatch
is a sticky ``ErrShape`` on the result, never an exception.
"""
from __future__ import annotations

import torch

from .. import tensor as T
from ..tensor import errors as E

F = torch.nn.functional
_core = T.core


def _f32(x):
    return x if x.dtype == T.float32 or x.dtype == torch.float64 else T.cast(x, T.float32)


def _pair(what, a, b):
    """Both operands as float tensors of one shape, or a sticky error."""
    for t in (a, b):
        if t._err is not None:
            return None, None, t
    if tuple(a.shape) != tuple(b.shape):
        return None, None, _core._error_tensor(E.ErrShape(f"loss: {what} of shapes {tuple(a.shape)} and {tuple(b.shape)}"))
    a = _f32(a)
    b = _f32(b) if b.dtype != a.dtype else b
    return a, b, None


def _classes(what, scores, target):
    """Checks ``scores [N, C, ...]`` against integer ``target [N, ...]``; returns a sticky error or None."""
    for t in (scores, target):
        if t._err is not None:
            return t
    s, g = tuple(scores.shape), tuple(target.shape)
    if len(s) < 2 or s[:1] + s[2:] != g:
        return _core._error_tensor(E.ErrShape(f"loss: {what} of scores {s} for targets {g}, want [N, C, ...] and [N, ...]"))
    if target.dtype.is_floating_point or target.dtype == torch.bool:
        return _core._error_tensor(E.ErrDType(f"loss: {what} wants integer class indices, got {target.dtype}"))
    return None


def _picked(values, target):
    """``values[n, target[n], ...]``: the entry of the target class."""
    return T.squeeze(T.gather(values, 1, T.unsqueeze(target, 1)), 1)


# ------------------------------------------------------------------ class scores
def cross_entropy(logits, target):
    """Mean softmax cross-entropy of logits ``[N, C]`` (or ``[N, C, d1, ...]``) against integer class
    targets.  2-D bf16 CUDA logits whose class count is a multiple of 8 run the fused native kernel (loss and d(loss)/d(logits) in one pass over the
    logits, no fp32 copy of them); rows with a negative target are ignored there."""
    def run(l, t):
        if l.dim() == 2 and _core._native_ok(l) and t.is_cuda and l.shape[-1] % 8 == 0 and l.numel():
            from ..ops import functional as NF
            return NF.cross_entropy(l, t)
        return F.cross_entropy(l.float(), t.long())
    # a scalar float32 result whenever the operands fit; a misfit goes through the inference and
    # comes back as a sticky error
    known = None
    if logits._err is None and target._err is None and len(logits.shape) >= 2 and logits.dtype.is_floating_point \
            and not target.dtype.is_floating_point and tuple(target.shape) == tuple(logits.shape[:1]) + tuple(logits.shape[2:]):
        known = ((), T.float32)
    return _core._node(run, (logits, target), {}, "cross_entropy", known=known)


def nll(logp, target):
    """Negative log-likelihood of the target classes under log-probabilities ``[N, C, ...]``."""
    err = _classes("negative log-likelihood", logp, target)
    if err is not None:
        return err
    return T.neg(T.mean(_picked(_f32(logp), target)))


def label_smoothing(eps):
    """Cross-entropy against targets smoothed by ``eps``: (1 - eps) on the class, eps / C everywhere."""
    def f(logits, target):
        err = _classes("label-smoothed cross-entropy", logits, target)
        if err is not None:
            return err
        logp = T.log_softmax(_f32(logits), 1)
        hard = T.neg(T.mean(_picked(logp, target)))
        soft = T.neg(T.mean(T.mean(logp, 1)))            # -(1/C) sum_c logp, averaged over the batch
        return hard * (1.0 - eps) + soft * eps
    return f


def focal(gamma):
    """Focal loss: cross-entropy weighted by (1 - p_target)^gamma."""
    def f(logits, target):
        err = _classes("focal loss", logits, target)
        if err is not None:
            return err
        logp = _picked(T.log_softmax(_f32(logits), 1), target)
        weight = T.pow_(1.0 - T.exp(logp), float(gamma))
        return T.neg(T.mean(weight * logp))
    return f


def hinge(scores, target):
    """Multi-class hinge (Crammer-Singer sum form): sum over the other classes of max(0, 1 + s_c - s_target)."""
    err = _classes("hinge loss", scores, target)
    if err is not None:
        return err
    s = _f32(scores)
    correct = T.gather(s, 1, T.unsqueeze(target, 1))
    margins = T.relu(s - correct + 1.0)                  # the target's own column contributes exactly 1
    return T.mean(T.sum_(margins, 1) - 1.0)


def dice(logits, target, eps=1.0):
    """1 - Dice coefficient of softmax probabilities ``[N, C, d...]`` against integer masks ``[N, d...]``,
    averaged over batch and classes."""
    err = _classes("dice loss", logits, target)
    if err is not None:
        return err
    p = T.softmax(_f32(logits), 1)
    nd = len(logits.shape)
    oh = T.one_hot(target, logits.shape[1])              # [N, d..., C]
    oh = T.permute(oh, (0, nd - 1) + tuple(range(1, nd - 1)))
    space = tuple(range(2, nd))
    inter, ps, ts = p * oh, p, oh
    for d in reversed(space):
        inter, ps, ts = T.sum_(inter, d), T.sum_(ps, d), T.sum_(ts, d)
    return T.mean(1.0 - (inter * 2.0 + eps) / (ps + ts + eps))


# ------------------------------------------------------------------ elementwise, averaged over everything
def bce_with_logits(logits, target):
    """Binary cross-entropy of sigmoid(logits), computed from the logits: max(x, 0) - x y + log(1 + e^-|x|)."""
    x, y, err = _pair("binary cross-entropy", logits, target)
    if err is not None:
        return err
    return T.mean(T.relu(x) - x * y + T.log1p(T.exp(T.neg(T.abs_(x)))))


def bce(pred, target):
    """Binary cross-entropy of probabilities; logarithms are clamped at -100 like PyTorch's."""
    p, y, err = _pair("binary cross-entropy", pred, target)
    if err is not None:
        return err
    lp = T.clamp(T.log(p), -100.0, None)
    lq = T.clamp(T.log(1.0 - p), -100.0, None)
    return T.neg(T.mean(y * lp + (1.0 - y) * lq))


def mse(pred, target):
    p, y, err = _pair("mean squared error", pred, target)
    if err is not None:
        return err
    d = p - y
    return T.mean(d * d)


def l1(pred, target):
    p, y, err = _pair("mean absolute error", pred, target)
    if err is not None:
        return err
    return T.mean(T.abs_(p - y))


def huber(pred, target, delta=1.0):
    """Squared error below ``delta``, linear above: 0.5 d^2 or delta (|d| - 0.5 delta)."""
    p, y, err = _pair("Huber loss", pred, target)
    if err is not None:
        return err
    a = T.abs_(p - y)
    small = T.minimum(a, float(delta))                   # 0.5 m^2 + delta (a - m) with m = min(a, delta)
    return T.mean(small * small * 0.5 + (a - small) * float(delta))


def smooth_l1(beta=1.0):
    """Huber divided by ``beta``: 0.5 d^2 / beta below beta, |d| - 0.5 beta above."""
    def f(pred, target):
        if beta == 0:
            return l1(pred, target)
        return huber(pred, target, beta) * (1.0 / beta)
    return f


def kl_div(logp, target):
    """KL(target || exp(logp)) summed over classes and averaged over the batch (``batchmean``); entries
    with zero target probability contribute nothing."""
    l, y, err = _pair("KL divergence", logp, target)
    if err is not None:
        return err
    pos = T.less(0.0 * y, y)
    term = T.where(pos, y * (T.log(T.where(pos, y, y * 0.0 + 1.0)) - l), y * 0.0)
    n = logp.shape[0] if len(logp.shape) else 1
    return T.sum_(term) * (1.0 / n)


def poisson_nll(log_rate, target):
    """Poisson negative log-likelihood of counts under exp(log_rate), without the Stirling term."""
    l, y, err = _pair("Poisson negative log-likelihood", log_rate, target)
    if err is not None:
        return err
    return T.mean(T.exp(l) - y * l)


def gaussian_nll(mean, variance, target):
    """0.5 (log max(var, 1e-6) + (mean - target)^2 / max(var, 1e-6)), averaged."""
    m, y, err = _pair("Gaussian negative log-likelihood", mean, target)
    if err is not None:
        return err
    if variance._err is not None:
        return variance
    v = T.clamp(_f32(variance), 1e-6, None)
    d = m - y
    return T.mean((T.log(v) + d * d / v) * 0.5)


def binary_focal(gamma, alpha):
    def f(logits, target):
        x, y, err = _pair("binary focal loss", logits, target)
        if err is not None:
            return err
        p = T.sigmoid(x)
        pt = p * y + (1.0 - p) * (1.0 - y)
        a = y * float(alpha) + (1.0 - y) * (1.0 - float(alpha))
        ce = T.relu(x) - x * y + T.log1p(T.exp(T.neg(T.abs_(x))))
        return T.mean(a * T.pow_(1.0 - pt, float(gamma)) * ce)
    return f


def binary_dice(logits, target, eps=1.0):
    x, y, err = _pair("binary dice loss", logits, target)
    if err is not None:
        return err
    n = logits.shape[0]
    p = T.reshape(T.sigmoid(x), (n, -1))
    y = T.reshape(y, (n, -1))
    return T.mean(1.0 - (T.sum_(p * y, 1) * 2.0 + eps) / (T.sum_(p, 1) + T.sum_(y, 1) + eps))


# ------------------------------------------------------------------ pairs and triplets
def margin_ranking(margin):
    """max(0, -y (a - b) + margin) for y in {-1, +1}."""
    def f(a, b, y):
        a, b, err = _pair("margin ranking loss", a, b)
        if err is not None:
            return err
        return T.mean(T.relu(T.neg(_f32(y) * (a - b)) + float(margin)))
    return f


def _norm2(x, eps=0.0):
    return T.sqrt(T.sum_(x * x, -1) + eps) if eps else T.sqrt(T.sum_(x * x, -1))


def triplet(margin):
    """max(0, |a - p| - |a - n| + margin) with Euclidean distances (1e-6 added to every difference, like PyTorch)."""
    def f(a, p, n):
        a1, p1, err = _pair("triplet loss", a, p)
        if err is not None:
            return err
        a2, n1, err = _pair("triplet loss", a, n)
        if err is not None:
            return err
        dp = _norm2(a1 - p1 + 1e-6)
        dn = _norm2(a2 - n1 + 1e-6)
        return T.mean(T.relu(dp - dn + float(margin)))
    return f


def cosine_embedding(margin):
    """1 - cos(a, b) for y = +1, max(0, cos(a, b) - margin) for y = -1."""
    def f(a, b, y):
        a, b, err = _pair("cosine embedding loss", a, b)
        if err is not None:
            return err
        eps = 1e-12                                        # under the square roots, as PyTorch has it
        cos = T.sum_(a * b, -1) / T.sqrt((T.sum_(a * a, -1) + eps) * (T.sum_(b * b, -1) + eps))
        y = _f32(y)
        pos = T.less(y * 0.0, y)
        return T.mean(T.where(pos, 1.0 - cos, T.relu(cos - float(margin))))
    return f


ALL = ["cross_entropy", "nll", "bce_with_logits", "mse", "l1", "huber", "label_smoothing", "focal",
       "binary_focal", "bce", "kl_div", "smooth_l1", "hinge", "margin_ranking", "triplet",
       "cosine_embedding", "poisson_nll", "gaussian_nll", "dice", "binary_dice"]
