"""Losses over lazy tensors (reference: nn/loss/loss.go:35-96, more.go:66-296).
Every loss returns the mean over the batch.  Class targets are integer tensors."""
from __future__ import annotations

import torch

from .. import tensor as T

F = torch.nn.functional


def _op(name, fn, *ts):
    return T.core._node(fn, ts, {}, name)


def cross_entropy(logits, target):
    """Mean softmax cross-entropy of logits ``[N, C]`` (or ``[N, C, d1, ...]``) against integer class
    targets.  2-D bf16 CUDA logits whose class count is a multiple of 8 run the fused native kernel (loss and d(loss)/d(logits) in one pass over the
    logits, no fp32 copy of them); rows with a negative target are ignored there."""
    def run(l, t):
        if l.dim() == 2 and T.core._native_ok(l) and t.is_cuda and l.shape[-1] % 8 == 0 and l.numel():
            from ..ops import functional as NF
            return NF.cross_entropy(l, t)
        return F.cross_entropy(l.float(), t.long())
    return _op("cross_entropy", run, logits, target)
def nll(logp, target): return _op("nll", lambda l, t: F.nll_loss(l.float(), t.long()), logp, target)
def bce_with_logits(logits, target): return _op("bce_with_logits", lambda l, t: F.binary_cross_entropy_with_logits(l.float(), t.float()), logits, target)
def bce(pred, target): return _op("bce", lambda p, t: F.binary_cross_entropy(p.float(), t.float()), pred, target)
def mse(pred, target): return _op("mse", lambda p, t: F.mse_loss(p.float(), t.float()), pred, target)
def l1(pred, target): return _op("l1", lambda p, t: F.l1_loss(p.float(), t.float()), pred, target)
def huber(pred, target, delta=1.0): return _op("huber", lambda p, t: F.huber_loss(p.float(), t.float(), delta=delta), pred, target)
def smooth_l1(beta=1.0): return lambda pred, target: _op("smooth_l1", lambda p, t: F.smooth_l1_loss(p.float(), t.float(), beta=beta), pred, target)
def kl_div(logp, target): return _op("kl_div", lambda l, t: F.kl_div(l.float(), t.float(), reduction="batchmean"), logp, target)
def label_smoothing(eps): return lambda logits, target: _op("label_smoothing", lambda l, t: F.cross_entropy(l.float(), t.long(), label_smoothing=eps), logits, target)


def focal(gamma):
    def f(l, t):
        logp = F.log_softmax(l.float(), -1).gather(-1, t.long().unsqueeze(-1)).squeeze(-1)
        return (-(1 - logp.exp()) ** gamma * logp).mean()
    return lambda logits, target: _op("focal", f, logits, target)


def binary_focal(gamma, alpha):
    def f(l, t):
        t = t.float()
        p = torch.sigmoid(l.float())
        pt = p * t + (1 - p) * (1 - t)
        a = alpha * t + (1 - alpha) * (1 - t)
        return (a * (1 - pt) ** gamma * F.binary_cross_entropy_with_logits(l.float(), t, reduction="none")).mean()
    return lambda logits, target: _op("binary_focal", f, logits, target)


def hinge(scores, target):
    def f(s, t):
        s = s.float()
        correct = s.gather(-1, t.long().unsqueeze(-1))
        m = (1 + s - correct).clamp_min(0)
        m = m.scatter(-1, t.long().unsqueeze(-1), 0.0)
        return m.sum(-1).mean()
    return _op("hinge", f, scores, target)


def margin_ranking(margin): return lambda a, b, y: _op("margin_ranking", lambda u, v, w: F.margin_ranking_loss(u.float(), v.float(), w.float(), margin=margin), a, b, y)
def triplet(margin): return lambda a, p, n: _op("triplet", lambda u, v, w: F.triplet_margin_loss(u.float(), v.float(), w.float(), margin=margin), a, p, n)
def cosine_embedding(margin): return lambda a, b, y: _op("cosine_embedding", lambda u, v, w: F.cosine_embedding_loss(u.float(), v.float(), w.float(), margin=margin), a, b, y)
def poisson_nll(log_rate, target): return _op("poisson_nll", lambda l, t: F.poisson_nll_loss(l.float(), t.float(), log_input=True), log_rate, target)
def gaussian_nll(mean, variance, target): return _op("gaussian_nll", lambda m, v, t: F.gaussian_nll_loss(m.float(), t.float(), v.float()), mean, variance, target)


def dice(logits, target, eps=1.0):
    def f(l, t):
        p = torch.softmax(l.float(), 1)
        oh = F.one_hot(t.long(), l.shape[1]).movedim(-1, 1).float()
        dims = tuple(range(2, l.dim()))
        inter = (p * oh).sum(dims)
        return (1 - (2 * inter + eps) / (p.sum(dims) + oh.sum(dims) + eps)).mean()
    return _op("dice", f, logits, target)


def binary_dice(logits, target, eps=1.0):
    def f(l, t):
        p, t = torch.sigmoid(l.float()).flatten(1), t.float().flatten(1)
        return (1 - (2 * (p * t).sum(1) + eps) / (p.sum(1) + t.sum(1) + eps)).mean()
    return _op("binary_dice", f, logits, target)


ALL = ["cross_entropy", "nll", "bce_with_logits", "mse", "l1", "huber", "label_smoothing", "focal",
       "binary_focal", "bce", "kl_div", "smooth_l1", "hinge", "margin_ranking", "triplet",
       "cosine_embedding", "poisson_nll", "gaussian_nll", "dice", "binary_dice"]
