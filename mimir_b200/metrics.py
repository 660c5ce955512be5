"""Streaming metrics and classical scores (reference: metrics/, metrics/score.go)."""
from __future__ import annotations

import math

import torch


class Metric:
    name = "metric"

    def update(self, pred: torch.Tensor, target: torch.Tensor) -> None:
        raise NotImplementedError

    def value(self) -> float:
        raise NotImplementedError

    def reset(self) -> None:
        pass


class Accuracy(Metric):
    name = "accuracy"

    def __init__(self):
        self.correct = self.total = 0

    def update(self, pred, target):
        p = pred.argmax(-1) if pred.dim() > target.dim() else (pred > 0.5).long()
        self.correct += int((p.long() == target.long()).sum())
        self.total += target.numel()

    def value(self):
        return self.correct / max(self.total, 1)

    def reset(self):
        self.correct = self.total = 0


def _t(x):
    return torch.as_tensor(x)


def class_accuracy(pred, y): return float((_t(pred).long() == _t(y).long()).float().mean())


def confusion(pred, y, classes=None):
    pred, y = _t(pred).long(), _t(y).long()
    k = classes or int(max(pred.max(), y.max())) + 1
    return torch.bincount(y * k + pred, minlength=k * k).view(k, k)


def per_class(pred, y, classes=None):
    c = confusion(pred, y, classes).float()
    tp = c.diag()
    prec = tp / c.sum(0).clamp_min(1)
    rec = tp / c.sum(1).clamp_min(1)
    f1 = 2 * prec * rec / (prec + rec).clamp_min(1e-12)
    return prec, rec, f1


def precision(pred, y, classes=None): return float(per_class(pred, y, classes)[0].mean())
def recall(pred, y, classes=None): return float(per_class(pred, y, classes)[1].mean())
def f1(pred, y, classes=None): return float(per_class(pred, y, classes)[2].mean())


def roc_auc(scores, y):
    s, y = _t(scores).double(), _t(y).long()
    order = torch.argsort(s)
    ranks = torch.empty_like(s)
    ranks[order] = torch.arange(1, s.numel() + 1, dtype=torch.double)
    # average ranks of ties
    uniq, inv = torch.unique(s, return_inverse=True)
    sums = torch.zeros(uniq.numel(), dtype=torch.double).index_add_(0, inv, ranks)
    cnt = torch.bincount(inv).double()
    ranks = (sums / cnt)[inv]
    npos, nneg = int(y.sum()), int((1 - y).sum())
    if npos == 0 or nneg == 0:
        return float("nan")
    return float((ranks[y == 1].sum() - npos * (npos + 1) / 2) / (npos * nneg))


def log_loss(prob, y, eps=1e-15):
    p, y = _t(prob).double().clamp(eps, 1 - eps), _t(y).long()
    if p.dim() == 1:
        return float(-(y * p.log() + (1 - y) * (1 - p).log()).mean())
    return float(-p.gather(1, y[:, None]).log().mean())


def mae(pred, y): return float((_t(pred).double() - _t(y).double()).abs().mean())
def rmse(pred, y): return math.sqrt(float(((_t(pred).double() - _t(y).double()) ** 2).mean()))


def r2(pred, y):
    p, y = _t(pred).double(), _t(y).double()
    return float(1 - ((y - p) ** 2).sum() / ((y - y.mean()) ** 2).sum().clamp_min(1e-300))
