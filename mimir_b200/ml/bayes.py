"""Naive Bayes classifiers (reference: bayes/bayes.go): a product of one simple distribution per
feature, fitted in one pass.  Gaussian suits measurements, multinomial counts (how often each word
appears), Bernoulli presence (whether it appears at all).

Every kind's log-likelihood of class c for a row x is
``prior[c] + sum_j (square[c, j] x_j^2 + linear[c, j] x_j + const[c, j])`` over the features that are
not missing (x_j first binarized for Bernoulli), so one model class and one ``nn.Module`` serve all
three.  A missing value (NaN) is left out of a row's likelihood."""
from __future__ import annotations

import math

import torch

from .base import CLASSIFICATION, Model, as_rows, count_classes

GAUSSIAN, MULTINOMIAL, BERNOULLI = "gaussian", "multinomial", "bernoulli"


class NaiveBayes(Model):
    FIELDS = ("kind", "features", "classes", "prior", "square", "linear", "const", "binarize")

    def log_likelihood(self, X) -> torch.Tensor:
        """``[rows, classes]`` joint log-likelihoods (prior included)."""
        X = as_rows(X, self.features).double()
        have = ~torch.isnan(X)
        x = torch.where(have, X, torch.zeros_like(X))
        if self.kind == BERNOULLI:
            x = (x > self.binarize).double()
        h = have.double()
        return self.prior + (x * x * h) @ self.square.t() + (x * h) @ self.linear.t() + h @ self.const.t()

    def predict(self, X) -> torch.Tensor:
        return torch.softmax(self.log_likelihood(X), 1).float()

    def module(self):
        from .modules import BayesModule
        return BayesModule.of(self)


def _start(d, classes, priors):
    d.check(CLASSIFICATION)
    K = count_classes(d.Y, classes)
    if K < 1:
        raise ValueError("bayes: no classes")
    y = d.Y.long()
    counts = torch.bincount(y, minlength=K).double()
    if priors is not None:
        p = torch.as_tensor(priors, dtype=torch.double)
        if p.numel() != K or (p < 0).any() or abs(float(p.sum()) - 1) > 1e-6:
            raise ValueError(f"bayes: {p.numel()} priors for {K} classes, or priors that do not sum to 1")
        prior = p.clamp_min(1e-300).log()
    else:
        prior = (counts / counts.sum()).clamp_min(1e-300).log()
    onehot = torch.nn.functional.one_hot(y, K).double()
    X = d.X.double()
    have = ~torch.isnan(X)
    return K, prior, onehot, torch.where(have, X, torch.zeros_like(X)), have.double()


def _model(kind, F, K, prior, sq, lin, const, binarize=0.0):
    m = NaiveBayes()
    m.kind, m.features, m.classes, m.prior, m.square, m.linear, m.const, m.binarize = kind, F, K, prior, sq, lin, const, float(binarize)
    return m


def gaussian(d, var_smoothing: float = 1e-9, classes: int = 0, priors=None) -> NaiveBayes:
    """A normal distribution per feature and class; ``var_smoothing`` times the largest feature variance is
    added to every variance."""
    if var_smoothing < 0:
        raise ValueError("bayes: smoothing must not be negative")
    K, prior, onehot, x, h = _start(d, classes, priors)
    n = (onehot.t() @ h).clamp_min(1)                                  # rows of class c that have feature j
    mean = (onehot.t() @ x) / n
    var = (onehot.t() @ (x * x)) / n - mean * mean
    tot = h.sum(0).clamp_min(1)
    gvar = (x * x).sum(0) / tot - ((x.sum(0) / tot) ** 2)
    var = var.clamp_min(0) + var_smoothing * float(gvar.max().clamp_min(0)) + 1e-300
    # -0.5 log(2 pi var) - (x - mean)^2 / (2 var), expanded in powers of x
    sq, lin = -0.5 / var, mean / var
    const = -0.5 * torch.log(2 * math.pi * var) - 0.5 * mean * mean / var
    return _model(GAUSSIAN, d.n_features, K, prior, sq, lin, const)


def multinomial(d, alpha: float = 1.0, classes: int = 0, priors=None) -> NaiveBayes:
    """Each class's share of the total of each feature (counts that are 0 or more), with additive smoothing."""
    if alpha < 0:
        raise ValueError("bayes: alpha must not be negative")
    K, prior, onehot, x, h = _start(d, classes, priors)
    if (x < 0).any():
        raise ValueError("bayes: multinomial features must not be negative")
    cnt = onehot.t() @ x + alpha
    logp = (cnt / cnt.sum(1, keepdim=True)).clamp_min(1e-300).log()
    z = torch.zeros_like(logp)
    return _model(MULTINOMIAL, d.n_features, K, prior, z, logp, z.clone())


def bernoulli(d, alpha: float = 1.0, binarize: float = 0.0, classes: int = 0, priors=None) -> NaiveBayes:
    """Whether each feature is present (above ``binarize``) in each class."""
    if alpha < 0:
        raise ValueError("bayes: alpha must not be negative")
    K, prior, onehot, x, h = _start(d, classes, priors)
    present = (x > binarize).double() * h
    n = onehot.t() @ h
    p = ((onehot.t() @ present + alpha) / (n + 2 * alpha).clamp_min(1e-300)).clamp(1e-300, 1 - 1e-16)
    # x log p + (1 - x) log(1 - p)
    return _model(BERNOULLI, d.n_features, K, prior, torch.zeros_like(p), p.log() - torch.log1p(-p), torch.log1p(-p), binarize)
