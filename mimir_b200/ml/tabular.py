"""Tabular data helpers (reference: tabular/): ``Data{X, Features, Y}``, ``split``, ``take``,
``cross_validate``, ``fit_scaler``."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class Data:
    X: torch.Tensor
    Y: torch.Tensor | None = None
    features: list = field(default_factory=list)

    def take(self, idx) -> "Data":
        idx = torch.as_tensor(idx)
        return Data(self.X[idx], None if self.Y is None else self.Y[idx], self.features)

    def __len__(self):
        return self.X.shape[0]


def split(d: Data, test: float = 0.2, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(len(d), generator=g)
    n = int(round(len(d) * (1 - test)))
    return d.take(perm[:n]), d.take(perm[n:])


class Scaler:
    def __init__(self, mean, std):
        self.mean, self.std = mean, std

    def transform(self, X):
        return (X - self.mean) / self.std

    def inverse(self, X):
        return X * self.std + self.mean


def fit_scaler(X) -> Scaler:
    X = torch.as_tensor(X).float()
    return Scaler(X.mean(0), X.std(0).clamp_min(1e-8))


def cross_validate(fit, score, d: Data, folds: int = 5, seed: int = 0):
    """``fit(train) -> model``, ``score(model, test) -> float``; returns the per-fold scores."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(len(d), generator=g)
    out = []
    for k in range(folds):
        test_idx = perm[k::folds]
        mask = torch.ones(len(d), dtype=torch.bool)
        mask[test_idx] = False
        out.append(score(fit(d.take(perm[mask[perm]])), d.take(test_idx)))
    return out
