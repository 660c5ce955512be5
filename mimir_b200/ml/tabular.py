"""Tabular data (reference: tabular/tabular.go, tabular/scale.go): a table of float features with one
answer per row, seeded splits and cross-validation, and a feature scaler."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .base import CLASSIFICATION, REGRESSION, Standard, Task, as_rows, as_task, count_classes  # noqa: F401


@dataclass
class Data:
    """``X [rows, features]`` (a flat list with ``n_features`` works too) and ``Y [rows]``: a value per row
    for regression, a class 0, 1, ... for classification.  NaN in ``X`` marks a missing value."""

    X: torch.Tensor
    Y: torch.Tensor | None = None
    features: list = field(default_factory=list)          # optional feature names
    n_features: int | None = None

    def __post_init__(self):
        self.X = as_rows(self.X, self.n_features)
        self.n_features = self.X.shape[1]
        if self.Y is not None:
            self.Y = torch.as_tensor(self.Y).reshape(-1)

    def __len__(self):
        return self.X.shape[0]

    @property
    def rows(self) -> int:
        return self.X.shape[0]

    def row(self, i: int) -> torch.Tensor:
        return self.X[i]

    def check(self, task=None) -> None:
        """Raises ``ValueError`` unless the table can be fitted for ``task``: at least one row and one
        feature, an answer per row, finite answers, whole-number classes for classification."""
        if self.rows == 0 or self.n_features == 0:
            raise ValueError(f"table of {self.rows} rows and {self.n_features} features")
        if torch.isinf(self.X).any():
            raise ValueError("a feature is infinite")
        if task is None:
            return
        if self.Y is None or self.Y.numel() != self.rows:
            raise ValueError(f"{0 if self.Y is None else self.Y.numel()} answers for {self.rows} rows")
        y = self.Y.double()
        if not torch.isfinite(y).all():
            raise ValueError("an answer is NaN or infinite")
        if as_task(task) is CLASSIFICATION:
            count_classes(self.Y)

    def classes(self) -> int:
        """One more than the largest class in ``Y``."""
        return count_classes(self.Y) if self.Y is not None else 0

    def take(self, idx) -> "Data":
        idx = torch.as_tensor(idx, dtype=torch.long)
        return Data(self.X[idx], None if self.Y is None else self.Y[idx], self.features)

    def split(self, test: float = 0.2, seed: int = 0):
        """``(train, held)``: a seeded shuffle cut so that ``held`` has ``round(test * rows)`` rows; every
        row lands in exactly one part."""
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(self.rows, generator=g)
        n_test = min(self.rows, max(0, int(round(self.rows * test))))
        return self.take(perm[n_test:]), self.take(perm[:n_test])


def split(d: Data, test: float = 0.2, seed: int = 0):
    return d.split(test, seed)


class Scaler:
    def __init__(self, mean, std):
        self.mean, self.std = mean, std

    def transform(self, X):
        return (torch.as_tensor(X).float() - self.mean) / self.std

    def inverse(self, X):
        return torch.as_tensor(X).float() * self.std + self.mean


def fit_scaler(X, features: int | None = None) -> Scaler:
    """Mean and deviation of each feature over the rows that have it; a constant feature keeps scale 1."""
    s = Standard.fit(as_rows(X, features))
    return Scaler(s.mean, s.scale)


def cross_validate(fit, score, d: Data, folds: int = 5, seed: int = 0):
    """``fit(train) -> model``, ``score(model, held) -> float``; every row is held out exactly once over
    the ``folds`` seeded folds.  Returns the score of each fold."""
    if folds < 2 or folds > len(d):
        raise ValueError(f"{folds} folds of {len(d)} rows")
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(len(d), generator=g)
    out = []
    for k in range(folds):
        held = perm[k::folds]
        mask = torch.ones(len(d), dtype=torch.bool)
        mask[held] = False
        out.append(float(score(fit(d.take(perm[mask[perm]])), d.take(held))))
    return out
