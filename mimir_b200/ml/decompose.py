"""Principal component analysis (reference: decompose/pca.go): the directions a table's rows vary in
most, on standardized features (so the directions are those of the correlations, not of the units); a
missing value counts as the feature's mean."""
from __future__ import annotations

import torch

from .base import Model, Standard, as_rows


class Components(Model):
    """``k`` directions of ``features`` numbers each, in standardized units, from the most varied;
    ``variance[i]`` is the variance of the rows along direction i and ``ratio[i]`` its share of the total."""

    FIELDS = ("features", "directions", "variance", "ratio", "standard")

    @property
    def k(self) -> int:
        return int(self.directions.shape[0])

    def transform(self, X) -> torch.Tensor:
        """Each row as ``k`` numbers: its standardized values along each direction."""
        return self.standard.apply(as_rows(X, self.features)) @ self.directions.t()

    def inverse(self, Y) -> torch.Tensor:
        """Each row of ``k`` numbers back as ``features`` numbers in the features' own units."""
        Y = as_rows(Y, self.k)
        return (Y @ self.directions) * self.standard.scale + self.standard.mean

    def ranked(self, d: int) -> list:
        """The features by how much they weigh in direction ``d``, the most first."""
        return torch.argsort(self.directions[d].abs(), descending=True, stable=True).tolist()


def pca_fit(X, k: int, features: int | None = None) -> Components:
    X = as_rows(X, features)
    n, F = X.shape
    if n < 2 or k < 1 or k > min(n, F) or torch.isinf(X).any():
        raise ValueError(f"pca: {k} components of a table of {n} rows and {F} features")
    std = Standard.fit(X)
    Z = std.apply(X).double()
    Z = Z - Z.mean(0)
    # the eigenvectors of the smaller of the two Gram matrices
    if F <= n:
        w, V = torch.linalg.eigh(Z.t() @ Z / (n - 1))
        w, V = w.flip(0), V.flip(1)
        dirs = V.t()
    else:
        w, U = torch.linalg.eigh(Z @ Z.t() / (n - 1))
        w, U = w.flip(0).clamp_min(0), U.flip(1)
        dirs = (Z.t() @ U / (w * (n - 1)).sqrt().clamp_min(1e-300)).t()
    dirs = dirs[:k]
    # a fixed sign: the largest entry of each direction is positive
    big = dirs.abs().argmax(1)
    sign = torch.sign(dirs.gather(1, big[:, None]))
    dirs = dirs * torch.where(sign == 0, torch.ones_like(sign), sign)
    m = Components()
    total = float(w.clamp_min(0).sum()) or 1.0
    m.features, m.directions, m.variance, m.ratio, m.standard = F, dirs.float(), w[:k].clamp_min(0).float(), (w[:k].clamp_min(0) / total).float(), std
    return m
