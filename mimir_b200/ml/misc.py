"""Forecasting, recommendation, association rules, AutoML (reference: forecast/, recommend/,
rules/, automl/)."""
from __future__ import annotations

import itertools

import torch

from . import linear, neighbors, tree


# ---------------------------------------------------------------- forecast
class HoltWinters:
    """Additive triple exponential smoothing with period ``m`` (m=0: double smoothing)."""

    def __init__(self, alpha=0.3, beta=0.1, gamma=0.1, period=0):
        self.alpha, self.beta, self.gamma, self.m = alpha, beta, gamma, period

    def fit(self, y):
        y = [float(v) for v in y]
        m = self.m
        level = sum(y[:m]) / m if m else y[0]
        trend = (sum(y[m:2 * m]) - sum(y[:m])) / (m * m) if m and len(y) >= 2 * m else (y[1] - y[0] if len(y) > 1 else 0.0)
        season = [y[i] - level for i in range(m)] if m else []
        for t, v in enumerate(y):
            s = season[t % m] if m else 0.0
            last = level
            level = self.alpha * (v - s) + (1 - self.alpha) * (level + trend)
            trend = self.beta * (level - last) + (1 - self.beta) * trend
            if m:
                season[t % m] = self.gamma * (v - level) + (1 - self.gamma) * s
        self.level, self.trend, self.season, self.n = level, trend, season, len(y)
        return self

    def forecast(self, steps):
        return torch.tensor([self.level + (h + 1) * self.trend + (self.season[(self.n + h) % self.m] if self.m else 0.0)
                             for h in range(steps)])


def autoregressive(y, lags=4, l2=0.0):
    """AR(lags) by least squares; returns ``forecast(steps)``."""
    y = torch.as_tensor(y).float()
    X = torch.stack([y[i:len(y) - lags + i] for i in range(lags)], 1)
    m = linear.ridge(X, y[lags:], l2)

    def forecast(steps):
        hist = y[-lags:].clone()
        out = []
        for _ in range(steps):
            nxt = m.predict(hist[None])[0]
            out.append(nxt)
            hist = torch.cat([hist[1:], nxt[None]])
        return torch.stack(out)
    return forecast


# ---------------------------------------------------------------- recommend
class ALS:
    """Alternating least squares matrix factorisation on (user, item, rating) triples."""

    def __init__(self, users, items, factors=16, l2=0.1, iters=10, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.U = torch.randn(users, factors, generator=g) * 0.1
        self.V = torch.randn(items, factors, generator=g) * 0.1
        self.l2, self.iters = l2, iters

    def fit(self, u, i, r):
        u, i, r = torch.as_tensor(u).long(), torch.as_tensor(i).long(), torch.as_tensor(r).float()
        R = torch.zeros(self.U.shape[0], self.V.shape[0])
        M = torch.zeros_like(R)
        R[u, i], M[u, i] = r, 1.0
        eye = self.l2 * torch.eye(self.U.shape[1])
        for _ in range(self.iters):
            for A, B, Rm, Mm in ((self.U, self.V, R, M), (self.V, self.U, R.t(), M.t())):
                G = torch.einsum("nk,mn,nl->mkl", B, Mm, B) + eye
                rhs = (Rm * Mm) @ B
                A.copy_(torch.linalg.solve(G, rhs.unsqueeze(-1)).squeeze(-1))
        return self

    def predict(self, u, i):
        return (self.U[u] * self.V[i]).sum(-1)

    def recommend(self, user, k=10):
        return torch.topk(self.V @ self.U[user], k).indices


# ---------------------------------------------------------------- rules
def apriori(transactions, min_support=0.1, min_confidence=0.5, max_len=3):
    """Frequent itemsets and association rules ``(antecedent, consequent, support, confidence, lift)``."""
    n = len(transactions)
    sets = [frozenset(t) for t in transactions]
    items = sorted({x for t in sets for x in t})
    support = {}
    level = [frozenset([x]) for x in items]
    k = 1
    while level and k <= max_len:
        keep = []
        for c in level:
            s = sum(1 for t in sets if c <= t) / n
            if s >= min_support:
                support[c] = s
                keep.append(c)
        k += 1
        level = list({a | b for a, b in itertools.combinations(keep, 2) if len(a | b) == k})
    out = []
    for s, sup in support.items():
        if len(s) < 2:
            continue
        for r in range(1, len(s)):
            for ante in map(frozenset, itertools.combinations(sorted(s), r)):
                conf = sup / support[ante]
                if conf >= min_confidence:
                    cons = s - ante
                    out.append((set(ante), set(cons), sup, conf, conf / support[cons]))
    return support, sorted(out, key=lambda r: -r[3])


# ---------------------------------------------------------------- automl
def automl(X, y, classes=0, folds=3, seed=0, time_budget=None):
    """Fits a small portfolio (linear / logistic, boosted trees at two depths, forest, k-NN) and
    returns ``(best_name, best_model, leaderboard)`` by cross-validated score (R^2 or accuracy)."""
    from .tabular import Data, cross_validate
    X, y = torch.as_tensor(X).float(), torch.as_tensor(y)
    d = Data(X, y)
    cands = {}
    if classes:
        cands["logistic"] = lambda t: linear.logistic(t.X, t.Y, classes)
        cands["gbdt_d3"] = lambda t: tree.gradient_boosting(t.X, t.Y, trees=50, max_depth=3, classes=classes, seed=seed)
        cands["gbdt_d6"] = lambda t: tree.gradient_boosting(t.X, t.Y, trees=50, max_depth=6, classes=classes, seed=seed)
        cands["knn"] = lambda t: neighbors.KNN(t.X, t.Y, 5, classes)
        score = lambda m, t: float((m.classify(t.X) == t.Y).float().mean())
    else:
        cands["ridge"] = lambda t: linear.ridge(t.X, t.Y, 1e-3)
        cands["gbdt_d3"] = lambda t: tree.gradient_boosting(t.X, t.Y, trees=50, max_depth=3, seed=seed)
        cands["gbdt_d6"] = lambda t: tree.gradient_boosting(t.X, t.Y, trees=50, max_depth=6, seed=seed)
        cands["forest"] = lambda t: tree.random_forest(t.X, t.Y, trees=30, seed=seed)
        cands["knn"] = lambda t: neighbors.KNN(t.X, t.Y, 5)
        score = lambda m, t: float(1 - ((m.predict(t.X) - t.Y.float()) ** 2).sum() / ((t.Y.float() - t.Y.float().mean()) ** 2).sum())
    board = {name: sum(s := cross_validate(fit, score, d, folds, seed)) / len(s) for name, fit in cands.items()}
    best = max(board, key=board.get)
    return best, cands[best](d), board
