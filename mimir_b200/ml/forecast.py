"""Forecasting series measured at equal steps (reference: forecast/forecast.go, forecast/smooth.go).

``fit`` is a *global* model: gradient-boosted trees over each step's recent values, learned from every
series at once.  Each series is scaled by the mean size of its values, so series in thousands and in
tens teach the same shapes; NaN marks a missing value.  It forecasts one step at a time, feeding each
forecast back as the next step's latest value.  ``smooth`` is additive Holt-Winters exponential
smoothing of one series with its smoothing weights chosen by a search over the one-step error."""
from __future__ import annotations

import itertools
import math

import torch

from . import tree
from .base import Model


def _scale(s: torch.Tensor) -> float:
    v = s[~torch.isnan(s)].abs()
    m = float(v.mean()) if v.numel() else 0.0
    return m if m > 0 else 1.0


def _features(lags: int, season: int) -> int:
    return lags + (2 if season > 0 else 0) + 2


class Forecaster(Model):
    """The boosted trees and what a step's features are: the ``lags`` latest values (scaled), their mean and
    spread, and with a ``season`` the phase of the step in its cycle as a sine / cosine pair."""

    FIELDS = ("lags", "season", "trees_json")

    @property
    def features(self) -> int:
        return _features(self.lags, self.season)

    @property
    def trees(self):
        t = getattr(self, "_trees", None)
        if t is None:
            t = self._trees = tree.Model.from_json(self.trees_json)
        return t

    def _row(self, s: torch.Tensor, t: int) -> torch.Tensor:
        """Features of the step at ``t`` of the scaled series ``s`` whose earlier steps are ``s[:t]``."""
        recent = s[t - self.lags:t]
        have = recent[~torch.isnan(recent)]
        extra = [float(have.mean()) if have.numel() else math.nan, float(have.std(unbiased=False)) if have.numel() else math.nan]
        if self.season > 0:
            ph = 2 * math.pi * (t % self.season) / self.season
            extra += [math.sin(ph), math.cos(ph)]
        return torch.cat([recent, torch.tensor(extra)])

    def rows(self, history):
        """For the step after ``history``: the features the trees read and the scale their answer is in."""
        h = torch.as_tensor(history, dtype=torch.float32)
        if h.numel() < self.lags:
            raise ValueError(f"forecast: a history of {h.numel()} steps, the model reads {self.lags}")
        sc = _scale(h)
        return self._row(h / sc, h.numel()), sc

    def forecast(self, history, steps: int) -> torch.Tensor:
        h = torch.as_tensor(history, dtype=torch.float32)
        if h.numel() < self.lags or steps < 0:
            raise ValueError(f"forecast: a history of {h.numel()} steps, the model reads {self.lags}")
        sc = _scale(h)
        s = torch.cat([h / sc, torch.zeros(steps)])
        n = h.numel()
        for k in range(steps):
            s[n + k] = self.trees.predict(self._row(s, n + k)[None])[0]
        return s[n:] * sc


def fit(series, lags: int | None = None, season: int = 0, holdout: int = 0, **tree_options) -> Forecaster:
    """``series``: a list of 1-D sequences, each at least ``lags + 2`` steps long.  ``lags`` defaults to twice
    the season and at least 14; the last ``holdout`` steps of each series (default a tenth of its steps, up
    to the season or 14) tell when more trees stop helping.  Other keywords go to the boosted trees."""
    if season < 0:
        raise ValueError("forecast: the season must not be negative")
    lags = max(2 * season, 14) if lags is None else int(lags)
    if lags < 1 or not len(series):
        raise ValueError("forecast: no series, or lags below 1")
    m = Forecaster()
    m.lags, m.season = lags, int(season)
    Xt, yt, Xv, yv = [], [], [], []
    for raw in series:
        s = torch.as_tensor(raw, dtype=torch.float32).reshape(-1)
        if s.numel() < lags + 2:
            raise ValueError(f"forecast: a series of {s.numel()} steps, want at least {lags + 2}")
        s = s / _scale(s)
        hold = holdout if holdout > 0 else min(max(s.numel() // 10, 1), season if season > 0 else 14)
        hold = min(hold, s.numel() - lags - 1)
        for t in range(lags, s.numel()):
            if torch.isnan(s[t]):
                continue
            (Xv if t >= s.numel() - hold else Xt).append(m._row(s, t))
            (yv if t >= s.numel() - hold else yt).append(s[t])
    if not Xt:
        raise ValueError("forecast: no step has a value to learn from")
    opts = dict(trees=300, max_depth=5, learning_rate=0.1, patience=20)
    opts.update(tree_options)
    val = (torch.stack(Xv), torch.stack(yv)) if Xv else None
    model = tree.gradient_boosting(torch.stack(Xt), torch.stack(yt), validation=val, **opts)
    m.trees_json, m._trees = model.to_json(), model
    return m


# ------------------------------------------------------------------ exponential smoothing
class Smoothing(Model):
    """Additive Holt-Winters state after the last step: level, trend, one offset per phase of the season."""

    FIELDS = ("alpha", "beta", "gamma", "season", "level", "trend", "offsets", "steps", "error")

    def forecast(self, steps: int) -> torch.Tensor:
        out = [self.level + (h + 1) * self.trend + (self.offsets[(self.steps + h) % self.season] if self.season else 0.0)
               for h in range(steps)]
        return torch.tensor(out, dtype=torch.float32)


def _run(y, season, alpha, beta, gamma):
    """The state after the series and the sum of squared one-step errors after the first season (or step),
    which the state is set from.  A missing value only carries the state forward."""
    m = season
    first = [v for v in y[:max(m, 1)] if v == v]
    level = sum(first) / len(first) if first else 0.0
    if m and len(y) >= 2 * m:
        second = [v for v in y[m:2 * m] if v == v]
        trend = ((sum(second) / len(second) if second else level) - level) / m
    else:
        trend = 0.0 if m or len(y) < 2 or y[1] != y[1] or y[0] != y[0] else y[1] - y[0]
    offsets = [(y[i] - level) if y[i] == y[i] else 0.0 for i in range(m)] if m else []
    sse = 0.0
    for t in range(max(m, 1), len(y)):
        v = y[t]
        s = offsets[t % m] if m else 0.0
        pred = level + trend + s
        if v != v:
            level += trend
            continue
        sse += (v - pred) ** 2
        last = level
        level = alpha * (v - s) + (1 - alpha) * (level + trend)
        trend = beta * (level - last) + (1 - beta) * trend
        if m:
            offsets[t % m] = gamma * (v - level) + (1 - gamma) * s
    return level, trend, offsets, sse


def smooth(series, season: int = 0, alpha=None, beta=None, gamma=None) -> Smoothing:
    """Weights that are not given are chosen from a grid by the smallest sum of squared one-step errors."""
    y = [float(v) for v in torch.as_tensor(series, dtype=torch.float64).reshape(-1).tolist()]
    if season < 0 or len(y) < max(2, 2 * season) or all(v != v for v in y):
        raise ValueError(f"smooth: {len(y)} steps for a season of {season}, or no values")
    grid = (0.05, 0.1, 0.2, 0.3, 0.5, 0.7, 0.9)
    best = None
    for a, b, g in itertools.product([alpha] if alpha is not None else grid, [beta] if beta is not None else (0.0, 0.01, 0.05, 0.1, 0.3),
                                     [gamma] if gamma is not None else (grid if season else (0.0,))):
        level, trend, offsets, sse = _run(y, season, a, b, g)
        if best is None or sse < best[0]:
            best = (sse, a, b, g, level, trend, offsets)
    m = Smoothing()
    m.error, m.alpha, m.beta, m.gamma, m.level, m.trend, m.offsets = best
    m.season, m.steps = int(season), len(y)
    return m
