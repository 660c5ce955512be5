"""Picking and tuning a model for a table (reference: automl/automl.go): boosted trees, random forests,
linear models, support vector machines, nearest neighbours and naive Bayes are each tried with their
defaults, then boosted trees with random settings, up to ``trials`` candidates.  Each is scored on rows
it did not learn from (log loss for classification, RMSE for regression, lower is better; k-fold
cross-validation on tables of up to 20,000 rows, one held-out fifth on larger ones), and the best is
fitted to the whole table."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field

import torch

from . import bayes, linear, neighbors, svm, tree
from .base import CLASSIFICATION, REGRESSION, as_task, count_classes
from .tabular import Data

BOOST, FOREST, LINEAR, SVM, NEIGHBORS, BAYES = "boost", "forest", "linear", "svm", "neighbors", "bayes"
FAMILIES = (BOOST, FOREST, LINEAR, SVM, NEIGHBORS, BAYES)
SVM_ROWS, NEIGHBOR_ROWS, FOLD_ROWS = 20_000, 100_000, 20_000


@dataclass
class Candidate:
    family: str
    settings: dict = field(default_factory=dict)

    def __str__(self):
        return self.family + ("(" + ", ".join(f"{k}={v}" for k, v in sorted(self.settings.items())) + ")" if self.settings else "")


@dataclass
class Trial:
    candidate: Candidate
    score: float            # log loss or RMSE on held-out rows; lower is better
    seconds: float

    @property
    def name(self):
        return str(self.candidate)


@dataclass
class Result:
    best: object            # the winner, fitted to every row
    candidate: Candidate
    score: float
    trials: list
    task: object


def _fitter(c: Candidate, task, classes, seed):
    s = c.settings
    if c.family == BOOST:
        return lambda d: tree.boosting(d, task, classes=classes, seed=seed, **s)
    if c.family == FOREST:
        return lambda d: tree.forest(d, task, classes=classes, seed=seed, **s)
    if c.family == LINEAR:
        return (lambda d: linear.logistic_fit(d, classes=classes, **s)) if classes else (lambda d: linear.regression(d, **s))
    if c.family == SVM:
        return lambda d: svm.fit(d, task, classes=classes, **s)
    if c.family == NEIGHBORS:
        return lambda d: neighbors.fit(d, task, classes=classes, **s)
    if c.family == BAYES:
        return lambda d: bayes.gaussian(d, classes=classes, **s)
    raise ValueError(f"automl: unknown family {c.family!r}: want some of {FAMILIES}")


def _score(model, held: Data, classes) -> float:
    p = model.predict(held.X)
    if classes:
        q = p.double().clamp(1e-15, 1.0)
        return float(-q.gather(1, held.Y.long()[:, None]).log().mean())
    return math.sqrt(float(((p.double() - held.Y.double()) ** 2).mean()))


def _candidates(task, rows, families, trials, seed):
    out = []
    defaults = {BOOST: dict(trees=100, max_depth=6, learning_rate=0.1), FOREST: dict(trees=100, max_depth=10), LINEAR: {},
                SVM: {}, NEIGHBORS: dict(k=5), BAYES: {}}
    for f in families:
        if f == SVM and rows > SVM_ROWS or f == NEIGHBORS and rows > NEIGHBOR_ROWS or f == BAYES and task is REGRESSION:
            continue
        out.append(Candidate(f, dict(defaults[f])))
    g = torch.Generator().manual_seed(seed)
    if BOOST in families:
        while len(out) < trials:
            u = torch.rand(5, generator=g).tolist()
            out.append(Candidate(BOOST, dict(trees=int(50 + 250 * u[0]), max_depth=int(2 + 7 * u[1]), learning_rate=round(0.02 * (15 ** u[2]), 4),
                                             subsample=round(0.6 + 0.4 * u[3], 2), colsample=round(0.5 + 0.5 * u[4], 2))))
    return out[:max(trials, 1)]


def search(d: Data, task, trials: int = 12, folds: int = 3, classes: int = 0, seed: int = 1, budget: float | None = None,
           families=None, progress=None) -> Result:
    """``budget`` (seconds) stops trying candidates once that much time has passed (the best so far wins);
    ``progress(done, total)`` is told after each one."""
    task = as_task(task)
    d.check(task)
    families = tuple(families) if families else FAMILIES
    for f in families:
        if f not in FAMILIES:
            raise ValueError(f"automl: unknown family {f!r}: want some of {FAMILIES}")
    if trials < 1 or folds < 2:
        raise ValueError("automl: at least one trial and two folds")
    K = count_classes(d.Y, classes) if task is CLASSIFICATION else 0
    cands = _candidates(task, d.rows, families, trials, seed)
    if not cands:
        raise ValueError("automl: no family fits this table and task")
    start, done = time.monotonic(), []
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(d.rows, generator=g)
    if d.rows <= FOLD_ROWS:
        k = min(folds, d.rows)
        parts = [(perm[torch.arange(d.rows) % k != i], perm[i::k]) for i in range(k)]
    else:
        cut = d.rows // 5
        parts = [(perm[cut:], perm[:cut])]
    for n, c in enumerate(cands):
        if budget is not None and done and time.monotonic() - start > budget:
            break
        t0 = time.monotonic()
        fit = _fitter(c, task, K, seed)
        try:
            score = sum(_score(fit(d.take(tr)), d.take(te), K) for tr, te in parts) / len(parts)
        except (ValueError, RuntimeError):
            score = math.inf                                 # a family that cannot fit this table loses
        done.append(Trial(c, score, time.monotonic() - t0))
        if progress is not None:
            progress(n + 1, len(cands))
    best = min(done, key=lambda t: t.score)
    if not math.isfinite(best.score):
        raise ValueError("automl: no candidate could be fitted")
    return Result(_fitter(best.candidate, task, K, seed)(d), best.candidate, best.score, done, task)
