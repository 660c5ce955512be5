"""Histogram-based trees (reference: tree/): DecisionTree, RandomForest, GradientBoosting,
IsolationForest.  Features are binned into at most 255 bins once; split search works on
per-node gradient / hessian histograms (the reference accelerates the same histograms
with AVX2 assembly, tree/hist_amd64.go; here they are ``torch.bincount`` calls, which run
on the GPU when the data lives there)."""
from __future__ import annotations

import json
import math

import torch


def _bin(X, bins=255):
    X = X.float()
    qs = torch.linspace(0, 1, bins + 1)[1:-1]
    edges = torch.quantile(X, qs.to(X.device), dim=0).t().contiguous()  # [F, bins-1]
    B = torch.searchsorted(edges, X.t().contiguous()).t().contiguous()
    return B.to(torch.int64), edges


class _Tree:
    """Regression tree on gradients/hessians (second-order gain with L2)."""

    def __init__(self, max_depth=6, min_leaf=1, min_gain=0.0, l2=1.0, bins=255, colsample=1.0, gen=None):
        self.max_depth, self.min_leaf, self.min_gain, self.l2, self.bins = max_depth, min_leaf, min_gain, l2, bins
        self.colsample, self.gen = colsample, gen
        self.nodes = []  # (feature, bin, left, right, value)
        self.importance = None

    def fit(self, B, g, h):
        n, F = B.shape
        self.importance = torch.zeros(F)
        self.nodes = []
        self._grow(B, g, h, torch.arange(n, device=B.device), 0)
        return self

    def _grow(self, B, g, h, idx, depth):
        G, H = g[idx].sum(), h[idx].sum()
        node = len(self.nodes)
        self.nodes.append([-1, 0, -1, -1, float(-G / (H + self.l2))])
        if depth >= self.max_depth or idx.numel() < 2 * self.min_leaf:
            return node
        F = B.shape[1]
        feats = torch.arange(F)
        if self.colsample < 1.0:
            k = max(1, int(F * self.colsample))
            feats = torch.randperm(F, generator=self.gen)[:k]
        Bi = B[idx][:, feats]
        flat = Bi + torch.arange(feats.numel(), device=B.device) * self.bins
        hg = torch.bincount(flat.reshape(-1), weights=g[idx].repeat_interleave(feats.numel()), minlength=feats.numel() * self.bins)
        hh = torch.bincount(flat.reshape(-1), weights=h[idx].repeat_interleave(feats.numel()), minlength=feats.numel() * self.bins)
        hc = torch.bincount(flat.reshape(-1), minlength=feats.numel() * self.bins)
        GL = hg.view(-1, self.bins).cumsum(1)
        HL = hh.view(-1, self.bins).cumsum(1)
        CL = hc.view(-1, self.bins).cumsum(1)
        GR, HR, CR = G - GL, H - HL, idx.numel() - CL
        gain = GL ** 2 / (HL + self.l2) + GR ** 2 / (HR + self.l2) - G ** 2 / (H + self.l2)
        gain[(CL < self.min_leaf) | (CR < self.min_leaf)] = -1
        best = int(gain.argmax())
        bg = float(gain.reshape(-1)[best])
        if bg <= self.min_gain:
            return node
        f, b = feats[best // self.bins].item(), best % self.bins
        self.importance[f] += bg
        go_left = B[idx, f] <= b
        self.nodes[node][0], self.nodes[node][1] = f, b
        self.nodes[node][2] = self._grow(B, g, h, idx[go_left], depth + 1)
        self.nodes[node][3] = self._grow(B, g, h, idx[~go_left], depth + 1)
        return node

    def predict_binned(self, B):
        out = torch.zeros(B.shape[0])
        node = torch.zeros(B.shape[0], dtype=torch.int64)
        active = torch.ones(B.shape[0], dtype=torch.bool)
        tbl = torch.tensor(self.nodes, dtype=torch.float64)
        for _ in range(self.max_depth + 1):
            f = tbl[node, 0].long()
            leaf = f < 0
            done = active & leaf
            out[done] = tbl[node[done], 4].float()
            active = active & ~leaf
            if not active.any():
                break
            ai = active.nonzero().squeeze(1)
            fa = f[ai]
            left = B[ai, fa] <= tbl[node[ai], 1].long()
            node[ai] = torch.where(left, tbl[node[ai], 2].long(), tbl[node[ai], 3].long())
        return out


class Model:
    """A fitted ensemble: ``predict`` (regression value / class probabilities), ``classify``,
    ``importance``, JSON round trip."""

    def __init__(self, trees, edges, lr, base, classes=0, kind="gbdt"):
        self.trees, self.edges, self.lr, self.base, self.classes, self.kind = trees, edges, lr, base, classes, kind

    def _binned(self, X):
        return torch.searchsorted(self.edges, torch.as_tensor(X).float().t().contiguous()).t().contiguous()

    def raw(self, X):
        B = self._binned(X)
        if self.classes > 2:
            out = self.base.clone().repeat(B.shape[0], 1)
            for round_trees in self.trees:
                for k, t in enumerate(round_trees):
                    out[:, k] += self.lr * t.predict_binned(B)
            return out
        out = torch.full((B.shape[0],), float(self.base))
        scale = self.lr if self.kind == "gbdt" else 1.0 / max(len(self.trees), 1)
        for t in self.trees:
            out += scale * t.predict_binned(B)
        return out

    def predict(self, X):
        r = self.raw(X)
        if self.classes == 2:
            return torch.sigmoid(r)
        if self.classes > 2:
            return torch.softmax(r, 1)
        return r

    def classify(self, X):
        p = self.predict(X)
        return (p > 0.5).long() if self.classes == 2 else p.argmax(1)

    def importance(self):
        trees = [t for r in self.trees for t in (r if isinstance(r, list) else [r])]
        imp = sum(t.importance for t in trees)
        return imp / imp.sum().clamp_min(1e-12)

    def to_json(self) -> str:
        def enc(t):
            return t.nodes
        trees = [[enc(t) for t in r] if isinstance(r, list) else enc(r) for r in self.trees]
        return json.dumps(dict(trees=trees, edges=self.edges.tolist(), lr=self.lr,
                               base=self.base.tolist() if torch.is_tensor(self.base) else self.base,
                               classes=self.classes, kind=self.kind,
                               depth=(self.trees[0][0] if isinstance(self.trees[0], list) else self.trees[0]).max_depth))

    @staticmethod
    def from_json(s: str) -> "Model":
        d = json.loads(s)

        def dec(nodes):
            t = _Tree(max_depth=d["depth"])
            t.nodes, t.importance = nodes, torch.zeros(len(d["edges"]))
            return t
        trees = [[dec(n) for n in r] if r and isinstance(r[0][0], list) else dec(r) for r in d["trees"]]
        base = torch.tensor(d["base"]) if isinstance(d["base"], list) else d["base"]
        return Model(trees, torch.tensor(d["edges"]), d["lr"], base, d["classes"], d["kind"])


def gradient_boosting(X, y, trees=100, learning_rate=0.1, max_depth=6, min_leaf=1, min_gain=0.0, l2=1.0, bins=255,
                      subsample=1.0, colsample=1.0, classes=0, seed=0, validation=None, progress=None) -> Model:
    """Second-order boosting: squared error (classes=0), logistic (2) or softmax (>2)."""
    X, y = torch.as_tensor(X).float(), torch.as_tensor(y)
    gen = torch.Generator().manual_seed(seed)
    B, edges = _bin(X, bins)
    n = X.shape[0]
    out_trees = []
    if classes > 2:
        base = torch.zeros(classes)
        F = torch.zeros(n, classes)
        oh = torch.nn.functional.one_hot(y.long(), classes).float()
    else:
        yf = y.float()
        base = float(yf.mean()) if classes == 0 else float(torch.logit(yf.mean().clamp(1e-6, 1 - 1e-6)))
        F = torch.full((n,), base)
    for it in range(trees):
        rows = torch.arange(n) if subsample >= 1.0 else torch.randperm(n, generator=gen)[: max(1, int(n * subsample))]
        if classes > 2:
            p = torch.softmax(F, 1)
            round_trees = []
            for k in range(classes):
                g, h = (p[:, k] - oh[:, k]), (p[:, k] * (1 - p[:, k])).clamp_min(1e-6)
                t = _Tree(max_depth, min_leaf, min_gain, l2, bins, colsample, gen).fit(B[rows], g[rows], h[rows])
                F[:, k] += learning_rate * t.predict_binned(B)
                round_trees.append(t)
            out_trees.append(round_trees)
        else:
            if classes == 2:
                p = torch.sigmoid(F)
                g, h = p - yf, (p * (1 - p)).clamp_min(1e-6)
            else:
                g, h = F - yf, torch.ones(n)
            t = _Tree(max_depth, min_leaf, min_gain, l2, bins, colsample, gen).fit(B[rows], g[rows], h[rows])
            F += learning_rate * t.predict_binned(B)
            out_trees.append(t)
        if progress is not None and (it + 1) % 10 == 0:
            progress.write(f"tree {it + 1}/{trees}\n")
    return Model(out_trees, edges, learning_rate, base, classes, "gbdt")


def decision_tree(X, y, max_depth=8, min_leaf=1, classes=0, **kw) -> Model:
    return gradient_boosting(X, y, trees=1, learning_rate=1.0, max_depth=max_depth, min_leaf=min_leaf, l2=0.0,
                             classes=classes, **kw)


def random_forest(X, y, trees=100, max_depth=10, min_leaf=1, colsample=None, bootstrap=True, classes=0, seed=0, bins=255) -> Model:
    """Bagged trees on bootstrap samples with per-node feature sampling; averages the trees."""
    X, y = torch.as_tensor(X).float(), torch.as_tensor(y).float()
    gen = torch.Generator().manual_seed(seed)
    B, edges = _bin(X, bins)
    n, F = X.shape
    colsample = colsample or (math.sqrt(F) / F if classes else 1.0 / 3 if F >= 3 else 1.0)
    out = []
    for _ in range(trees):
        rows = torch.randint(0, n, (n,), generator=gen) if bootstrap else torch.arange(n)
        t = _Tree(max_depth, min_leaf, 0.0, 0.0, bins, colsample, gen).fit(B[rows], -y[rows], torch.ones(n))
        out.append(t)
    m = Model(out, edges, 1.0, 0.0, 0, "forest")
    m.forest_classes = classes
    return m


class IsolationForestModel:
    def __init__(self, trees, sample):
        self.trees, self.sample = trees, sample

    def score(self, X):
        """Anomaly score in (0, 1): higher = more isolated."""
        X = torch.as_tensor(X).float()
        depth = torch.zeros(X.shape[0])
        for t in self.trees:
            depth += self._path(t, X)
        c = 2 * (math.log(self.sample - 1) + 0.5772156649) - 2 * (self.sample - 1) / self.sample if self.sample > 2 else 1.0
        return torch.pow(2.0, -(depth / len(self.trees)) / c)

    @staticmethod
    def _path(tree, X):
        out = torch.zeros(X.shape[0])
        stack = [(0, torch.arange(X.shape[0]), 0)]
        while stack:
            node, idx, d = stack.pop()
            f, thr, l, r, size = tree[node]
            if f < 0 or idx.numel() == 0:
                extra = 2 * (math.log(size - 1) + 0.5772156649) - 2 * (size - 1) / size if size > 2 else (1.0 if size == 2 else 0.0)
                out[idx] = d + extra
                continue
            left = X[idx, f] < thr
            stack.append((l, idx[left], d + 1))
            stack.append((r, idx[~left], d + 1))
        return out


def isolation_forest(X, trees=100, samples=256, seed=0) -> IsolationForestModel:
    X = torch.as_tensor(X).float()
    gen = torch.Generator().manual_seed(seed)
    n = X.shape[0]
    samples = min(samples, n)
    limit = math.ceil(math.log2(max(samples, 2)))
    forest = []
    for _ in range(trees):
        rows = torch.randperm(n, generator=gen)[:samples]
        nodes = []

        def grow(idx, depth):
            me = len(nodes)
            nodes.append([-1, 0.0, -1, -1, idx.numel()])
            if depth >= limit or idx.numel() <= 1:
                return me
            f = int(torch.randint(0, X.shape[1], (1,), generator=gen))
            lo, hi = X[idx, f].min().item(), X[idx, f].max().item()
            if hi <= lo:
                return me
            thr = lo + (hi - lo) * float(torch.rand(1, generator=gen))
            left = X[idx, f] < thr
            nodes[me][0], nodes[me][1] = f, thr
            nodes[me][2] = grow(idx[left], depth + 1)
            nodes[me][3] = grow(idx[~left], depth + 1)
            return me
        grow(rows, 0)
        forest.append(nodes)
    return IsolationForestModel(forest, samples)
