"""Fitted classical models as ``nn.Module``s (reference: the ``module.go`` of tree/, linear/, svm/,
neighbors/, bayes/, cluster/ and recommend/).

A module trains nowhere but runs, saves and loads wherever a network does: its tables are buffers,
``forward`` maps ``x [batch, features]`` to ``[batch, classes]`` logits whose softmax is the model's
probabilities (``[batch, 1]`` values for regression) in lazy tensor ops, and ``Module.empty(shape)``
builds one with zero tables of the right sizes for saved weights to load into.  ``shape`` is the dict
of sizes that ``module.shape`` returns."""
from __future__ import annotations

import math

import torch

from .. import tensor as T
from ..nn.module import Module
from ..tensor.autograd import Buffer
from .base import CLASSIFICATION, REGRESSION

_TINY = 1e-30


def _buf(t, name):
    return Buffer(torch.as_tensor(t).clone(), name)


def _log_probs(p):
    """Logits whose softmax is ``p`` (rows of probabilities)."""
    return T.log(T.maximum(p, _TINY))


def _standardize(x, mean, scale):
    """``(x - mean) / scale`` with a missing value (NaN) as the mean."""
    z = (x - mean.value()) / scale.value()
    return T.where(T.equal(z, z), z, 0.0)


class _Tables(Module):
    """Shared plumbing: ``shape`` and ``empty``."""

    SIZES: tuple = ()

    @property
    def shape(self) -> dict:
        return dict(self._nn_skip_shape)

    @classmethod
    def empty(cls, shape: dict):
        return cls(**shape)


# ------------------------------------------------------------------ linear
class LinearModule(_Tables):
    def __init__(self, features: int, outputs: int, link: str):
        self._nn_skip_shape = dict(features=features, outputs=outputs, link=link)
        self.link = link
        self.weight, self.bias = _buf(torch.zeros(outputs, features), "weight"), _buf(torch.zeros(outputs), "bias")
        self.fill = _buf(torch.zeros(features), "fill")

    @classmethod
    def of(cls, m):
        mod = cls(m.features, int(m.weights.shape[0]), m.link)
        mod.weight.set(m.weights)
        mod.bias.set(m.bias)
        mod.fill.set(m.fill)
        return mod

    def forward(self, x):
        x = T.where(T.equal(x, x), x, self.fill.value())
        z = T.matmul_t(x, self.weight.value(), self.bias.value())
        if self.link == "sigmoid":                      # logits of [1 - p, p] are [0, z]
            return T.cat([z * 0.0, z], 1)
        return z


# ------------------------------------------------------------------ support vector machine
class SVMModule(_Tables):
    def __init__(self, features: int, outputs: int, support: int, kernel: str, gamma: float, coef0: float, degree: int,
                 classes: int, y_mean: float = 0.0, y_scale: float = 1.0):
        self._nn_skip_shape = dict(features=features, outputs=outputs, support=support, kernel=kernel, gamma=gamma, coef0=coef0,
                                   degree=degree, classes=classes, y_mean=y_mean, y_scale=y_scale)
        self.kernel, self.gamma, self.coef0, self.degree, self.classes = kernel, gamma, coef0, degree, classes
        self.y_mean, self.y_scale = y_mean, y_scale
        self.mean, self.scale = _buf(torch.zeros(features), "mean"), _buf(torch.ones(features), "scale")
        linear_classifier = kernel == "linear" and classes > 0
        self.support = _buf(torch.zeros(0 if linear_classifier else support, features), "support")
        self.coef = _buf(torch.zeros(outputs, features if linear_classifier else support), "coef")
        self.bias = _buf(torch.zeros(outputs), "bias")
        self.platt = _buf(torch.zeros(outputs if classes else 0, 2), "platt")

    @classmethod
    def of(cls, m):
        mod = cls(m.features, int(m.coef.shape[0]), m.support_vectors(), m.kernel, m.gamma, m.coef0, m.degree, m.classes,
                  float(m.y_mean), float(m.y_scale))
        mod.mean.set(m.standard.mean)
        mod.scale.set(m.standard.scale)
        mod.support.set(m.support.float())
        mod.coef.set(m.coef.float())
        mod.bias.set(m.bias.float())
        mod.platt.set(m.platt.float())
        return mod

    def forward(self, x):
        z = _standardize(x, self.mean, self.scale)
        if self.kernel == "linear" and self.classes > 0:
            f = T.matmul_t(z, self.coef.value(), self.bias.value())
        else:
            s = self.support.value()
            dot = T.matmul_t(z, s)
            if self.kernel == "rbf":
                d = T.sum_(z * z, 1, keepdim=True) - dot * 2.0 + T.unsqueeze(T.sum_(s * s, 1), 0)
                k = T.exp(T.maximum(d, 0.0) * -self.gamma)
            elif self.kernel == "polynomial":
                k = T.pow_(dot * self.gamma + self.coef0, float(self.degree))
            elif self.kernel == "sigmoid":
                k = T.tanh(dot * self.gamma + self.coef0)
            else:
                k = dot
            f = T.matmul_t(k, self.coef.value(), self.bias.value())
        if not self.classes:
            return f * self.y_scale + self.y_mean
        p = self.platt.value()
        a, b = T.shrink(p, ((0, p.shape[0]), (0, 1))), T.shrink(p, ((0, p.shape[0]), (1, 2)))
        g = T.neg(f * T.reshape(a, (1, -1)) + T.reshape(b, (1, -1)))          # log-odds of each output
        if self.classes == 2:
            return T.cat([g * 0.0, g], 1)
        return _log_probs(T.sigmoid(g))                                       # one against the rest, normalised by the softmax


# ------------------------------------------------------------------ nearest neighbours
class NeighborsModule(_Tables):
    def __init__(self, features: int, rows: int, k: int, classes: int, metric: str, by_distance: bool):
        self._nn_skip_shape = dict(features=features, rows=rows, k=k, classes=classes, metric=metric, by_distance=by_distance)
        self.k, self.classes, self.metric, self.by_distance = k, classes, metric, by_distance
        self.mean, self.scale = _buf(torch.zeros(features), "mean"), _buf(torch.ones(features), "scale")
        self.rows = _buf(torch.zeros(rows, features), "rows")
        self.answers = _buf(torch.zeros(rows, max(classes, 1)), "answers")      # one-hot classes, or the values

    @classmethod
    def of(cls, m):
        mod = cls(m.features, int(m.rows.shape[0]), m.k, m.classes, m.metric, m.by_distance)
        mod.mean.set(m.standard.mean)
        mod.scale.set(m.standard.scale)
        mod.rows.set(m.rows)
        mod.answers.set(torch.nn.functional.one_hot(m.answers, m.classes).float() if m.task is CLASSIFICATION
                        else m.answers.float()[:, None])
        return mod

    def forward(self, x):
        z, r = _standardize(x, self.mean, self.scale), self.rows.value()
        if self.metric == "cosine":
            zn = z / T.maximum(T.sqrt(T.sum_(z * z, 1, keepdim=True)), 1e-12)
            rn = r / T.maximum(T.sqrt(T.sum_(r * r, 1, keepdim=True)), 1e-12)
            dist = T.maximum(1.0 - T.matmul_t(zn, rn), 0.0)
        elif self.metric == "manhattan":
            dist = T.sum_(T.abs_(T.unsqueeze(z, 1) - T.unsqueeze(r, 0)), -1)
        else:
            d2 = T.sum_(z * z, 1, keepdim=True) - T.matmul_t(z, r) * 2.0 + T.unsqueeze(T.sum_(r * r, 1), 0)
            dist = T.sqrt(T.maximum(d2, 0.0))
        k = min(self.k, r.shape[0])
        near, idx = T.topk(dist, k, -1, False)
        if self.by_distance:
            exact = T.cast(T.less(near, 1e-12 + near * 0.0), T.float32)
            any_exact = T.max_(exact, 1, keepdim=True)
            w = T.where(T.less(any_exact * 0.0, any_exact), exact, T.recip(T.maximum(near, 1e-12)))
        else:
            w = near * 0.0 + 1.0
        width = self.answers.value().shape[1]
        ans = T.reshape(T.gather_rows(self.answers.value(), idx), (-1, k, width))
        votes = T.sum_(ans * T.unsqueeze(w, -1), 1) / T.sum_(w, 1, keepdim=True)
        return _log_probs(votes) if self.classes else votes


# ------------------------------------------------------------------ naive Bayes
class BayesModule(_Tables):
    def __init__(self, features: int, classes: int, kind: str, binarize: float = 0.0):
        self._nn_skip_shape = dict(features=features, classes=classes, kind=kind, binarize=binarize)
        self.kind, self.binarize = kind, binarize
        self.prior = _buf(torch.zeros(classes), "prior")
        self.square, self.linear, self.const = (_buf(torch.zeros(classes, features), n) for n in ("square", "linear", "const"))

    @classmethod
    def of(cls, m):
        mod = cls(m.features, m.classes, m.kind, m.binarize)
        for name in ("prior", "square", "linear", "const"):
            getattr(mod, name).set(getattr(m, name).float())
        return mod

    def forward(self, x):
        have = T.cast(T.equal(x, x), T.float32)
        v = T.where(T.equal(x, x), x, 0.0)
        if self.kind == "bernoulli":
            v = T.cast(T.less(v * 0.0 + self.binarize, v), T.float32)
        v = v * have
        return (T.matmul_t(v * v, self.square.value()) + T.matmul_t(v, self.linear.value()) + T.matmul_t(have, self.const.value())
                + self.prior.value())


# ------------------------------------------------------------------ groups (k-means, mixtures)
class GroupsModule(_Tables):
    """Logits whose largest is the row's group: for k-means minus half the squared standardized distance to
    each center; for a mixture each group's log-likelihood plus log weight."""

    def __init__(self, features: int, k: int, mixture: bool):
        self._nn_skip_shape = dict(features=features, k=k, mixture=mixture)
        self.mixture = mixture
        self.mean, self.scale = _buf(torch.zeros(features), "mean"), _buf(torch.ones(features), "scale")
        self.centers = _buf(torch.zeros(k, features), "centers")
        self.variances = _buf(torch.ones(k, features), "variances")
        self.log_weights = _buf(torch.zeros(k), "log_weights")

    @classmethod
    def of(cls, m):
        mixture = hasattr(m, "weights")
        mod = cls(m.features, m.k, mixture)
        mod.mean.set(m.standard.mean)
        mod.scale.set(m.standard.scale)
        mod.centers.set(m.means if mixture else m.centers)
        if mixture:
            mod.variances.set(m.variances)
            mod.log_weights.set(m.weights.log())
        return mod

    def forward(self, x):
        z = _standardize(x, self.mean, self.scale)
        c, v = self.centers.value(), self.variances.value()
        inv = T.recip(v)
        quad = T.matmul_t(z * z, inv) - T.matmul_t(z, c * inv) * 2.0 + T.unsqueeze(T.sum_(c * c * inv, 1), 0)
        out = quad * -0.5
        if self.mixture:
            out = out - T.unsqueeze(T.sum_(T.log(v * (2 * math.pi)), 1), 0) * 0.5 + self.log_weights.value()
        return out


# ------------------------------------------------------------------ recommendation
class FactorsModule(_Tables):
    """``forward(pairs [batch, 2] of (user, item) indices) -> [batch, 1]`` scores."""

    def __init__(self, users: int, items: int, factors: int, mean: float = 0.0):
        self._nn_skip_shape = dict(users=users, items=items, factors=factors, mean=mean)
        self.mean = mean
        self.user_factors, self.item_factors = _buf(torch.zeros(users, factors), "user_factors"), _buf(torch.zeros(items, factors), "item_factors")

    @classmethod
    def of(cls, m):
        mod = cls(m.users, m.items, m.factors, float(m.mean) if m.ratings else 0.0)
        mod.user_factors.set(m.user_factors)
        mod.item_factors.set(m.item_factors)
        return mod

    def forward(self, pairs):
        pairs = T.cast(pairs, T.int32) if pairs.dtype.is_floating_point else pairs
        n = pairs.shape[0]
        u = T.reshape(T.shrink(pairs, ((0, n), (0, 1))), (n,))
        i = T.reshape(T.shrink(pairs, ((0, n), (1, 2))), (n,))
        s = T.sum_(T.gather_rows(self.user_factors.value(), u) * T.gather_rows(self.item_factors.value(), i), 1, keepdim=True)
        return s + self.mean


# ------------------------------------------------------------------ trees
class TreeModule(_Tables):
    """Every tree is walked one level a step, every row and tree at once, by gathering the node's feature,
    threshold and children; a leaf leads to itself, so ``depth`` steps reach every leaf.  ``outputs`` trees
    per round add into each output."""

    def __init__(self, features: int, trees: int, nodes: int, depth: int, outputs: int, classes: int, scale: float = 1.0):
        self._nn_skip_shape = dict(features=features, trees=trees, nodes=nodes, depth=depth, outputs=outputs, classes=classes, scale=scale)
        self.depth, self.outputs, self.classes, self.scale = depth, outputs, classes, scale
        self.feature = _buf(torch.zeros(trees, nodes, dtype=torch.int64), "feature")
        self.threshold = _buf(torch.full((trees, nodes), math.inf), "threshold")
        self.left = _buf(torch.zeros(trees, nodes, dtype=torch.int64), "left")
        self.right = _buf(torch.zeros(trees, nodes, dtype=torch.int64), "right")
        self.value = _buf(torch.zeros(trees, nodes), "value")
        self.base = _buf(torch.zeros(outputs), "base")

    @classmethod
    def of(cls, m):
        """From a ``tree.Model`` (boosted trees, a forest or one tree)."""
        flat = [t for r in m.trees for t in (r if isinstance(r, list) else [r])]
        outputs = m.classes if m.classes > 2 else 1
        nodes = max(len(t.nodes) for t in flat)
        depth = max(t.max_depth for t in flat)
        forest = m.kind != "gbdt"
        scale = (1.0 / max(len(flat), 1)) if forest else float(m.lr)
        classes = getattr(m, "forest_classes", m.classes) if forest else m.classes
        mod = cls(int(m.edges.shape[0]), len(flat), nodes, depth, outputs, int(classes), scale)
        feat = torch.zeros(len(flat), nodes, dtype=torch.int64)
        thr = torch.full((len(flat), nodes), math.inf)
        left = torch.arange(nodes).repeat(len(flat), 1)
        right = left.clone()
        val = torch.zeros(len(flat), nodes)
        edges = m.edges
        for t, tr in enumerate(flat):
            for i, (f, b, l, r, v) in enumerate(tr.nodes):
                val[t, i] = v
                if f >= 0:
                    feat[t, i], left[t, i], right[t, i] = f, l, r
                    thr[t, i] = edges[f, b] if b < edges.shape[1] else math.inf
        for name, v in (("feature", feat), ("threshold", thr), ("left", left), ("right", right), ("value", val)):
            getattr(mod, name).set(v)
        mod.base.set(m.base.float() if torch.is_tensor(m.base) else torch.full((outputs,), float(m.base)))
        mod._nn_skip_forest = forest
        return mod

    def forward(self, x):
        """Only operations of the exported graph vocabulary are used (a table lookup is a row gather of the
        flattened table at ``tree * nodes + node``; a row's value of a node's feature is picked by comparing the
        feature number with 0..F-1), so the module exports like a network."""
        feat, thr, left, right, value = (b.value() for b in (self.feature, self.threshold, self.left, self.right, self.value))
        trees, nodes = feat.shape
        features = x.shape[1]
        dev = x.device
        flat = lambda t: T.reshape(t, (trees * nodes,))  # noqa: E731
        base = T.tensor(torch.arange(trees, dtype=torch.int64)[:, None] * nodes, device=dev)          # [trees, 1]
        which = T.tensor(torch.arange(features, dtype=torch.int64).reshape(1, 1, features), device=dev)
        xb = T.unsqueeze(x, 0)                                                                        # [1, n, F]
        # every row starts at the root of every tree: node 0
        zero_col = T.cast(T.unsqueeze(T.sum_(T.where(T.equal(x, x), x, 0.0), 1), 0) * 0.0, torch.int64)  # [1, n] zeros, batch-sized
        pos = base * 0 + zero_col                                                                     # [trees, n]
        for _ in range(self.depth):
            at = pos + base
            f = T.gather_rows(flat(feat), at)                                                         # [trees, n]
            picked = T.where(T.equal(T.unsqueeze(f, -1), which), xb, 0.0)                             # [trees, n, F]
            xv = T.sum_(picked, -1)
            missing = T.logical_not(T.equal(xv, xv))
            go_left = T.logical_and(T.logical_not(T.less(T.gather_rows(flat(thr), at), xv)), T.logical_not(missing))
            pos = T.where(go_left, T.gather_rows(flat(left), at), T.gather_rows(flat(right), at))
        leaf = T.gather_rows(flat(value), pos + base)                                                 # [trees, n]
        per_out = T.sum_(T.reshape(leaf, (trees // self.outputs, self.outputs, -1)), 0)               # rounds add up per output
        out = T.transpose(per_out, 0, 1) * self.scale + self.base.value()
        if self.classes == 2 and self.outputs == 1 and not getattr(self, "_nn_skip_forest", False):
            return T.cat([out * 0.0, out], 1)
        return out
