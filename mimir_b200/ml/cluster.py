"""Groups in tables without answers (reference: cluster/): k-means, diagonal Gaussian mixtures,
DBSCAN, Ward's agglomerative hierarchy, and the silhouette that scores a grouping.

Every fit standardizes the features first and counts a missing value as the feature's mean.  Distances
are one matrix product plus two norms, so the heavy step of k-means, the mixture and the silhouette is
a GEMM.  ``Means`` and ``Mixture`` convert to an ``nn.Module`` whose logits' largest is the row's group."""
from __future__ import annotations

import math

import torch

from .base import Model, Standard, as_rows

NOISE = -1


def _sq(A, B):
    from .neighbors import pairwise_sq
    return pairwise_sq(A, B).clamp_min_(0)


def _table(X, features, what):
    X = as_rows(X, features)
    if X.shape[0] == 0 or X.shape[1] == 0 or torch.isinf(X).any():
        raise ValueError(f"{what}: a table of {X.shape[0]} rows and {X.shape[1]} features, or an infinite value")
    return X


# ------------------------------------------------------------------ k-means
class Means(Model):
    """Each row belongs to the nearest of ``k`` centers (kept in standardized units)."""

    FIELDS = ("features", "centers", "standard", "inertia")

    @property
    def k(self) -> int:
        return int(self.centers.shape[0])

    def assign(self, X) -> torch.Tensor:
        return _sq(self.standard.apply(as_rows(X, self.features)), self.centers).argmin(1)

    def predict(self, X) -> torch.Tensor:
        """``k`` numbers per row: 1 for its group, 0 for the others."""
        return torch.nn.functional.one_hot(self.assign(X), self.k).float()

    def module(self):
        from .modules import GroupsModule
        return GroupsModule.of(self)


def _extend(Z):
    """Rows as ``[z, |z|^2, 1]``: their squared distances to centers are then one product with ``_centers_ext``."""
    z2 = (Z * Z).sum(1, keepdim=True)
    return torch.cat([Z, z2, torch.ones_like(z2)], 1)


def _to_centers(Zx, C):
    """``[rows, k]`` squared distances of extended rows to the centers ``C``."""
    Cx = torch.cat([C * -2.0, torch.ones(C.shape[0], 1, dtype=C.dtype), (C * C).sum(1, keepdim=True)], 1)
    return (Zx @ Cx.t()).clamp_min_(0)


def _draw(weights, g):
    """One index with a chance in proportion to ``weights`` (a cumulative sum and a binary search)."""
    cum = torch.cumsum(weights.double(), 0)
    total = float(cum[-1])
    if not total > 0:
        return int(torch.randint(0, weights.numel(), (1,), generator=g))
    u = torch.rand(1, generator=g, dtype=torch.double) * total
    return min(int(torch.searchsorted(cum, u)), weights.numel() - 1)


def _plus_plus(Z, Zx, k, g):
    if Z.shape[0] > 100_000:
        pick = torch.randperm(Z.shape[0], generator=g)[:100_000]
        Z, Zx = Z[pick], Zx[pick]
    centers = Z[int(torch.randint(0, Z.shape[0], (1,), generator=g))][None]
    d = _to_centers(Zx, centers)[:, 0]
    for _ in range(1, k):
        nxt = Z[_draw(d, g)][None]
        centers = torch.cat([centers, nxt])
        d = torch.minimum(d, _to_centers(Zx, nxt)[:, 0])
    return centers


def _lloyd(Z, Zx, centers, max_iter, tol):
    k = centers.shape[0]
    for _ in range(max_iter):
        d = _to_centers(Zx, centers)
        a = d.argmin(1)
        onehot = torch.zeros(Z.shape[0], k, dtype=Z.dtype)
        onehot.scatter_(1, a[:, None], 1.0)
        cnt = onehot.sum(0)
        new = (onehot.t() @ Z) / cnt.clamp_min(1)[:, None]         # the sums of each group's rows as one product
        empty = cnt == 0
        if empty.any():
            # a center that lost every row restarts at the row farthest from its center
            far = d.min(1).values.topk(int(empty.sum())).indices
            new[empty] = Z[far]
        moved = float((new - centers).norm(dim=1).max())
        centers = new
        if moved <= tol:
            break
    d = _to_centers(Zx, centers)
    return centers, float(d.min(1).values.sum())


def kmeans_fit(X, k: int, features: int | None = None, inits: int = 4, max_iter: int = 300, tol: float = 1e-4, seed: int = 1) -> Means:
    """Lloyd's algorithm from ``inits`` k-means++ starts, keeping the grouping with the smallest sum of
    squared distances."""
    X = _table(X, features, "k-means")
    if k < 1 or k > X.shape[0] or inits < 1 or max_iter < 1 or tol < 0:
        raise ValueError(f"k-means: {k} groups of {X.shape[0]} rows, or a bad option")
    std = Standard.fit(X)
    Z = std.apply(X)
    g = torch.Generator().manual_seed(seed)
    Zx = _extend(Z)
    best = None
    for _ in range(inits):
        centers, inertia = _lloyd(Z, Zx, _plus_plus(Z, Zx, k, g), max_iter, tol)
        if best is None or inertia < best[1]:
            best = (centers, inertia)
    m = Means()
    m.features, m.centers, m.standard, m.inertia = X.shape[1], best[0], std, best[1]
    return m


# ------------------------------------------------------------------ Gaussian mixture
MIN_VAR = 1e-6


class Mixture(Model):
    """Each group is a normal distribution with its own mean and a variance per feature, and a weight
    (scikit-learn's ``GaussianMixture`` with ``covariance_type="diag"``)."""

    FIELDS = ("features", "weights", "means", "variances", "standard", "log_likelihood")

    @property
    def k(self) -> int:
        return int(self.weights.numel())

    def _log_joint(self, Z):
        """``[rows, k]``: log weight + log density of each group."""
        Z = Z.double()
        v = self.variances.double()
        quad = (Z * Z) @ (1 / v).t() - 2 * Z @ (self.means.double() / v).t() + (self.means.double() ** 2 / v).sum(1)
        return self.weights.double().log() - 0.5 * (quad + torch.log(2 * math.pi * v).sum(1))

    def probabilities(self, X) -> torch.Tensor:
        return torch.softmax(self._log_joint(self.standard.apply(as_rows(X, self.features))), 1).float()

    predict = probabilities

    def assign(self, X) -> torch.Tensor:
        return self._log_joint(self.standard.apply(as_rows(X, self.features))).argmax(1)

    def log_density(self, X) -> torch.Tensor:
        """The log-likelihood of each row in standardized units: low for rows unlike any group."""
        return torch.logsumexp(self._log_joint(self.standard.apply(as_rows(X, self.features))), 1)

    def module(self):
        from .modules import GroupsModule
        return GroupsModule.of(self)


def gaussian_mixture(X, k: int, features: int | None = None, max_iter: int = 300, tol: float = 1e-4, seed: int = 1, inits: int = 4) -> Mixture:
    """Expectation-maximization from a k-means grouping until the mean log-likelihood rises by less than ``tol``."""
    km = kmeans_fit(X, k, features, inits=inits, max_iter=max_iter, tol=tol, seed=seed)
    X = as_rows(X, features)
    Z = km.standard.apply(X).double()
    n = Z.shape[0]
    resp = torch.nn.functional.one_hot(_sq(Z.float(), km.centers).argmin(1), k).double()
    m = Mixture()
    m.features, m.standard = X.shape[1], km.standard
    last = -math.inf
    for _ in range(max_iter):
        nk = resp.sum(0).clamp_min(1e-12)
        m.weights = (nk / n).float()
        mean = (resp.t() @ Z) / nk[:, None]
        var = (resp.t() @ (Z * Z)) / nk[:, None] - mean * mean
        m.means, m.variances = mean.float(), (var.clamp_min(0) + MIN_VAR).float()
        lj = m._log_joint(Z)
        ll = float(torch.logsumexp(lj, 1).mean())
        resp = torch.softmax(lj, 1)
        if ll - last < tol:
            last = ll
            break
        last = ll
    m.log_likelihood = last
    return m


# ------------------------------------------------------------------ DBSCAN
class Density(Model):
    """Rows with at least ``min_rows`` rows within ``eps`` (themselves included) are cores; a group is the
    cores that reach one another and the rows they reach; the rest is ``NOISE``."""

    FIELDS = ("features", "eps", "min_rows", "labels", "cores", "core_labels", "standard")

    @property
    def groups(self) -> int:
        return int(self.labels.max()) + 1 if self.labels.numel() else 0

    def assign(self, X) -> torch.Tensor:
        """The group of the nearest core within ``eps`` of each row, or ``NOISE``."""
        Z = self.standard.apply(as_rows(X, self.features))
        if self.cores.shape[0] == 0:
            return torch.full((Z.shape[0],), NOISE, dtype=torch.long)
        d, i = _sq(Z, self.cores).min(1)
        return torch.where(d <= self.eps * self.eps, self.core_labels[i], torch.full_like(i, NOISE))


def dbscan_fit(X, eps: float, features: int | None = None, min_rows: int = 5, native: bool = True) -> Density:
    """``eps`` is in standardized units.  On the host the search is native code: rows are compared tile by tile,
    cores within reach of one another are joined as they are met, and nothing but the table is held in memory.
    ``native=False`` (and other devices) finds neighbours block by block of rows against the table (a GEMM each)
    and grows groups from each unvisited core by repeated frontier expansion: the same groups, the same numbers."""
    X = _table(X, features, "dbscan")
    if eps <= 0 or min_rows < 1:
        raise ValueError("dbscan: eps must be positive and min_rows at least 1")
    std = Standard.fit(X)
    Z = std.apply(X)
    n = Z.shape[0]
    if native and Z.device.type == "cpu" and n < 2 ** 31:
        # the whole search in native code: no list of neighbours is kept (``mimir_cpu_dbscan``)
        import ctypes
        from .. import _native
        lib = _native.lib()
        if not getattr(lib, "_dbscan_bound", False):
            lib.mimir_cpu_dbscan.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p,
                                             ctypes.c_void_p]
            lib.mimir_cpu_dbscan.restype = ctypes.c_longlong
            lib._dbscan_bound = True
        Zc = Z.float().contiguous()
        labels = torch.empty(n, dtype=torch.long)
        core8 = torch.empty(n, dtype=torch.uint8)
        if lib.mimir_cpu_dbscan(Zc.data_ptr(), n, Zc.shape[1], float(eps) * float(eps), int(min_rows), labels.data_ptr(), core8.data_ptr()) < 0:
            raise ValueError("dbscan: the native search refused its arguments")
        core = core8.bool()
        m = Density()
        m.features, m.eps, m.min_rows, m.labels, m.standard = X.shape[1], float(eps), int(min_rows), labels, std
        m.cores, m.core_labels = Z[core], labels[core]
        return m
    block = max(1, (1 << 25) // max(n, 1))
    near = []                                    # per row: indices within eps
    for s in range(0, n, block):
        hit = _sq(Z[s:s + block], Z) <= eps * eps
        near.extend(torch.nonzero(r, as_tuple=False)[:, 0] for r in hit)
    core = torch.tensor([len(r) >= min_rows for r in near])
    labels = torch.full((n,), NOISE, dtype=torch.long)
    group = 0
    for i in range(n):
        if labels[i] != NOISE or not core[i]:
            continue
        labels[i] = group
        frontier = [i]
        while frontier:
            reach = torch.unique(torch.cat([near[j] for j in frontier]))
            fresh = reach[labels[reach] == NOISE]
            labels[fresh] = group
            frontier = fresh[core[fresh]].tolist()
        group += 1
    m = Density()
    m.features, m.eps, m.min_rows, m.labels, m.standard = X.shape[1], float(eps), int(min_rows), labels, std
    m.cores, m.core_labels = Z[core], labels[core]
    return m


# ------------------------------------------------------------------ Ward's hierarchy
class Linkage(Model):
    """The hierarchy Ward's method builds over the training rows: ``merges[i] = (a, b)`` joins clusters a
    and b (rows are 0..n-1, merge i makes cluster n+i) at ``heights()[i]``.  It is cut into any number of
    groups afterwards; ``means`` holds the centers at the ``k`` it was fitted for."""

    FIELDS = ("features", "rows", "merges", "merge_heights", "means", "standard")

    @property
    def k(self) -> int:
        return self.means.k

    def heights(self) -> torch.Tensor:
        """The heights of the merges, rising; a large jump after the merge i from the end suggests i+1 groups."""
        return self.merge_heights.clone()

    def cut(self, k: int) -> torch.Tensor:
        """The group of each training row with the hierarchy cut into ``k`` groups (one when ``k`` is out of
        range), numbered by first row."""
        n = self.rows
        if k < 1 or k > n:
            k = 1
        parent = list(range(2 * n - 1))

        def find(x):
            while parent[x] != x:
                parent[x] = parent[parent[x]]
                x = parent[x]
            return x
        for i in range(n - k):
            a, b = int(self.merges[i, 0]), int(self.merges[i, 1])
            parent[find(a)] = n + i
            parent[find(b)] = n + i
        names, out = {}, torch.empty(n, dtype=torch.long)
        for r in range(n):
            out[r] = names.setdefault(find(r), len(names))
        return out

    def centers(self, X, k: int) -> Means:
        """The centers of the ``k`` groups the hierarchy of the training rows ``X`` cuts into, to assign new
        rows and to score the cut."""
        Z = self.standard.apply(as_rows(X, self.features))
        if Z.shape[0] != self.rows:
            raise ValueError(f"{Z.shape[0]} rows, the hierarchy was built over {self.rows}")
        lab = self.cut(k)
        kk = int(lab.max()) + 1
        c = torch.zeros(kk, Z.shape[1]).index_add_(0, lab, Z) / torch.bincount(lab, minlength=kk)[:, None]
        m = Means()
        m.features, m.centers, m.standard = self.features, c, self.standard
        m.inertia = float(_sq(Z, c).min(1).values.sum())
        return m

    def assign(self, X) -> torch.Tensor:
        return self.means.assign(X)


def agglomerative(X, k: int, features: int | None = None, native: bool = True) -> Linkage:
    """Ward's minimum-variance hierarchy by the nearest-neighbour chain algorithm.  The distance between clusters
    A and B is ``|A||B| / (|A| + |B|) |mean_A - mean_B|^2``.  On the host the chain runs in native code straight
    from the clusters' means: time grows with the square of the rows, memory with the rows.  ``native=False`` (and
    other devices) keeps an n x n matrix up to date by the Lance-Williams update: the same hierarchy up to
    rounding."""
    X = _table(X, features, "agglomerative")
    n = X.shape[0]
    if k < 1 or k > n:
        raise ValueError(f"agglomerative: {k} groups of {n} rows")
    std = Standard.fit(X)
    Z = std.apply(X).double()
    if native and Z.device.type == "cpu":
        # the chain in native code over the clusters' means, with no distance matrix (``mimir_cpu_ward_means``)
        import ctypes
        from .. import _native
        lib = _native.lib()
        if not getattr(lib, "_ward_bound", False):
            lib.mimir_cpu_ward_means.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
            lib._ward_bound = True
        Zc = Z.contiguous()
        pairs = torch.empty(max(n - 1, 0), 2, dtype=torch.long)
        hs = torch.empty(max(n - 1, 0), dtype=torch.double)
        if lib.mimir_cpu_ward_means(Zc.data_ptr(), n, Zc.shape[1], pairs.data_ptr(), hs.data_ptr()) != 0:
            raise ValueError("agglomerative: the native chain refused its arguments")
        return _linkage(X, std, k, [tuple(p) for p in pairs.tolist()], hs.tolist())
    D = 0.5 * _sq(Z, Z)                               # Ward distance between single rows
    D.fill_diagonal_(math.inf)
    size = torch.ones(n, dtype=torch.double)
    alive = torch.ones(n, dtype=torch.bool)
    name = list(range(n))                             # the cluster id held at each slot
    merges, heights, chain = [], [], []
    for step in range(n - 1):
        if not chain:
            chain.append(int(torch.nonzero(alive)[0]))
        while True:
            a = chain[-1]
            row = D[a]
            b = int(row.argmin())
            if len(chain) > 1 and row[chain[-2]] <= row[b]:
                b = chain[-2]                         # ties keep the previous link, so the chain ends
            if len(chain) > 1 and b == chain[-2]:
                break
            chain.append(b)
        a = chain.pop()
        b = chain.pop()
        h = float(D[a, b])
        merges.append((name[a], name[b]))
        heights.append(h)
        others = alive.clone()
        others[a] = others[b] = False
        sa, sb, so = size[a], size[b], size[others]
        D[a, others] = D[others, a] = ((sa + so) * D[a, others] + (sb + so) * D[b, others] - so * h) / (sa + sb + so)
        D[b, :] = math.inf
        D[:, b] = math.inf
        alive[b] = False
        size[a] = sa + sb
        name[a] = n + step
    return _linkage(X, std, k, merges, heights)


def _linkage(X, std, k, merges, heights) -> Linkage:
    """The hierarchy from the merges in the order the chain found them."""
    n = X.shape[0]
    order = sorted(range(n - 1), key=lambda i: heights[i])
    # reducible linkage: the chain finds merges out of height order; renumber them rising
    remap = {}
    sorted_merges = []
    for new, old in enumerate(order):
        remap[n + old] = n + new
    for old in order:
        a, b = merges[old]
        sorted_merges.append((remap.get(a, a), remap.get(b, b)))
    m = Linkage()
    m.features, m.rows, m.standard = X.shape[1], n, std
    m.merges = torch.tensor(sorted_merges, dtype=torch.long).reshape(-1, 2)
    m.merge_heights = torch.tensor([heights[i] for i in order], dtype=torch.double)
    m.means = None
    m.means = m.centers(X, k)
    return m


# ------------------------------------------------------------------ silhouette
SILHOUETTE_ROWS = 5000


def silhouette_of(Z, labels, seed: int = 1) -> float:
    """Mean silhouette of standardized rows ``Z`` in the groups ``labels``: for each row, how much nearer it is
    to its own group than to the next nearest, from -1 to 1.  Noise rows are left out; a row alone in its
    group scores 0; over 5,000 rows a seeded sample is scored."""
    labels = torch.as_tensor(labels).long()
    keep = labels != NOISE
    Z, labels = Z[keep], labels[keep]
    if Z.shape[0] > SILHOUETTE_ROWS:
        pick = torch.randperm(Z.shape[0], generator=torch.Generator().manual_seed(seed))[:SILHOUETTE_ROWS]
        Z, labels = Z[pick], labels[pick]
    if Z.shape[0] == 0:
        return 0.0
    _, labels = torch.unique(labels, return_inverse=True)
    k = int(labels.max()) + 1
    if k < 2:
        return 0.0
    D = _sq(Z, Z).sqrt()
    onehot = torch.nn.functional.one_hot(labels, k).to(D.dtype)
    sums, cnt = D @ onehot, onehot.sum(0)
    own = cnt[labels]
    a = sums.gather(1, labels[:, None])[:, 0] / (own - 1).clamp_min(1)
    other = sums / cnt.clamp_min(1)
    other.scatter_(1, labels[:, None], math.inf)
    b = other.min(1).values
    s = torch.where(own > 1, (b - a) / torch.maximum(a, b).clamp_min(1e-300), torch.zeros_like(a))
    return float(s.mean())


def silhouette(model, X, seed: int = 1) -> float:
    """The silhouette of the rows of ``X`` in the groups ``model`` (``Means``, ``Mixture``, ``Density`` or
    ``Linkage``) assigns them."""
    Z = model.standard.apply(as_rows(X, model.features))
    return silhouette_of(Z, model.assign(X), seed)
