"""k-nearest neighbours, naive Bayes, k-means / DBSCAN, PCA (reference: neighbors/, bayes/,
cluster/, decomp/).  Distances are one GEMM plus two norms, so they run on the tensor
cores when the data is on the GPU."""
from __future__ import annotations

import torch


def pairwise_sq(A, B):
    """Squared Euclidean distances ``[rows of A, rows of B]`` as ONE matrix product: the rows are extended to
    ``[a, |a|^2, 1]`` and ``[-2 b, 1, |b|^2]``, so the result is written once instead of being built from
    three full-size temporaries."""
    a2, b2 = (A * A).sum(1, keepdim=True), (B * B).sum(1, keepdim=True)
    one_a, one_b = torch.ones_like(a2), torch.ones_like(b2)
    return torch.cat([A, a2, one_a], 1) @ torch.cat([B * -2.0, one_b, b2], 1).t()


class KNN:
    def __init__(self, X, y, k=5, classes=0):
        self.X, self.y, self.k, self.classes = torch.as_tensor(X).float(), torch.as_tensor(y), k, classes

    def kneighbors(self, Q):
        d = pairwise_sq(torch.as_tensor(Q).float(), self.X)
        return torch.topk(d, self.k, dim=1, largest=False)

    def predict(self, Q):
        _, idx = self.kneighbors(Q)
        yn = self.y[idx]
        if self.classes:
            return torch.nn.functional.one_hot(yn.long(), self.classes).float().mean(1)
        return yn.float().mean(1)

    def classify(self, Q):
        return self.predict(Q).argmax(1)


class GaussianNB:
    def __init__(self, X, y, classes, smoothing=1e-9):
        X, y = torch.as_tensor(X).float(), torch.as_tensor(y).long()
        self.mu = torch.stack([X[y == c].mean(0) for c in range(classes)])
        self.var = torch.stack([X[y == c].var(0, unbiased=False) for c in range(classes)]) + smoothing * X.var(0).max()
        self.prior = torch.bincount(y, minlength=classes).float().div(len(y)).log()

    def log_prob(self, X):
        X = torch.as_tensor(X).float()[:, None]
        return self.prior - 0.5 * (torch.log(2 * torch.pi * self.var) + (X - self.mu) ** 2 / self.var).sum(-1)

    def predict(self, X):
        return torch.softmax(self.log_prob(X), 1)

    def classify(self, X):
        return self.log_prob(X).argmax(1)


class MultinomialNB:
    def __init__(self, X, y, classes, alpha=1.0):
        X, y = torch.as_tensor(X).float(), torch.as_tensor(y).long()
        cnt = torch.stack([X[y == c].sum(0) for c in range(classes)]) + alpha
        self.logp = (cnt / cnt.sum(1, keepdim=True)).log()
        self.prior = torch.bincount(y, minlength=classes).float().div(len(y)).log()

    def classify(self, X):
        return (torch.as_tensor(X).float() @ self.logp.t() + self.prior).argmax(1)


class KMeansModel:
    def __init__(self, centers, inertia):
        self.centers, self.inertia = centers, inertia

    def assign(self, X):
        return pairwise_sq(torch.as_tensor(X).float(), self.centers).argmin(1)


def kmeans(X, k, iters=100, seed=0, tol=1e-6) -> KMeansModel:
    """k-means++ seeding, Lloyd iterations."""
    X = torch.as_tensor(X).float()
    g = torch.Generator().manual_seed(seed)
    centers = X[torch.randint(0, len(X), (1,), generator=g)]
    for _ in range(1, k):
        d = pairwise_sq(X, centers).min(1).values.clamp_min(0)
        centers = torch.cat([centers, X[torch.multinomial(d / d.sum(), 1, generator=g)]])
    for _ in range(iters):
        a = pairwise_sq(X, centers).argmin(1)
        new = torch.zeros_like(centers).index_add_(0, a, X)
        cnt = torch.bincount(a, minlength=k).clamp_min(1)[:, None]
        new = new / cnt
        moved = (new - centers).abs().max()
        centers = new
        if moved < tol:
            break
    d = pairwise_sq(X, centers).min(1).values
    return KMeansModel(centers, float(d.sum()))


def dbscan(X, eps, min_samples=5):
    """Labels in [0, n_clusters) with -1 = noise."""
    X = torch.as_tensor(X).float()
    near = pairwise_sq(X, X) <= eps * eps
    core = near.sum(1) >= min_samples
    labels = torch.full((len(X),), -1, dtype=torch.long)
    c = 0
    for i in range(len(X)):
        if labels[i] >= 0 or not core[i]:
            continue
        frontier = torch.zeros(len(X), dtype=torch.bool)
        frontier[i] = True
        member = frontier.clone()
        while frontier.any():
            reach = near[frontier & core].any(0) & ~member
            member |= reach
            frontier = reach
        labels[member & (labels < 0)] = c
        c += 1
    return labels


class PCAModel:
    def __init__(self, mean, components, variance):
        self.mean, self.components, self.variance = mean, components, variance

    def transform(self, X):
        return (torch.as_tensor(X).float() - self.mean) @ self.components.t()

    def inverse(self, Z):
        return Z @ self.components + self.mean


def pca(X, k) -> PCAModel:
    X = torch.as_tensor(X).float()
    mu = X.mean(0)
    _, S, Vt = torch.linalg.svd(X - mu, full_matrices=False)
    return PCAModel(mu, Vt[:k], (S[:k] ** 2) / (len(X) - 1))


class GMMModel:
    def __init__(self, weights, means, covs):
        self.weights, self.means, self.covs = weights, means, covs

    def log_prob(self, X):
        """[n, k] log of weight_k * N(x | mean_k, cov_k)."""
        X = torch.as_tensor(X).float()
        d = torch.distributions.MultivariateNormal(self.means, covariance_matrix=self.covs)
        return d.log_prob(X[:, None, :]) + self.weights.log()

    def predict(self, X):
        return torch.softmax(self.log_prob(X), 1)

    def assign(self, X):
        return self.log_prob(X).argmax(1)

    def score(self, X):
        return float(torch.logsumexp(self.log_prob(X), 1).mean())


def gmm(X, k, iters=100, seed=0, tol=1e-5, reg=1e-6) -> GMMModel:
    """Full-covariance Gaussian mixture by expectation-maximisation, seeded with k-means."""
    X = torch.as_tensor(X).float()
    n, d = X.shape
    km = kmeans(X, k, seed=seed)
    a = km.assign(X)
    means = km.centers.clone()
    weights = torch.bincount(a, minlength=k).float().clamp_min(1) / n
    covs = torch.stack([torch.cov(X[a == j].t()) + reg * torch.eye(d) if (a == j).sum() > d else torch.eye(d) for j in range(k)])
    last = -float("inf")
    for _ in range(iters):
        model = GMMModel(weights, means, covs)
        lp = model.log_prob(X)
        ll = float(torch.logsumexp(lp, 1).mean())
        r = torch.softmax(lp, 1)                                  # responsibilities
        nk = r.sum(0).clamp_min(1e-8)
        weights = nk / n
        means = (r.t() @ X) / nk[:, None]
        diff = X[:, None, :] - means[None]
        covs = torch.einsum("nk,nki,nkj->kij", r, diff, diff) / nk[:, None, None] + reg * torch.eye(d)
        if abs(ll - last) < tol:
            break
        last = ll
    return GMMModel(weights, means, covs)


def ward(X, k):
    """Agglomerative clustering with Ward's minimum-variance linkage (Lance-Williams update); labels [n]."""
    X = torch.as_tensor(X).double()
    n = X.shape[0]
    D = pairwise_sq(X, X).clamp_min(0)      # squared Euclidean = Ward distance between singletons (times 1/2)
    D.fill_diagonal_(float("inf"))
    size = torch.ones(n, dtype=torch.double)
    alive = torch.ones(n, dtype=torch.bool)
    label = torch.arange(n)
    for _ in range(n - k):
        flat = int(D.argmin())
        i, j = flat // n, flat % n
        if i > j:
            i, j = j, i
        ni, nj = size[i], size[j]
        others = alive.clone()
        others[i] = others[j] = False
        nk = size[others]
        new = ((ni + nk) * D[i, others] + (nj + nk) * D[j, others] - nk * D[i, j]) / (ni + nj + nk)
        D[i, others] = new
        D[others, i] = new
        D[j, :] = float("inf")
        D[:, j] = float("inf")
        alive[j] = False
        size[i] = ni + nj
        label[label == label[j]] = label[i]
    _, out = torch.unique(label, return_inverse=True)
    return out


# ---------------------------------------------------------------------------------------------
# k nearest neighbours over a table (reference: neighbors/neighbors.go)
# ---------------------------------------------------------------------------------------------
from .base import CLASSIFICATION, REGRESSION, Model, Standard, as_rows, as_task, count_classes  # noqa: E402

EUCLIDEAN, MANHATTAN, COSINE = "euclidean", "manhattan", "cosine"
METRICS = (EUCLIDEAN, MANHATTAN, COSINE)


def distances(metric: str, Q: torch.Tensor, R: torch.Tensor) -> torch.Tensor:
    """``[queries, rows]`` distances: Euclidean and cosine are one matrix product plus norms; Manhattan
    sums absolute differences in blocks of queries."""
    if metric == EUCLIDEAN:
        return pairwise_sq(Q, R).clamp_min(0).sqrt()
    if metric == COSINE:
        qn = Q / Q.norm(dim=1, keepdim=True).clamp_min(1e-12)
        rn = R / R.norm(dim=1, keepdim=True).clamp_min(1e-12)
        return (1.0 - qn @ rn.t()).clamp_min(0)
    if metric == MANHATTAN:
        block = max(1, (1 << 24) // max(R.numel(), 1))
        return torch.cat([(Q[i:i + block, None, :] - R[None]).abs().sum(-1) for i in range(0, Q.shape[0], block)]) \
            if Q.shape[0] else torch.zeros(0, R.shape[0])
    raise ValueError(f"unknown metric {metric!r}: want one of {METRICS}")


def _smallest(D, k: int, group: int = 64):
    """The ``k`` smallest of each row of ``D`` with their columns, smallest first.  Wide rows are searched in
    two steps: the minimum of every group of 64 columns (one vectorised pass), then only the ``k`` groups
    with the smallest minima, which must hold the ``k`` smallest values (the k-th smallest value cannot
    exceed the k-th smallest group minimum)."""
    q, n = D.shape
    if n <= 8192 or k * group >= n:
        return torch.topk(D, k, dim=1, largest=False)
    full = n // group * group
    mins = D[:, :full].reshape(q, -1, group).amin(2)
    tail = D[:, full:]
    groups = torch.topk(mins, k, dim=1, largest=False).indices                    # [q, k]
    cols = (groups[:, :, None] * group + torch.arange(group)[None, None]).reshape(q, -1)
    cand, cand_cols = D.gather(1, cols), cols
    if tail.shape[1]:
        cand = torch.cat([cand, tail], 1)
        cand_cols = torch.cat([cols, torch.arange(full, n).expand(q, -1)], 1)
    d, j = torch.topk(cand, k, dim=1, largest=False)
    return d, cand_cols.gather(1, j)


class Neighbors(Model):
    """The kept rows (standardized unless ``raw``) and their answers.  ``predict`` gives ``classes``
    probabilities per row (the neighbours' votes, weighted by inverse distance with ``by_distance``) or
    the neighbours' mean answer for regression."""

    FIELDS = ("task", "features", "classes", "k", "by_distance", "metric", "rows", "answers", "standard")

    def neighbors(self, X):
        """For each row of ``X`` its ``k`` nearest kept rows: ``(index [q, k], distance [q, k])``, nearest first."""
        Q = self.standard.apply(as_rows(X, self.features))
        k = min(self.k, self.rows.shape[0])
        # tiles of 256 queries by 4096 kept rows stay in cache: each tile is one small matrix product and gives
        # its k nearest; the candidates of a query block are merged at the end.  Euclidean neighbours are
        # chosen on squared distances and only the chosen take a square root.
        n = self.rows.shape[0]
        qb, rb = 256, (4096 if n > 32768 else max(n, 1))
        ext = None
        if self.metric == EUCLIDEAN:
            ext = getattr(self, "_ext", None)
            if ext is None or ext.shape[0] != n:
                r2 = (self.rows * self.rows).sum(1, keepdim=True)
                ext = self._ext = torch.cat([self.rows * -2.0, torch.ones_like(r2), r2], 1).contiguous()
        ds, ids = [], []
        for s in range(0, Q.shape[0], qb):
            q = Q[s:s + qb]
            if ext is not None:
                q2 = (q * q).sum(1, keepdim=True)
                q = torch.cat([q, q2, torch.ones_like(q2)], 1)
            cd, ci = [], []
            for r in range(0, n, rb):
                tile = q @ ext[r:r + rb].t() if ext is not None else distances(self.metric, q, self.rows[r:r + rb])
                d, i = _smallest(tile, min(k, tile.shape[1]))
                cd.append(d)
                ci.append(i + r)
            d, i = torch.cat(cd, 1), torch.cat(ci, 1)
            if d.shape[1] > k:
                d, j = torch.topk(d, k, dim=1, largest=False)
                i = i.gather(1, j)
            ds.append(d.clamp_min(0).sqrt() if ext is not None else d)
            ids.append(i)
        if not ds:
            return torch.zeros(0, k, dtype=torch.long), torch.zeros(0, k)
        return torch.cat(ids), torch.cat(ds)

    def predict(self, X) -> torch.Tensor:
        i, d = self.neighbors(X)
        if self.by_distance:
            w = 1.0 / d.clamp_min(1e-12)
            exact = d <= 1e-12                    # a row at distance zero answers alone, with its twins
            w = torch.where(exact.any(1, keepdim=True), exact.float(), w)
        else:
            w = torch.ones_like(d)
        ans = self.answers[i]
        if self.task is REGRESSION:
            return (w * ans.float()).sum(1) / w.sum(1)
        votes = torch.zeros(i.shape[0], self.classes).scatter_add_(1, ans.long(), w)
        return votes / votes.sum(1, keepdim=True)

    def module(self):
        from .modules import NeighborsModule
        return NeighborsModule.of(self)


def fit(d, task, k: int = 5, by_distance: bool = False, metric: str = EUCLIDEAN, raw: bool = False, classes: int = 0) -> Neighbors:
    task = as_task(task)
    d.check(task)
    if k < 1 or metric not in METRICS:
        raise ValueError(f"neighbors: k must be at least 1 and the metric one of {METRICS}")
    m = Neighbors()
    m.task, m.features, m.k, m.by_distance, m.metric = task, d.n_features, int(k), bool(by_distance), metric
    m.standard = Standard.fit(d.X, raw=raw)
    m.rows = m.standard.apply(d.X)
    m.classes = count_classes(d.Y, classes) if task is CLASSIFICATION else 0
    m.answers = d.Y.long() if task is CLASSIFICATION else d.Y.float()
    return m
