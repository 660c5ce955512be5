"""k-nearest neighbours, naive Bayes, k-means / DBSCAN, PCA (reference: neighbors/, bayes/,
cluster/, decomp/).  Distances are one GEMM plus two norms, so they run on the tensor
cores when the data is on the GPU."""
from __future__ import annotations

import torch


def pairwise_sq(A, B):
    return (A * A).sum(1, keepdim=True) - 2 * A @ B.t() + (B * B).sum(1)[None]


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
