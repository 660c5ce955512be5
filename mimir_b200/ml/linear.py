"""Linear models (reference: linear/, logistic/, svm/): ridge (closed form on the normal
equations), lasso / elastic net (coordinate descent), logistic and softmax regression
(full-batch L-BFGS on the device of the data), linear SVM (squared hinge)."""
from __future__ import annotations

import torch


class LinearModel:
    def __init__(self, w, b):
        self.w, self.b = w, b

    def predict(self, X):
        return torch.as_tensor(X).to(self.w) @ self.w + self.b


def ridge(X, y, l2: float = 0.0) -> LinearModel:
    X, y = torch.as_tensor(X).double(), torch.as_tensor(y).double()
    mu, ym = X.mean(0), y.mean(0)
    Xc = X - mu
    A = Xc.t() @ Xc + l2 * torch.eye(X.shape[1], dtype=X.dtype, device=X.device)
    w = torch.linalg.lstsq(A, (Xc.t() @ (y - ym)).unsqueeze(-1) if y.dim() == 1 else Xc.t() @ (y - ym), driver='gelsd').solution
    w = w.squeeze(-1) if y.dim() == 1 else w
    return LinearModel(w.float(), (ym - mu @ w).float())


def elastic_net(X, y, l1: float = 0.0, l2: float = 0.0, iters: int = 200, tol: float = 1e-7) -> LinearModel:
    """Coordinate descent on 1/(2n)||y - Xw - b||^2 + l1 |w|_1 + l2/2 |w|^2."""
    X, y = torch.as_tensor(X).double(), torch.as_tensor(y).double()
    n, F = X.shape
    mu, ym = X.mean(0), y.mean()
    Xc, yc = X - mu, y - ym
    sq = (Xc ** 2).sum(0) / n
    w = torch.zeros(F, dtype=X.dtype)
    r = yc.clone()
    for _ in range(iters):
        delta = 0.0
        for j in range(F):
            if sq[j] == 0:
                continue
            rho = (Xc[:, j] @ r) / n + sq[j] * w[j]
            new = torch.sign(rho) * torch.clamp(rho.abs() - l1, min=0) / (sq[j] + l2)
            if new != w[j]:
                r -= Xc[:, j] * (new - w[j])
                delta = max(delta, float((new - w[j]).abs()))
                w[j] = new
        if delta < tol:
            break
    return LinearModel(w.float(), (ym - mu @ w).float())


def lasso(X, y, l1: float, **kw) -> LinearModel:
    return elastic_net(X, y, l1=l1, l2=0.0, **kw)


class LogisticModel:
    def __init__(self, W, b):
        self.W, self.b = W, b

    def predict(self, X):
        z = torch.as_tensor(X).to(self.W) @ self.W + self.b
        return torch.sigmoid(z.squeeze(-1)) if self.W.shape[1] == 1 else torch.softmax(z, -1)

    def classify(self, X):
        p = self.predict(X)
        return (p > 0.5).long() if p.dim() == 1 else p.argmax(-1)


def logistic(X, y, classes: int = 2, l2: float = 1e-4, iters: int = 100) -> LogisticModel:
    X, y = torch.as_tensor(X).float(), torch.as_tensor(y)
    k = 1 if classes == 2 else classes
    W = torch.zeros(X.shape[1], k, device=X.device, requires_grad=True)
    b = torch.zeros(k, device=X.device, requires_grad=True)
    opt = torch.optim.LBFGS([W, b], max_iter=iters, line_search_fn="strong_wolfe")

    def closure():
        opt.zero_grad()
        z = X @ W + b
        loss = (torch.nn.functional.binary_cross_entropy_with_logits(z.squeeze(-1), y.float()) if k == 1
                else torch.nn.functional.cross_entropy(z, y.long())) + 0.5 * l2 * (W ** 2).sum()
        loss.backward()
        return loss
    opt.step(closure)
    return LogisticModel(W.detach(), b.detach())


class SVMModel(LinearModel):
    def classify(self, X):
        return (self.predict(X) > 0).long()


def linear_svm(X, y, c: float = 1.0, iters: int = 100) -> SVMModel:
    """Squared-hinge linear SVM; labels in {0, 1}."""
    X, t = torch.as_tensor(X).float(), torch.as_tensor(y).float() * 2 - 1
    w = torch.zeros(X.shape[1], requires_grad=True)
    b = torch.zeros((), requires_grad=True)
    opt = torch.optim.LBFGS([w, b], max_iter=iters, line_search_fn="strong_wolfe")

    def closure():
        opt.zero_grad()
        loss = 0.5 * (w ** 2).sum() + c * torch.clamp(1 - t * (X @ w + b), min=0).pow(2).mean()
        loss.backward()
        return loss
    opt.step(closure)
    return SVMModel(w.detach(), b.detach())


def fista_lasso(X, y, l1: float, iters: int = 500, tol: float = 1e-8) -> LinearModel:
    """Lasso by the accelerated proximal gradient method (FISTA) on centred data."""
    X, y = torch.as_tensor(X).double(), torch.as_tensor(y).double()
    n = X.shape[0]
    mu, ym = X.mean(0), y.mean()
    Xc, yc = X - mu, y - ym
    L = float(torch.linalg.matrix_norm(Xc, 2) ** 2 / n)          # Lipschitz constant of the smooth part
    w = torch.zeros(X.shape[1], dtype=X.dtype)
    z, t = w.clone(), 1.0
    for _ in range(iters):
        grad = Xc.t() @ (Xc @ z - yc) / n
        u = z - grad / L
        new = torch.sign(u) * torch.clamp(u.abs() - l1 / L, min=0)
        t_new = (1 + (1 + 4 * t * t) ** 0.5) / 2
        z = new + (t - 1) / t_new * (new - w)
        done = float((new - w).abs().max()) < tol
        w, t = new, t_new
        if done:
            break
    return LinearModel(w.float(), (ym - mu @ w).float())


class KernelSVM:
    """C-SVM with an RBF or linear kernel trained by sequential minimal optimisation (Platt's
    simplified SMO with the maximal-violating-pair choice); labels in {0, 1}."""

    def __init__(self, c: float = 1.0, kernel: str = "rbf", gamma: float | None = None, tol: float = 1e-3, max_iter: int = 20000):
        self.c, self.kernel, self.gamma, self.tol, self.max_iter = c, kernel, gamma, tol, max_iter

    def _k(self, A, B):
        if self.kernel == "linear":
            return A @ B.t()
        d = (A * A).sum(1, keepdim=True) - 2 * A @ B.t() + (B * B).sum(1)[None]
        return torch.exp(-self.gamma * d.clamp_min(0))

    def fit(self, X, y):
        X = torch.as_tensor(X).double()
        t = torch.as_tensor(y).double() * 2 - 1
        n = X.shape[0]
        if self.gamma is None:
            self.gamma = 1.0 / (X.shape[1] * float(X.var()) + 1e-12)
        Kmat = self._k(X, X)
        alpha = torch.zeros(n, dtype=torch.double)
        g = -torch.ones(n, dtype=torch.double)           # gradient of the dual objective
        for _ in range(self.max_iter):
            up = ((t > 0) & (alpha < self.c)) | ((t < 0) & (alpha > 0))
            low = ((t > 0) & (alpha > 0)) | ((t < 0) & (alpha < self.c))
            score = -t * g
            i = int(torch.where(up, score, torch.full_like(score, -float("inf"))).argmax())
            j = int(torch.where(low, score, torch.full_like(score, float("inf"))).argmin())
            if score[i] - score[j] < self.tol:
                break
            eta = Kmat[i, i] + Kmat[j, j] - 2 * Kmat[i, j]
            step = (score[i] - score[j]) / max(float(eta), 1e-12)
            # keep both multipliers inside [0, C] along the feasible direction (t_i, -t_j)
            hi_i = (self.c - alpha[i]) if t[i] > 0 else alpha[i]
            hi_j = alpha[j] if t[j] > 0 else (self.c - alpha[j])
            step = min(float(step), float(hi_i), float(hi_j))
            alpha[i] += t[i] * step
            alpha[j] -= t[j] * step
            g += step * (Kmat[:, i] - Kmat[:, j]) * t
        sv = alpha > 1e-8
        self.sv, self.coef = X[sv], (alpha * t)[sv]
        free = sv & (alpha < self.c - 1e-8)
        idx = free if free.any() else sv
        self.b = float((t[idx] - (Kmat[idx][:, sv] @ self.coef)).mean()) if idx.any() else 0.0
        return self

    def decision(self, X):
        return (self._k(torch.as_tensor(X).double(), self.sv) @ self.coef + self.b).float()

    def classify(self, X):
        return (self.decision(X) > 0).long()
