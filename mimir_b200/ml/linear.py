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


# ---------------------------------------------------------------------------------------------
# Fitted linear models over a table (reference: linear/linear.go, linear/fit.go, linear/lbfgs.go)
# ---------------------------------------------------------------------------------------------
from .base import CLASSIFICATION, REGRESSION, Model, Standard, as_rows, count_classes  # noqa: E402


class Linear(Model):
    """For each output a weight per feature and a bias, in the features' own units, passed through
    ``link`` ("identity", "sigmoid" for two classes, "softmax" for more).  ``predict`` returns one value
    per row for regression and ``classes`` probabilities per row for classification."""

    FIELDS = ("task", "features", "classes", "weights", "bias", "link", "fill")

    def weight(self, o: int, j: int) -> float:
        return float(self.weights[o, j])

    def decision(self, X) -> torch.Tensor:
        X = as_rows(X, self.features)
        X = torch.where(torch.isnan(X), self.fill.to(X), X) if torch.isnan(X).any() else X
        return X @ self.weights.t().to(X) + self.bias.to(X)

    def predict(self, X) -> torch.Tensor:
        z = self.decision(X)
        if self.link == "identity":
            return z[:, 0]
        if self.link == "sigmoid":
            p = torch.sigmoid(z[:, 0])
            return torch.stack([1 - p, p], 1)
        return torch.softmax(z, 1)

    def module(self):
        from .modules import LinearModule
        return LinearModule.of(self)


def _unscale(w_std, b_std, std: Standard):
    """Weights of standardized features as weights of the features themselves."""
    w = w_std / std.scale.double()
    return w.float(), (b_std - w @ std.mean.double()).float()


def _native_cd(G, c, l1, l2, tol, max_iter, w) -> bool:
    """Coordinate descent on the Gram matrix in native code; False when the library is missing."""
    import ctypes
    from .. import _native
    if not _native.available():
        return False
    lib = _native.lib()
    if not getattr(lib, "_cd_bound", False):
        lib.mimir_cpu_elastic_cd.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_double, ctypes.c_double,
                                             ctypes.c_double, ctypes.c_int, ctypes.c_void_p]
        lib.mimir_cpu_elastic_cd.restype = ctypes.c_int
        lib._cd_bound = True
    Gc, cc = G.contiguous(), c.contiguous()
    return lib.mimir_cpu_elastic_cd(Gc.data_ptr(), cc.data_ptr(), Gc.shape[0], float(l1), float(l2), float(tol), int(max_iter), w.data_ptr()) >= 0


def regression(d, l1: float = 0.0, l2: float = 0.0, max_iter: int = 1000, tol: float = 1e-6) -> Linear:
    """Least squares with optional lasso (``l1``) and ridge (``l2``) penalties on standardized features:
    ``1/(2n) |y - Xw - b|^2 + l1 |w|_1 + l2/2 |w|^2``.  Without ``l1`` the normal equations are solved
    directly; with it, coordinate descent runs on the Gram matrix until a pass changes no weight by more
    than ``tol``."""
    d.check(REGRESSION)
    if l1 < 0 or l2 < 0 or max_iter < 1 or tol < 0:
        raise ValueError("penalties, passes and tolerance must not be negative")
    std = Standard.fit(d.X)
    Z = std.apply(d.X).double()
    y = d.Y.double()
    n, F = Z.shape
    ym = y.mean()
    G, c = Z.t() @ Z / n, Z.t() @ (y - ym) / n
    if l1 == 0:
        A = G + l2 * torch.eye(F, dtype=torch.double)
        w = torch.linalg.lstsq(A, c.unsqueeze(1)).solution[:, 0] if l2 == 0 else torch.linalg.solve(A, c)
    else:
        w = torch.zeros(F, dtype=torch.double)
        diag = G.diagonal()
        for _ in range(0 if _native_cd(G, c, l1, l2, tol, max_iter, w) else max_iter):
            moved = 0.0
            for j in range(F):
                if diag[j] <= 0:
                    continue
                rho = float(c[j] - G[j] @ w + diag[j] * w[j])
                new = (abs(rho) - l1) / float(diag[j] + l2)
                new = 0.0 if new <= 0 else (new if rho > 0 else -new)
                moved = max(moved, abs(new - float(w[j])))
                w[j] = new
            if moved <= tol:
                break
    wt, b = _unscale(w.unsqueeze(0), ym.unsqueeze(0), std)
    m = Linear()
    m.task, m.features, m.classes, m.weights, m.bias, m.link, m.fill = REGRESSION, F, 0, wt, b, "identity", std.mean
    return m


def _lbfgs(f, x0, max_iter, tol, history=10):
    """Limited-memory BFGS with a backtracking Armijo line search; ``f(x) -> (value, gradient)``.  Stops
    once no part of the gradient exceeds ``tol``."""
    x = x0.clone()
    fx, g = f(x)
    S, Y = [], []
    for _ in range(max_iter):
        if float(g.abs().max()) <= tol:
            break
        q = g.clone()
        alphas = []
        for s, yv in zip(reversed(S), reversed(Y)):
            a = (s @ q) / (yv @ s)
            alphas.append(a)
            q -= a * yv
        if S:
            q *= (S[-1] @ Y[-1]) / (Y[-1] @ Y[-1])
        for (s, yv), a in zip(zip(S, Y), reversed(alphas)):
            q += (a - (yv @ q) / (yv @ s)) * s
        p = -q
        slope = float(g @ p)
        if slope >= 0:                      # not a descent direction: restart from the gradient
            p, slope, S, Y = -g, -float(g @ g), [], []
        step, ok = 1.0 if S else min(1.0, 1.0 / max(float(g.norm()), 1e-12)), False
        for _ in range(40):
            xn = x + step * p
            fn, gn = f(xn)
            if float(fn) <= float(fx) + 1e-4 * step * slope:
                ok = True
                break
            step *= 0.5
        if not ok:
            break
        s, yv = xn - x, gn - g
        if float(s @ yv) > 1e-12:
            S.append(s)
            Y.append(yv)
            if len(S) > history:
                S.pop(0)
                Y.pop(0)
        x, fx, g = xn, fn, gn
    return x


def logistic_fit(d, l1: float = 0.0, l2: float | None = None, classes: int = 0, max_iter: int = 1000,
                 tol: float = 1e-6) -> Linear:
    """Logistic (two classes) or softmax regression on standardized features.  ``l2`` defaults to one over
    the number of rows (the penalty of scikit-learn's ``C = 1``).  Without ``l1`` the loss is minimised by
    L-BFGS until no part of the gradient exceeds ``tol``; with it by accelerated proximal gradient steps
    whose soft threshold drives the weights of unhelpful features to exactly zero."""
    d.check(CLASSIFICATION)
    K = count_classes(d.Y, classes)
    if K < 2:
        raise ValueError("logistic regression needs at least two classes")
    std = Standard.fit(d.X)
    Z = std.apply(d.X).double()
    n, F = Z.shape
    l2 = 1.0 / n if l2 is None else l2
    if l1 < 0 or l2 < 0:
        raise ValueError("penalties must not be negative")
    outs = 1 if K == 2 else K
    y = d.Y.long()
    onehot = torch.nn.functional.one_hot(y, K).double()

    def smooth(theta):
        W, b = theta[:outs * F].reshape(outs, F), theta[outs * F:]
        z = Z @ W.t() + b
        if outs == 1:
            t = onehot[:, 1]
            loss = (torch.clamp(z[:, 0], min=0) - z[:, 0] * t + torch.log1p(torch.exp(-z[:, 0].abs()))).mean()
            r = (torch.sigmoid(z[:, 0]) - t).unsqueeze(1)
        else:
            lp = torch.log_softmax(z, 1)
            loss = -(lp * onehot).sum(1).mean()
            r = lp.exp() - onehot
        gW = r.t() @ Z / n + l2 * W
        return loss + 0.5 * l2 * (W * W).sum(), torch.cat([gW.reshape(-1), r.mean(0)])

    theta = torch.zeros(outs * F + outs, dtype=torch.double)
    if l1 == 0:
        theta = _lbfgs(smooth, theta, max_iter, tol)
    else:
        # FISTA with backtracking on the smooth part; the bias is not penalised
        mask = torch.cat([torch.ones(outs * F), torch.zeros(outs)]).double()
        L, t, zk = 1.0, 1.0, theta.clone()
        for _ in range(max_iter):
            fz, gz = smooth(zk)
            while True:
                u = zk - gz / L
                new = torch.where(mask > 0, torch.sign(u) * torch.clamp(u.abs() - l1 / L, min=0), u)
                diff = new - zk
                if float(smooth(new)[0]) <= float(fz + gz @ diff + 0.5 * L * (diff @ diff)) + 1e-12:
                    break
                L *= 2.0
            t_new = (1 + (1 + 4 * t * t) ** 0.5) / 2
            zk = new + (t - 1) / t_new * (new - theta)
            moved = float((new - theta).abs().max())
            theta, t = new, t_new
            if moved <= tol:
                break
    W, b = theta[:outs * F].reshape(outs, F), theta[outs * F:]
    scale = std.scale.double()
    Wu = W / scale
    m = Linear()
    m.task, m.features, m.classes = CLASSIFICATION, F, K
    m.weights, m.bias = Wu.float(), (b - Wu @ std.mean.double()).float()
    m.link, m.fill = ("sigmoid" if outs == 1 else "softmax"), std.mean
    return m
