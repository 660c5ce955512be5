"""Support vector machines (reference: svm/svm.go, svm/solve.go).

``fit(d, task, ...)`` standardizes the features (a missing value counts as the mean), then

* a kernel machine (RBF by default, polynomial, sigmoid, or a linear kernel for regression) is solved
  by sequential minimal optimization with second-order working-set selection (Fan, Chen, Lin 2005) on
  kernel rows computed by one matrix product each and kept in a cache;
* a linear classifier by dual coordinate descent in native code (``mimir_cpu_svm_dcd``), which needs
  no kernel matrix and reads the table once per pass;
* more than two classes are one against the rest; probabilities come from Platt scaling of each
  decision value; regression is the epsilon-insensitive machine with ``epsilon`` in standard
  deviations of the answers.

The decision value of output o is ``sum_s coef[o, s] K(x, support[s]) + bias[o]`` on standardized x.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .base import CLASSIFICATION, REGRESSION, Model, Standard, as_rows, as_task, count_classes

LINEAR, RBF, POLYNOMIAL, SIGMOID = "linear", "rbf", "polynomial", "sigmoid"
KERNELS = (LINEAR, RBF, POLYNOMIAL, SIGMOID)


def kernel_matrix(kind, A, B, gamma, coef0, degree):
    if kind == LINEAR:
        return A @ B.t()
    if kind == RBF:
        d = (A * A).sum(1, keepdim=True) - 2.0 * (A @ B.t()) + (B * B).sum(1)[None]
        return torch.exp(-gamma * d.clamp_min(0))
    if kind == POLYNOMIAL:
        return (gamma * (A @ B.t()) + coef0) ** degree
    if kind == SIGMOID:
        return torch.tanh(gamma * (A @ B.t()) + coef0)
    raise ValueError(f"unknown kernel {kind!r}: want one of {KERNELS}")


class _Rows:
    """Rows of the kernel matrix of ``Z`` on demand, the most recent kept within ``cache_mb``."""

    def __init__(self, Z, kind, gamma, coef0, degree, cache_mb):
        self.Z, self.args = Z, (kind, gamma, coef0, degree)
        n = Z.shape[0]
        self.full = None
        if n * n * 4 <= cache_mb * (1 << 20):
            # single precision holds twice the rows and is what the native solver reads
            Zf = Z.float()
            self.full = kernel_matrix(kind, Zf, Zf, gamma, coef0, degree)
        self.cap = max(2, int(cache_mb * (1 << 20) // max(8 * n, 1)))
        self.cache: dict = {}
        self.diag = self.full.diagonal().double() if self.full is not None else \
            torch.stack([kernel_matrix(kind, Z[i:i + 1], Z[i:i + 1], gamma, coef0, degree)[0, 0] for i in range(n)])

    def row(self, i: int):
        if self.full is not None:
            return self.full[i].double()
        r = self.cache.pop(i, None)
        if r is None:
            kind, gamma, coef0, degree = self.args
            r = kernel_matrix(kind, self.Z[i:i + 1], self.Z, gamma, coef0, degree)[0]
            if len(self.cache) >= self.cap:
                self.cache.pop(next(iter(self.cache)))
        self.cache[i] = r                       # most recently used last
        return r


def _smo(rows: _Rows, idx, y, p, c, tol, max_iter):
    """min 0.5 a'Qa + p'a with Q[s, t] = y_s y_t K[idx_s, idx_t], 0 <= a <= c, y'a = 0.  ``idx`` maps the
    variables to kernel rows (regression has two variables per row).  Returns ``(a, bias)``."""
    l = y.numel()
    a = torch.zeros(l, dtype=torch.double)
    G = p.clone()
    if rows.full is not None and _native_smo(rows, idx, y, c, tol, max_iter, a, G):
        return a, _bias(a, G, y, c)
    diag = rows.diag[idx]
    tau = 1e-12
    for _ in range(max_iter):
        score = -y * G
        up = ((y > 0) & (a < c)) | ((y < 0) & (a > 0))
        low = ((y > 0) & (a > 0)) | ((y < 0) & (a < c))
        s_up = torch.where(up, score, torch.full_like(score, -math.inf))
        i = int(s_up.argmax())
        gmax = float(s_up[i])
        s_low = torch.where(low, score, torch.full_like(score, math.inf))
        gmin = float(s_low.min())
        if gmax - gmin < tol:
            break
        Ki = rows.row(int(idx[i]))[idx]
        # second-order choice of j: the largest decrease of the objective among the violators
        b = gmax - score
        quad = (diag[i] + diag - 2.0 * Ki).clamp_min(tau)
        gain = torch.where(low & (b > 0), -(b * b) / quad, torch.full_like(score, math.inf))
        j = int(gain.argmin())
        if not math.isfinite(float(gain[j])):
            break
        Kj = rows.row(int(idx[j]))[idx]
        step = float(b[j] / quad[j])
        room_i = float(c - a[i]) if y[i] > 0 else float(a[i])
        room_j = float(a[j]) if y[j] > 0 else float(c - a[j])
        step = min(step, room_i, room_j)
        a[i] += y[i] * step
        a[j] -= y[j] * step
        G += (step * y) * (Ki - Kj)
    return a, _bias(a, G, y, c)


def _bias(a, G, y, c) -> float:
    """``-y_t G_t`` at a free multiplier (their mean), or the midpoint of the violating pair's bounds."""
    score = -y * G
    free = (a > 1e-12 * c) & (a < c * (1 - 1e-12))
    if free.any():
        return float(score[free].mean())
    up = ((y > 0) & (a < c)) | ((y < 0) & (a > 0))
    low = ((y > 0) & (a > 0)) | ((y < 0) & (a < c))
    hi = float(score[up].max()) if up.any() else 0.0
    lo = float(score[low].min()) if low.any() else hi
    return 0.5 * (hi + lo)


def _native_smo(rows, idx, y, c, tol, max_iter, a, G) -> bool:
    """The solver's loop in native code over the kernel matrix in memory; False when the library is missing."""
    from .. import _native
    if not _native.available():
        return False
    lib = _native.lib()
    if not getattr(lib, "_smo_bound", False):
        lib.mimir_cpu_svm_smo.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                                          ctypes.c_double, ctypes.c_double, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
        lib.mimir_cpu_svm_smo.restype = ctypes.c_longlong
        lib._smo_bound = True
    K32 = rows.full
    idx64, yd = idx.to(torch.int64).contiguous(), y.double().contiguous()
    return lib.mimir_cpu_svm_smo(K32.data_ptr(), K32.shape[0], idx64.data_ptr(), yd.data_ptr(), yd.numel(), float(c), float(tol),
                                 int(max_iter), a.data_ptr(), G.data_ptr()) >= 0


def _dcd(Z, y, c, tol, max_iter, seed):
    """The linear classifier's weights and bias by native dual coordinate descent."""
    from .. import _native
    n, F = Z.shape
    X1 = torch.cat([Z.float(), torch.ones(n, 1)], 1).contiguous()
    yf = y.float().contiguous()
    alpha = torch.zeros(n, dtype=torch.double)
    w = torch.zeros(F + 1, dtype=torch.double)
    if _native.available():
        lib = _native.lib()
        if not getattr(lib, "_svm_bound", False):
            lib.mimir_cpu_svm_dcd.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_double,
                                              ctypes.c_double, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
            lib.mimir_cpu_svm_dcd.restype = ctypes.c_int
            lib._svm_bound = True
        passes = lib.mimir_cpu_svm_dcd(X1.data_ptr(), yf.data_ptr(), n, F + 1, float(c), float(tol), int(min(max_iter, 2**31 - 1)),
                                       int(seed), alpha.data_ptr(), w.data_ptr())
        if passes < 0:
            raise ValueError("svm: bad sizes for the linear solver")
        return w[:F], float(w[F])
    g = torch.Generator().manual_seed(seed)
    qd = (X1.double() ** 2).sum(1)
    Xd = X1.double()
    for _ in range(min(max_iter, 200)):
        worst = 0.0
        for i in torch.randperm(n, generator=g).tolist():
            gi = float(yf[i]) * float(w @ Xd[i]) - 1.0
            ai = float(alpha[i])
            pg = min(gi, 0.0) if ai <= 0 else (max(gi, 0.0) if ai >= c else gi)
            worst = max(worst, abs(pg))
            if pg != 0.0:
                new = min(max(ai - gi / float(qd[i]), 0.0), c)
                w += (new - ai) * float(yf[i]) * Xd[i]
                alpha[i] = new
        if worst <= tol:
            break
    return w[:F], float(w[F])


def _platt(f, t):
    """A, B of ``P(y=1 | f) = 1 / (1 + exp(A f + B))`` by Newton's method with backtracking on the
    regularized targets of Platt (as improved by Lin, Lin and Weng 2007)."""
    f, pos = f.double(), t > 0
    n1, n0 = float(pos.sum()), float((~pos).sum())
    target = torch.where(pos, torch.tensor((n1 + 1) / (n1 + 2)), torch.tensor(1 / (n0 + 2))).double()
    A, B = 0.0, math.log((n0 + 1) / (n1 + 1))

    def loss(A, B):
        z = A * f + B
        return float((torch.clamp(z, min=0) + torch.log1p(torch.exp(-z.abs())) - (1 - target) * z).sum())       # -sum t log p + (1-t) log(1-p)
    cur = loss(A, B)
    for _ in range(100):
        z = A * f + B
        p = torch.sigmoid(-z)                     # P(y = 1)
        d1 = target - p
        gA, gB = float((f * d1).sum()), float(d1.sum())
        if abs(gA) < 1e-5 and abs(gB) < 1e-5:
            break
        h = p * (1 - p)
        hAA, hBB, hAB = float((f * f * h).sum()) + 1e-12, float(h.sum()) + 1e-12, float((f * h).sum())
        det = hAA * hBB - hAB * hAB
        dA, dB = -(hBB * gA - hAB * gB) / det, -(hAA * gB - hAB * gA) / det
        step, moved = 1.0, False
        while step >= 1e-10:
            nl = loss(A + step * dA, B + step * dB)
            if nl < cur + 1e-4 * step * (gA * dA + gB * dB):
                A, B, cur, moved = A + step * dA, B + step * dB, nl, True
                break
            step /= 2
        if not moved:
            break
    return A, B


class SVM(Model):
    FIELDS = ("task", "features", "classes", "kernel", "gamma", "coef0", "degree", "support", "coef", "bias",
              "platt", "standard", "y_mean", "y_scale")

    def support_vectors(self) -> int:
        return int(self.support.shape[0])

    def decision(self, X) -> torch.Tensor:
        """``[rows, outputs]`` decision values: one output for two classes or regression, one per class for more."""
        Z = self.standard.apply(as_rows(X, self.features)).double()
        if self.kernel == LINEAR and self.task is CLASSIFICATION:
            return Z @ self.coef.t() + self.bias               # coef holds the weights: no support vectors are kept
        K = kernel_matrix(self.kernel, Z, self.support, self.gamma, self.coef0, self.degree)
        return K @ self.coef.t() + self.bias

    def predict(self, X) -> torch.Tensor:
        f = self.decision(X)
        if self.task is REGRESSION:
            return (f[:, 0] * self.y_scale + self.y_mean).float()
        A, B = self.platt[:, 0], self.platt[:, 1]
        p = torch.sigmoid(-(f * A + B))
        if self.classes == 2:
            return torch.stack([1 - p[:, 0], p[:, 0]], 1).float()
        return (p / p.sum(1, keepdim=True).clamp_min(1e-300)).float()

    def module(self):
        from .modules import SVMModule
        return SVMModule.of(self)


def fit(d, task, c: float = 1.0, kernel: str = RBF, gamma: float | None = None, coef0: float = 0.0, degree: int = 3,
        epsilon: float = 0.1, tol: float = 1e-3, max_iter: int | None = None, classes: int = 0, cache_mb: int = 256,
        seed: int = 0) -> SVM:
    task = as_task(task)
    d.check(task)
    if c <= 0 or tol <= 0 or epsilon < 0 or degree < 1 or cache_mb < 1 or kernel not in KERNELS:
        raise ValueError("svm: C, tolerance and cache must be positive, epsilon not negative, the kernel one of " + ", ".join(KERNELS))
    if gamma is not None and gamma <= 0:
        raise ValueError("svm: gamma must be positive")
    std = Standard.fit(d.X)
    Z = std.apply(d.X).double()
    n, F = Z.shape
    gamma = 1.0 / F if gamma is None else float(gamma)
    max_iter = max(10_000_000, 100 * n) if max_iter is None else int(max_iter)
    m = SVM()
    m.task, m.features, m.kernel, m.gamma, m.coef0, m.degree, m.standard = task, F, kernel, gamma, float(coef0), int(degree), std
    m.y_mean, m.y_scale, m.classes = 0.0, 1.0, 0
    if task is REGRESSION:
        y = d.Y.double()
        m.y_mean = float(y.mean())
        m.y_scale = float(y.std(unbiased=False)) or 1.0
        t = (y - m.y_mean) / m.y_scale
        rows = _Rows(Z, kernel, gamma, coef0, degree, cache_mb)
        idx = torch.cat([torch.arange(n), torch.arange(n)])
        sign = torch.cat([torch.ones(n), -torch.ones(n)]).double()
        p = torch.cat([epsilon - t, epsilon + t])
        a, bias = _smo(rows, idx, sign, p, c, tol, max_iter)
        beta = a[:n] - a[n:]
        keep = beta.abs() > 1e-12
        m.support, m.coef, m.bias = Z[keep], beta[keep].unsqueeze(0), torch.tensor([bias], dtype=torch.double)
        m.platt = torch.zeros(0, 2, dtype=torch.double)
        return m
    K = count_classes(d.Y, classes)
    if K < 2:
        raise ValueError("svm: classification needs at least two classes")
    m.classes = K
    labels = d.Y.long()
    outs = [1] if K == 2 else list(range(K))
    coefs, biases, platt = [], [], []
    rows = None if kernel == LINEAR else _Rows(Z, kernel, gamma, coef0, degree, cache_mb)
    used = torch.zeros(n, dtype=torch.bool)
    alphas = []
    for o in outs:
        y = torch.where(labels == o, 1.0, -1.0).double()
        if kernel == LINEAR:
            w, b = _dcd(Z, y, c, tol, min(max_iter, 1000), seed + o)
            coefs.append(w)
            biases.append(b)
            f = Z @ w + b
        else:
            a, b = _smo(rows, torch.arange(n), y, -torch.ones(n, dtype=torch.double), c, tol, max_iter)
            beta = a * y
            alphas.append(beta)
            used |= beta.abs() > 1e-12
            biases.append(b)
            f = None
        if f is None:
            f = torch.stack([rows.row(i) for i in range(n)]) @ beta + b if rows.full is None else (rows.full @ beta.float()).double() + b
        platt.append(_platt(f, y))
    if kernel == LINEAR:
        m.support, m.coef = torch.zeros(0, F, dtype=torch.double), torch.stack(coefs)
    else:
        m.support, m.coef = Z[used], torch.stack([b[used] for b in alphas])
    m.bias, m.platt = torch.tensor(biases, dtype=torch.double), torch.tensor(platt, dtype=torch.double)
    return m
