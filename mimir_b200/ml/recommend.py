"""Recommendation by matrix factorization with alternating least squares (reference:
recommend/recommend.go): implicit events (clicks, views, purchases) as Hu, Koren and Volinsky do, where
an event counts ``1 + alpha * value`` times more than its absence, and explicit ratings learned from
the rated pairs only.  Users and items are indices from 0; each gets ``factors`` numbers and the score
of an item for a user is their dot product."""
from __future__ import annotations

import torch

from .base import Model


class Factors(Model):
    FIELDS = ("users", "items", "factors", "ratings", "user_factors", "item_factors", "mean")

    def score(self, user: int, item: int) -> float:
        """The predicted rating for a ratings model; a preference near 0 to 1 otherwise."""
        return float(self.user_factors[user] @ self.item_factors[item]) + (self.mean if self.ratings else 0.0)

    def scores(self, user: int) -> torch.Tensor:
        return self.item_factors @ self.user_factors[user] + (self.mean if self.ratings else 0.0)

    def recommend(self, user: int, n: int, skip=()) -> list:
        """The ``n`` items of highest score for ``user``, highest first, leaving out ``skip``."""
        s = self.scores(user).clone()
        if len(skip):
            s[torch.as_tensor(list(skip), dtype=torch.long)] = -float("inf")
        k = min(n, self.items - len(set(skip)))
        return torch.topk(s, max(k, 0)).indices.tolist() if k > 0 else []

    def similar(self, item: int, n: int) -> list:
        """The ``n`` items whose factors point most nearly the way ``item``'s do (cosine), ``item`` left out."""
        V = self.item_factors / self.item_factors.norm(dim=1, keepdim=True).clamp_min(1e-12)
        s = V @ V[item]
        s[item] = -float("inf")
        return torch.topk(s, min(n, self.items - 1)).indices.tolist()

    def hit_rate(self, train, held, n: int) -> float:
        """Recall at ``n``: the share of held-out events whose item is among the ``n`` recommended for the
        event's user, skipping the items each user's training events name."""
        seen: dict = {}
        for u, i, *_ in train:
            seen.setdefault(int(u), set()).add(int(i))
        hits = sum(1 for u, i, *_ in held if int(i) in self.recommend(int(u), n, seen.get(int(u), ())))
        return hits / max(len(held), 1)

    def module(self):
        from .modules import FactorsModule
        return FactorsModule.of(self)


def _solve_side(A, B, idx_rows, idx_cols, conf, target, l2, implicit, native=True):
    """Sets each row of ``A`` to the least-squares fit against the fixed ``B`` of what it has events with.
    Implicit: (B'B + B_u'(C_u - I)B_u + l2 I) x = B_u' C_u p_u with one shared B'B."""
    k = B.shape[1]
    eye = l2 * torch.eye(k, dtype=B.dtype)
    order = torch.argsort(idx_rows, stable=True)
    rows, cols, conf, target = idx_rows[order], idx_cols[order], conf[order], target[order]
    counts = torch.bincount(rows, minlength=A.shape[0])
    BtB = B.t() @ B if implicit else None
    if native and A.device.type == "cpu" and A.dtype == torch.double and A.is_contiguous():
        # each row's normal equations built and solved (Cholesky) by the worker that owns the row (``mimir_cpu_als_side``)
        import ctypes
        from .. import _native
        lib = _native.lib()
        if not getattr(lib, "_als_bound", False):
            lib.mimir_cpu_als_side.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_double]
            lib._als_bound = True
        start = torch.zeros(A.shape[0] + 1, dtype=torch.long)
        start[1:] = counts.cumsum(0)
        Bc = B.contiguous()
        w = (conf - (1.0 if implicit else 0.0)).double().contiguous()
        t = (conf * target).double().contiguous()
        cols = cols.contiguous()
        base = BtB.contiguous() if implicit else None
        if lib.mimir_cpu_als_side(A.data_ptr(), A.shape[0], Bc.data_ptr(), Bc.shape[0], k, start.data_ptr(), cols.data_ptr(), w.data_ptr(),
                                  t.data_ptr(), base.data_ptr() if base is not None else None, float(l2)) != 0:
            raise ValueError("recommend: the native solver refused its arguments")
        return
    # outer products of the event rows, summed per row of A
    Bc = B[cols]
    outer = torch.zeros(A.shape[0], k, k, dtype=B.dtype).index_add_(0, rows, (conf - (1.0 if implicit else 0.0))[:, None, None] * Bc[:, :, None] * Bc[:, None, :])
    rhs = torch.zeros(A.shape[0], k, dtype=B.dtype).index_add_(0, rows, (conf * target)[:, None] * Bc)
    G = outer + eye + (BtB if implicit else 0.0)
    has = counts > 0
    sol = torch.linalg.solve(G[has], rhs[has].unsqueeze(-1)).squeeze(-1)
    A[has] = sol
    A[~has] = 0.0


def fit(users: int, items: int, events, factors: int = 32, iterations: int = 15, l2: float = 0.1, alpha: float = 10.0,
        ratings: bool = False, seed: int = 1) -> Factors:
    """``events``: ``(user, item, value)`` triples (a pair listed several times adds up)."""
    ev = torch.as_tensor([[float(u), float(i), float(v)] for u, i, v in events], dtype=torch.double).reshape(-1, 3)
    if users < 1 or items < 1 or factors < 1 or iterations < 1 or l2 < 0 or ev.shape[0] == 0:
        raise ValueError("recommend: users, items, factors and iterations must be positive and events not empty")
    u, i, v = ev[:, 0].long(), ev[:, 1].long(), ev[:, 2]
    if (u < 0).any() or (u >= users).any() or (i < 0).any() or (i >= items).any() or not torch.isfinite(v).all():
        raise ValueError("recommend: an event names a user or item out of range, or a value that is not finite")
    if not ratings and (v < 0).any():
        raise ValueError("recommend: implicit events must not be negative")
    key, inv = torch.unique(u * items + i, return_inverse=True)
    v = torch.zeros(key.numel(), dtype=torch.double).index_add_(0, inv, v)
    u, i = key // items, key % items
    g = torch.Generator().manual_seed(seed)
    U = torch.randn(users, factors, generator=g, dtype=torch.double) * 0.1
    V = torch.randn(items, factors, generator=g, dtype=torch.double) * 0.1
    mean = float(v.mean()) if ratings else 0.0
    conf = torch.ones_like(v) if ratings else 1.0 + alpha * v
    target = v - mean if ratings else torch.ones_like(v)
    for _ in range(iterations):
        _solve_side(U, V, u, i, conf, target, l2, not ratings)
        _solve_side(V, U, i, u, conf, target, l2, not ratings)
    m = Factors()
    m.users, m.items, m.factors, m.ratings = users, items, factors, bool(ratings)
    m.user_factors, m.item_factors, m.mean = U.float(), V.float(), mean
    return m
