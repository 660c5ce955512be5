"""Histogram-based trees (reference: tree/): DecisionTree, RandomForest, GradientBoosting,
IsolationForest.  Features are binned into at most 255 bins once; split search works on
per-node gradient / hessian histograms (the reference accelerates the same histograms
with AVX2 assembly, tree/hist_amd64.go; on the host the binning, the trees and whole boosting
loops are native code, ``csrc/cpu_hist.cc``; elsewhere the histograms are ``torch.bincount``
calls, which run on the GPU when the data lives there)."""
from __future__ import annotations

import json
import math

import torch


def _bin(X, bins=255):
    X = X.float()
    qs = torch.linspace(0, 1, bins + 1)[1:-1]
    # the bin edges come from at most 65,536 rows (evenly spaced ones): enough for 255 quantiles, and the sort
    # of every column is the most expensive step of a fit on a large table
    S = X if X.shape[0] <= 65536 else X[torch.linspace(0, X.shape[0] - 1, 65536).long()]
    edges = torch.quantile(S, qs.to(X.device), dim=0).t().contiguous()  # [F, bins-1]
    if bins <= 256 and X.device.type == "cpu":
        # one byte per value, written by rows (what prediction walks) and by columns (what the grower reads)
        B, cols = bin_table(X, edges, columns=True)
        _COLUMNS["last"] = ((B.data_ptr(), tuple(B.shape), B._version), cols, B)
        return B, edges
    B = torch.searchsorted(edges, X.t().contiguous()).t().contiguous()
    return B.to(torch.uint8 if bins <= 256 else torch.int64), edges


def bin_table(X, edges, columns=False):
    """The bin of every value of ``X [n, F]``: the number of its feature's ``edges [F, bins - 1]`` below it, as
    uint8 ``[n, F]`` (``torch.searchsorted`` per feature, done by ``mimir_cpu_bin_table`` over the worker pool).
    ``columns=True`` also returns the same table held one column per feature, ``[F, n]``."""
    import ctypes
    from .. import _native
    X, edges = X.float().contiguous(), edges.float().contiguous()
    n, F = X.shape
    if edges.shape[0] != F or edges.shape[1] > 255:
        raise ValueError(f"edges of shape {tuple(edges.shape)} for {F} features")
    lib = _native.lib()
    if not getattr(lib, "_bin_bound", False):
        lib.mimir_cpu_bin_table.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                            ctypes.c_void_p]
        lib._bin_bound = True
    B = torch.empty(n, F, dtype=torch.uint8)
    cols = torch.empty(F, n, dtype=torch.uint8) if columns else None
    if lib.mimir_cpu_bin_table(X.data_ptr(), n, F, edges.data_ptr(), edges.shape[1], B.data_ptr(), cols.data_ptr() if columns else None) != 0:
        raise ValueError("bin_table: bad arguments")
    return (B, cols) if columns else B


_COLUMNS: dict = {}


def _columns(B):
    """``B`` with one column per feature in memory (``[F, n]`` contiguous), which is what the native grower
    reads; kept for the latest table so the trees of one ensemble share it."""
    key = (B.data_ptr(), tuple(B.shape), B._version)
    hit = _COLUMNS.get("last")
    if hit is not None and hit[0] == key:
        return hit[1]
    cols = B.t().contiguous()
    _COLUMNS["last"] = (key, cols, B)          # B is kept alive so its address cannot be reused under the key
    return cols


def _histogram(B, idx, g, h, bins):
    """Sums of g, sums of h and counts per (feature, bin) over the rows ``idx``: ``[3, F, bins]`` float64.
    uint8 bins on the CPU take the native multi-threaded pass (``csrc/cpu_hist.cc``)."""
    F = B.shape[1]
    if B.dtype == torch.uint8 and B.device.type == "cpu" and B.is_contiguous() and bins <= 256:
        import ctypes
        from .. import _native
        lib = _native.lib()
        if not getattr(lib, "_hist_bound", False):
            lib.mimir_cpu_hist.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
            lib._hist_bound = True
        out = torch.empty(3, F, bins, dtype=torch.float64)
        idx = idx.contiguous()
        g32 = g if g.dtype == torch.float32 and g.is_contiguous() else g.float().contiguous()
        h32 = h if h.dtype == torch.float32 and h.is_contiguous() else h.float().contiguous()
        rc = lib.mimir_cpu_hist(B.data_ptr(), F, idx.data_ptr(), idx.numel(), g32.data_ptr(), h32.data_ptr(), bins, out.data_ptr())
        if rc == 0:
            return out
    Bi = B[idx].long()
    flat = (Bi + torch.arange(F, device=B.device) * bins).reshape(-1)
    hg = torch.bincount(flat, weights=g[idx].double().repeat_interleave(F), minlength=F * bins)
    hh = torch.bincount(flat, weights=h[idx].double().repeat_interleave(F), minlength=F * bins)
    hc = torch.bincount(flat, minlength=F * bins).double()
    return torch.stack([hg, hh, hc]).view(3, F, bins)


class _Tree:
    """Regression tree on gradients/hessians (second-order gain with L2)."""

    def __init__(self, max_depth=6, min_leaf=1, min_gain=0.0, l2=1.0, bins=255, colsample=1.0, gen=None, min_weight=0.0, allowed=None):
        """``colsample``: the share of the features drawn afresh at every node; ``allowed``: the features (ascending
        numbers) this tree may split on at all, None for every one; ``min_weight``: the smallest sum of hessians a
        child may hold."""
        self.max_depth, self.min_leaf, self.min_gain, self.l2, self.bins = max_depth, min_leaf, min_gain, l2, bins
        self.colsample, self.gen, self.min_weight = colsample, gen, float(min_weight)
        self.allowed = None if allowed is None else torch.as_tensor(allowed, dtype=torch.int32).contiguous()
        self.nodes = []  # (feature, bin, left, right, value)
        self.importance = None

    def fit(self, B, g, h, rows=None):
        """Grows the tree on the rows ``rows`` of ``B`` (all of them when None); ``g`` and ``h`` are indexed by
        row number.  After a native fit on all rows ``self.answers`` holds the tree's value for each row."""
        n, F = B.shape
        self.importance = torch.zeros(F)
        self.nodes = []
        self.answers = None
        if g.dtype != torch.float64:
            g, h = g.float().contiguous(), h.float().contiguous()
        if B.dtype == torch.uint8 and B.device.type == "cpu" and B.is_contiguous() and self.bins <= 256 and g.dtype == torch.float32 \
                and self._grow_native(B, g, h, rows):
            return self
        self._grow(B, g, h, torch.arange(n, device=B.device) if rows is None else rows.to(B.device), 0)
        return self

    def _grow_native(self, B, g, h, rows=None) -> bool:
        """The whole tree grown by ``csrc/cpu_hist.cc`` (histograms over the worker pool, the larger
        child's histogram by subtraction, rows partitioned in place).  Feature subsets per node are drawn
        from a seed taken from this tree's generator."""
        import ctypes
        from .. import _native
        lib = _native.lib()
        if not getattr(lib, "_tree_bound", False):
            c = ctypes
            lib.mimir_cpu_grow_tree_answers.argtypes = [c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_longlong, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                                                        c.c_longlong, c.c_double, c.c_double, c.c_int, c.c_ulonglong, c.c_void_p, c.c_int,
                                                        c.c_void_p, c.c_void_p, c.c_double, c.c_void_p, c.c_int]
            lib._tree_bound = True
        total, F = B.shape
        n = total if rows is None else int(rows.numel())
        k = 0
        seed = 0
        universe = F if self.allowed is None else int(self.allowed.numel())
        if self.colsample < 1.0:
            k = max(1, int(universe * self.colsample))
            seed = int(torch.randint(0, 2 ** 62, (1,), generator=self.gen))
        max_nodes = int(min(2 ** (self.max_depth + 1) - 1, 2 * n + 1))
        nodes = torch.empty(max_nodes, 5, dtype=torch.float64)
        imp = torch.zeros(F, dtype=torch.float64)
        idx = torch.arange(n, dtype=torch.int64) if rows is None else rows.to(torch.int64).clone()
        answers = torch.empty(total) if rows is None else None
        cols = _columns(B)
        cnt = lib.mimir_cpu_grow_tree_answers(cols.data_ptr(), total, F, idx.data_ptr(), n, g.data_ptr(), h.data_ptr(), self.bins, self.max_depth,
                                              max(int(self.min_leaf), 1) if self.min_leaf >= 1 else 0, float(self.min_gain), float(self.l2),
                                              k, seed, nodes.data_ptr(), max_nodes, imp.data_ptr(),
                                              answers.data_ptr() if answers is not None else None, self.min_weight,
                                              self.allowed.data_ptr() if self.allowed is not None else None, universe)
        if cnt <= 0:
            return False
        self.answers = answers
        rows = nodes[:cnt]
        self.nodes = [[int(r[0]), int(r[1]), int(r[2]), int(r[3]), float(r[4])] for r in rows.tolist()]
        self.importance = imp.float()
        return True

    def _grow(self, B, g, h, idx, depth, hist=None):
        """``hist``: this node's histogram when the parent already has it (a child's histogram is the
        parent's minus its sibling's, so only the smaller child is ever counted)."""
        if hist is not None:
            G, H = hist[0, 0].sum().to(g.dtype), hist[1, 0].sum().to(g.dtype)      # every row falls in some bin of feature 0
        else:
            G, H = g[idx].sum(), h[idx].sum()
        node = len(self.nodes)
        self.nodes.append([-1, 0, -1, -1, float(-G / (H + self.l2))])
        if depth >= self.max_depth or idx.numel() < 2 * self.min_leaf:
            return node
        feats = torch.arange(B.shape[1]) if self.allowed is None else self.allowed.long()
        if self.colsample < 1.0:
            k = max(1, int(feats.numel() * self.colsample))
            feats = feats[torch.randperm(feats.numel(), generator=self.gen)[:k]]
        if hist is None:
            hist = _histogram(B, idx, g, h, self.bins)
        sel = hist[:, feats].to(g.dtype if g.dtype == torch.float64 else torch.float32)
        hg, hh, hc = sel[0].reshape(-1), sel[1].reshape(-1), hist[2, feats].reshape(-1).long()
        GL = hg.view(-1, self.bins).cumsum(1)
        HL = hh.view(-1, self.bins).cumsum(1)
        CL = hc.view(-1, self.bins).cumsum(1)
        GR, HR, CR = G - GL, H - HL, idx.numel() - CL
        gain = GL ** 2 / (HL + self.l2) + GR ** 2 / (HR + self.l2) - G ** 2 / (H + self.l2)
        gain[(CL < self.min_leaf) | (CR < self.min_leaf) | (HL < self.min_weight) | (HR < self.min_weight)] = -1
        best = int(gain.argmax())
        bg = float(gain.reshape(-1)[best])
        if bg <= self.min_gain:
            return node
        f, b = feats[best // self.bins].item(), best % self.bins
        self.importance[f] += bg
        go_left = B[idx, f] <= b
        self.nodes[node][0], self.nodes[node][1] = f, b
        li, ri = idx[go_left], idx[~go_left]
        lh = rh = None
        if depth + 1 < self.max_depth and min(li.numel(), ri.numel()) >= 2 * self.min_leaf:
            if li.numel() <= ri.numel():
                lh = _histogram(B, li, g, h, self.bins)
                rh = hist - lh
            else:
                rh = _histogram(B, ri, g, h, self.bins)
                lh = hist - rh
        self.nodes[node][2] = self._grow(B, g, h, li, depth + 1, lh)
        self.nodes[node][3] = self._grow(B, g, h, ri, depth + 1, rh)
        return node

    def predict_binned(self, B):
        if B.dtype == torch.uint8 and B.device.type == "cpu" and B.is_contiguous() and self.nodes:
            import ctypes
            from .. import _native
            lib = _native.lib()
            if not getattr(lib, "_predict_bound", False):
                lib.mimir_cpu_tree_predict.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int,
                                                       ctypes.c_void_p]
                lib._predict_bound = True
            tbl = torch.tensor(self.nodes, dtype=torch.float64)
            out = torch.empty(B.shape[0])
            if lib.mimir_cpu_tree_predict(B.data_ptr(), B.shape[1], B.shape[0], tbl.data_ptr(), tbl.shape[0], out.data_ptr()) == 0:
                return out
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
        X = torch.as_tensor(X).float()
        if X.device.type == "cpu" and self.edges.shape[1] <= 255:
            return bin_table(X, self.edges)
        return torch.searchsorted(self.edges, X.t().contiguous()).t().contiguous()

    @staticmethod
    def _sum_of(trees, B):
        """The sum of the trees' values for every row of ``B``: one native pass over all trees for byte bins
        on the host (``mimir_cpu_trees_predict``), else tree by tree."""
        if B.dtype == torch.uint8 and B.device.type == "cpu" and B.is_contiguous() and trees and all(t.nodes for t in trees):
            import ctypes
            from .. import _native
            lib = _native.lib()
            if not getattr(lib, "_trees_bound", False):
                lib.mimir_cpu_trees_predict.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p,
                                                        ctypes.c_int, ctypes.c_void_p]
                lib._trees_bound = True
            tbl = torch.tensor([q for t in trees for q in t.nodes], dtype=torch.float64)
            offsets = torch.tensor([0] + [len(t.nodes) for t in trees], dtype=torch.int64).cumsum(0).contiguous()
            out = torch.empty(B.shape[0])
            if lib.mimir_cpu_trees_predict(B.data_ptr(), B.shape[1], B.shape[0], tbl.data_ptr(), offsets.data_ptr(), len(trees),
                                           out.data_ptr()) == 0:
                return out
        out = torch.zeros(B.shape[0])
        for t in trees:
            out += t.predict_binned(B)
        return out

    def raw(self, X):
        B = self._binned(X)
        if self.classes > 2:
            out = self.base.clone().repeat(B.shape[0], 1)
            for k in range(self.classes):
                out[:, k] += self.lr * self._sum_of([r[k] for r in self.trees], B)
            return out
        scale = self.lr if self.kind == "gbdt" else 1.0 / max(len(self.trees), 1)
        return float(self.base) + scale * self._sum_of(self.trees, B)

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

    def module(self):
        """This ensemble as an ``nn.Module`` that walks every tree in tensor ops (``ml/modules.py``)."""
        from .modules import TreeModule
        return TreeModule.of(self)

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


def _boost_native(B, y, score, kind, rounds, lr, max_depth, min_leaf, min_gain, l2, bins, colsample, gen, min_weight=0.0, per_tree=1.0,
                  classes=0):
    """``rounds`` rounds grown one after another by ``mimir_cpu_boost`` (``csrc/cpu_hist.cc``) on all rows of ``B``,
    or, with ``classes`` above two, by ``mimir_cpu_boost_classes`` (one tree per class and round; the result is a
    list of rounds, each a list of trees).  ``score`` is updated in place.  Feature lists and feature-draw seeds
    come from ``gen`` in the order the per-round loop draws them."""
    import ctypes
    from .. import _native
    lib = _native.lib()
    if not getattr(lib, "_boost_bound", False):
        c = ctypes
        lib.mimir_cpu_boost.argtypes = [c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_double, c.c_int, c.c_int,
                                        c.c_longlong, c.c_double, c.c_double, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p,
                                        c.c_double, c.c_void_p, c.c_int]
        lib.mimir_cpu_boost_classes.argtypes = [c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_double, c.c_int,
                                                c.c_int, c.c_longlong, c.c_double, c.c_double, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p,
                                                c.c_void_p, c.c_double, c.c_void_p, c.c_int]
        lib._boost_bound = True
    total, F = B.shape
    per_round = classes if classes > 2 else 1
    k, seeds, allowed = 0, None, None
    universe = F if per_tree >= 1.0 else max(1, int(F * per_tree))
    if colsample < 1.0 or per_tree < 1.0:
        # the draws of each round in the order the per-round loop makes them: the tree's features, then its seed
        k = max(1, int(universe * colsample)) if colsample < 1.0 else 0
        lists, seeds = [], []
        for _ in range(rounds):
            if per_tree < 1.0:
                lists.append(_draw_features(F, per_tree, gen))
            seeds += [int(torch.randint(0, 2 ** 62, (1,), generator=gen)) if colsample < 1.0 else 0 for _ in range(per_round)]
        seeds = torch.tensor(seeds, dtype=torch.int64)
        allowed = torch.stack(lists).contiguous() if lists else None
    max_nodes = int(min(2 ** (max_depth + 1) - 1, 2 * total + 1))
    grown = rounds * per_round
    nodes = torch.empty(grown, max_nodes, 5, dtype=torch.float64)
    counts = torch.zeros(grown, dtype=torch.int32)
    imp = torch.empty(grown, F, dtype=torch.float64)
    cols = _columns(B)
    tail = (float(lr), bins, max_depth, max(int(min_leaf), 1) if min_leaf >= 1 else 0, float(min_gain), float(l2), k,
            seeds.data_ptr() if seeds is not None else None, nodes.data_ptr(), max_nodes, counts.data_ptr(), imp.data_ptr(),
            float(min_weight), allowed.data_ptr() if allowed is not None else None, universe)
    if classes > 2:
        y = y.long().contiguous()
        if not score.is_contiguous() or tuple(score.shape) != (total, classes):
            raise ValueError("boosting: scores must be a contiguous [rows, classes] table")
        done = lib.mimir_cpu_boost_classes(cols.data_ptr(), total, F, y.data_ptr(), score.data_ptr(), classes, rounds, *tail)
    else:
        y = y.float().contiguous()
        done = lib.mimir_cpu_boost(cols.data_ptr(), total, F, y.data_ptr(), score.data_ptr(), kind, rounds, *tail)
    if done != rounds:
        raise RuntimeError("boosting: the native grower refused its arguments")
    out = []
    for r in range(grown):
        t = _Tree(max_depth, min_leaf, min_gain, l2, bins, colsample, gen, min_weight, None if allowed is None else allowed[r // per_round])
        t.nodes = [[int(q[0]), int(q[1]), int(q[2]), int(q[3]), float(q[4])] for q in nodes[r, : int(counts[r])].tolist()]
        t.importance = imp[r].float()
        t.answers = None
        out.append(t)
    return out if per_round == 1 else [out[r: r + per_round] for r in range(0, grown, per_round)]


def _draw_features(F, share, gen):
    """The features one tree may split on: ``share`` of all, drawn without repeats, ascending (None: all)."""
    if share >= 1.0:
        return None
    return torch.randperm(F, generator=gen)[: max(1, int(F * share))].sort().values.to(torch.int32).contiguous()


def gradient_boosting(X, y, trees=100, learning_rate=0.1, max_depth=6, min_leaf=1, min_gain=0.0, l2=1.0, bins=255,
                      subsample=1.0, colsample=1.0, classes=0, seed=0, validation=None, patience=10, progress=None,
                      native_rounds=True, min_weight=0.0, per_tree=1.0) -> Model:
    """Second-order boosting: squared error (classes=0), logistic (2) or softmax (>2).  ``subsample`` draws
    that share of the rows for each tree, ``per_tree`` that share of the features for each tree (tree/options.go:
    ColSample) and ``colsample`` that share of a tree's features afresh at every node; ``min_weight`` is the
    smallest sum of hessians a child may hold (XGBoost's min_child_weight; tree/options.go: MinWeight).
    ``validation`` (a table, or ``(X, y)``) is scored after every round (squared error or log loss): boosting
    stops once ``patience`` rounds in a row have not improved it, and the model keeps the best round's trees
    (tree/boost.go: Validation).  Without row sampling and validation every round runs inside one native
    call; ``native_rounds=False`` keeps the per-round loop (the same trees up to the
    rounding of the sigmoid)."""
    X, y = torch.as_tensor(X).float(), torch.as_tensor(y)
    gen = torch.Generator().manual_seed(seed)
    B, edges = _bin(X, bins)
    n = X.shape[0]
    out_trees = []
    held = None
    if validation is not None:
        Xv, yv = (validation.X, validation.Y) if hasattr(validation, "X") else validation
        Xv, yv = torch.as_tensor(Xv).float(), torch.as_tensor(yv)
        Bv = torch.searchsorted(edges, Xv.t().contiguous()).t().contiguous()
        held = dict(B=Bv, y=yv, best=math.inf, at=0, bad=0)
    if classes > 2:
        base = torch.zeros(classes)
        F = torch.zeros(n, classes)
        oh = torch.nn.functional.one_hot(y.long(), classes).float()
    else:
        yf = y.float()
        base = float(yf.mean()) if classes == 0 else float(torch.logit(yf.mean().clamp(1e-6, 1 - 1e-6)))
        F = torch.full((n,), base)
    if held is not None:
        held["F"] = base.clone().repeat(held["B"].shape[0], 1) if classes > 2 else torch.full((held["B"].shape[0],), base)
    if native_rounds and subsample >= 1.0 and held is None and B.dtype == torch.uint8 and B.device.type == "cpu" and bins <= 256:
        # every round in native code (``mimir_cpu_boost``): the loop below is its oracle
        span = 10 if progress is not None else trees
        for it in range(0, trees, span):
            out_trees += _boost_native(B, y if classes > 2 else yf, F, 0 if classes == 0 else 1, min(span, trees - it), learning_rate,
                                       max_depth, min_leaf, min_gain, l2, bins, colsample, gen, min_weight, per_tree, classes)
            if progress is not None and len(out_trees) % 10 == 0:
                progress.write(f"tree {len(out_trees)}/{trees}\n")
        trees = 0
    for it in range(trees):
        rows = None if subsample >= 1.0 else torch.randperm(n, generator=gen)[: max(1, int(n * subsample))]
        allowed = _draw_features(X.shape[1], per_tree, gen)
        if classes > 2:
            p = torch.softmax(F, 1)
            round_trees = []
            for k in range(classes):
                g, h = (p[:, k] - oh[:, k]), (p[:, k] * (1 - p[:, k])).clamp_min(1e-6)
                t = _Tree(max_depth, min_leaf, min_gain, l2, bins, colsample, gen, min_weight, allowed).fit(B, g, h, rows)
                F[:, k] += learning_rate * (t.answers if t.answers is not None else t.predict_binned(B))
                if held is not None:
                    held["F"][:, k] += learning_rate * t.predict_binned(held["B"])
                round_trees.append(t)
            out_trees.append(round_trees)
        else:
            if classes == 2:
                p = torch.sigmoid(F)
                g, h = p - yf, (p * (1 - p)).clamp_min(1e-6)
            else:
                g, h = F - yf, torch.ones(n)
            t = _Tree(max_depth, min_leaf, min_gain, l2, bins, colsample, gen, min_weight, allowed).fit(B, g, h, rows)
            F += learning_rate * (t.answers if t.answers is not None else t.predict_binned(B))
            if held is not None:
                held["F"] += learning_rate * t.predict_binned(held["B"])
            out_trees.append(t)
        if progress is not None and (it + 1) % 10 == 0:
            progress.write(f"tree {it + 1}/{trees}\n")
        if held is not None:
            if classes > 2:
                loss = float(torch.nn.functional.cross_entropy(held["F"], held["y"].long()))
            elif classes == 2:
                loss = float(torch.nn.functional.binary_cross_entropy_with_logits(held["F"], held["y"].float()))
            else:
                loss = float(((held["F"] - held["y"].float()) ** 2).mean())
            if loss < held["best"] - 1e-12:
                held["best"], held["at"], held["bad"] = loss, it + 1, 0
            else:
                held["bad"] += 1
                if held["bad"] >= max(int(patience), 1):
                    break
    if held is not None and held["at"] > 0:
        out_trees = out_trees[:held["at"]]
    m = Model(out_trees, edges, learning_rate, base, classes, "gbdt")
    m.validation_loss = held["best"] if held is not None else None
    return m


def decision_tree(X, y, max_depth=8, min_leaf=1, classes=0, **kw) -> Model:
    return gradient_boosting(X, y, trees=1, learning_rate=1.0, max_depth=max_depth, min_leaf=min_leaf, l2=0.0,
                             classes=classes, **kw)


def _forest_native(B, rows, g, h, seeds, max_depth, min_leaf, bins, colsample, gen):
    """One tree per row of ``rows [trees, n]`` (row numbers of ``B``, repeats allowed), grown side by side."""
    import ctypes
    from .. import _native
    lib = _native.lib()
    if not getattr(lib, "_forest_bound", False):
        c = ctypes
        lib.mimir_cpu_grow_forest.argtypes = [c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_void_p, c.c_int,
                                              c.c_int, c.c_longlong, c.c_double, c.c_double, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p,
                                              c.c_void_p, c.c_double, c.c_void_p, c.c_int]
        lib._forest_bound = True
    total, F = B.shape
    count, n = rows.shape
    k = max(1, int(F * colsample)) if colsample < 1.0 else 0
    max_nodes = int(min(2 ** (max_depth + 1) - 1, 2 * n + 1))
    nodes = torch.empty(count, max_nodes, 5, dtype=torch.float64)
    counts = torch.zeros(count, dtype=torch.int32)
    imp = torch.empty(count, F, dtype=torch.float64)
    rows = rows.to(torch.int64).contiguous()
    seed_t = torch.tensor(seeds, dtype=torch.int64)
    cols = _columns(B)
    rc = lib.mimir_cpu_grow_forest(cols.data_ptr(), total, F, rows.data_ptr(), n, count, g.data_ptr(), h.data_ptr(), bins, max_depth,
                                   max(int(min_leaf), 1) if min_leaf >= 1 else 0, 0.0, 0.0, k, seed_t.data_ptr(), nodes.data_ptr(), max_nodes,
                                   counts.data_ptr(), imp.data_ptr(), 0.0, None, 0)
    if rc != 0:
        raise RuntimeError("forest: the native grower refused its arguments")
    out = []
    for r in range(count):
        t = _Tree(max_depth, min_leaf, 0.0, 0.0, bins, colsample, gen)
        t.nodes = [[int(q[0]), int(q[1]), int(q[2]), int(q[3]), float(q[4])] for q in nodes[r, : int(counts[r])].tolist()]
        t.importance = imp[r].float()
        t.answers = None
        out.append(t)
    return out


def random_forest(X, y, trees=100, max_depth=10, min_leaf=1, colsample=None, bootstrap=True, classes=0, seed=0, bins=255,
                  native_trees=True, per_node=None) -> Model:
    """Bagged trees on bootstrap samples with per-node feature sampling; averages the trees.  ``per_node``
    features are drawn at each node (tree/options.go: PerNode), or the share ``colsample`` of them; by default the
    square root of the features for classification and a third for regression.  On the host the trees grow side
    by side in native code; ``native_trees=False`` grows them one by one (the same trees)."""
    X, y = torch.as_tensor(X).float(), torch.as_tensor(y).float()
    gen = torch.Generator().manual_seed(seed)
    B, edges = _bin(X, bins)
    n, F = X.shape
    if per_node is not None:
        if not 1 <= int(per_node) <= F:
            raise ValueError(f"per_node {per_node} of {F} features")
        colsample = (int(per_node) + 0.5) / F if per_node < F else 1.0
    colsample = colsample or (math.sqrt(F) / F if classes else 1.0 / 3 if F >= 3 else 1.0)
    out = []
    if native_trees and B.dtype == torch.uint8 and B.device.type == "cpu" and bins <= 256:
        # the trees of a chunk grow side by side in native code, one whole tree per worker (``mimir_cpu_grow_forest``)
        g, h = (-y).contiguous(), torch.ones(n)
        for t0 in range(0, trees, 32):
            rows, seeds = [], []
            for _ in range(min(32, trees - t0)):         # the draws in the order the per-tree loop makes them
                rows.append(torch.randint(0, n, (n,), generator=gen) if bootstrap else torch.arange(n))
                seeds.append(int(torch.randint(0, 2 ** 62, (1,), generator=gen)) if colsample < 1.0 else 0)
            out += _forest_native(B, torch.stack(rows), g, h, seeds, max_depth, min_leaf, bins, colsample, gen)
        trees = 0
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
        depth = self._paths_native(X) if X.device.type == "cpu" and self.trees else None
        if depth is None:
            depth = torch.zeros(X.shape[0])
            for t in self.trees:
                depth += self._path(t, X)
        c = 2 * (math.log(self.sample - 1) + 0.5772156649) - 2 * (self.sample - 1) / self.sample if self.sample > 2 else 1.0
        return torch.pow(2.0, -(depth / len(self.trees)) / c)

    @staticmethod
    def _extra(size):
        """The expected further depth of a leaf that still holds ``size`` rows."""
        return 2 * (math.log(size - 1) + 0.5772156649) - 2 * (size - 1) / size if size > 2 else (1.0 if size == 2 else 0.0)

    def _paths_native(self, X):
        """The summed path lengths of every row over all trees in one native pass (``mimir_cpu_paths_sum``), or
        None when the library refuses the tables."""
        import ctypes
        from .. import _native
        lib = _native.lib()
        if not getattr(lib, "_paths_bound", False):
            lib.mimir_cpu_paths_sum.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                                ctypes.c_void_p]
            lib._paths_bound = True
        tbl = torch.tensor([[q[0], q[1], q[2], q[3], self._extra(q[4]) if q[0] < 0 else 0.0] for t in self.trees for q in t], dtype=torch.float64)
        offsets = torch.tensor([0] + [len(t) for t in self.trees], dtype=torch.int64).cumsum(0).contiguous()
        X = X.contiguous()
        out = torch.empty(X.shape[0])
        rc = lib.mimir_cpu_paths_sum(X.data_ptr(), X.shape[1], X.shape[0], tbl.data_ptr(), offsets.data_ptr(), len(self.trees), out.data_ptr())
        return out if rc == 0 else None

    @staticmethod
    def _path(tree, X):
        out = torch.zeros(X.shape[0])
        stack = [(0, torch.arange(X.shape[0]), 0)]
        while stack:
            node, idx, d = stack.pop()
            f, thr, l, r, size = tree[node]
            if f < 0 or idx.numel() == 0:
                out[idx] = d + IsolationForestModel._extra(size)
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


# ---------------------------------------------------------------------------------------------
# Table-level entry points (reference: tree/boost.go, tree/forest.go, tree/tree.go, tree/options.go)
# ---------------------------------------------------------------------------------------------
class Ensemble:
    """Trees fitted to a table for a task: ``predict`` gives ``classes`` probabilities per row for
    classification and one value per row for regression, whatever the kind of ensemble underneath (boosted
    rounds, or one forest per class).  ``importance()`` is each feature's share of the total gain."""

    def __init__(self, task, classes: int, models: list, kind: str):
        self.task, self.classes, self.models, self.kind = task, classes, models, kind

    def predict(self, X):
        X = torch.as_tensor(X).float()
        if not self.classes:
            return self.models[0].predict(X)
        if self.kind == "forest":
            p = torch.stack([m.predict(X) for m in self.models], 1).clamp_min(0)
            return p / p.sum(1, keepdim=True).clamp_min(1e-12)
        p = self.models[0].predict(X)
        return torch.stack([1 - p, p], 1) if p.dim() == 1 else p

    def classify(self, X):
        p = self.predict(X)
        return p.argmax(1) if p.dim() == 2 else p

    def importance(self):
        imp = sum(m.importance() for m in self.models)
        return imp / imp.sum().clamp_min(1e-12)

    def module(self):
        """The ensemble as an ``nn.Module`` (boosted trees and single trees; a forest of several classes is
        served one class at a time by its members' modules)."""
        if len(self.models) != 1:
            raise ValueError("a forest of several classes has one module per class: use models[k].module()")
        return self.models[0].module()

    def to_json(self) -> str:
        return json.dumps({"task": str(self.task), "classes": self.classes, "kind": self.kind,
                           "models": [json.loads(m.to_json()) for m in self.models]})

    @staticmethod
    def from_json(s: str) -> "Ensemble":
        from .base import as_task
        d = json.loads(s)
        return Ensemble(as_task(d["task"]), d["classes"], [Model.from_json(json.dumps(m)) for m in d["models"]], d["kind"])


def _table(d, task, classes):
    from .base import CLASSIFICATION, as_task, count_classes
    task = as_task(task)
    d.check(task)
    return task, (count_classes(d.Y, classes) if task is CLASSIFICATION else 0)


class _workers:
    """``with _workers(n):`` the native tree code uses ``n`` threads inside (None: as many as it has now;
    tree/options.go: Workers)."""

    def __init__(self, n):
        self.n, self.had = n, None

    def __enter__(self):
        if self.n is not None:
            from ..ops import quant_cpu
            self.had = quant_cpu.set_threads(int(self.n))

    def __exit__(self, *exc):
        if self.n is not None:
            from ..ops import quant_cpu
            quant_cpu.set_threads(self.had)


def boosting(d, task, classes: int = 0, **options) -> Ensemble:
    """Gradient boosting on a table: squared error for regression, logistic loss for two classes, softmax for
    more.  Options are ``gradient_boosting``'s (``trees``, ``learning_rate``, ``max_depth``, ``min_leaf``,
    ``min_gain``, ``min_weight``, ``l2``, ``subsample``, ``per_tree``, ``colsample``, ``bins``, ``seed``, ``validation``
    with ``patience``), and ``workers``: the threads the native code uses."""
    task, k = _table(d, task, classes)
    with _workers(options.pop("workers", None)):
        return Ensemble(task, k, [gradient_boosting(d.X, d.Y, classes=k, **options)], "boost")


def forest(d, task, classes: int = 0, **options) -> Ensemble:
    """A random forest on a table; for classification one regression forest per class on its indicator, whose
    averaged leaves are the class's probability."""
    task, k = _table(d, task, classes)
    seed = options.pop("seed", 0)
    with _workers(options.pop("workers", None)):
        if not k:
            return Ensemble(task, 0, [random_forest(d.X, d.Y, seed=seed, **options)], "forest")
        return Ensemble(task, k, [random_forest(d.X, (d.Y == c).float(), seed=seed + c, **options) for c in range(k)], "forest")


def single(d, task, classes: int = 0, **options) -> Ensemble:
    """One decision tree on a table."""
    task, k = _table(d, task, classes)
    return Ensemble(task, k, [decision_tree(d.X, d.Y, classes=k, **options)], "tree")
