"""Classical models on the host against scikit-learn on the same synthetic tables.

    python -m mimir_b200.utils.bench_ml [--rows 20000] [--repeat 3] [--only NAME ...]

Prints one JSON line per model: fit seconds here and in scikit-learn (the best of ``--repeat`` runs, after
one warm-up) and a quality figure of each (accuracy, R^2, inertia ratio), so a speed-up that costs quality
shows.  ``--gate 2`` makes it a check: the exit code is 1 when some model takes more than twice scikit-learn's
time.  scikit-learn is optional: without it only this library's figures are printed."""
from __future__ import annotations

import argparse
import json
import math
import time

import torch


def _best(fn, repeat):
    fn()
    best, out = math.inf, None
    for _ in range(repeat):
        t = time.perf_counter()
        out = fn()
        best = min(best, time.perf_counter() - t)
    return best, out


def _tables(rows, seed=0):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(rows, 20, generator=g)
    w = torch.randn(20, generator=g)
    y_reg = X @ w + torch.sin(X[:, 0] * 2) * 3 + 0.1 * torch.randn(rows, generator=g)
    y_cls = ((X @ w + X[:, 0] * X[:, 1] * 2) > 0).long()
    centers = torch.randn(8, 20, generator=g) * 4
    which = torch.randint(0, 8, (rows,), generator=g)
    blobs = centers[which] + torch.randn(rows, 20, generator=g)
    return X, y_reg, y_cls, blobs, which


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=20000)
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--only", nargs="*", default=None)
    ap.add_argument("--gate", type=float, default=0.0, help="exit 1 when a model takes more than this many times scikit-learn's time")
    a = ap.parse_args(argv)
    from .. import ml
    from ..ml import cluster, decompose, linear, neighbors, svm, tree
    try:
        import sklearn.cluster
        import sklearn.decomposition
        import sklearn.ensemble
        import sklearn.linear_model
        import sklearn.neighbors
        import sklearn.svm
        sk = sklearn
    except ImportError:
        sk = None
    X, y_reg, y_cls, blobs, which = _tables(a.rows)
    Xn, yrn, ycn, bn = X.numpy(), y_reg.numpy(), y_cls.numpy(), blobs.numpy()
    half = a.rows // 2
    acc = lambda p, y: float((p == y).float().mean())  # noqa: E731
    r2 = lambda p, y: float(1 - ((p - y) ** 2).sum() / ((y - y.mean()) ** 2).sum())  # noqa: E731
    d_cls, d_reg = ml.Data(X[:half], y_cls[:half]), ml.Data(X[:half], y_reg[:half])

    cases = {
        "logistic": (lambda: linear.logistic_fit(d_cls), lambda m: acc(m.classify(X[half:]), y_cls[half:]),
                     lambda: sk.linear_model.LogisticRegression(max_iter=1000).fit(Xn[:half], ycn[:half]),
                     lambda m: float(m.score(Xn[half:], ycn[half:]))),
        "ridge": (lambda: linear.regression(d_reg, l2=1e-3), lambda m: r2(m.predict(X[half:]), y_reg[half:]),
                  lambda: sk.linear_model.Ridge(alpha=1e-3 * half).fit(Xn[:half], yrn[:half]), lambda m: float(m.score(Xn[half:], yrn[half:]))),
        "lasso": (lambda: linear.regression(d_reg, l1=0.05), lambda m: r2(m.predict(X[half:]), y_reg[half:]),
                  lambda: sk.linear_model.Lasso(alpha=0.05).fit(Xn[:half], yrn[:half]), lambda m: float(m.score(Xn[half:], yrn[half:]))),
        "linear_svm": (lambda: svm.fit(d_cls, "classification", kernel="linear"), lambda m: acc(m.classify(X[half:]), y_cls[half:]),
                       lambda: sk.svm.LinearSVC(loss="hinge", dual=True, max_iter=1000).fit(Xn[:half], ycn[:half]),
                       lambda m: float(m.score(Xn[half:], ycn[half:]))),
        "rbf_svm_4k": (lambda: svm.fit(ml.Data(X[:4000], y_cls[:4000]), "classification"), lambda m: acc(m.classify(X[half:half + 4000]), y_cls[half:half + 4000]),
                       lambda: sk.svm.SVC(probability=False).fit(Xn[:4000], ycn[:4000]), lambda m: float(m.score(Xn[half:half + 4000], ycn[half:half + 4000]))),
        "boosting": (lambda: tree.gradient_boosting(X[:half], y_cls[:half], trees=50, max_depth=6, classes=2, min_leaf=20, l2=0.0),
                     lambda m: acc(m.classify(X[half:]), y_cls[half:]),
                     lambda: sk.ensemble.HistGradientBoostingClassifier(max_iter=50, max_depth=6, early_stopping=False).fit(Xn[:half], ycn[:half]),
                     lambda m: float(m.score(Xn[half:], ycn[half:]))),
        "forest": (lambda: tree.random_forest(X[:half], y_cls[:half], trees=50, max_depth=10, classes=2),
                   lambda m: acc((m.raw(X[half:]) > 0.5).long(), y_cls[half:]),
                   lambda: sk.ensemble.RandomForestClassifier(50, max_depth=10, n_jobs=-1).fit(Xn[:half], ycn[:half]),
                   lambda m: float(m.score(Xn[half:], ycn[half:]))),
        "kmeans": (lambda: cluster.kmeans_fit(blobs, 8, inits=4), lambda m: m.inertia / a.rows,
                   lambda: sk.cluster.KMeans(8, n_init=4, random_state=0).fit(sklearn.preprocessing.scale(bn)), lambda m: float(m.inertia_) / a.rows),
        "dbscan_10k": (lambda: cluster.dbscan_fit(blobs[:10000], eps=3.0, min_rows=5), lambda m: float(m.groups),
                       lambda: sk.cluster.DBSCAN(eps=3.0, min_samples=5).fit(sklearn.preprocessing.scale(bn[:10000])),
                       lambda m: float(m.labels_.max() + 1)),
        "ward_5k": (lambda: cluster.agglomerative(blobs[:5000], 8), lambda m: m.means.inertia / 5000,
                    lambda: sk.cluster.AgglomerativeClustering(8).fit(sklearn.preprocessing.scale(bn[:5000])),
                    lambda m: float(sum(((sklearn.preprocessing.scale(bn[:5000])[m.labels_ == c] - sklearn.preprocessing.scale(bn[:5000])[m.labels_ == c].mean(0)) ** 2).sum()
                                        for c in range(8))) / 5000),
        "knn_predict": (lambda: neighbors.fit(d_cls, "classification").classify(X[half:half + 2000]), lambda p: acc(p, y_cls[half:half + 2000]),
                        lambda: sk.neighbors.KNeighborsClassifier(5, algorithm="brute").fit(Xn[:half], ycn[:half]).predict(Xn[half:half + 2000]),
                        lambda p: float((torch.as_tensor(p) == y_cls[half:half + 2000]).float().mean())),
        "pca": (lambda: decompose.pca_fit(X, 5), lambda m: float(m.ratio.sum()),
                lambda: sk.decomposition.PCA(5).fit(sklearn.preprocessing.scale(Xn)), lambda m: float(m.explained_variance_ratio_.sum())),
    }
    if sk is not None:
        import sklearn.preprocessing  # noqa: F401
    slow = []
    for name, (ours, q_ours, theirs, q_theirs) in cases.items():
        if a.only and name not in a.only:
            continue
        t, m = _best(ours, a.repeat)
        line = {"model": name, "rows": a.rows, "seconds": round(t, 4), "quality": round(q_ours(m), 4)}
        if sk is not None:
            t2, m2 = _best(theirs, a.repeat)
            line.update(sklearn_seconds=round(t2, 4), sklearn_quality=round(q_theirs(m2), 4), speedup=round(t2 / t, 2))
            if a.gate > 0 and t > a.gate * t2:
                slow.append(name)
        print(json.dumps(line), flush=True)
    if slow:
        raise SystemExit(f"slower than {a.gate} x scikit-learn: {', '.join(slow)}")


if __name__ == "__main__":
    main()
