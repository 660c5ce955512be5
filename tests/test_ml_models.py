"""The table-level models: what each recovers on data whose answer is known, options, missing values,
JSON round trips, errors, and that a model's ``nn.Module`` answers as its ``predict`` does (the
categories of the reference's tests under linear/, svm/, neighbors/, bayes/, cluster/, decompose/,
forecast/, recommend/, rules/, automl/ and tabular/)."""
import math

import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200 import ml
from mimir_b200.ml import automl, bayes, cluster, decompose, forecast, linear, neighbors, recommend, rules, svm, tree
from mimir_b200.ml.tabular import Data, cross_validate


def blobs(n=150, d=4, gap=1.5, seed=0):
    g = torch.Generator().manual_seed(seed)
    X = torch.cat([torch.randn(n, d, generator=g) + gap, torch.randn(n, d, generator=g) - gap])
    return X, (torch.arange(2 * n) >= n).long()


def three(seed=1):
    g = torch.Generator().manual_seed(seed)
    C = torch.cat([torch.randn(80, 2, generator=g) * 0.5 + torch.tensor([4.0, 0.0]), torch.randn(80, 2, generator=g) * 0.5 - torch.tensor([4.0, 0.0]),
                   torch.randn(80, 2, generator=g) * 0.5 + torch.tensor([0.0, 5.0])])
    return C, torch.arange(3).repeat_interleave(80)


def pure(assign, truth, k=3):
    return all(len(set(assign[truth == j].tolist())) == 1 for j in range(k)) and len(set(assign.tolist())) == k


def module_matches(model, Q, soft=True, tol=1e-4):
    out = model.module()(T.tensor(Q)).data()
    want = model.predict(Q)
    got = torch.softmax(out, 1) if soft else out[:, 0]
    return float((got - want).abs().max()) < tol


# ------------------------------------------------------------------ tabular
def test_table_checks_splits_and_cross_validation():
    X, y = blobs(20)
    d = Data(X, y)
    d.check("classification")
    assert d.rows == 40 and d.classes() == 2 and d.n_features == 4
    assert Data(X.reshape(-1).tolist(), y, n_features=4).rows == 40
    tr, te = d.split(0.25, seed=3)
    both = torch.cat([tr.X, te.X])
    assert len(te) == 10 and len(tr) == 30 and torch.equal(both.sort(0).values, X.sort(0).values)      # every row exactly once
    seen = []
    scores = cross_validate(lambda t: len(t), lambda m, h: seen.append(h.X) or m, d, folds=4)
    assert scores == [30.0] * 4 and torch.equal(torch.cat(seen).sort(0).values, X.sort(0).values)
    with pytest.raises(ValueError):
        Data(X, y.float() + 0.5).check("classification")
    with pytest.raises(ValueError):
        Data(X, y[:3]).check("regression")
    with pytest.raises(ValueError):
        Data(torch.zeros(0, 3), torch.zeros(0)).check()
    with pytest.raises(ValueError):
        cross_validate(None, None, d, folds=1)


# ------------------------------------------------------------------ linear
def test_least_squares_ridge_and_lasso():
    g = torch.Generator().manual_seed(0)
    X = torch.randn(400, 6, generator=g) * torch.tensor([1, 5, 0.1, 2, 1, 1.0]) + 3
    w = torch.tensor([2.0, -1, 0, 0, 0.5, 0])
    y = X @ w + 1 + 0.01 * torch.randn(400, generator=g)
    m = linear.regression(Data(X, y))
    assert torch.allclose(m.weights[0], w, atol=0.02) and abs(float(m.bias) - 1) < 0.05 and abs(m.weight(0, 1) + 1) < 0.02
    # ridge against its closed form on standardized features
    l2 = 0.5
    mu, sd = X.double().mean(0), X.double().std(0, unbiased=False)
    Z = (X.double() - mu) / sd
    ws = torch.linalg.solve(Z.t() @ Z / 400 + l2 * torch.eye(6, dtype=torch.double), Z.t() @ (y.double() - y.double().mean()) / 400)
    assert torch.allclose(linear.regression(Data(X, y), l2=l2).weights[0].double(), ws / sd, atol=1e-5)
    lasso = linear.regression(Data(X, y), l1=0.05)
    assert (lasso.weights[0][[2, 3, 5]] == 0).all() and (lasso.weights[0][[0, 1, 4]].abs() > 0.3).all()


def test_logistic_recovers_log_odds_classes_and_sparsity():
    g = torch.Generator().manual_seed(1)
    X = torch.randn(4000, 3, generator=g)
    w = torch.tensor([1.5, -2.0, 0.0])
    yc = (torch.rand(4000, generator=g) < torch.sigmoid(X @ w + 0.5)).long()
    m = linear.logistic_fit(Data(X, yc), l2=1e-6)
    assert torch.allclose(m.weights[0], w, atol=0.15) and abs(float(m.bias) - 0.5) < 0.15
    p = m.predict(X[:5])
    assert p.shape == (5, 2) and torch.allclose(p.sum(1), torch.ones(5))
    C, truth = three()
    m3 = linear.logistic_fit(Data(C, truth))
    assert (m3.classify(C) == truth).float().mean() > 0.99 and m3.predict(C).shape == (240, 3)
    sparse = linear.logistic_fit(Data(X, yc), l1=0.05)
    assert sparse.weights[0, 2] == 0 and sparse.weights[0, 0] > 0.5 and sparse.weights[0, 1] < -0.5
    assert module_matches(m, X[:9]) and module_matches(m3, C[::20]) and module_matches(linear.regression(Data(X, X @ w)), X[:9], soft=False)


def test_missing_and_constant_features_json_and_bad_input():
    X, y = blobs()
    X = torch.cat([X, torch.full((300, 1), 7.0)], 1)            # a constant feature
    Xn = X.clone()
    Xn[::5, 0] = math.nan
    m = linear.logistic_fit(Data(Xn, y))
    assert (m.classify(Xn) == y).float().mean() > 0.97 and m.weights[0, 4] == 0 and torch.isfinite(m.predict(Xn)).all()
    again = linear.Linear.from_json(m.to_json())
    assert torch.equal(again.predict(Xn), m.predict(Xn))
    with pytest.raises(ValueError):
        linear.Linear.from_json(svm.fit(Data(X, y), "classification", kernel="linear").to_json())
    with pytest.raises(ValueError):
        linear.regression(Data(X, y.float()), l1=-1)
    with pytest.raises(ValueError):
        linear.logistic_fit(Data(X, torch.zeros(300)))


# ------------------------------------------------------------------ svm
def test_kernels_separate_rings_and_linear_separates_blobs():
    g = torch.Generator().manual_seed(0)
    r = torch.cat([torch.rand(150, generator=g), 2 + torch.rand(150, generator=g)])
    th = torch.rand(300, generator=g) * 2 * math.pi
    P, lab = torch.stack([r * th.cos(), r * th.sin()], 1), (torch.arange(300) >= 150).long()
    for kernel, kw in (("rbf", {}), ("polynomial", dict(coef0=1.0, degree=2))):
        m = svm.fit(Data(P, lab), "classification", kernel=kernel, c=10.0, **kw)
        assert (m.classify(P) == lab).float().mean() > 0.98 and 0 < m.support_vectors() < 150
        assert module_matches(m, P[::17], tol=1e-3)
    assert (svm.fit(Data(P, lab), "classification", kernel="linear").classify(P) == lab).float().mean() < 0.8     # no line splits rings
    X, y = blobs(2000, 5)
    lin = svm.fit(Data(X, y), "classification", kernel="linear")
    assert (lin.classify(X) == y).float().mean() > 0.99 and lin.support_vectors() == 0 and module_matches(lin, X[::333], tol=1e-3)
    C, truth = three()
    m3 = svm.fit(Data(C, truth), "classification")
    p = m3.predict(C)
    assert (p.argmax(1) == truth).float().mean() > 0.99 and torch.allclose(p.sum(1), torch.ones(240), atol=1e-5)
    assert module_matches(m3, C[::20], tol=1e-3)
    assert torch.allclose(svm.SVM.from_json(m3.to_json()).predict(C), p)


def test_support_vector_regression_and_bad_options():
    x = torch.linspace(-3, 3, 200)[:, None]
    y = torch.sin(x[:, 0]) * 2 + 5
    m = svm.fit(Data(x, y), "regression", c=10.0, epsilon=0.05)
    assert float(((m.predict(x) - y) ** 2).mean().sqrt()) < 0.15 and m.support_vectors() < 60
    assert module_matches(m, x[::20], soft=False, tol=1e-3)
    for bad in (dict(c=0), dict(kernel="wavelet"), dict(gamma=-1.0), dict(epsilon=-0.1)):
        with pytest.raises(ValueError):
            svm.fit(Data(x, y), "regression", **bad)


# ------------------------------------------------------------------ neighbours and naive Bayes
def test_neighbours_classify_regress_and_list():
    X, y = blobs()
    m = neighbors.fit(Data(X, y), "classification", k=7, by_distance=True)
    assert (m.classify(X) == y).all()                                        # each row is its own nearest neighbour
    idx, dist = m.neighbors(X[:3])
    assert idx[:, 0].tolist() == [0, 1, 2] and float(dist[:, 0].max()) < 1e-3 and (dist[:, 1:] >= dist[:, :-1]).all()
    for metric in neighbors.METRICS:
        mm = neighbors.fit(Data(X, y), "classification", metric=metric, raw=metric == "manhattan")
        assert (mm.classify(X) == y).float().mean() > 0.97 and module_matches(mm, X[::31])
    r = neighbors.fit(Data(X, X[:, 0] * 2), "regression", k=3)
    assert float(((r.predict(X) - X[:, 0] * 2) ** 2).mean()) < 0.3 and module_matches(r, X[::31], soft=False)
    assert module_matches(m, X[::31])
    with pytest.raises(ValueError):
        neighbors.fit(Data(X, y), "classification", k=0)
    with pytest.raises(ValueError):
        neighbors.fit(Data(X, y), "classification", metric="chebyshev")


def test_naive_bayes_kinds_priors_and_missing_values():
    X, y = blobs()
    g = bayes.gaussian(Data(X, y))
    assert (g.classify(X) == y).float().mean() > 0.98 and module_matches(g, X[::31])
    Xn = X[:4].clone()
    Xn[0, 1] = math.nan                                                      # left out of the row's likelihood
    keep = [0, 2, 3]
    sub = bayes.gaussian(Data(X[:, keep], y))
    assert torch.allclose(g.log_likelihood(Xn)[0], sub.log_likelihood(X[:1][:, keep])[0], atol=1e-9)
    gen = torch.Generator().manual_seed(0)
    counts = torch.poisson(torch.cat([torch.tensor([[5.0, 1, 1]]).repeat(100, 1), torch.tensor([[1.0, 1, 5]]).repeat(100, 1)]), generator=gen)
    yc = (torch.arange(200) >= 100).long()
    mn, bn = bayes.multinomial(Data(counts, yc)), bayes.bernoulli(Data(counts, yc), binarize=2.5)
    assert (mn.classify(counts) == yc).float().mean() > 0.9 and (bn.classify(counts) == yc).float().mean() > 0.85
    assert module_matches(mn, counts[::13]) and module_matches(bn, counts[::13])
    skew = bayes.gaussian(Data(X, y), priors=[0.999, 0.001])
    assert (skew.classify(X) == 0).sum() >= (g.classify(X) == 0).sum()
    assert torch.allclose(bayes.NaiveBayes.from_json(mn.to_json()).predict(counts), mn.predict(counts))
    with pytest.raises(ValueError):
        bayes.multinomial(Data(-counts, yc))
    with pytest.raises(ValueError):
        bayes.gaussian(Data(X, y), priors=[0.5, 0.2])


# ------------------------------------------------------------------ cluster, decompose
def test_groupings_find_the_blobs():
    C, truth = three()
    km = cluster.kmeans_fit(C, 3)
    assert pure(km.assign(C), truth) and km.predict(C).sum(1).eq(1).all() and cluster.silhouette(km, C) > 0.7
    mx = cluster.gaussian_mixture(C, 3)
    assert pure(mx.assign(C), truth) and torch.allclose(mx.weights, torch.full((3,), 1 / 3), atol=1e-3)
    assert float(mx.log_density(torch.tensor([[20.0, 20.0]]))) < float(mx.log_density(C[:1])) - 100
    assert torch.equal(km.module()(T.tensor(C)).data().argmax(1), km.assign(C)) and module_matches(mx, C[::20])
    db = cluster.dbscan_fit(torch.cat([C, torch.tensor([[40.0, 40.0]])]), 0.3)
    assert db.groups == 3 and db.labels[-1] == cluster.NOISE and pure(db.labels[:-1], truth)
    assert db.assign(torch.tensor([[4.0, 0.0], [30.0, 30.0]])).tolist() == [int(db.labels[0]), cluster.NOISE]
    ag = cluster.agglomerative(C, 3)
    h = ag.heights()
    assert pure(ag.cut(3), truth) and (h[1:] >= h[:-1]).all() and h[-2] > 20 * h[-3]       # two big jumps: three groups
    assert ag.cut(0).unique().tolist() == [0] and pure(ag.assign(C), truth) and ag.cut(240).unique().numel() == 240
    assert cluster.silhouette(ag.centers(C, 2), C) < cluster.silhouette(ag, C)
    for model, cls in ((km, cluster.Means), (mx, cluster.Mixture), (db, cluster.Density), (ag, cluster.Linkage)):
        again = cls.from_json(model.to_json())
        assert torch.equal(again.assign(C), model.assign(C))
    for bad in (lambda: cluster.kmeans_fit(C, 0), lambda: cluster.kmeans_fit(C, 500), lambda: cluster.dbscan_fit(C, -1.0),
                lambda: cluster.agglomerative(C, 0), lambda: cluster.kmeans_fit(torch.zeros(0, 2), 1)):
        with pytest.raises(ValueError):
            bad()


def test_pca_finds_the_shared_direction():
    g = torch.Generator().manual_seed(0)
    X = torch.randn(300, 1, generator=g) @ torch.tensor([[1.0, 2, 0.5]]) + 0.1 * torch.randn(300, 3, generator=g)
    p = decompose.pca_fit(X, 2)
    assert p.k == 2 and p.ratio[0] > 0.95 and torch.allclose(p.directions[0].abs(), torch.full((3,), 3 ** -0.5), atol=0.02)
    assert sorted(p.ranked(0)) == [0, 1, 2] and abs(float(p.directions[0] @ p.directions[1])) < 1e-5
    full = decompose.pca_fit(X, 3)
    assert torch.allclose(full.inverse(full.transform(X)), X, atol=1e-4)
    wide = decompose.pca_fit(torch.randn(5, 12, generator=g), 3)                 # more features than rows
    assert wide.transform(torch.randn(2, 12)).shape == (2, 3)
    with pytest.raises(ValueError):
        decompose.pca_fit(X, 4)


# ------------------------------------------------------------------ forecast, recommend, rules, automl
def test_forecast_learns_the_week_with_gaps():
    g = torch.Generator().manual_seed(0)
    week = torch.tensor([5.0, 6, 7, 8, 9, 3, 2])
    series = [week.repeat(20) * s + 0.1 * s * torch.randn(140, generator=g) for s in (1.0, 10.0, 300.0)]
    series[0][30:33] = math.nan
    m = forecast.fit(series, season=7, trees=80)
    f = m.forecast(series[1][:133], 7)
    assert float((f - week * 10).abs().max()) < 2.0 and m.features == 18
    row, scale = m.rows(series[1][:133])
    assert row.shape == (18,) and abs(float(m.trees.predict(row[None])[0]) * scale - float(f[0])) < 1e-4
    assert torch.allclose(forecast.Forecaster.from_json(m.to_json()).forecast(series[1][:133], 3), f[:3])
    s = forecast.smooth(week.repeat(10) + torch.arange(70) * 0.1, season=7)
    assert torch.allclose(s.forecast(7), week + 7.0 + torch.arange(7) * 0.1, atol=0.2)
    with pytest.raises(ValueError):
        forecast.fit([torch.arange(5.0)])
    with pytest.raises(ValueError):
        forecast.smooth([1.0, 2.0], season=7)


def test_recommendations_beat_popularity_and_ratings_predict():
    g = torch.Generator().manual_seed(0)
    events = []
    for u in range(40):
        for i in (range(0, 10) if u % 2 == 0 else range(10, 20)):
            if torch.rand(1, generator=g) < 0.6:
                events.append((u, i, 1.0))
    held = [(u, i, 1.0) for u in range(0, 40, 2) for i in range(10) if (u, i, 1.0) not in events][:20]
    m = recommend.fit(40, 20, events, factors=4, iterations=10)
    assert m.hit_rate(events, held, 5) >= 0.8                                   # popularity alone would name the other taste half the time
    seen = [i for u, i, _ in events if u == 0]
    top = m.recommend(0, 3, seen)
    assert all(i < 10 and i not in seen for i in top) and all(i < 10 for i in m.similar(0, 3))
    assert m.score(0, top[0]) > m.score(0, 15)
    pairs = torch.tensor([[0, 1], [3, 12]])
    out = m.module()(T.tensor(pairs)).data()[:, 0]
    assert torch.allclose(out, torch.tensor([m.score(0, 1), m.score(3, 12)]), atol=1e-6)
    r = recommend.fit(3, 3, [(0, 0, 5), (0, 1, 3), (1, 0, 4), (1, 1, 2), (2, 1, 1), (2, 2, 5)], factors=2, ratings=True, l2=0.01, iterations=30)
    assert abs(r.score(0, 0) - 5) < 0.1 and abs(r.score(1, 1) - 2) < 0.1
    for bad in ([(0, 99, 1.0)], [(0, 0, -1.0)], []):
        with pytest.raises(ValueError):
            recommend.fit(3, 3, bad)


def test_rules_find_what_goes_together():
    baskets = [["bread", "butter"], ["bread", "butter", "jam"], ["bread"], ["butter", "jam"], ["bread", "butter"], ["tea"]]
    out = rules.mine(baskets, 0.3, 0.6)
    first = out[0]
    assert first.if_ == ("jam",) and first.then == ("butter",) and first.confidence == 1.0 and abs(first.lift - 1.5) < 1e-9
    assert all(a.lift >= b.lift for a, b in zip(out, out[1:])) and len(rules.mine(baskets, 0.3, 0.6, top=1)) == 1
    assert not any("tea" in r.if_ + r.then for r in out)
    with pytest.raises(ValueError):
        rules.mine([], 0.3)
    with pytest.raises(ValueError):
        rules.mine(baskets, 0.0)


def test_search_picks_what_fits():
    g = torch.Generator().manual_seed(0)
    X = torch.randn(300, 5, generator=g)
    y = X @ torch.tensor([1.0, -2, 0.5, 0, 0]) + 0.01 * torch.randn(300, generator=g)
    told = []
    r = automl.search(Data(X, y), "regression", trials=5, folds=2, progress=lambda a, b: told.append((a, b)))
    assert r.candidate.family == automl.LINEAR and r.score < 0.05 and told[-1] == (5, 5) and len(r.trials) == 5
    assert float(((r.best.predict(X) - y) ** 2).mean()) < 0.01
    step = (X[:, 0] * X[:, 1] > 0).long()                                     # no line splits it
    rc = automl.search(Data(X, step), "classification", trials=6, folds=2, families=(automl.BOOST, automl.LINEAR))
    assert rc.candidate.family == automl.BOOST and {t.candidate.family for t in rc.trials} == {automl.BOOST, automl.LINEAR}
    assert (rc.best.classify(X) == step).float().mean() > 0.95 and str(rc.candidate).startswith("boost(")
    quick = automl.search(Data(X, y), "regression", trials=12, budget=0.0)
    assert len(quick.trials) == 1
    with pytest.raises(ValueError):
        automl.search(Data(X, y), "regression", families=("oracle",))


def test_boosting_stops_when_a_validation_table_stops_improving():
    g = torch.Generator().manual_seed(0)
    X = torch.randn(600, 5, generator=g)
    y = torch.sin(X[:, 0]) * 2 + X[:, 1] + 0.3 * torch.randn(600, generator=g)
    m = tree.gradient_boosting(X[:400], y[:400], trees=300, max_depth=4, validation=(X[400:], y[400:]), patience=5)
    assert len(m.trees) < 150 and abs(m.validation_loss - float(((m.predict(X[400:]) - y[400:]) ** 2).mean())) < 1e-5
    out = m.module()(T.tensor(X[:7])).data()[:, 0]
    assert torch.allclose(out, m.predict(X[:7]), atol=1e-5)
    y3 = torch.bucketize(X[:, 0].contiguous(), torch.tensor([-0.5, 0.5]))
    m3 = tree.gradient_boosting(X, y3, trees=8, max_depth=3, classes=3)
    assert torch.allclose(torch.softmax(m3.module()(T.tensor(X[:7])).data(), 1), m3.predict(X[:7]), atol=1e-6)
    empty = type(m3.module()).empty(m3.module().shape)
    empty.load_state_dict(m3.module().state_dict())
    assert torch.equal(empty(T.tensor(X[:7])).data(), m3.module()(T.tensor(X[:7])).data())


def test_table_level_trees_answer_with_probabilities_and_round_trip():
    g = torch.Generator().manual_seed(0)
    X = torch.randn(400, 5, generator=g)
    y3 = torch.bucketize(X[:, 0].contiguous(), torch.tensor([-0.5, 0.5]))
    yr = X[:, 0] * 2 + X[:, 1]
    for make, kw in ((tree.boosting, dict(trees=15)), (tree.forest, dict(trees=15)), (tree.single, {})):
        m = make(Data(X, y3), "classification", **kw)
        p = m.predict(X)
        assert p.shape == (400, 3) and torch.allclose(p.sum(1), torch.ones(400), atol=1e-5)
        assert (m.classify(X) == y3).float().mean() > 0.95 and int(m.importance().argmax()) == 0
        assert torch.allclose(tree.Ensemble.from_json(m.to_json()).predict(X), p)
        r = make(Data(X, yr), "regression", **kw)
        assert r.predict(X).shape == (400,) and float(((r.predict(X) - yr) ** 2).mean()) < 0.5
    two = tree.boosting(Data(X, (X[:, 1] > 0).long()), "classification", trees=10, max_depth=3)
    assert two.predict(X).shape == (400, 2)
    assert torch.allclose(torch.softmax(two.module()(T.tensor(X[:5])).data(), 1), two.predict(X[:5]), atol=1e-6)
    with pytest.raises(ValueError):
        tree.boosting(Data(X, yr), "classification")


def test_modules_save_load_and_export_like_networks(tmp_path):
    """A fitted model's module keeps its tables in a .mim file, loads into an empty module of the same shape,
    and exports as a graph that the interpreter runs on another batch size (missing values included)."""
    import os
    from mimir_b200.io import export, mim
    g = torch.Generator().manual_seed(0)
    X = torch.randn(300, 5, generator=g)
    y, y3 = (X[:, 0] > 0).long(), torch.bucketize(X[:, 1].contiguous(), torch.tensor([-0.5, 0.5]))
    d = Data(X, y)
    Q = torch.randn(7, 5, generator=g)
    Q[0, 0] = math.nan
    models = {
        "logistic": linear.logistic_fit(d), "svm": svm.fit(d, "classification"), "bayes": bayes.gaussian(d),
        "knn": neighbors.fit(d, "classification", by_distance=True), "knn_manhattan": neighbors.fit(Data(X, X[:, 0]), "regression", metric="manhattan"),
        "kmeans": cluster.kmeans_fit(X, 3), "mixture": cluster.gaussian_mixture(X, 2),
        "boost2": tree.gradient_boosting(X, y, trees=5, max_depth=3, classes=2), "boost3": tree.gradient_boosting(X, y3, trees=4, max_depth=3, classes=3),
        "forest": tree.random_forest(X, X[:, 0] * 2, trees=5, max_depth=4),
    }
    for name, model in models.items():
        mod = model.module()
        want = mod(T.tensor(Q)).data()
        assert torch.isfinite(want).all(), name
        path = os.path.join(tmp_path, name + ".mim")
        mim.save(path, mod)
        fresh = type(mod).empty(mod.shape)
        with mim.open(path) as f:
            fresh.load_state_dict(f.load())
        assert torch.equal(fresh(T.tensor(Q)).data(), want), name
        graph = os.path.join(tmp_path, name + "-graph.mim")
        export.export(graph, mod, X[:4], input_name="x", output_name="y", dynamic={"x": {0: ("batch", 64)}})
        with mim.open(graph) as f:
            got = f.run({"x": Q})["y"].data()
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-4), (name, float((got - want).abs().max()))


@pytest.mark.parametrize("kw", [dict(classes=2), dict(classes=0), dict(classes=2, colsample=0.5)])
def test_boosting_rounds_in_one_native_call_grow_the_trees_of_the_per_round_loop(kw):
    """Regression and two-class boosting without row sampling or validation run every round inside one native
    call; the per-round loop is the oracle: the same splits in every tree, leaf values within float rounding
    (the native sigmoid and PyTorch's differ in the last bit), the same importances."""
    from mimir_b200.ml import tree
    g = torch.Generator().manual_seed(5)
    X = torch.randn(6000, 8, generator=g)
    score = X[:, 0] * 2 + X[:, 1] * X[:, 2] + 0.1 * torch.randn(6000, generator=g)
    y = (score > 0).long() if kw["classes"] else score
    a = tree.gradient_boosting(X, y, trees=12, max_depth=4, min_leaf=5, seed=3, **kw)
    b = tree.gradient_boosting(X, y, trees=12, max_depth=4, min_leaf=5, seed=3, native_rounds=False, **kw)
    assert len(a.trees) == len(b.trees) == 12
    for ta, tb in zip(a.trees, b.trees):
        assert [q[:4] for q in ta.nodes] == [q[:4] for q in tb.nodes]
        assert max(abs(p[4] - q[4]) for p, q in zip(ta.nodes, tb.nodes)) < 1e-5
    assert float((a.raw(X) - b.raw(X)).abs().max()) < 1e-4
    assert torch.allclose(a.importance(), b.importance(), atol=1e-5)
    lines = []

    class Sink:
        def write(self, s):
            lines.append(s)
    tree.gradient_boosting(X, y, trees=20, max_depth=3, progress=Sink(), **kw)
    assert lines == ["tree 10/20\n", "tree 20/20\n"]


def test_native_binning_and_ensemble_prediction_agree_with_the_tensor_ops():
    """``bin_table`` is ``torch.searchsorted`` per feature (NaN after every edge, infinities, repeated edges),
    by rows and by columns; the one-pass ensemble prediction is the sum of the trees walked one by one, for two
    classes, several classes and forests; a table that is not a tree is refused, not walked."""
    from mimir_b200.ml import tree
    g = torch.Generator().manual_seed(9)
    X = torch.randn(5003, 7, generator=g)
    X[::11, 2] = float("nan")
    X[5, 1], X[6, 1] = float("inf"), -float("inf")
    edges = torch.quantile(torch.randn(4096, 7, generator=g), torch.linspace(0, 1, 256)[1:-1], dim=0).t().contiguous()
    edges[3, 100:110] = edges[3, 100]
    B, C = tree.bin_table(X, edges, columns=True)
    assert B.dtype == torch.uint8 and torch.equal(B.long(), torch.searchsorted(edges, X.t().contiguous()).t())
    assert torch.equal(B.t(), C)
    assert torch.equal(tree.bin_table(X, edges[:, :0]), torch.zeros(5003, 7, dtype=torch.uint8))
    Xc = torch.nan_to_num(X, nan=0.0, posinf=3.0, neginf=-3.0)
    y3 = (Xc[:, 0] > 0.5).long() + (Xc[:, 1] > 0).long()
    for m in (tree.gradient_boosting(Xc, (y3 > 0).long(), trees=8, max_depth=4, classes=2),
              tree.gradient_boosting(Xc, y3, trees=5, max_depth=3, classes=3),
              tree.random_forest(Xc, Xc[:, 0] * Xc[:, 1], trees=6, max_depth=5)):
        Bm = m._binned(X)
        groups = [[r[k] for r in m.trees] for k in range(3)] if m.classes > 2 else [m.trees]
        for trees in groups:
            want = sum(t.predict_binned(Bm).double() for t in trees)
            assert torch.allclose(tree.Model._sum_of(trees, Bm).double(), want, atol=1e-5)
        assert m.raw(X).shape[0] == 5003
    t0 = m.trees[0]
    good = t0.nodes
    t0.nodes = [[0, 3, 0, 0, 0.0]] + [list(q) for q in good[1:]]      # a node that is its own child
    lib_answer = tree.Model._sum_of(m.trees, Bm)                        # falls back to the walks with a step limit
    assert torch.isfinite(lib_answer).all()
    t0.nodes = good


def test_forest_trees_grown_side_by_side_are_the_trees_grown_one_by_one():
    """A forest's trees grow in one native call, whole trees sharing the workers; growing them one at a time
    from the same generator gives the same trees, with and without bootstrap samples."""
    from mimir_b200.ml import tree
    g = torch.Generator().manual_seed(2)
    X = torch.randn(3000, 9, generator=g)
    y = X[:, 0] * X[:, 1] + X[:, 2]
    for kw in (dict(), dict(bootstrap=False), dict(colsample=0.8), dict(classes=2)):
        yy = (y > 0).float() if kw.get("classes") else y
        a = tree.random_forest(X, yy, trees=7, max_depth=6, seed=4, **kw)
        b = tree.random_forest(X, yy, trees=7, max_depth=6, seed=4, native_trees=False, **kw)
        assert [t.nodes for t in a.trees] == [t.nodes for t in b.trees], kw
        assert torch.allclose(a.importance(), b.importance(), atol=1e-6)
    r2 = 1 - ((a.raw(X) - yy) ** 2).sum() / ((yy - yy.mean()) ** 2).sum()
    assert float(r2) > 0.5


def test_tree_options_features_per_tree_features_per_node_smallest_child_weight_and_workers():
    """The reference's options: a share of the features per boosted tree, a count of features per forest node,
    the smallest hessian sum of a child, the number of threads (tree/options.go: ColSample, PerNode, MinWeight,
    Workers).  The native rounds and the per-round loop agree under each."""
    from mimir_b200.ml import tree
    from mimir_b200.ops import quant_cpu
    g = torch.Generator().manual_seed(0)
    X = torch.randn(3000, 10, generator=g)
    y = (X[:, 0] * X[:, 1] + X[:, 2] > 0).long()
    for kw in (dict(per_tree=0.5), dict(per_tree=0.5, colsample=0.6), dict(min_weight=5.0)):
        a = tree.gradient_boosting(X, y, trees=8, max_depth=4, classes=2, seed=1, **kw)
        b = tree.gradient_boosting(X, y, trees=8, max_depth=4, classes=2, seed=1, native_rounds=False, **kw)
        for ta, tb in zip(a.trees, b.trees):
            assert [q[:4] for q in ta.nodes] == [q[:4] for q in tb.nodes], kw
            if "per_tree" in kw:
                assert ta.allowed.numel() == 5 and {q[0] for q in ta.nodes if q[0] >= 0} <= set(ta.allowed.tolist())
        if "per_tree" in kw:
            assert len({tuple(t.allowed.tolist()) for t in a.trees}) > 1        # drawn afresh for each tree
    one = tree.gradient_boosting(X, y, trees=1, max_depth=8, classes=2, min_weight=5.0)
    leaf = one.trees[0].predict_binned(one._binned(X))
    assert min(int((leaf == v).sum()) for v in leaf.unique()) >= 20                # a hessian is at most 1/4
    f = tree.random_forest(X, y.float(), trees=4, max_depth=5, per_node=3)
    assert all(max(1, int(10 * t.colsample)) == 3 for t in f.trees)
    with pytest.raises(ValueError):
        tree.random_forest(X, y.float(), trees=1, per_node=11)
    had = quant_cpu.set_threads(0)
    quant_cpu.set_threads(had)
    e1 = tree.boosting(ml.Data(X, y), "classification", trees=5, workers=1)
    e4 = tree.boosting(ml.Data(X, y), "classification", trees=5, workers=4)
    assert torch.equal(e1.predict(X), e4.predict(X))                               # the trees do not depend on the threads
    assert quant_cpu.set_threads(had) == had                                       # and the setting is put back


def test_isolation_scores_in_one_native_pass_equal_the_tree_by_tree_walk():
    from mimir_b200.ml import tree
    g = torch.Generator().manual_seed(0)
    X = torch.randn(3000, 6, generator=g)
    X[:20] += 6
    X[40, 2] = float("nan")                                           # goes right at every cut on feature 2, in both walks
    m = tree.isolation_forest(X, trees=30, samples=128)
    walked = sum(m._path(t, X).double() for t in m.trees)
    assert torch.allclose(m._paths_native(X).double(), walked, atol=1e-3)
    s = m.score(X)
    assert float(s[:20].mean()) > float(s[100:].mean()) + 0.1


def test_native_density_groups_and_ward_chain_equal_the_tensor_op_paths():
    """DBSCAN on the host joins cores concurrently without keeping neighbour lists, Ward's chain runs from the
    clusters' means without a distance matrix; the tensor-op paths (neighbour lists and frontier growth; an
    n x n matrix under the Lance-Williams update) are their oracles: the same labels, noise and borders included,
    and the same merges at the same heights."""
    g = torch.Generator().manual_seed(4)
    centers = torch.randn(5, 4, generator=g) * 3
    X = centers[torch.randint(0, 5, (1500,), generator=g)] + 0.6 * torch.randn(1500, 4, generator=g)
    noise = borders = 0
    for eps, rows in ((0.25, 6), (0.4, 8), (0.6, 30)):
        a = cluster.dbscan_fit(X, eps=eps, min_rows=rows)
        b = cluster.dbscan_fit(X, eps=eps, min_rows=rows, native=False)
        assert torch.equal(a.labels, b.labels) and torch.equal(a.core_labels, b.core_labels) and a.groups == b.groups
        assert torch.equal(a.assign(X[:50]), b.assign(X[:50])) and a.groups >= 1
        noise += int((a.labels < 0).sum())
        borders += int((a.labels >= 0).sum()) - int(a.cores.shape[0])
    assert noise > 0 and borders > 0                                         # every kind of row was compared
    w = cluster.agglomerative(X[:700], 5)
    v = cluster.agglomerative(X[:700], 5, native=False)
    assert torch.equal(w.merges, v.merges) and torch.allclose(w.merge_heights, v.merge_heights, rtol=1e-9, atol=1e-9)
    assert torch.equal(w.cut(5), v.cut(5)) and torch.equal(w.cut(40), v.cut(40))
    one = cluster.agglomerative(X[:1], 1)
    assert one.merges.shape == (0, 2)


def test_native_least_squares_side_and_rules_counted_by_matrix_products():
    """One side of alternating least squares solved row by row in native code equals the batched tensor solve,
    with and without the shared B'B of implicit feedback and for rows without events; item sets counted by matrix
    products give the counts of a basket-by-basket count, with item names whose text order is not their numeric
    order and sets of up to four items."""
    import itertools
    g = torch.Generator().manual_seed(0)
    U, I, E, k = 120, 90, 2500, 6
    u, i = torch.randint(0, U - 5, (E,), generator=g), torch.randint(0, I, (E,), generator=g)      # the last five rows have no events
    for implicit in (True, False):
        A1 = torch.randn(U, k, generator=g, dtype=torch.double)
        A2, B = A1.clone(), torch.randn(I, k, generator=g, dtype=torch.double)
        conf, target = 1 + 10 * torch.rand(E, generator=g, dtype=torch.double), torch.rand(E, generator=g, dtype=torch.double)
        recommend._solve_side(A1, B, u, i, conf, target, 0.1, implicit)
        recommend._solve_side(A2, B, u, i, conf, target, 0.1, implicit, native=False)
        assert torch.allclose(A1, A2, atol=1e-10) and float(A1[-5:].abs().max()) == 0.0
    baskets = [torch.randint(0, 120, (5,), generator=g).tolist() + [7, 100][: int(r % 3 == 0) * 2] for r in range(1500)]
    found = rules.mine(baskets, min_support=0.004, min_confidence=0.0, max_items=4)
    sets = [frozenset(b) for b in baskets]
    assert found and max(len(r.if_) + len(r.then) for r in found) >= 3
    for r in found[:40] + found[-40:]:
        both = sum(1 for b in sets if set(r.if_) | set(r.then) <= b)
        first = sum(1 for b in sets if set(r.if_) <= b)
        assert abs(r.support - both / len(sets)) < 1e-12 and abs(r.confidence - both / first) < 1e-12
    pairs = {frozenset(r.if_ + r.then) for r in found if len(r.if_) + len(r.then) == 2}
    want = {frozenset(p) for p in itertools.combinations(range(120), 2) if sum(1 for b in sets if set(p) <= b) >= 0.004 * len(sets)}
    assert pairs == want


def test_softmax_boosting_rounds_in_one_native_call_grow_the_trees_of_the_per_round_loop():
    from mimir_b200.ml import tree
    g = torch.Generator().manual_seed(8)
    centers = torch.randn(4, 6, generator=g) * 2
    y = torch.randint(0, 4, (2500,), generator=g)
    X = centers[y] + torch.randn(2500, 6, generator=g)
    for kw in (dict(), dict(colsample=0.6, per_tree=0.7), dict(min_weight=2.0)):
        a = tree.gradient_boosting(X, y, trees=6, max_depth=4, classes=4, seed=2, **kw)
        b = tree.gradient_boosting(X, y, trees=6, max_depth=4, classes=4, seed=2, native_rounds=False, **kw)
        assert len(a.trees) == len(b.trees) == 6 and all(len(r) == 4 for r in a.trees)
        for ra, rb in zip(a.trees, b.trees):
            for ta, tb in zip(ra, rb):
                assert [q[:4] for q in ta.nodes] == [q[:4] for q in tb.nodes], kw
        assert float((a.raw(X) - b.raw(X)).abs().max()) < 1e-4
        assert torch.allclose(a.importance(), b.importance(), atol=1e-5)
    assert float((a.classify(X) == y).float().mean()) > 0.8
