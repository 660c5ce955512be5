"""Classical ML on small synthetic problems (reference: tree/*_test.go, linear/*_test.go, ...)."""
import torch

from mimir_b200 import distributions as D
from mimir_b200 import ml
import mimir_b200.tensor as T


def _reg():
    torch.manual_seed(0)
    X = torch.randn(400, 4)
    w = torch.tensor([1.0, -2.0, 0.0, 0.5])
    return X, X @ w + 3 + 0.01 * torch.randn(400), w


def test_linear_family():
    X, y, w = _reg()
    m = ml.ridge(X, y)
    assert torch.allclose(m.w, w, atol=5e-3) and abs(float(m.b) - 3) < 5e-3
    l = ml.lasso(X, y, 0.05)
    assert l.w[2] == 0 and l.w[0] > 0.8
    yc = (X @ w > 0).long()
    assert (ml.logistic(X, yc).classify(X) == yc).float().mean() > 0.97
    y3 = torch.bucketize(X @ w, torch.tensor([-1.0, 1.0]))
    assert (ml.logistic(X, y3, 3).classify(X) == y3).float().mean() > 0.97
    assert (ml.linear_svm(X, yc).classify(X) == yc).float().mean() > 0.9


def test_trees():
    X, y, _ = _reg()
    y = y + X[:, 1] ** 2
    m = ml.gradient_boosting(X, y, trees=40, max_depth=4)
    assert ((m.predict(X) - y) ** 2).mean().sqrt() < 0.4
    assert m.importance()[2] < 0.05
    m2 = ml.tree.Model.from_json(m.to_json())
    assert torch.allclose(m2.predict(X), m.predict(X))
    yc = (X[:, 0] + X[:, 3] > 0).long()
    assert (ml.gradient_boosting(X, yc, trees=30, max_depth=3, classes=2).classify(X) == yc).float().mean() > 0.95
    y3 = torch.bucketize(X[:, 0], torch.tensor([-0.5, 0.5]))
    assert (ml.gradient_boosting(X, y3, trees=15, max_depth=2, classes=3).classify(X) == y3).float().mean() > 0.95
    assert (ml.decision_tree(X, yc, max_depth=6, classes=2).classify(X) == yc).float().mean() > 0.9
    rf = ml.random_forest(X, y, trees=20, max_depth=6)
    assert ((rf.predict(X) - y) ** 2).mean() < y.var()
    pts = torch.cat([torch.randn(200, 2), torch.tensor([[8.0, 8.0]])])
    s = ml.isolation_forest(pts, trees=50).score(pts)
    assert s.argmax() == 200


def test_neighbors_cluster_decomp():
    X, y, w = _reg()
    yc = (X @ w > 0).long()
    assert (ml.KNN(X, yc, 5, 2).classify(X) == yc).float().mean() > 0.9
    assert (ml.GaussianNB(X, yc, 2).classify(X) == yc).float().mean() > 0.85
    C = torch.cat([torch.randn(100, 2) + 5, torch.randn(100, 2) - 5])
    km = ml.kmeans(C, 2)
    assert sorted(km.centers[:, 0].round().tolist()) == [-5.0, 5.0]
    assert ml.dbscan(C, 1.5, 4).max() == 1
    p = ml.pca(X, 2)
    assert p.transform(X).shape == (400, 2) and p.variance[0] >= p.variance[1]


def test_splits_and_scaler():
    X, y, _ = _reg()
    tr, te = ml.split(ml.Data(X, y), 0.25)
    assert len(tr) == 300 and len(te) == 100
    sc = ml.fit_scaler(X)
    assert torch.allclose(sc.inverse(sc.transform(X)), X, atol=1e-5)


def test_distributions():
    mu = T.Param(torch.tensor([0.5]))
    d = D.Normal(mu.value(), T.tensor([2.0]))
    lp = d.log_prob(T.tensor([1.0]))
    T.backward(lp.sum())
    g = mu.grad()
    assert abs(float(g.data()) - 0.125) < 1e-6
    k = D.kl(D.Normal(T.tensor([0.0]), T.tensor([1.0])), D.Normal(T.tensor([1.0]), T.tensor([2.0])))
    assert abs(float(k.data()) - 0.4431) < 1e-3
    assert D.Normal(T.tensor([0.0]), T.tensor([1.0])).rsample((3,), seed=1).shape == (3, 1)
    assert isinstance(D.kl(D.Poisson(T.tensor([1.0])), D.Dirichlet(T.tensor([1.0, 1.0]))).err, D.ErrNoKL)
    c = D.Categorical(probs=T.tensor([0.2, 0.8]))
    assert abs(float(c.entropy().data()) - 0.5004) < 1e-3


def test_gmm_ward_fista_kernel_svm():
    torch.manual_seed(1)
    C = torch.cat([torch.randn(80, 2) * 0.5 + torch.tensor([4.0, 0.0]), torch.randn(80, 2) * 0.5 - torch.tensor([4.0, 0.0]),
                   torch.randn(80, 2) * 0.5 + torch.tensor([0.0, 5.0])])
    truth = torch.arange(3).repeat_interleave(80)
    m = ml.gmm(C, 3)
    a = m.assign(C)
    assert all(len(set(a[truth == k].tolist())) == 1 for k in range(3)) and len(set(a.tolist())) == 3
    assert abs(float(m.weights.sum()) - 1) < 1e-5 and m.score(C) > -3.5
    w = ml.ward(C, 3)
    assert all(len(set(w[truth == k].tolist())) == 1 for k in range(3)) and len(set(w.tolist())) == 3
    X, y, wt = _reg()
    f = ml.fista_lasso(X, y, 0.05)
    c = ml.lasso(X, y, 0.05)
    assert torch.allclose(f.w, c.w, atol=2e-3) and f.w[2] == 0
    # a ring inside a ring: not linearly separable
    r = torch.cat([torch.rand(100) * 1.0, 2.5 + torch.rand(100) * 1.0])
    th = torch.rand(200) * 6.283
    P = torch.stack([r * th.cos(), r * th.sin()], 1)
    lab = (torch.arange(200) >= 100).long()
    svm = ml.KernelSVM(c=10.0, kernel="rbf", gamma=1.0).fit(P, lab)
    assert (svm.classify(P) == lab).float().mean() > 0.98
    lin = ml.KernelSVM(c=1.0, kernel="linear").fit(X[:150], (X[:150] @ wt > 0).long())
    assert (lin.classify(X[:150]) == (X[:150] @ wt > 0).long()).float().mean() > 0.95


def test_native_tree_growth_equals_the_reference_path():
    """The tree grown by the native code (histograms over the worker pool, sibling subtraction, in-place
    row partition) against the same learner on the PyTorch path (bins as int64)."""
    from mimir_b200.ml import tree as TR
    torch.manual_seed(3)
    X = torch.randn(3000, 9)
    y = X[:, 0] * 2 - X[:, 4] + (X[:, 2] > 0.3).float() * 3 + 0.1 * torch.randn(3000)
    B, _ = TR._bin(X, 64)
    assert B.dtype == torch.uint8
    g, h = (0.0 - y), torch.ones(3000)
    fast = TR._Tree(5, 3, 0.0, 1.0, 64).fit(B, g, h)
    slow = TR._Tree(5, 3, 0.0, 1.0, 64).fit(B.long(), g, h)            # int64 bins: the PyTorch path
    assert len(fast.nodes) == len(slow.nodes) > 20
    for a, b in zip(fast.nodes, slow.nodes):
        assert a[:4] == b[:4] and abs(a[4] - b[4]) < 1e-4 * max(1.0, abs(b[4])), (a, b)
    assert torch.allclose(fast.predict_binned(B), slow.predict_binned(B.long()), atol=1e-4)
    assert torch.allclose(fast.importance, slow.importance, rtol=1e-3, atol=1e-3)
    # feature sampling per node: deterministic for a seed, and it does restrict the features
    g1 = torch.Generator().manual_seed(5)
    g2 = torch.Generator().manual_seed(5)
    t1 = TR._Tree(4, 1, 0.0, 1.0, 64, colsample=0.3, gen=g1).fit(B, g, h)
    t2 = TR._Tree(4, 1, 0.0, 1.0, 64, colsample=0.3, gen=g2).fit(B, g, h)
    assert t1.nodes == t2.nodes and t1.nodes != fast.nodes
