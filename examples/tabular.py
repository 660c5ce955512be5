"""Classical models on a table (reference: the tabular / tree / linear / automl packages and their README
walk-through): split, fit a boosted ensemble and a linear model, search over model families, then serve the winner
as an ``nn.Module`` and as one exported ``.mim`` file run back through the graph runtime."""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def table(rows=4000, seed=0):
    """Twelve features, two of them informative through an interaction, some values missing."""
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(rows, 12, generator=g)
    y = ((X[:, 0] * X[:, 1] + 0.5 * X[:, 2] + 0.1 * torch.randn(rows, generator=g)) > 0).long()
    X[torch.rand(rows, generator=g) < 0.02, 5] = float("nan")
    return X, y


def main(rows=4000, budget=20.0, log=print):
    import mimir_b200.tensor as T
    from mimir_b200 import ml
    from mimir_b200.io import export, mim
    from mimir_b200.ml import automl, linear, tree
    X, y = table(rows)
    train, held = ml.Data(X, y).split(test=0.25, seed=1)
    train.check("classification")
    accuracy = lambda pred, want: float((pred == want).float().mean())  # noqa: E731

    filled = torch.nan_to_num(train.X, nan=0.0)
    boosted = tree.gradient_boosting(filled, train.Y, trees=60, max_depth=4, classes=2)
    a_boost = accuracy(boosted.classify(torch.nan_to_num(held.X, nan=0.0)), held.Y)
    logit = linear.logistic_fit(train)
    a_lin = accuracy(logit.classify(held.X), held.Y)
    log(f"boosted trees {a_boost:.3f}, logistic regression {a_lin:.3f} (the answer is an interaction: a line cannot see it)")
    top = boosted.importance().argsort(descending=True)[:3].tolist()
    log(f"most useful features: {top}")

    found = automl.search(train, "classification", trials=8, folds=3, budget=budget, seed=0)
    a_auto = accuracy(found.best.classify(held.X), held.Y)
    log(f"search picked {found.candidate} (cross-validated log loss {found.score:.3f}); held-out accuracy {a_auto:.3f}")

    # the fitted model as a network module, then as a file with its graph, run back without the library's model code
    net = found.best.module()
    rows = T.from_torch(held.X[:64].contiguous())
    probs = T.softmax(net(rows), -1).data()
    agree = accuracy(probs.argmax(-1), found.best.classify(held.X[:64]))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "model.mim")
        export.export(path, net, rows, input_name="features", output_name="logits", dynamic={"features": {0: ("batch", 4096)}})
        with mim.open(path) as model:
            out = model.run({"features": T.from_torch(held.X[:200].contiguous())})["logits"].data()
        err = float((out - net(T.from_torch(held.X[:200].contiguous())).data()).abs().max())
    log(f"module agrees with the model on {agree:.0%} of rows; the exported file reproduces it within {err:.1e}")
    return a_boost, a_lin, a_auto, agree, err


if __name__ == "__main__":
    main()
