"""Host training-step benchmarks: the rows of the reference's own table (tools/bench/README.md:30-66:
MNIST MLP, MNIST CNN, ResNet-18 at 224 x 224, a deep tabular MLP; one step = forward, cross-entropy,
backward, AdamW update) through this package's public API, next to the same step in plain PyTorch
on the same box.

    python -m mimir_b200.utils.bench_cpu [--only mlp,cnn,deep,resnet18,gcn] [--steps 10] [--threads 0]

``gcn`` is a two-layer graph convolution over a random graph of 100,000 nodes and 1,000,000 edges (64 -> 64 -> 8
features): this package's ``nn.GCNConv`` (segment kernel over sorted entries) against the same layer written
on ``torch.sparse`` CSR products, the faster of PyTorch's two ways to aggregate neighbours.

One JSON line per model: best and median milliseconds of both arms (synthetic inputs, random-init
weights of the same shapes).
"""
from __future__ import annotations

import argparse
import json
import statistics
import time

import torch

from .. import nn, optim, vision
from .. import tensor as T
from ..nn import loss as L


def _ours_mlp(sizes):
    layers = []
    for i in range(len(sizes) - 1):
        layers.append(nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2:
            layers.append(nn.ReLU())
    return nn.Sequential(*layers)


def _torch_mlp(sizes):
    layers = []
    for i in range(len(sizes) - 1):
        layers.append(torch.nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2:
            layers.append(torch.nn.ReLU())
    return torch.nn.Sequential(*layers)


def _torch_resnet18(classes=1000):
    tn = torch.nn

    class Block(tn.Module):
        def __init__(self, cin, cout, stride):
            super().__init__()
            self.c1, self.b1 = tn.Conv2d(cin, cout, 3, stride, 1, bias=False), tn.BatchNorm2d(cout)
            self.c2, self.b2 = tn.Conv2d(cout, cout, 3, 1, 1, bias=False), tn.BatchNorm2d(cout)
            self.down = None
            if stride != 1 or cin != cout:
                self.down = tn.Sequential(tn.Conv2d(cin, cout, 1, stride, bias=False), tn.BatchNorm2d(cout))

        def forward(self, x):
            y = torch.relu(self.b1(self.c1(x)))
            y = self.b2(self.c2(y))
            return torch.relu(y + (x if self.down is None else self.down(x)))
    layers = [tn.Conv2d(3, 64, 7, 2, 3, bias=False), tn.BatchNorm2d(64), tn.ReLU(), tn.MaxPool2d(3, 2, 1)]
    cin = 64
    for cout, stride in ((64, 1), (128, 2), (256, 2), (512, 2)):
        layers += [Block(cin, cout, stride), Block(cout, cout, 1)]
        cin = cout
    layers += [tn.AdaptiveAvgPool2d(1), tn.Flatten(), tn.Linear(512, classes)]
    return tn.Sequential(*layers)


MODELS = {
    "mlp": dict(shape=(128, 784), classes=10,
                ours=lambda: _ours_mlp([784, 128, 10]), theirs=lambda: _torch_mlp([784, 128, 10])),
    "cnn": dict(shape=(128, 1, 28, 28), classes=10,
                ours=lambda: nn.Sequential(nn.Conv2d(1, 32, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(32, 64, 3, padding=1),
                                           nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(), nn.Linear(3136, 128), nn.ReLU(), nn.Linear(128, 10)),
                theirs=lambda: torch.nn.Sequential(torch.nn.Conv2d(1, 32, 3, padding=1), torch.nn.ReLU(), torch.nn.MaxPool2d(2),
                                                   torch.nn.Conv2d(32, 64, 3, padding=1), torch.nn.ReLU(), torch.nn.MaxPool2d(2),
                                                   torch.nn.Flatten(), torch.nn.Linear(3136, 128), torch.nn.ReLU(), torch.nn.Linear(128, 10))),
    "deep": dict(shape=(512, 20), classes=3,
                 ours=lambda: _ours_mlp([20, 1024, 1024, 1024, 512, 256, 3]), theirs=lambda: _torch_mlp([20, 1024, 1024, 1024, 512, 256, 3])),
    "resnet18": dict(shape=(16, 3, 224, 224), classes=1000, ours=lambda: vision.resnet18(1000), theirs=_torch_resnet18),
}


def _gcn_case(steps, warmup):
    g = torch.Generator().manual_seed(0)
    n, e, f, hidden, classes = 100_000, 1_000_000, 64, 64, 8
    src, dst = torch.randint(0, n, (e,), generator=g), torch.randint(0, n, (e,), generator=g)
    x, y = torch.randn(n, f, generator=g), torch.randint(0, classes, (n,), generator=g)
    nn.manual_seed(0)
    graph = nn.Graph(n, src, dst)
    l1, l2 = nn.GCNConv(f, hidden), nn.GCNConv(hidden, classes)
    opt = optim.AdamW(l1.parameters() + l2.parameters(), lr=1e-3, weight_decay=0.01)
    xt, yt = T.from_torch(x), T.from_torch(y)

    def ours_step():
        L.cross_entropy(l2.convolve(graph, T.relu(l1.convolve(graph, xt))), yt).backward()
        opt.step()
        opt.zero_grad()
    ob, om = _time(ours_step, steps, warmup)
    # the same layer on torch.sparse: self loops (existing ones dropped), D^-1/2 A D^-1/2 as one CSR matrix
    keep = src != dst
    loop = torch.arange(n)
    s2, d2 = torch.cat([src[keep], loop]), torch.cat([dst[keep], loop])
    dinv = torch.bincount(d2, minlength=n).float().clamp_min(1).rsqrt()
    adj = torch.sparse_coo_tensor(torch.stack([d2, s2]), dinv[d2] * dinv[s2], (n, n)).coalesce().to_sparse_csr()
    torch.manual_seed(0)
    w1, w2 = torch.nn.Linear(f, hidden), torch.nn.Linear(hidden, classes)
    topt = torch.optim.AdamW(list(w1.parameters()) + list(w2.parameters()), lr=1e-3, weight_decay=0.01)

    def torch_step():
        topt.zero_grad(set_to_none=True)
        h = torch.relu(adj @ (x @ w1.weight.t()) + w1.bias)
        torch.nn.functional.cross_entropy(adj @ (h @ w2.weight.t()) + w2.bias, y).backward()
        topt.step()
    tb, tm = _time(torch_step, steps, warmup)
    return n, ob, om, tb, tm


def _time(step, steps, warmup):
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        step()
        if i >= warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    return min(times), statistics.median(times)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="mlp,cnn,deep,resnet18")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--threads", type=int, default=0)
    a = ap.parse_args(argv)
    if a.threads:
        torch.set_num_threads(a.threads)
    T.set_default_device(T.CPU())
    for name in a.only.split(","):
        if name == "gcn":
            n, ob, om, tb, tm = _gcn_case(max(3, a.steps // 2), a.warmup)
            print(json.dumps({"metric": "cpu_train_step_ms", "model": "gcn", "batch": n, "ours_best_ms": round(ob, 2),
                              "ours_median_ms": round(om, 2), "pytorch_best_ms": round(tb, 2), "pytorch_median_ms": round(tm, 2),
                              "ours_over_pytorch": round(om / tm, 3), "threads": torch.get_num_threads(), "data": "synthetic"}), flush=True)
            continue
        m = MODELS[name]
        g = torch.Generator().manual_seed(0)
        x = torch.randn(*m["shape"], generator=g)
        y = torch.randint(0, m["classes"], (m["shape"][0],), generator=g)
        steps = max(3, a.steps // 3) if name == "resnet18" else a.steps
        nn.manual_seed(0)
        net = m["ours"]()
        net.train() if hasattr(net, "train") else None
        opt = optim.AdamW(net.parameters(), lr=1e-3, weight_decay=0.01)
        xt, yt = T.from_torch(x), T.from_torch(y)

        def ours_step():
            L.cross_entropy(net(xt), yt).backward()
            opt.step()
            opt.zero_grad()
        ob, om = _time(ours_step, steps, a.warmup)
        torch.manual_seed(0)
        tnet = m["theirs"]()
        topt = torch.optim.AdamW(tnet.parameters(), lr=1e-3, weight_decay=0.01)

        def torch_step():
            topt.zero_grad(set_to_none=True)
            torch.nn.functional.cross_entropy(tnet(x), y).backward()
            topt.step()
        tb, tm = _time(torch_step, steps, a.warmup)
        print(json.dumps({"metric": "cpu_train_step_ms", "model": name, "batch": m["shape"][0], "ours_best_ms": round(ob, 2),
                          "ours_median_ms": round(om, 2), "pytorch_best_ms": round(tb, 2), "pytorch_median_ms": round(tm, 2),
                          "ours_over_pytorch": round(om / tm, 3), "threads": torch.get_num_threads(), "steps": steps,
                          "data": "synthetic"}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
