"""MNIST-shaped CNN training step (reference: tools/bench/train_step.py and the table in
tools/bench/README.md: conv 1->32, pool, conv 32->64, pool, linear 3136->128, linear 128->10,
batch 128, AdamW lr 1e-3 weight decay 0.01, forward + cross-entropy + backward + update).

    python -m mimir_b200.utils.bench_mnist --device cpu      # lazy-tensor layer on the host cores
    python -m mimir_b200.utils.bench_mnist --device gpu      # native conv / pool / GEMM kernels

Prints one JSON line with the mean and median milliseconds per step over ``--steps`` steps after
``--warmup`` untimed ones; synthetic images, random-init weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=["cpu", "gpu"])
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline"],
                    help="baseline = the same network and step in plain PyTorch (cuDNN / cuBLAS, or MKL on the host)")
    a = ap.parse_args()
    if a.threads:
        torch.set_num_threads(a.threads)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(a.batch, 1, 28, 28, generator=gen)
    y = torch.randint(0, 10, (a.batch,), generator=gen)
    times = []
    if a.impl == "baseline":
        import sys
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline"))
        import torch_baselines as TB
        dev = "cuda" if a.device == "gpu" else "cpu"
        torch.manual_seed(0)
        net = TB.MnistCNN().to(dev)
        opt = torch.optim.AdamW(net.parameters(), lr=1e-3, weight_decay=0.01, fused=dev == "cuda")
        xd, yd = x.to(dev), y.to(dev)
        for i in range(a.warmup + a.steps):
            if dev == "cuda":
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            opt.zero_grad(set_to_none=True)
            net(xd, yd).backward()
            opt.step()
            if dev == "cuda":
                torch.cuda.synchronize()
            if i >= a.warmup:
                times.append((time.perf_counter() - t0) * 1e3)
        launches = 0
    elif a.device == "gpu":
        from ..models.cnn import MnistCNN
        eng = MnistCNN(a.batch, "cuda", lr=1e-3, weight_decay=0.01)
        xd, yd = x.cuda(), y.cuda()
        for i in range(a.warmup + a.steps):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.train_step(xd, yd)
            e1.record()
            torch.cuda.synchronize()
            if i >= a.warmup:
                times.append(e0.elapsed_time(e1))
        launches = int(eng.launches_per_step)
    else:
        from .. import nn, optim
        from .. import tensor as T
        nn.manual_seed(0)
        net = nn.Sequential(nn.Conv2d(1, 32, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(32, 64, 3, padding=1),
                            nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(), nn.Linear(3136, 128), nn.ReLU(), nn.Linear(128, 10))
        opt = optim.AdamW(net.parameters(), lr=1e-3, weight_decay=0.01)
        xt, yt = T.from_torch(x), T.from_torch(y)
        for i in range(a.warmup + a.steps):
            t0 = time.perf_counter()
            loss = nn.loss.cross_entropy(net(xt), yt)
            loss.backward()
            opt.step()
            opt.zero_grad()
            if i >= a.warmup:
                times.append((time.perf_counter() - t0) * 1e3)
        launches = 0
    print(json.dumps({"metric": "mnist_cnn_ms_per_step", "impl": a.impl, "device": a.device, "batch": a.batch, "steps": a.steps,
                      "mean_ms": sum(times) / len(times), "median_ms": statistics.median(times), "gpu_launches": launches,
                      "threads": torch.get_num_threads(), "cpu_count": os.cpu_count(), "data": "synthetic"}))


if __name__ == "__main__":
    main()
