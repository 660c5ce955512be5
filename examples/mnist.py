"""MNIST classifier (reference: examples/mnist/main.go): MLP or CNN through ``train.fit``; with
``--device gpu`` the CNN runs on the native convolution / pooling / GEMM kernels.

    python examples/mnist.py --data /path/to/mnist --model cnn --epochs 2
    python examples/mnist.py                                   # synthetic digits when no data directory is given
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def synthetic(rows=256, seed=0):
    """Ten classes of 28x28 images: a bright bar whose position encodes the label, plus noise."""
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, 10, (rows,), generator=g)
    x = 0.3 * torch.randn(rows, 1, 28, 28, generator=g)
    for i, c in enumerate(y.tolist()):
        x[i, 0, 2 * c + 4: 2 * c + 7] += 1.5
    return x, y


def main(data=None, model="cnn", epochs=2, batch=32, log=print):
    from mimir_b200 import metrics, nn, optim, train
    from mimir_b200.data import Tensors, datasets
    nn.manual_seed(0)
    if data:
        tr_ds, ev_ds = datasets.mnist(data, True, batch), datasets.mnist(data, False, batch, shuffle=False)
    else:
        x, y = synthetic(320)
        tr_ds, ev_ds = Tensors(x[:256], y[:256], batch_size=batch, seed=0), Tensors(x[256:], y[256:], batch_size=64, shuffle=False)
    if model == "mlp":
        net = nn.Sequential(nn.Flatten(), nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 10))
    else:
        net = nn.Sequential(nn.Conv2d(1, 32, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(32, 64, 3, padding=1),
                            nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(), nn.Linear(3136, 128), nn.ReLU(), nn.Linear(128, 10))
    opt = optim.AdamW(net.parameters(), lr=1e-3, weight_decay=0.01)
    reports = train.fit(net, opt, tr_ds, loss=nn.loss.cross_entropy, epochs=epochs, eval=ev_ds,
                        metrics=[metrics.Accuracy()] if hasattr(metrics, "Accuracy") else ())
    for r in reports:
        log(f"epoch {r.epoch} loss {r.loss:.4f} {r.metrics}")
    return reports


def gpu_main(steps=50, batch=128, log=print):
    from mimir_b200.models.cnn import MnistCNN
    x, y = synthetic(batch)
    eng = MnistCNN(batch, "cuda")
    xd, yd = x.cuda(), y.cuda()
    losses = [float(eng.train_step(xd, yd).item()) for _ in range(steps)]
    log(f"first loss {losses[0]:.3f}, last loss {losses[-1]:.3f}")
    return losses


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--data")
    ap.add_argument("--model", default="cnn", choices=["cnn", "mlp"])
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--device", default="cpu", choices=["cpu", "gpu"])
    a = ap.parse_args()
    gpu_main() if a.device == "gpu" else main(a.data, a.model, a.epochs)
