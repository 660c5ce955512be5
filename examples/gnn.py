"""Node classification with a two-layer GCN on a synthetic community graph (reference: examples/gnn)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(steps=60, log=print):
    import mimir_b200.tensor as T
    from mimir_b200 import nn, optim
    from mimir_b200.nn.gnn import GCNConv, Graph
    nn.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    n, classes = 120, 3
    y = torch.arange(n) % classes
    src, dst = [], []
    for i in range(n):
        for j in torch.randint(0, n, (8,), generator=g).tolist():
            same = y[i] == y[j]
            if torch.rand(1, generator=g).item() < (0.9 if same else 0.05):
                src += [i, j]
                dst += [j, i]
    graph = Graph(n, src, dst)
    x = T.from_torch(torch.randn(n, 8, generator=g))
    l1, l2 = GCNConv(8, 16), GCNConv(16, classes)
    opt = optim.Adam(l1.parameters() + l2.parameters(), lr=2e-2)
    train_mask = torch.arange(n) < 60
    acc = 0.0
    for s in range(steps):
        logits = l2(T.relu(l1(x, graph)), graph)
        loss = nn.loss.cross_entropy(logits[train_mask], T.from_torch(y[train_mask]))
        loss.backward()
        pred = logits.data().argmax(1)
        acc = float((pred[~train_mask] == y[~train_mask]).float().mean())
        opt.step()
        opt.zero_grad()
    log(f"gnn: held-out accuracy {acc:.2f}")
    return acc


if __name__ == "__main__":
    main()
