"""Functions run on CPU ranks by tests/test_group.py (module-level so that they pickle)."""
import torch

import mimir_b200.tensor as T


def collectives(g):
    rank, world = g.rank, g.size
    x = T.tensor([float(rank + 1)] * 4)
    out = {"sum": g.all_reduce(x).data().tolist(), "mean": g.all_reduce(x, "mean").data().tolist(),
           "max": g.all_reduce(x, "max").data().tolist(),
           "bcast": g.broadcast(x, root=1).data().tolist(),
           "gather": g.all_gather(T.tensor([[float(rank)]])).data().reshape(-1).tolist(),
           "rs": g.reduce_scatter(T.tensor([[1.0 + rank]] * world)).data().reshape(-1).tolist()}
    return out


def grads(g):
    rank, world = g.rank, g.size
    torch.manual_seed(rank)
    ps = [T.Param(torch.randn(5, 3)), T.Param(torch.randn(7))]
    g.broadcast_params(ps, root=0)
    same = [p.value().data().clone() for p in ps]
    for p in ps:
        p._grad = torch.full(tuple(p.shape), float(rank + 1))
    g.all_reduce_grads(ps)
    return {"p0": same[0].sum().item(), "g": [p.grad().data().flatten()[0].item() for p in ps],
            "calls": g.traffic["all_reduce"]}


def dp_fit(g, mode):
    """Trains a small MLP data-parallel; returns the losses and a parameter checksum."""
    from mimir_b200 import nn, optim, train
    from mimir_b200.data import Tensors
    nn.manual_seed(g.rank + 5)          # different initial weights per rank: the broadcast must fix that
    model = nn.Sequential(nn.Linear(6, 16), nn.Tanh(), nn.Linear(16, 3))
    gen = torch.Generator().manual_seed(0)
    x, y = torch.randn(40, 6, generator=gen), torch.randint(0, 3, (40,), generator=gen)
    ds = Tensors(x, y, batch_size=10, shuffle=True, seed=1)
    opt = optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    from mimir_b200.parallel.replicas import fit_data_parallel
    reps = fit_data_parallel(model, opt, ds, nn.loss.cross_entropy, 3, g, mode=mode)
    return {"loss": [r.loss for r in reps], "w": [float(p._data.double().sum()) for p in model.parameters()]}


def single_fit():
    from mimir_b200 import nn, optim, train
    from mimir_b200.data import Tensors
    nn.manual_seed(5)
    model = nn.Sequential(nn.Linear(6, 16), nn.Tanh(), nn.Linear(16, 3))
    gen = torch.Generator().manual_seed(0)
    x, y = torch.randn(40, 6, generator=gen), torch.randint(0, 3, (40,), generator=gen)
    ds = Tensors(x, y, batch_size=10, shuffle=True, seed=1)
    opt = optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    reps = train.fit(model, opt, ds, loss=nn.loss.cross_entropy, epochs=3)
    return {"loss": [r.loss for r in reps], "w": [float(p._data.double().sum()) for p in model.parameters()]}
