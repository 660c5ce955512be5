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
