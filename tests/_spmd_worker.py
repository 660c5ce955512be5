"""CPU worker (gloo): a model with an embedding, layer norms, attention, reshapes and a loss over a
``P("data")`` batch, partitioned over a mesh by the layout rules alone (no sharded layer classes)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build():
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    nn.manual_seed(13)

    class Net(nn.Module):
        def __init__(self):
            self.wte = nn.Embedding(48, 32)
            self.wpe = nn.Embedding(8, 32)
            self.block = nn.DecoderBlock(32, 4, hidden=64, style="gpt2")
            self.lnf = nn.LayerNorm(32)
            self.head = nn.Linear(32, 16)
            self._nn_skip_pos = torch.arange(8, dtype=torch.int64)

        def forward(self, tok):
            x = self.wte(tok) + self.wpe(T.from_torch(self._nn_skip_pos))
            return self.head(self.lnf(self.block(x)))
    return Net()


def loss_fn(out, y):
    import mimir_b200.tensor as T
    from mimir_b200.nn import loss as L
    return L.cross_entropy(T.reshape(out, (-1, 16)), T.reshape(y, (-1,)))


def fit_sharded(rank, world):
    """``fit(sharded=(mesh, rule))`` equals ``fit`` on one device (train/sharded_test.go:165-196)."""
    import mimir_b200.tensor as T
    from mimir_b200 import data, optim
    from mimir_b200.parallel import mesh as M
    from mimir_b200.train import fit
    T.set_default_device(T.CPU())
    g = torch.Generator().manual_seed(2)
    X = torch.randint(0, 48, (16, 8), generator=g)
    Y = torch.randint(0, 16, (16, 8), generator=g)
    ds = data.Tensors(X, Y, batch_size=8, shuffle=False)
    one = build()
    # SGD is linear in the gradients, so parity stays at rounding level
    r1 = fit(one, optim.SGD(one.parameters(), lr=0.05, momentum=0.9), ds, loss=loss_fn, epochs=2)
    mesh = M.Mesh((2, world // 2), ("data", "model"))
    model = build()
    r2 = fit(model, optim.SGD(model.parameters(), lr=0.05, momentum=0.9), ds, loss=loss_fn, epochs=2,
             sharded=(mesh, M.rules(M.tensor_parallel("model"), M.fully_shard("data"))))
    diff = max((M.gather_param(p) - q._data).abs().max().item()
               for (_, p), (_, q) in zip(model.named_params(), one.named_params()))
    os.write(1, ("RESULT " + json.dumps({"rank": rank, "diff": diff, "l1": [r.loss for r in r1],
                                  "l2": [r.loss for r in r2]}) + "\n").encode())
    dist.destroy_process_group()


def main():
    strategy = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    import mimir_b200.tensor as T
    from mimir_b200 import optim
    from mimir_b200.parallel import mesh as M
    from mimir_b200.parallel import spmd as S
    T.set_default_device(T.CPU())
    if strategy == "fit":
        return fit_sharded(rank, world)
    shape = {"dp": (world, 1), "tp": (1, world), "fsdp": (world, 1), "dpxtp": (2, world // 2),
             "fsdpxtp": (2, world // 2)}[strategy]
    mesh = M.Mesh(shape, ("data", "model"))
    rule = {"dp": None, "tp": M.tensor_parallel("model"), "fsdp": M.fully_shard("data"),
            "dpxtp": M.tensor_parallel("model"),
            "fsdpxtp": M.rules(M.tensor_parallel("model"), M.fully_shard("data"))}[strategy]
    g = torch.Generator().manual_seed(1)
    X = torch.randint(0, 48, (8, 8), generator=g)
    Y = torch.randint(0, 16, (8, 8), generator=g)
    ref = build()
    ropt = optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    ref_losses = []
    for _ in range(3):
        l = loss_fn(ref(T.from_torch(X)), T.from_torch(Y))
        l.backward()
        ropt.step()
        ropt.zero_grad()
        ref_losses.append(l.item())
    model = build()
    S.shard_params(model, mesh, rule)
    opt = optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    batch = M.P("data") if mesh.axis_size("data") > 1 else None
    # forward only, results left where the rules put them
    mesh.traffic.reset()
    (blk, lay), = S.realize_blocks(model(S.place(X, mesh, batch)))
    fwd = dict(ar=mesh.traffic.all_reduce, ag=mesh.traffic.all_gather, rs=mesh.traffic.reduce_scatter)
    out_layout = [str(a) for a in lay.dims]
    # the same forward, gathered: equals one device
    whole = model(S.place(X, mesh, batch)).data()
    ref0 = build()
    fdiff = (whole - ref0(T.from_torch(X)).data()).abs().max().item()
    losses, step_traffic = [], None
    before = S.stats()["analysed"]
    for i in range(3):
        mesh.traffic.reset()
        losses.append(S.sharded_step(model, opt, mesh, loss_fn, X, Y))
        if i == 0:
            step_traffic = dict(ar=mesh.traffic.all_reduce, ag=mesh.traffic.all_gather, rs=mesh.traffic.reduce_scatter)
    analysed = S.stats()["analysed"] - before
    diff = 0.0
    for (n, p), (_, q) in zip(model.named_params(), ref.named_params()):
        diff = max(diff, (M.gather_param(p) - q._data).abs().max().item())
    nparams = len(list(model.named_params(buffers=False)))
    os.write(1, ("RESULT " + json.dumps({"rank": rank, "strategy": strategy, "diff": diff, "fdiff": fdiff, "losses": losses,
                                  "ref_losses": ref_losses, "fwd": fwd, "step": step_traffic, "params": nparams,
                                  "out_layout": out_layout, "analysed": analysed}) + "\n").encode())
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
