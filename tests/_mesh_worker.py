"""CPU worker (gloo) for the mesh tests: trains a small block under one sharding strategy."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build():
    from mimir_b200 import nn
    nn.manual_seed(7)

    class Net(nn.Module):
        def __init__(self):
            self.block = nn.DecoderBlock(32, 4, hidden=64, style="gpt2")
            self.head = nn.Linear(32, 8)

        def forward(self, x):
            return self.head(self.block(x))
    return Net()


def sharded_tensor_layouts(rank, world):
    """shard / unshard / with_sharding of plain tensors, with a sectioned split."""
    import torch
    import mimir_b200.tensor as T
    from mimir_b200.parallel import mesh as M
    mesh = M.Mesh((2, 2), ("data", "model"))
    full = torch.arange(8 * 6, dtype=torch.float32).view(8, 6)
    x = M.shard(T.from_torch(full), mesh, M.P("data", "model"))
    ok = tuple(x.shape) == (4, 3) and x.sharding[1] == M.P("data", "model")
    ok = ok and torch.equal(M.unshard(x).data(), full)
    y = M.with_sharding(x, mesh, M.P("model", None))               # the split moves to the other axis
    ok = ok and tuple(y.shape) == (4, 6) and torch.equal(M.unshard(y).data(), full)
    spec = M.P("model", None).with_sections(0, 4, 2, 2)            # [Q | K | V]-style rows
    z = M.shard(T.from_torch(full), mesh, spec)
    ok = ok and tuple(z.shape) == (4, 6) and torch.equal(M.unshard(z).data(), full)
    i = mesh.axis_index("model")
    ok = ok and torch.equal(z.data()[:2], full[2 * i: 2 * i + 2]) and torch.equal(z.data()[2:3], full[4 + i: 5 + i])
    return {"ok": bool(ok)}


def main():
    strategy = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    if strategy == "layouts":
        out = sharded_tensor_layouts(rank, world)
        os.write(1, ("RESULT " + json.dumps(dict(out, rank=rank)) + "\n").encode())
        dist.destroy_process_group()
        return
    import mimir_b200.tensor as T
    from mimir_b200 import optim
    from mimir_b200.nn import loss as L
    from mimir_b200.parallel import mesh as M
    T.set_default_device(T.CPU())
    shape = {"dp": (world, 1), "tp": (1, world), "fsdp": (world, 1), "dpxtp": (2, world // 2), "fsdpxtp": (2, world // 2)}[strategy]
    mesh = M.Mesh(shape, ("data", "model"))
    rule = {"dp": None, "tp": M.tensor_parallel("model"), "fsdp": M.fully_shard("data"),
            "dpxtp": M.tensor_parallel("model"),
            "fsdpxtp": M.rules(M.tensor_parallel("model"), M.fully_shard("data"))}[strategy]
    torch.manual_seed(0)
    X = torch.randn(8, 6, 32)
    Y = torch.randn(8, 6, 8)
    # one device, whole batch
    ref = build()
    ropt = optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)  # linear in the gradients: parity stays at rounding level
    ref_losses = []
    for _ in range(3):
        l = L.mse(ref(T.tensor(X)), T.tensor(Y))
        l.backward()
        ropt.step()
        ropt.zero_grad()
        ref_losses.append(l.item())
    # sharded
    model = build()
    M.shard_module(model, mesh, rule)
    opt = optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    dp, di = mesh.axis_size("data"), mesh.axis_index("data")
    per = X.shape[0] // dp
    xs, ys = X[di * per:(di + 1) * per], Y[di * per:(di + 1) * per]
    mesh.traffic.reset()
    out = model(T.tensor(xs))
    out.realize()
    fwd = dict(ar=mesh.traffic.all_reduce, ag=mesh.traffic.all_gather, rs=mesh.traffic.reduce_scatter)
    losses = []
    step_traffic = None
    for i in range(3):
        mesh.traffic.reset()
        losses.append(M.sharded_step(model, opt, mesh, L.mse, T.tensor(xs), T.tensor(ys)))
        if i == 0:
            step_traffic = dict(ar=mesh.traffic.all_reduce, ag=mesh.traffic.all_gather, rs=mesh.traffic.reduce_scatter)
    diff = 0.0
    for (n, p), (_, q) in zip(model.named_params(), ref.named_params()):
        diff = max(diff, (M.gather_param(p) - q._data).abs().max().item())
    nparams = len(list(model.named_params(buffers=False)))
    os.write(1, ("RESULT " + json.dumps({"rank": rank, "strategy": strategy, "diff": diff, "losses": losses,
                                  "ref_losses": ref_losses, "fwd": fwd, "step": step_traffic, "params": nparams}) + "\n").encode())  # one write: lines of different ranks never interleave
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
