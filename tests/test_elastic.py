"""Recovery after a lost rank on CPU ranks (gloo): a rank leaves between two steps, the survivors learn
it from the heartbeat before their next collective, shrink the group, reload the last checkpoint and
end with the weights of an uninterrupted run.  No GPU is involved."""
import multiprocessing as mp
import os
import time
from datetime import timedelta

import torch
import torch.distributed as dist

STEPS, LEAVE_AFTER, CKPT_EVERY = 6, 3, 2


def _batch(step):
    g = torch.Generator().manual_seed(100 + step)
    x = torch.randn(12, 8, generator=g)
    return x, (x @ torch.ones(8, 3)).tanh()


def _build():
    from mimir_b200 import nn, optim
    nn.manual_seed(5)
    m = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 3))
    return m, optim.SGD(m.parameters(), lr=0.1, momentum=0.9)


def _rank(rank, world, port, ckpt, q):
    import mimir_b200.tensor as T
    from mimir_b200.nn import loss as L
    from mimir_b200.parallel import elastic, health
    from mimir_b200.parallel.replicas import Parallel
    from mimir_b200.tensor.group import Group
    from mimir_b200.train.fit import save_checkpoint
    T.set_default_device(T.CPU())
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=30),
                          wait_for_workers=False)
    dist.init_process_group("gloo", store=dist.PrefixStore("gen0", store), rank=rank, world_size=world,
                            timeout=timedelta(seconds=20))
    hb = health.Heartbeat(store, rank, world, interval=0.05, timeout=0.6)
    hb.wait_all(20)
    model, opt = _build()
    par = Parallel(model, Group())
    my_rank, my_world, step, generation, recovered = rank, world, 0, 0, 0
    while step < STEPS:
        if rank == 2 and step == LEAVE_AFTER:
            hb.stop()                         # leaves between steps: nothing of it is in flight
            q.put((rank, "left", step, None))
            return
        dead = []
        try:
            hb.check()                        # on the host, before the next collective
            x, y = _batch(step)
            par.backward(T.from_torch(x), T.from_torch(y), L.mse)
            par.step(opt)
        except health.RankLost as lost:
            dead = lost.ranks
        except RuntimeError:
            # the collective itself ended with an error (the peer's connection closed, or the group's
            # short timeout ran out): ask the heartbeat who is gone
            dead = elastic.detect(hb, 5.0)
            if not dead:
                raise
        if dead:
            generation += 1
            my_rank, my_world, tr = elastic.recover(store, my_rank, my_world, dead, model, opt, ckpt,
                                                    generation=generation, timeout=timedelta(seconds=20))
            hb.stop()
            hb = health.Heartbeat(store, my_rank, my_world, interval=0.05, timeout=0.6, prefix=f"hb{generation}")
            hb.wait_all(20)
            par = Parallel(model, Group())
            step = int(tr["steps"]) if tr else 0
            recovered += 1
            continue
        step += 1
        if step % CKPT_EVERY == 0 and my_rank == 0:
            save_checkpoint(ckpt, model, opt, epoch=0, steps=step)
    hb.stop()
    q.put((rank, "done", recovered, [p._data.clone() for p in model.parameters()]))
    if rank == 0:
        time.sleep(1.0)
    dist.destroy_process_group()


def test_survivors_shrink_the_group_and_resume_from_the_checkpoint(tmp_path):
    import mimir_b200.tensor as T
    from mimir_b200.nn import loss as L
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 3, 29931, str(tmp_path), q)) for r in range(3)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(3):
        r, what, n, params = q.get(timeout=120)
        got[r] = (what, n, params)
    for p in procs:
        p.join(30)
    assert got[2][0] == "left"
    assert got[0][0] == got[1][0] == "done" and got[0][1] == got[1][1] == 1     # one recovery each
    # an uninterrupted single-device run on the same batches
    T.set_default_device(T.CPU())
    model, opt = _build()
    for s in range(STEPS):
        x, y = _batch(s)
        L.mse(model(T.from_torch(x)), T.from_torch(y)).backward()
        opt.step()
        opt.zero_grad()
    for a, b, c in zip(got[0][2], got[1][2], model.parameters()):
        assert torch.equal(a, b)                                   # the survivors stayed identical
        assert torch.allclose(a, c._data, atol=2e-6), (a - c._data).abs().max()
    assert os.path.exists(os.path.join(str(tmp_path), "checkpoint.mim"))
