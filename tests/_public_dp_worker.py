"""Worker: ``fit(data_parallel=group)`` on the fused peer-memory path for an ``nn`` model."""
import json
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import mimir_b200.tensor as T
    from mimir_b200 import _native, data, nn, optim
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.tensor.group import Group
    from mimir_b200.train import fit
    from _tiny_gpt import TinyGPT, loss_fn
    _native.lib().mimir_set_device(local)
    T.set_default_device(T.GPU(local))
    g = torch.Generator().manual_seed(21)
    tok = torch.randint(0, 512, (32, 128), generator=g)
    tgt = torch.roll(tok, -1, 1)

    def build():
        nn.manual_seed(17)
        m = TinyGPT()
        m.cast(torch.bfloat16).to(T.GPU(local))
        return m, optim.AdamW(m.parameters(), lr=1e-3, weight_decay=0.01, master_weights=True)
    m, opt = build()
    ds = data.Tensors(tok, tgt, batch_size=8, shuffle=False)
    reps = fit(m, opt, ds, loss=loss_fn(m.vocab), epochs=2, data_parallel=Group())
    torch.cuda.synchronize()
    res = {"rank": rank, "err": check_error_word(), "loss": [r.loss for r in reps], "steps": opt.steps}
    mine = torch.cat([p._data.reshape(-1) for p in m.parameters()]).view(torch.uint8).clone()
    ref = mine.clone()
    dist.broadcast(ref, 0)
    res["identical"] = bool(torch.equal(mine, ref))
    res["state_names"] = sorted(opt.snapshot())[:3]
    if rank == 0:
        m1, o1 = build()
        r1 = fit(m1, o1, ds, loss=loss_fn(m1.vocab), epochs=2, device=T.GPU(local))
        res["single_loss"] = [r.loss for r in r1]
        res["max_param_diff"] = max((a._data.float() - b._data.float()).abs().max().item()
                                    for a, b in zip(m.parameters(), m1.parameters()))
        res["moment_diff"] = max((opt.state[i]["exp_avg"] - o1.state[i]["exp_avg"]).abs().max().item()
                                 for i in range(len(opt.params)))
    dist.barrier()
    dist.destroy_process_group()
    os.write(1, ("RESULT " + json.dumps(res) + "\n").encode())


if __name__ == "__main__":
    main()
