"""Worker for the multi-GPU data-parallel test (launched by torch.distributed.run)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    use_graph = os.environ.get("MIMIR_TEST_GRAPH", "1") == "1"
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mimir_b200 import _native
    from mimir_b200.models.gpt2 import GPT2Config, GPT2Engine
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.parallel.dp import FusedDataParallel
    from mimir_b200.train import FusedTrainer
    _native.lib().mimir_set_device(local)
    cfg = GPT2Config(n_layer=2, n_head=2, d_model=128, vocab=512, ctx=128)
    Bl, T, steps = 2, 128, 6
    gen = torch.Generator().manual_seed(7)
    tok = torch.randint(0, cfg.vocab, (Bl * world, T), generator=gen)
    tgt = torch.roll(tok, -1, 1)
    dp = FusedDataParallel(rank, world, local)
    eng = GPT2Engine(cfg, Bl, T, device=f"cuda:{local}", seed=5, flat_alloc=dp.alloc_shared)
    dp.attach(eng)
    tr = FusedTrainer(eng, lr=2e-3, dp=dp, use_graph=use_graph)
    my = slice(rank * Bl, (rank + 1) * Bl)
    losses = [tr.step(tok[my], tgt[my]) for _ in range(steps)]
    torch.cuda.synchronize()
    err = check_error_word()
    # replicas must be bit-identical
    mine = eng.params.clone().view(torch.uint8).clone()
    ref = mine.clone()
    dist.broadcast(ref, 0)
    identical = bool((mine == ref).all().item())
    lt = torch.tensor(losses, device="cuda")
    dist.all_reduce(lt)
    mean_losses = (lt / world).tolist()
    result = {"rank": rank, "err": err, "identical": identical, "losses": mean_losses}
    if rank == 0:
        # the same training on one device with the whole batch
        e1 = GPT2Engine(cfg, Bl * world, T, device=f"cuda:{local}", seed=5)
        t1 = FusedTrainer(e1, lr=2e-3, use_graph=False)
        result["single"] = [t1.step(tok, tgt) for _ in range(steps)]
        diff = (e1.params.float() - eng.params.float()).abs().max().item()
        result["max_param_diff"] = diff
    # ---- checkpoint under data parallelism: save, one more step; fresh replica, load, same step
    sd = {k: v.clone() for k, v in eng.state_dict().items()}
    count = eng.step_count
    tr.step(tok[my], tgt[my])
    torch.cuda.synchronize()
    after = eng.params.clone()
    dp2 = FusedDataParallel(rank, world, local)
    eng2 = GPT2Engine(cfg, Bl, T, device=f"cuda:{local}", seed=99, flat_alloc=dp2.alloc_shared)   # other weights
    dp2.attach(eng2)
    eng2.load_state_dict(sd)
    eng2.step_count = count
    # the restore itself is exact: what the fresh replica would save equals what was saved
    sd2 = eng2.state_dict()
    result["restore_exact"] = all(torch.equal(sd[k], sd2[k]) for k in sd) and len(sd) == len(sd2)
    tr2 = FusedTrainer(eng2, lr=2e-3, dp=dp2, use_graph=False)
    tr2.step(tok[my], tgt[my])
    torch.cuda.synchronize()
    # the next step agrees up to the order of the embedding gradient's atomic adds (a bf16 ulp here and there)
    d = (after.float() - eng2.params.float()).abs()
    result["resume_max_diff"] = d.max().item()
    result["resume_frac_diff"] = (d > 0).float().mean().item()
    result["ckpt_names"] = sorted(sd)[:3]
    result["err2"] = check_error_word()
    dp2.close()
    dp.close()
    dist.destroy_process_group()
    os.write(1, ("RESULT " + json.dumps(result) + "\n").encode())  # one write: lines of different ranks never interleave


if __name__ == "__main__":
    main()
