"""Worker of the sharded Llama tests.  LLAMA_MODE=fsdp: two ranks, each with its own micro-batch, against
one single-device engine that sees both micro-batches.  LLAMA_MODE=tp: two tensor-parallel ranks on the
same batch against the single-device engine."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mimir_b200 import _native
    from mimir_b200.models.llama import LlamaEngine, LlamaTrainConfig
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.train import FusedTrainer
    _native.lib().mimir_set_device(local)
    cfg = LlamaTrainConfig.tiny()
    B, T = 2, 128
    gen = torch.Generator().manual_seed(0)
    tok_all = torch.randint(0, 64, (world * B, T), generator=gen)
    tgt_all = torch.roll(tok_all, -1, 1)
    mode = os.environ.get("LLAMA_MODE", "fsdp")
    if mode == "tp":
        return tensor_parallel(rank, world, cfg, B, T, tok_all[:B], tgt_all[:B])
    fs = LlamaEngine(cfg, B, T, seed=5, mode="fsdp", rank=rank, world=world)
    single = LlamaEngine(cfg, world * B, T, seed=5)
    fs.tokens.copy_(tok_all[rank * B:(rank + 1) * B].reshape(-1))
    fs.targets.copy_(tgt_all[rank * B:(rank + 1) * B].reshape(-1))
    single.tokens.copy_(tok_all.reshape(-1))
    single.targets.copy_(tgt_all.reshape(-1))
    for e in (fs, single):
        e.forward()
        e.loss_and_dlogits()
        e.backward()
    torch.cuda.synchronize()
    loss = fs.loss.clone()
    dist.all_reduce(loss)
    loss_fsdp = loss.item() / world
    loss_single = single.loss.item()      # before the optimizer steps below move it
    rows = single.g["h.0.wgu"].shape[0] // world
    a, b = fs.g["h.0.wgu"].float().flatten(), single.g["h.0.wgu"][rank * rows:(rank + 1) * rows].float().flatten()
    grad_cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
    # a few optimizer steps through the public trainer (no graph: NCCL calls sit inside the step)
    tr = FusedTrainer(fs, lr=3e-3, weight_decay=0.0, use_graph=False)
    tok = tok_all[rank * B:(rank + 1) * B].contiguous().pin_memory()
    tgt = tgt_all[rank * B:(rank + 1) * B].contiguous().pin_memory()
    losses = [tr.step(tok, tgt) for _ in range(6)]
    trs = FusedTrainer(single, lr=3e-3, weight_decay=0.0, use_graph=False)
    for _ in range(6):
        trs.step(tok_all.contiguous().pin_memory(), tgt_all.contiguous().pin_memory())
    rows = single.mv["h.1.wd"].shape[0] // world
    pa, pb = fs.mv["h.1.wd"].flatten(), single.mv["h.1.wd"][rank * rows:(rank + 1) * rows].flatten()
    param_cos = torch.nn.functional.cosine_similarity(pa, pb, dim=0).item()
    err = check_error_word()
    torch.cuda.synchronize()
    dist.barrier()
    fs.close()
    dist.destroy_process_group()
    os.write(1, ("RESULT " + json.dumps({"rank": rank, "loss_fsdp": loss_fsdp, "loss_single": loss_single,
                                         "grad_cos": grad_cos, "param_cos": param_cos, "losses": losses, "err": err}) + "\n").encode())


def tensor_parallel(rank, world, cfg, B, T, tok, tgt):
    from mimir_b200.models.llama import LlamaEngine
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.train import FusedTrainer
    tp = LlamaEngine(cfg, B, T, seed=5, mode="tp", rank=rank, world=world)
    single = LlamaEngine(cfg, B, T, seed=5)
    for e in (tp, single):
        e.tokens.copy_(tok.reshape(-1))
        e.targets.copy_(tgt.reshape(-1))
        e.forward()
        e.loss_and_dlogits()
        e.backward()
    torch.cuda.synchronize()
    F = tp.F
    a = tp.g["h.0.wd"].float().flatten()
    b = single.g["h.0.wd"][:, rank * F:(rank + 1) * F].float().flatten()
    grad_cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
    a2 = tp.g["h.1.wgu"][:F].float().flatten()
    b2 = single.g["h.1.wgu"][rank * F:(rank + 1) * F].float().flatten()
    grad_cos = min(grad_cos, torch.nn.functional.cosine_similarity(a2, b2, dim=0).item())
    a3, b3 = tp.g["wte"].float().flatten(), single.g["wte"].float().flatten()
    grad_cos = min(grad_cos, torch.nn.functional.cosine_similarity(a3, b3, dim=0).item())
    a4, b4 = tp.g["lm_head"].float().flatten(), single.g["lm_head"].float().flatten()   # summed over the ranks' row shares
    grad_cos = min(grad_cos, torch.nn.functional.cosine_similarity(a4, b4, dim=0).item())
    loss_tp, loss_single = tp.loss.item(), single.loss.item()
    tr = FusedTrainer(tp, lr=3e-3, weight_decay=0.0, use_graph=False)
    trs = FusedTrainer(single, lr=3e-3, weight_decay=0.0, use_graph=False)
    tokp, tgtp = tok.contiguous().pin_memory(), tgt.contiguous().pin_memory()
    losses = [tr.step(tokp, tgtp) for _ in range(6)]
    for _ in range(6):
        trs.step(tokp, tgtp)
    pa = tp.mv["h.1.wd"].flatten()
    pb = single.mv["h.1.wd"][:, rank * F:(rank + 1) * F].flatten()
    param_cos = torch.nn.functional.cosine_similarity(pa, pb, dim=0).item()
    err = check_error_word()
    torch.cuda.synchronize()
    dist.barrier()
    tp.close()
    dist.destroy_process_group()
    os.write(1, ("RESULT " + json.dumps({"rank": rank, "loss_fsdp": loss_tp, "loss_single": loss_single, "grad_cos": grad_cos,
                                         "param_cos": param_cos, "losses": losses, "err": err}) + "\n").encode())


if __name__ == "__main__":
    main()
