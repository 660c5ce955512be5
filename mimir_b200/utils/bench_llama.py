"""Llama training throughput on the native engine (``models/llama.py``).

    python -m mimir_b200.utils.bench_llama --model 1b3 --batch 8 --seq 2048                       # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m mimir_b200.utils.bench_llama --model 7b --mode fsdp --batch 1 --seq 4096              # fully sharded

Every rank trains on its own micro-batch of synthetic token ids (random-init weights).  ``--steps``
optimizer steps are timed with CUDA events after ``--warmup`` untimed ones, between barriers; the
slowest rank's time counts.  Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1b3", choices=["tiny", "1b3", "7b"])
    ap.add_argument("--mode", default="single", choices=["single", "fsdp", "tp"])
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel size (mode tp); the other ranks are data parallel")
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU and step")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--graph", action="store_true", help="replay the step as one CUDA graph (single mode)")
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline"],
                    help="baseline = plain PyTorch: cuBLAS, flash SDPA, fused AdamW, NCCL (FSDP / Megatron-style TP + DDP)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if a.impl == "baseline":
        return baseline(a, rank, world, local)
    from mimir_b200 import _native
    from mimir_b200.models.llama import LlamaEngine, LlamaTrainConfig
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.train import FusedTrainer
    lib = _native.lib()
    lib.mimir_set_device(local)
    cfg = {"tiny": LlamaTrainConfig.tiny, "1b3": LlamaTrainConfig.llama_1b3, "7b": LlamaTrainConfig.llama_7b}[a.model]()
    if a.layers:
        cfg.n_layer = a.layers
    mode = a.mode if world > 1 else "single"
    dp_world = 1
    if mode == "tp":
        tp = a.tp or world
        if world % tp:
            raise SystemExit(f"{world} ranks do not divide into tensor-parallel groups of {tp}")
        dp_world = world // tp
        tp_groups = [dist.new_group(list(range(g * tp, (g + 1) * tp))) for g in range(dp_world)]
        dp_groups = [dist.new_group(list(range(r, world, tp))) for r in range(tp)]
        eng = LlamaEngine(cfg, a.batch, a.seq, device=f"cuda:{local}", seed=0, mode="tp", rank=rank % tp, world=tp,
                          group=tp_groups[rank // tp], dp_group=dp_groups[rank % tp] if dp_world > 1 else None,
                          dp_world=dp_world)
    else:
        eng = LlamaEngine(cfg, a.batch, a.seq, device=f"cuda:{local}", seed=0, mode=mode, rank=rank, world=world)
    tr = FusedTrainer(eng, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, use_graph=a.graph and mode == "single")
    data_rank = rank // (a.tp or world) if mode == "tp" else rank      # tensor-parallel peers share their batch
    gen = torch.Generator().manual_seed(100 + data_rank)
    tok = torch.randint(0, cfg.vocab, (a.batch, a.seq), generator=gen).pin_memory()
    tgt = torch.roll(tok, -1, 1).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(max(a.warmup, 3)):
        loss = tr.step(tok, tgt)
    barrier()
    l0 = lib.mimir_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = tr.step(tok, tgt)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / a.steps
    tokens = a.batch * a.seq * (dp_world if mode == "tp" else world)
    params = cfg.param_count()
    flops = 6.0 * params * tokens + 12.0 * cfg.n_layer * cfg.d_model * a.seq * tokens / 2   # causal attention
    err = check_error_word()
    if rank == 0:
        print(json.dumps({
            "metric": "train_tokens_per_s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms,
            "n_gpus": world, "model_tflops_per_gpu": flops / (ms / 1e3) / 1e12 / world, "params": params, "loss": loss,
            "config": {"model": a.model, "layers": cfg.n_layer, "mode": mode, "tp": (a.tp or world) if mode == "tp" else 1, "micro_batch_per_gpu": a.batch,
                       "seq_len": a.seq, "global_batch": tokens // a.seq, "cuda_graph": bool(tr.graph)},
            "gpu_launches": int(lib.mimir_launch_count() - l0), "dtype": "bf16", "data": "synthetic", "error_word": err,
            "impl": "ours", "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}))
    if mode in ("fsdp", "tp"):
        barrier()
        eng.close()
    if world > 1:
        dist.destroy_process_group()


def baseline(a, rank, world, local):
    """The library arm: the same architecture, batch, optimizer, timing and output line in plain PyTorch.
    single: bf16 parameters + fp32 masters + fused AdamW, step in a CUDA graph.  fsdp: FSDP2
    (``fully_shard`` per block, fp32 sharded parameters computed in bf16).  tp: Megatron split with
    NCCL all-reduces inside tensor-parallel groups and DDP across them."""
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline"))
    import torch_baselines as TB
    shape = dict(TB.LLAMA_SHAPES[a.model])
    if a.layers:
        shape["n_layer"] = a.layers
    mode = a.mode if world > 1 else "single"
    torch.manual_seed(0)
    dp_world, tp = world, 1
    if mode == "tp":
        tp = a.tp or world
        dp_world = world // tp
        tp_groups = [dist.new_group(list(range(g * tp, (g + 1) * tp))) for g in range(dp_world)]
        dp_groups = [dist.new_group(list(range(r, world, tp))) for r in range(tp)]
        net = TB.Llama(seq=a.seq, tp=tp, group=tp_groups[rank // tp], **shape).cuda().to(torch.bfloat16)
        if dp_world > 1:
            net_run = torch.nn.parallel.DistributedDataParallel(net, device_ids=[local], process_group=dp_groups[rank % tp])
        else:
            net_run = net
        opt = TB.MasterAdamW(net.parameters(), 3e-4, (0.9, 0.95), 0.1)
        step_opt = opt.step
    elif mode == "fsdp":
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        net = TB.Llama(seq=a.seq, **shape).cuda()
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
        for blk in net.blocks:
            fully_shard(blk, mp_policy=mp)
        fully_shard(net, mp_policy=mp)
        net_run = net
        topt = torch.optim.AdamW(net.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

        def step_opt():
            topt.step()
            topt.zero_grad(set_to_none=True)
    else:
        net = TB.Llama(seq=a.seq, **shape).cuda().to(torch.bfloat16)
        net_run = net
        opt = TB.MasterAdamW(net.parameters(), 3e-4, (0.9, 0.95), 0.1)
        step_opt = opt.step
    data_rank = rank // tp if mode == "tp" else rank
    gen = torch.Generator().manual_seed(100 + data_rank)
    tok = torch.randint(0, shape["vocab"], (a.batch, a.seq), generator=gen).pin_memory()
    tgt = torch.roll(tok, -1, 1).pin_memory()
    dtok, dtgt = tok.cuda(), tgt.cuda()
    loss_dev = torch.zeros((), device="cuda")

    def device_step():
        loss = net_run(dtok, dtgt)
        loss.backward()
        step_opt()
        loss_dev.copy_(loss.detach())
    graph = None
    if mode == "single":
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                device_step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                device_step()
            graph = g
        except Exception as exc:  # noqa: BLE001
            sys.stderr.write(f"[baseline] step not captured: {exc}\n")
            torch.cuda.synchronize()

    def step():
        dtok.copy_(tok, non_blocking=True)
        dtgt.copy_(tgt, non_blocking=True)
        graph.replay() if graph is not None else device_step()
        return float(loss_dev.item())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(max(a.warmup, 3)):
        loss = step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / a.steps
    tokens = a.batch * a.seq * (dp_world if mode == "tp" else world)
    if rank == 0:
        print(json.dumps({
            "metric": "train_tokens_per_s", "impl": "baseline", "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms,
            "n_gpus": world, "loss": loss, "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
            "config": {"model": a.model, "layers": shape["n_layer"], "mode": mode, "tp": tp, "micro_batch_per_gpu": a.batch,
                       "seq_len": a.seq, "global_batch": tokens // a.seq, "cuda_graph": graph is not None,
                       "implementation": "plain PyTorch: cuBLAS bf16, flash SDPA, fused AdamW, NCCL"},
            "dtype": "bf16", "data": "synthetic"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
