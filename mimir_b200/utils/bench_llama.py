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
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
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
            "gpu_launches": int(lib.mimir_launch_count() - l0), "dtype": "bf16", "data": "synthetic", "error_word": err}))
    if mode in ("fsdp", "tp"):
        barrier()
        eng.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
