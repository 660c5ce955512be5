"""Tensor-parallel Llama decode benchmark (Llama-3-8B architecture, random-init
weights quantized to Q4_0, Q8_0 activations, fp16 KV cache).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m mimir_b200.utils.bench_decode --batch 1 --prompt 512 --gen 256

Device-timed with CUDA events, max over ranks; prints one JSON line on rank 0 with
decode tokens/s (batch * generated tokens / time) and prompt tokens/s.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--gen", type=int, default=256)
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "tiny"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the model's)")
    ap.add_argument("--engine", default="auto", choices=["auto", "tc", "dp4a"])
    ap.add_argument("--sequential-prefill", action="store_true", help="feed the prompt token by token")
    ap.add_argument("--primitives", action="store_true",
                    help="also time each kernel of the step on its own (at the final cache length)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mimir_b200 import _native
    from mimir_b200.llm import LlamaConfig, TPDecoder
    from mimir_b200.ops._util import check_error_word
    _native.lib().mimir_set_device(local)
    cfg = LlamaConfig.llama3_8b() if a.model == "llama3-8b" else LlamaConfig.tiny()
    if a.layers:
        cfg.n_layer = a.layers
    dec = TPDecoder(cfg, rank, world, batch=a.batch, cap=a.prompt + a.gen + 8, seed=0, engine=a.engine)
    prompt = torch.randint(0, cfg.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(1))

    def timed(fn):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    dec.reset()
    for _ in range(4):  # warm-up and graph capture
        dec.step()
    if not a.sequential_prefill:   # untimed pass: buffers and kernels of the GEMM path are warm afterwards
        dec.prefill_batched(prompt)
    dec.reset()
    ms_prompt = timed(lambda: (dec.prefill if a.sequential_prefill else dec.prefill_batched)(prompt))
    launches0 = _native.lib().mimir_launch_count()
    ms_gen = timed(lambda: [dec.step() for _ in range(a.gen)])
    launches = _native.lib().mimir_launch_count() - launches0
    prim = dec.primitive_times() if a.primitives else None
    err = check_error_word()
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": a.batch * a.gen / (ms_gen / 1e3), "unit": "tokens/s",
            "ms_per_token": ms_gen / a.gen, "prompt_tokens_per_s": a.batch * a.prompt / (ms_prompt / 1e3),
            "n_gpus": world, "batch": a.batch, "prompt": a.prompt, "gen": a.gen,
            "config": {"model": a.model, "layers": cfg.n_layer, "weights": "Q4_0", "activations": "Q8_0", "engine": dec.engine,
                       "kv_cache": "fp16", "parallelism": f"tp{world}"},
            "gpu_launches": int(launches), "launches_per_token": int(dec.launches_per_step), "primitive_us": prim, "error_word": err}))
    dec.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
