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
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline"],
                    help="baseline = plain PyTorch on weights expanded from Q4_0 to bf16 (cuBLAS, SDPA, NCCL all-reduce)")
    ap.add_argument("--primitives", action="store_true",
                    help="also time each kernel of the step on its own (at the final cache length)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if a.impl == "baseline":
        return baseline(a, rank, world)
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


def baseline(a, rank, world):
    """The library arm: same architecture, prompt and generation lengths, timing and output line."""
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline"))
    import torch_baselines as TB
    shape = dict(n_layer=32, d_model=4096, n_head=32, n_kv=8, ffn=14336, vocab=128256) if a.model == "llama3-8b" else \
        dict(n_layer=2, d_model=256, n_head=4, n_kv=2, ffn=512, vocab=1024)
    if a.layers:
        shape["n_layer"] = a.layers
    cap = a.prompt + a.gen + 8
    dec = TB.DecodeLlama(max_len=cap, batch=a.batch, rank=rank, world=world, **shape)
    prompt = torch.randint(0, shape["vocab"], (a.batch, a.prompt), generator=torch.Generator().manual_seed(1)).cuda()

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
    tok = torch.zeros(a.batch, 1, dtype=torch.int64, device="cuda")
    pos = torch.zeros((), dtype=torch.int64, device="cuda")
    out_tok = torch.zeros(a.batch, 1, dtype=torch.int64, device="cuda")

    def one_step():
        out_tok.copy_(dec.next_token(dec.step_static(tok, pos)))
    dec.pos = 0
    dec.forward(prompt)                       # warm-up of the prompt path
    for _ in range(3):
        one_step()
    graph = None
    try:
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            one_step()
        graph = g
    except Exception as exc:  # noqa: BLE001 - the baseline then runs eagerly
        import sys as _s
        _s.stderr.write(f"[baseline] decode step not captured: {exc}\n")
        torch.cuda.synchronize()
    dec.pos = 0
    ms_prompt = timed(lambda: dec.forward(prompt))

    def generate():
        for i in range(a.gen):
            pos.fill_(a.prompt + i)
            tok.copy_(out_tok)
            graph.replay() if graph is not None else one_step()
    ms_gen = timed(generate)
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": a.batch * a.gen / (ms_gen / 1e3), "unit": "tokens/s",
            "ms_per_token": ms_gen / a.gen, "prompt_tokens_per_s": a.batch * a.prompt / (ms_prompt / 1e3),
            "n_gpus": world, "batch": a.batch, "prompt": a.prompt, "gen": a.gen, "impl": "baseline",
            "config": {"model": a.model, "layers": shape["n_layer"], "weights": "Q4_0 expanded to bf16", "kv_cache": "fp16",
                       "parallelism": f"tp{world}", "cuda_graph": graph is not None,
                       "implementation": "plain PyTorch: cuBLAS bf16, SDPA, NCCL all-reduce"}}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
