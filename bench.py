#!/usr/bin/env python
"""Headline benchmark: GPT-2 small (12 layers, d=768, 12 heads, vocab 50257,
ctx 1024) data-parallel training in bf16 with fp32 master weights, sequence
1024, micro-batch 8 per GPU, synthetic token ids, random-init weights.

    python bench.py --gpus N --steps K --warmup W          (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \
        --master-addr 127.0.0.1 --master-port P bench.py --gpus N --steps K --warmup W

Rank 0 prints ONE JSON line.  ``value`` is the whole-job tokens/s of the
device-timed loop (CUDA events, max over ranks); ``e2e`` is the same metric
through ``FusedTrainer.step`` with the host->device copy of every batch from
pinned memory and the device->host read of the loss inside the timed region.
``--impl reference`` reports that the reference (a Go program) cannot run here.
``--impl baseline`` runs the same model, batch, optimizer and timing code in plain PyTorch
(cuBLAS bf16 products, flash SDPA, fused AdamW over fp32 masters, NCCL DDP; the step captured in
a CUDA graph on one GPU): ``baseline/torch_baselines.py``, which imports nothing of this package.
Its measured numbers are kept in ``baseline/measured.json``; the native arm reports
``vs_library_baseline`` against them.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "train_tokens_per_s"
MODEL = "gpt2-small(12L,d768,12h,vocab50257,ctx1024)"

SMI_QUERY = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU.  The process starts early (its
    start-up takes about a second) and keeps running; ``window(t0, t1)`` summarises the samples
    whose time stamps fall inside a timed region."""

    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.rows = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        self.proc = None
        import datetime
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                self.rows.append((ts, float(f[2]), float(f[3]), float(f[4]), [v.lower().startswith("active") for v in f[6:10]]))
            except ValueError:
                continue

    def window(self, t0: float, t1: float) -> dict:
        """Median SM clock, maximum clock, power and active throttle reasons between two ``time.time()`` stamps."""
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable or no samples"]}
        inside = [r for r in self.rows if t0 - 0.05 <= r[0] <= t1 + 0.05]
        note = None
        if not inside:      # region shorter than the sampling period: take the nearest sample
            inside = [min(self.rows, key=lambda r: abs(r[0] - (t0 + t1) / 2))]
            note = "nearest sample (timed region shorter than the 100 ms sampling period)"
        reasons = sorted({n for r in inside for n, on in zip(self.NAMES, r[4]) if on})
        out = {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": max(r[2] for r in inside),
               "reasons": reasons, "power_w_max": max(r[3] for r in inside), "samples": len(inside)}
        if note:
            out["note"] = note
        return out


def _against_library_baseline(world: int, value: float, e2e: float) -> dict:
    """Ratios against the recorded run of ``--impl baseline`` on the same number of GPUs
    (``baseline/measured.json``, written from that arm's output on the same kind of box)."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "measured.json")
    try:
        with open(path) as f:
            rec = json.load(f)["gpt2_small_dp"][str(world)]
    except (OSError, KeyError, ValueError):
        return {"vs_library_baseline": None}
    return {"vs_library_baseline": {"ratio": value / rec["value"], "e2e_ratio": e2e / rec["e2e"],
                                    "baseline_tokens_per_s": rec["value"], "baseline_e2e_tokens_per_s": rec["e2e"],
                                    "direction": "ours / baseline, higher is better"}}


def reference_arm(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": ("the reference is a Go 1.27 module with no setup.py/pyproject (pip: 'not "
                        "installable') and neither a Go toolchain nor its module cache exists offline"),
    }))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--attention", default="native")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--dp-blocks", type=int, default=0,
                    help="grid of the data-parallel bucket kernels that run beside backward (0 = two blocks per SM)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    # Libraries (NCCL's version banner among them) may write to stdout; the contract is
    # ONE JSON line there, so everything else goes to stderr until the result is printed.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # re-launch under torchrun so that there is one process per GPU
            os.dup2(real_stdout, 1)
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
                   os.environ.get("MASTER_PORT", "29517"), os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    warmup = max(args.warmup, 3)

    B, T = args.micro_batch, args.seq
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dp = None
    if args.impl == "baseline":
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
        import torch_baselines as TB
        torch.manual_seed(0)
        vocab = 50257
        net = TB.GPT2().cuda().to(torch.bfloat16)
        tr = TB.TorchTrainer(net, lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1, graph=not args.no_graph,
                             ddp=world > 1, local_rank=local_rank)
        tr.h2d_bytes_per_step, tr.d2h_bytes_per_step, tr.launches_per_step = 2 * B * T * 8, 4, 0
        launch_count = lambda: 0          # noqa: E731 - library kernels are not counted
        set_batch = lambda tok, tgt: tr.set_batch(tok, tgt)      # noqa: E731
        check_error_word = lambda: 0      # noqa: E731
    else:
        from mimir_b200 import _native
        from mimir_b200.models.gpt2 import GPT2Config, GPT2Engine
        from mimir_b200.ops._util import check_error_word
        from mimir_b200.train import FusedTrainer

        lib = _native.lib()
        lib.mimir_set_device(local_rank)
        flat_alloc = None
        if world > 1:
            from mimir_b200.parallel.dp import FusedDataParallel
            dp = FusedDataParallel(rank, world, local_rank, nblocks=args.dp_blocks)
            flat_alloc = dp.alloc_shared
        cfg = GPT2Config.small()
        vocab = cfg.vocab
        eng = GPT2Engine(cfg, B, T, device=f"cuda:{local_rank}", seed=0, flat_alloc=flat_alloc,
                         attention=args.attention)
        if dp is not None:
            dp.attach(eng)
        tr = FusedTrainer(eng, lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1, use_graph=not args.no_graph,
                          dp=dp)
        launch_count = lib.mimir_launch_count

        def set_batch(tok, tgt):
            eng.tokens.copy_(tok.view(-1))
            eng.targets.copy_(tgt.view(-1))

    gen = torch.Generator().manual_seed(1234 + rank)
    nbatch = 4
    toks = [torch.randint(0, vocab, (B, T), generator=gen).pin_memory() for _ in range(nbatch)]
    tgts = [torch.roll(t, -1, 1).pin_memory() for t in toks]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # warm-up through the public call (also captures the graph)
    for i in range(warmup):
        loss = tr.step(toks[i % nbatch], tgts[i % nbatch])

    def timed(fn):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = launch_count()
        w0, t0 = time.perf_counter(), time.time()
        e0.record()
        for i in range(args.steps):
            fn(i)
        e1.record()
        barrier()
        wall, t1 = time.perf_counter() - w0, time.time()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item(), launch_count() - l0, (t0, t1), wall

    # device-timed loop: batch already resident, no host round trip per step
    set_batch(toks[0], tgts[0])
    ms_dev, launches, win_dev, _ = timed(lambda i: tr.run_device_step())
    # end to end: H2D of the batch and D2H of the loss every step
    losses = []
    ms_e2e, _, win_e2e, wall_e2e = timed(lambda i: losses.append(tr.step(toks[i % nbatch], tgts[i % nbatch])))
    err = check_error_word()
    time.sleep(0.25)      # let the sampler print the last samples of the region
    sampler.stop()
    clocks, clocks_e2e = sampler.window(*win_dev), sampler.window(*win_e2e)

    tokens_per_step = B * T * world
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e = tokens_per_step * args.steps / (ms_e2e / 1e3)
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": MODEL, "global_batch": B * world, "micro_batch_per_gpu": B,
                       "seq_len": T, "parallelism": f"dp{world}", "optimizer": "AdamW fp32 master",
                       "l2": "per-step working set (~3 GB activations + 1.7 GB optimizer state) "
                             "exceeds the 126 MB L2, so no flush is needed between steps",
                       "cuda_graph": not args.no_graph, "attention": args.attention},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": tr.h2d_bytes_per_step,
                    "d2h_bytes_per_step": tr.d2h_bytes_per_step, "clocks": clocks_e2e,
                    "wall_s": wall_e2e},
            "gpu_launches": int(launches),
            "launches_per_step": int(tr.launches_per_step),
            "final_loss": losses[-1] if losses else None,
            "error_word": err,
            "impl": args.impl,
        }
        if args.impl == "baseline":
            out["config"]["implementation"] = ("plain PyTorch: cuBLAS bf16, flash SDPA, fused AdamW over fp32 masters, "
                                               "NCCL DDP; CUDA graph on one GPU: " + str(bool(getattr(tr, "graph", None))))
            out["gpu_launches"] = None
        else:
            out.update(_against_library_baseline(world, value, e2e))
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(out) + "\n").encode())
    if world > 1:
        if dp is not None:
            dp.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
