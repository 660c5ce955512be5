"""Fused compute + collective kernels against their roofline and against the NCCL lowering.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m mimir_b200.utils.bench_comm [--iters 20]

For each fused kernel: CUDA-event time (max over ranks, after warm-up, with a barrier on both
sides), the bytes every GPU must send and receive over NVLink (computed from the algorithm), the
product's FLOPs, and the roofline time = max(FLOPs / measured GEMM peak, NVLink bytes per direction
/ link bandwidth); ``frac`` = roofline / measured.  The same operation lowered to a library GEMM
plus an NCCL collective is timed next to it.  Prints one JSON line per kernel on rank 0.

Kernels: ``dp_bucket_kernel`` (gradient reduce-scatter + AdamW + parameter all-gather over the
whole GPT-2 small parameter buffer), ``gemm_comm_kernel<1>`` (all-gather -> GEMM) and
``gemm_comm_kernel<2>`` (GEMM -> reduce-scatter) on Llama-7B block shapes.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0          # measured peer copy per direction on this pool (900 nominal)


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mimir_b200 import _native
    from mimir_b200.ops import kernels as K
    from mimir_b200.ops._util import check_error_word, ptr
    from mimir_b200.ops.gemm import gemm
    from mimir_b200.parallel import fused_gemm as FG
    from mimir_b200.parallel.peer import SymmetricBuffer
    lib = _native.lib()
    lib.mimir_set_device(local)
    tflops, hbm, which = _peaks()

    def timed(fn, iters=a.iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e-3

    def report(name, sec, base_sec, flops, link_bytes, hbm_bytes, shape):
        roof = max(flops / (tflops * 1e12), link_bytes / (LINK_GBS * 1e9), hbm_bytes / (hbm * 1e9))
        if rank == 0:
            print(json.dumps({"kernel": name, "n_gpus": world, "shape": shape, "us": round(sec * 1e6, 1),
                              "nccl_lowering_us": round(base_sec * 1e6, 1), "speedup_vs_nccl": round(base_sec / sec, 3),
                              "flops": flops, "nvlink_bytes_per_direction": int(link_bytes), "hbm_bytes": int(hbm_bytes),
                              "roofline_us": round(roof * 1e6, 1), "frac_of_roofline": round(roof / sec, 3),
                              "bound": "compute" if roof == flops / (tflops * 1e12) else
                              ("nvlink" if roof == link_bytes / (LINK_GBS * 1e9) else "hbm"),
                              "peaks": {"bf16_tflops": tflops, "link_gbs": LINK_GBS, "hbm_gbs": hbm, "source": which},
                              "error_word": check_error_word()}), flush=True)

    # ------------------------------------------------------------------ dp bucket kernel
    n = 124_475_904 // (8 * world) * (8 * world)          # GPT-2 small parameter count
    pbuf, gbuf = SymmetricBuffer(n * 2, rank, world), SymmetricBuffer(n * 2, rank, world)
    sig = SymmetricBuffer(4096 * 4, rank, world)
    params, grads = pbuf.view(torch.bfloat16, 0, n), gbuf.view(torch.bfloat16, 0, n)
    grads.normal_(0, 1e-3)
    shard = n // world
    master = torch.zeros(shard, device="cuda")
    m, v = torch.zeros(shard, device="cuda"), torch.zeros(shard, device="cuda")
    hyper = torch.tensor([1e-4, 0.1, 0.2, 1.0 / world], device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    done = torch.tensor([1], dtype=torch.int32, device="cuda")
    pa, ga, sa = pbuf.ptr_array(), gbuf.ptr_array(), sig.ptr_array()
    nblocks = 2 * torch.cuda.get_device_properties(local).multi_processor_count
    st = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731

    def fused_dp():
        lib.mimir_dp_step_begin(ptr(epoch), ctypes.c_void_p(sig.local_ptr), 1, ptr(done), world, st())
        lib.mimir_dp_bucket(ga, pa, sa, ptr(master), ptr(m), ptr(v), ptr(hyper), ptr(epoch), ptr(counter), 0, n, n, 0,
                            0.9, 0.95, 1e-8, 0.1, rank, world, 0, 1, nblocks, st())
    g32 = torch.empty(shard, device="cuda", dtype=torch.bfloat16)

    def nccl_dp():
        dist.reduce_scatter_tensor(g32, grads)
        K.adamw_flat(master, params[rank * shard:(rank + 1) * shard], g32, m, v, lr=1e-4, step=1, gscale=1.0 / world)
        dist.all_gather_into_tensor(params, params[rank * shard:(rank + 1) * shard].clone())
    t_f, t_b = timed(fused_dp), timed(nccl_dp)
    link = (world - 1) / world * n * 2                      # gradients in, parameters out: each direction
    hbm_b = n * 2 + shard * (3 * 4 * 2) + n * 2             # own gradients read by peers, states, parameters written
    report("dp_bucket_kernel (reduce-scatter + AdamW + all-gather)", t_f, t_b, 0.0, link, hbm_b, {"elements": n})
    torch.cuda.synchronize()
    dist.barrier()

    # ------------------------------------------------------------------ all-gather -> GEMM, GEMM -> reduce-scatter
    for (M, N, Kd, tag) in ((4096, 11008, 4096, "llama-7b gate/up"), (4096, 4096, 4096, "llama-7b attention")):
        if N % world or (N // world) % 8:
            continue
        w = FG.ShardedWeight(N, Kd, rank, world)
        w.shard.normal_(0, 0.02)
        x = torch.randn(M, Kd, device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()
        t_f = timed(lambda: FG.gemm_allgather(x, w, out=out))
        t_b = timed(lambda: FG.gemm_allgather_baseline(x, w))
        report("gemm_comm_kernel<COMM=1> all-gather -> GEMM", t_f, t_b, 2.0 * M * N * Kd,
               (world - 1) / world * N * Kd * 2, (M * Kd + N * Kd + M * N) * 2, {"M": M, "N": N, "K": Kd, "what": tag})
        torch.cuda.synchronize()
        dist.barrier()
        w.close()
    for (M, N, Kd, tag) in ((4096, 4096, 11008 // world // 8 * 8, "llama-7b down (row parallel)"),
                            (11008 // (32 * world) * 32 * world, 4096, 4096, "llama-7b gate/up weight gradient")):
        if M % world or (M // world) % 32:
            continue
        rs = FG.ReduceScatterGemm(M, N, rank, world)
        aa = torch.randn(M, Kd, device="cuda").bfloat16()
        bb = (torch.randn(N, Kd, device="cuda") * 0.02).bfloat16()
        o = torch.empty(M // world, N, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()
        t_f = timed(lambda: rs(aa, bb, out=o))
        t_b = timed(lambda: FG.gemm_reduce_scatter_baseline(aa, bb, world))
        report("gemm_comm_kernel<COMM=2> GEMM -> reduce-scatter", t_f, t_b, 2.0 * M * N * Kd,
               (world - 1) / world * M * N * 2, (M * Kd + N * Kd) * 2 + 2 * M * N * 2, {"M": M, "N": N, "K": Kd, "what": tag})
        torch.cuda.synchronize()
        dist.barrier()
        rs.close()
    torch.cuda.synchronize()
    dist.barrier()
    for b in (pbuf, gbuf, sig):
        b.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
