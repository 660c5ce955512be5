"""Worker for the fused all-gather->GEMM and GEMM->reduce-scatter tests."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mimir_b200 import _native
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.parallel import fused_gemm as FG
    _native.lib().mimir_set_device(local)
    res = {"rank": rank}
    torch.manual_seed(3)
    # ---- all-gather -> GEMM
    M, N, K = 1024, 1536, 512
    w_full = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    dist.broadcast(w_full, 0)
    x = torch.randn(M, K, device="cuda").bfloat16()  # each rank its own activations
    w = FG.ShardedWeight(N, K, rank, world)
    w.shard.copy_(w_full[rank * w.rows: (rank + 1) * w.rows])
    dist.barrier()
    errs = []
    for _ in range(3):  # repeated calls reuse the counters
        w.full[: rank * w.rows].zero_()
        w.full[(rank + 1) * w.rows:].zero_()
        torch.cuda.synchronize()
        dist.barrier()
        y = FG.gemm_allgather(x, w)
        torch.cuda.synchronize()
        ref = x.float() @ w_full.float().t()
        errs.append(((y.float() - ref).abs().max() / ref.abs().max()).item())
        dist.barrier()
    res["ag_err"] = max(errs)
    base = FG.gemm_allgather_baseline(x, w)
    res["ag_vs_nccl"] = ((y.float() - base.float()).abs().max()).item()
    # ---- GEMM -> reduce-scatter (NT and TN)
    M2, N2, K2 = 2048, 768, 256
    a = torch.randn(M2, K2, device="cuda").bfloat16()
    b = (torch.randn(N2, K2, device="cuda") * 0.1).bfloat16()
    rs = FG.ReduceScatterGemm(M2, N2, rank, world)
    full = a.float() @ b.float().t()
    dist.all_reduce(full)
    rpr = M2 // world
    errs = []
    for _ in range(3):
        out = rs(a, b)
        torch.cuda.synchronize()
        ref = full[rank * rpr: (rank + 1) * rpr]
        errs.append(((out.float() - ref).abs().max() / ref.abs().max()).item())
        dist.barrier()
    res["rs_err"] = max(errs)
    at, bt = a.t().contiguous(), b.t().contiguous()  # stored [K, M], [K, N]
    out = rs(at, bt, transposed=True)
    torch.cuda.synchronize()
    res["rs_tn_err"] = ((out.float() - full[rank * rpr: (rank + 1) * rpr]).abs().max() / full.abs().max()).item()
    # ---- back-to-back calls on the same object with different inputs and NO host synchronisation or
    # barrier in between: a rank that runs ahead must not overwrite slabs its peer is still summing
    torch.cuda.synchronize()
    dist.barrier()
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    ins = [(torch.randn(M2, K2, device="cuda", generator=gen).bfloat16(),
            (torch.randn(N2, K2, device="cuda", generator=gen) * 0.1).bfloat16()) for _ in range(6)]
    outs = []
    for i, (ai, bi) in enumerate(ins):
        if i in (2, 4) and rank == (i // 2) % world:
            torch.cuda._sleep(40_000_000)          # this rank falls behind: its peers reach the next call first
        outs.append(rs(ai, bi))
    torch.cuda.synchronize()
    worst = 0.0
    for (ai, bi), o in zip(ins, outs):
        ref = FG.gemm_reduce_scatter_baseline(ai, bi, world)
        worst = max(worst, ((o.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-6)).item())
    res["rs_b2b_err"] = worst
    res["err"] = check_error_word()
    dist.barrier()
    w.close()
    rs.close()
    dist.destroy_process_group()
    os.write(1, ("RESULT " + json.dumps(res) + "\n").encode())  # one write: lines of different ranks never interleave


if __name__ == "__main__":
    main()
