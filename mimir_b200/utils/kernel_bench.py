"""Micro-benchmarks of the hand-written kernels against the library baselines.

    python -m mimir_b200.utils.kernel_bench gemm --m 8192 --n 2304 --k 768
    python -m mimir_b200.utils.kernel_bench attention --b 8 --t 1024 --h 12 --d 64

Times with CUDA events after warm-up; between timed iterations an L2-sized
buffer is overwritten so that no operand is served from a warm L2.  Prints one
JSON line per case with achieved TFLOP/s and the fraction of the measured cuBLAS
bf16 peak recorded in ``MEASURED_PEAKS.json`` (if present).
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except OSError:
        return {}


def time_ms(fn, iters: int, flush: torch.Tensor | None) -> float:
    """Mean device time of ``fn``; all iterations are queued before the one sync, so
    host launch latency never shows up as idle time between the two events."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs) / iters


def bench_gemm(a):
    from ..ops.gemm import gemm
    M, N, K = a.m, a.n, a.k
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    dy = torch.randn(M, N, device="cuda").bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if a.flush else None
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    dw = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
    peak = _peaks().get("bf16_tflops")
    cases = {
        "nt_forward": (lambda: gemm(x, w, out=out, bn=a.bn), lambda: torch.matmul(x, w.t(), out=out)),
        "nn_dgrad": (lambda: gemm(dy, w, b_mn=True, out=dx, bn=a.bn), lambda: torch.matmul(dy, w, out=dx)),
        "tn_wgrad": (lambda: gemm(dy, x, a_mn=True, b_mn=True, out=dw, bn=a.bn),
                     lambda: torch.matmul(dy.t(), x, out=dw)),
    }
    for name, (ours, lib) in cases.items():
        if a.only and a.only != name:
            continue
        t = time_ms(ours, a.iters, flush)
        rec = {"kernel": "gemm_bf16", "case": name, "M": M, "N": N, "K": K, "ms": t,
               "tflops": 2.0 * M * N * K / t / 1e9}
        if peak:
            rec["frac_of_measured_cublas_peak"] = rec["tflops"] / peak
        if not a.no_baseline:
            tl = time_ms(lib, a.iters, flush)
            rec["cublas_ms"] = tl
            rec["cublas_tflops"] = 2.0 * M * N * K / tl / 1e9
        print(json.dumps(rec), flush=True)


def bench_attention(a):
    from ..ops.attention import attention_bwd, attention_fwd
    B, T, H, D = a.b, a.t, a.h, a.d
    qkv = torch.randn(B, T, 3, H, D, device="cuda").bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    out = torch.empty(B, T, H, D, device="cuda", dtype=torch.bfloat16)
    do = torch.randn_like(out)
    lse = torch.empty(B, H, T, device="cuda")
    dsum = torch.empty(B, H, T, device="cuda")
    dqkv = torch.empty_like(qkv)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if a.flush else None
    flops_fwd = 4.0 * B * H * T * T * D / 2  # causal
    t = time_ms(lambda: attention_fwd(q, k, v, out, lse, causal=True), a.iters, flush)
    print(json.dumps({"kernel": "attention_fwd", "B": B, "T": T, "H": H, "D": D, "ms": t,
                      "tflops": flops_fwd / t / 1e9}), flush=True)
    t = time_ms(lambda: attention_bwd(q, k, v, out, do, lse, dsum, dqkv[:, :, 0], dqkv[:, :, 1],
                                      dqkv[:, :, 2], causal=True), a.iters, flush)
    print(json.dumps({"kernel": "attention_bwd", "B": B, "T": T, "H": H, "D": D, "ms": t,
                      "tflops": 2.5 * flops_fwd / t / 1e9}), flush=True)
    if not a.no_baseline:
        qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
        t = time_ms(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True),
                    a.iters, flush)
        print(json.dumps({"kernel": "torch_sdpa_fwd", "ms": t, "tflops": flops_fwd / t / 1e9}), flush=True)


def bench_q4(a):
    """Q4_0 weight x activation products of a decode step: the tensor-core kernel and the dp4a GEMV."""
    from ..ops import quant_cuda as Q
    N, K, B = a.n, a.k, a.b
    dev = "cuda"
    nb = N * K // 32
    planar = Q.PlanarQ4((torch.rand(nb, device=dev) * 0.01).half(), torch.randint(0, 256, (nb * 16,), device=dev, dtype=torch.uint8), N, K)
    tiled = Q.TiledQ4.from_planar(planar)
    x = torch.randn(B, K, device=dev).bfloat16()
    out = torch.empty(B, N, device=dev, dtype=torch.bfloat16)
    scratch = Q.TcScratch(B * N, dev)
    xq = torch.randint(-127, 127, (B, K), device=dev, dtype=torch.int8)
    xs = torch.rand(B, K // 32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    nbytes = N * K * 0.5625
    peak = _peaks().get("hbm_gbs")
    for name, fn in (("q4_tc", lambda: Q.q4_tc(tiled, x, out, scratch, splits=a.splits)),
                     ("q4_gemv_dp4a", lambda: Q.q4_gemv(planar, xq, xs, out))):
        if a.only and a.only != name:
            continue
        t = time_ms(fn, a.iters, flush)
        rec = {"kernel": name, "N": N, "K": K, "B": B, "us": t * 1e3, "weight_gbs": nbytes / t / 1e6}
        if peak:
            rec["frac_of_measured_hbm_copy"] = rec["weight_gbs"] / peak
        print(json.dumps(rec), flush=True)


def _finite_blocks(code, nblocks, dev):
    """Random ggml blocks with small finite scales (payload bytes are arbitrary)."""
    per = {64: 34, 65: 18, 66: 144, 67: 210}[code]
    raw = torch.randint(0, 256, (nblocks, per), dtype=torch.uint8, device=dev)
    d = torch.full((nblocks,), 0.01, device=dev).half().view(torch.uint8).reshape(nblocks, 2)
    if code == 67:
        raw[:, 208:210] = d
    else:
        raw[:, 0:2] = d
        if code == 66:
            raw[:, 2:4] = d
    return raw.reshape(-1)


def bench_qgemv(a):
    """GEMV over ggml blocks read in place (Q8_0 / Q4_0 / Q4_K / Q6_K), weights streamed from HBM."""
    from ..ops import quant_cuda as Q
    N, K, B = a.n, a.k, a.b
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    peak = _peaks().get("hbm_gbs")
    x = torch.randn(B, K, device=dev)
    for name, code, vals, per in (("q8_0", 64, 32, 34), ("q4_0", 65, 32, 18), ("q4_k", 66, 256, 144), ("q6_k", 67, 256, 210)):
        if a.only and a.only != name:
            continue
        raw = _finite_blocks(code, N * K // vals, dev)
        t = time_ms(lambda: Q.qgemv_ggml(code, raw, N, K, x), a.iters, flush)
        rec = {"kernel": "qgemv_ggml_" + name, "N": N, "K": K, "B": B, "us": t * 1e3,
               "weight_gbs": raw.numel() / t / 1e6}
        if peak:
            rec["frac_of_measured_hbm_copy"] = rec["weight_gbs"] / peak
        print(json.dumps(rec), flush=True)


def bench_sample(a):
    """The fused sampling kernel on [rows, vocab] logits."""
    from ..ops.sampling import sample
    x = (torch.randn(a.rows, a.vocab, device="cuda") * 3).bfloat16()
    out = torch.empty(a.rows, dtype=torch.int32, device="cuda")
    for name, kw in (("greedy", dict(temperature=0.0)), ("top_k40_top_p0.95", dict(temperature=0.8, top_k=40, top_p=0.95)),
                     ("top_p0.9", dict(temperature=1.0, top_k=0, top_p=0.9))):
        if a.only and a.only != name:
            continue
        t = time_ms(lambda: sample(x, out=out, **kw), a.iters, None)
        print(json.dumps({"kernel": "sample_" + name, "rows": a.rows, "vocab": a.vocab, "us": t * 1e3,
                          "logits_gbs": x.numel() * 2 / t / 1e6}), flush=True)


def bench_conv(a):
    """Implicit-GEMM convolution (forward, input gradient, weight gradient) against cuDNN through PyTorch."""
    from ..ops import conv as C
    N, Ci, Co, H, W, Kk = a.n, a.ci, a.co, a.h, a.w, a.ksize
    pad = Kk // 2
    x = torch.randn(N, Ci, H, W, device="cuda").bfloat16()
    w = (torch.randn(Co, Ci, Kk, Kk, device="cuda") * 0.05).bfloat16()
    xn, wp, wd = C.to_nhwc(x), C.pack_filter(w), C.pack_filter_dgrad(w)
    y = C.conv2d_fwd(xn, wp, Kk, Kk, pad)
    dy = torch.randn_like(y)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if a.flush else None
    flops = 2.0 * N * H * W * Co * Ci * Kk * Kk
    peak = _peaks().get("bf16_tflops")
    cases = {"conv_fwd": lambda: C.conv2d_fwd(xn, wp, Kk, Kk, pad, out=y),
             "conv_dgrad": lambda: C.conv2d_dgrad(dy, wd, Kk, Kk, pad),
             "conv_wgrad": lambda: C.conv2d_wgrad(dy, xn, Co, Kk, Kk, pad)}
    for name, fn in cases.items():
        if a.only and a.only != name:
            continue
        t = time_ms(fn, a.iters, flush)
        rec = {"kernel": name, "N": N, "Ci": Ci, "Co": Co, "H": H, "W": W, "k": Kk, "ms": t, "tflops": flops / t / 1e9}
        if peak:
            rec["frac_of_measured_cublas_peak"] = rec["tflops"] / peak
        print(json.dumps(rec), flush=True)
    if not a.no_baseline:
        xc, wc = x.contiguous(memory_format=torch.channels_last), w.contiguous(memory_format=torch.channels_last)
        t = time_ms(lambda: torch.nn.functional.conv2d(xc, wc, padding=pad), a.iters, flush)
        print(json.dumps({"kernel": "cudnn_conv_fwd(torch)", "ms": t, "tflops": flops / t / 1e9}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=2304)
    g.add_argument("--k", type=int, default=768)
    g.add_argument("--bn", type=int, default=0)
    g.add_argument("--only", default="")
    t = sub.add_parser("attention")
    t.add_argument("--b", type=int, default=8)
    t.add_argument("--t", type=int, default=1024)
    t.add_argument("--h", type=int, default=12)
    t.add_argument("--d", type=int, default=64)
    q = sub.add_parser("q4")
    q.add_argument("--n", type=int, default=28672)
    q.add_argument("--k", type=int, default=4096)
    q.add_argument("--b", type=int, default=1)
    q.add_argument("--splits", type=int, default=0)
    q.add_argument("--only", default="")
    c = sub.add_parser("conv")
    c.add_argument("--n", type=int, default=32)
    c.add_argument("--ci", type=int, default=128)
    c.add_argument("--co", type=int, default=128)
    c.add_argument("--h", type=int, default=56)
    c.add_argument("--w", type=int, default=56)
    c.add_argument("--ksize", type=int, default=3)
    c.add_argument("--only", default="")
    qg = sub.add_parser("qgemv")
    qg.add_argument("--n", type=int, default=65536)
    qg.add_argument("--k", type=int, default=4096)
    qg.add_argument("--b", type=int, default=1)
    qg.add_argument("--only", default="")
    sp = sub.add_parser("sample")
    sp.add_argument("--rows", type=int, default=32)
    sp.add_argument("--vocab", type=int, default=128256)
    sp.add_argument("--only", default="")
    for p in (g, t, q, c, qg, sp):
        p.add_argument("--iters", type=int, default=10)
        p.add_argument("--flush", action="store_true")
        p.add_argument("--no-baseline", action="store_true")
    a = ap.parse_args()
    {"gemm": bench_gemm, "attention": bench_attention, "q4": bench_q4, "conv": bench_conv, "qgemv": bench_qgemv,
     "sample": bench_sample}[a.cmd](a)


if __name__ == "__main__":
    main()
