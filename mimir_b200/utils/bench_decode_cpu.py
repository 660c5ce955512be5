"""Decode tokens/s on the host for a Llama-3.2-1B-shaped model with Q4_K_M-style weights (Q4_K
projections, Q6_K embedding / tied output head), the configuration the reference quotes its CPU
decode numbers on (README.md:449-454: about 1.15 x llama.cpp's time on one core).

    python -m mimir_b200.utils.bench_decode_cpu [--threads 1,4,8] [--gen 32] [--impl ours|baseline]

``ours``: ``llm.CPUDecoder`` over the blocks (native VNNI products).  ``baseline``: the same decode
loop in plain PyTorch over the same weights expanded to bfloat16 once (library matmuls), which is
what a framework without quantized host kernels does.  Random blocks with sane scales; one JSON line
per thread count.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from ..io import mim
from ..llm import Config, CPUDecoder
from ..ops import quant as Q
from ..ops import quant_cpu


def _blocks(code, n, k, gen):
    vals, nbytes = Q.BLOCK[code]
    raw = torch.randint(0, 256, (n * k // vals, nbytes), dtype=torch.uint8, generator=gen)
    d = (torch.rand(raw.shape[0], generator=gen) * 0.004 + 0.001).to(torch.float16).view(torch.uint8).reshape(-1, 2)
    if code == Q.Q4_K:
        raw[:, 0:2] = d
        raw[:, 2:4] = (torch.rand(raw.shape[0], generator=gen) * 0.002).to(torch.float16).view(torch.uint8).reshape(-1, 2)
    elif code == Q.Q6_K:
        raw[:, 208:210] = d
    else:
        raw[:, 0:2] = d
    return mim.QuantizedTensor(code, (n, k), raw.reshape(-1))


def model_tensors(c: Config, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    q, kv = c.heads * c.head_dim, c.kv_heads * c.head_dim
    t = {"token_embd.weight": _blocks(Q.Q6_K, c.vocab, c.embed, g), "output_norm.weight": torch.ones(c.embed)}
    for i in range(c.layers):
        p = f"blk.{i}."
        t[p + "attn_norm.weight"] = torch.ones(c.embed)
        t[p + "ffn_norm.weight"] = torch.ones(c.embed)
        t[p + "attn_q.weight"] = _blocks(Q.Q4_K, q, c.embed, g)
        t[p + "attn_k.weight"] = _blocks(Q.Q4_K, kv, c.embed, g)
        t[p + "attn_v.weight"] = _blocks(Q.Q4_K, kv, c.embed, g)
        t[p + "attn_output.weight"] = _blocks(Q.Q4_K, c.embed, q, g)
        t[p + "ffn_gate.weight"] = _blocks(Q.Q4_K, c.hidden, c.embed, g)
        t[p + "ffn_up.weight"] = _blocks(Q.Q4_K, c.hidden, c.embed, g)
        t[p + "ffn_down.weight"] = _blocks(Q.Q4_K, c.embed, c.hidden, g)
    return t


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--threads", default="1,4,8")
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--gen", type=int, default=32)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline"])
    ap.add_argument("--mode", default="auto")
    a = ap.parse_args(argv)
    c = Config(arch="llama", vocab=128256, context=256, embed=2048, hidden=8192, layers=a.layers, heads=32, kv_heads=8,
               head_dim=64, rope_dim=64, rope_base=500000.0)
    tensors = model_tensors(c)
    if a.impl == "baseline":
        tensors = {k: (v.dequantize(torch.bfloat16) if isinstance(v, mim.QuantizedTensor) else v) for k, v in tensors.items()}
        dec = CPUDecoder(c, tensors, cap=a.prompt + a.gen + 1, mode="exact", float_as="f32")
        for m in [dec.embed, dec.head] + [l[k] for l in dec.layers for k in ("qkv", "o", "gate_up", "down")]:
            m.data = m.data.bfloat16()                      # library path: bf16 weights, torch matmul
            m.mul = (lambda mm: (lambda x, mode: (x.bfloat16() @ mm.data.t()).float()))(m)
        dec.embed.rows = lambda idx, e=dec.embed: e.data[idx].float()
    else:
        dec = CPUDecoder(c, tensors, cap=a.prompt + a.gen + 1, mode=a.mode)
    prompt = torch.randint(0, c.vocab, (1, a.prompt))
    for th in [int(x) for x in a.threads.split(",")]:
        quant_cpu.set_threads(th)
        torch.set_num_threads(th)
        dec.reset()
        tp = time.perf_counter()
        logits = dec.prefill(prompt)
        tp = time.perf_counter() - tp
        t0 = time.perf_counter()
        for _ in range(a.gen):
            logits = dec.step(logits.argmax(-1))
        dt = (time.perf_counter() - t0) / a.gen
        print(json.dumps({"metric": "cpu_decode_tokens_per_s", "impl": a.impl, "value": 1.0 / dt, "ms_per_token": dt * 1e3,
                          "prompt_tokens_per_s": a.prompt / tp, "threads": th, "weight_gb": dec.weight_bytes() / 1e9, "weights_gb_per_s": dec.weight_bytes() / dt / 1e9,
                          "config": {"model": "llama-3.2-1b shape", "layers": c.layers, "weights": "Q4_K + Q6_K head" if a.impl == "ours" else "bf16",
                                     "mode": dec.mode, "prompt": a.prompt, "gen": a.gen}, "data": "synthetic"}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
