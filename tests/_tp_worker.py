"""Worker for the tensor-parallel decode test (one process per GPU)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def reference_logits(cfg, weights, tokens_seq):
    """fp32 Llama forward with the dequantised weights (no activation quantisation)."""
    from mimir_b200.ops.quant import dequantize_raw, quantize_q4_0, Q4_0
    def dq(w):
        return dequantize_raw(Q4_0, quantize_q4_0(w.float().cpu()), w.numel()).view(w.shape).cuda()
    D, H, Hk = cfg.head_dim, cfg.n_head, cfg.n_kv_head
    B, T = tokens_seq.shape
    x = weights["token_embd"].bfloat16().float()[tokens_seq]
    pos = torch.arange(T, device=x.device)
    inv = 1.0 / (cfg.rope_base ** (torch.arange(0, D, 2, device=x.device).float() / D))
    ang = pos[:, None].float() * inv[None]
    def rope(t):
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack([a * ang.cos() - b * ang.sin(), a * ang.sin() + b * ang.cos()], -1).flatten(-2)
    def rms(v, g):
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps)) * g
    for l in range(cfg.n_layer):
        a = rms(x, weights[f"blk.{l}.attn_norm"])
        qkv = a @ dq(weights[f"blk.{l}.qkv"]).t()
        q, k, v = qkv.split([H * D, Hk * D, Hk * D], -1)
        q = rope(q.view(B, T, H, D).transpose(1, 2))
        k = rope(k.view(B, T, Hk, D).transpose(1, 2)).repeat_interleave(H // Hk, 1)
        v = v.view(B, T, Hk, D).transpose(1, 2).repeat_interleave(H // Hk, 1)
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + o.transpose(1, 2).reshape(B, T, H * D) @ dq(weights[f"blk.{l}.o"]).t()
        a = rms(x, weights[f"blk.{l}.ffn_norm"])
        g, u = (a @ dq(weights[f"blk.{l}.gate_up"]).t()).chunk(2, -1)
        x = x + (torch.nn.functional.silu(g) * u) @ dq(weights[f"blk.{l}.down"]).t()
    x = rms(x, weights["output_norm"])
    return x @ dq(weights["output"]).t()


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mimir_b200 import _native
    from mimir_b200.llm import LlamaConfig, TPDecoder
    from mimir_b200.ops._util import check_error_word
    _native.lib().mimir_set_device(local)
    cfg = LlamaConfig.tiny()
    g = torch.Generator(device="cuda").manual_seed(11)
    D, d = cfg.head_dim, cfg.d_model
    def rnd(*s):
        return torch.randn(*s, generator=g, device="cuda") * 0.05
    weights = {"token_embd": rnd(cfg.vocab, d), "output": rnd(cfg.vocab, d), "output_norm": 1 + rnd(d)}
    for l in range(cfg.n_layer):
        weights[f"blk.{l}.qkv"] = rnd((cfg.n_head + 2 * cfg.n_kv_head) * D, d)
        weights[f"blk.{l}.o"] = rnd(d, cfg.n_head * D)
        weights[f"blk.{l}.gate_up"] = rnd(2 * cfg.ffn, d)
        weights[f"blk.{l}.down"] = rnd(d, cfg.ffn)
        weights[f"blk.{l}.attn_norm"] = 1 + rnd(d)
        weights[f"blk.{l}.ffn_norm"] = 1 + rnd(d)
    B, T = 3, 9
    dec = TPDecoder(cfg, rank, world, batch=B, cap=32, weights=weights, engine=os.environ.get("DECODE_ENGINE", "tc"))
    assert dec.engine == os.environ.get("DECODE_ENGINE", "tc")
    prompt = torch.randint(0, cfg.vocab, (B, T), generator=torch.Generator().manual_seed(5))
    dec.reset()
    logits = []
    for t in range(T):
        dec.tokens.copy_(prompt[:, t].cuda())
        dec.step()
        torch.cuda.synchronize()
        logits.append(dec.logits_all.view(torch.float32).view(world, B, dec.Vl).permute(1, 0, 2).reshape(B, -1).clone())
    got = torch.stack(logits, 1)  # [B, T, V]
    want = reference_logits(cfg, weights, prompt.cuda())
    cos = torch.nn.functional.cosine_similarity(got.flatten(1), want.flatten(1), dim=1).min().item()
    rel = ((got - want).norm() / want.norm()).item()
    dec.reset()
    dec.prefill_batched(prompt)          # GEMM path over the first T-1 tokens + one decode step
    torch.cuda.synchronize()
    last = dec.logits_all.view(torch.float32).view(world, B, dec.Vl).permute(1, 0, 2).reshape(B, -1)
    cos_prefill = torch.nn.functional.cosine_similarity(last, want[:, -1], dim=1).min().item()
    gen = dec.generate(prompt, 6).cpu().tolist()
    err = check_error_word()
    dec.close()
    # the same prompt with the fused sampling kernel inside the step: two decoders with one seed
    from mimir_b200.llm.generate import Sampler
    sampled = []
    for _ in range(2):
        d2 = TPDecoder(cfg, rank, world, batch=B, cap=32, weights=weights, engine=os.environ.get("DECODE_ENGINE", "tc"),
                       sampler=Sampler(temperature=1.5, top_k=50, top_p=0.95, seed=7))
        sampled.append(d2.generate(prompt, 6).cpu().tolist())
        err |= check_error_word()
        d2.close()
    if world > 1:
        dist.destroy_process_group()
    os.write(1, ("RESULT " + json.dumps({"rank": rank, "cos": cos, "rel": rel, "err": err, "gen": gen, "sampled": sampled, "vocab": cfg.vocab, "cos_prefill": cos_prefill,
                                  "launches": int(dec.launches_per_step)}) + "\n").encode())  # one write: lines of different ranks never interleave


if __name__ == "__main__":
    main()
