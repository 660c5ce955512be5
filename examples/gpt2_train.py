"""GPT-2 training (reference: examples/gpt2/train.go): warm-up + cosine learning rate, AdamW,
gradient clipping, checkpoint, then greedy / sampled continuation.

    python examples/gpt2_train.py --steps 30                  # CPU, nn layers through the lazy tensor API
    python examples/gpt2_train.py --device gpu --steps 100    # native engine, whole step as one CUDA graph
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def schedule(step, peak, warm, total, floor=0.1):
    if step < warm:
        return peak * (step + 1) / warm
    return peak * (floor + (1 - floor) * 0.5 * (1 + math.cos(math.pi * (step - warm) / max(1, total - warm))))


def cpu_main(steps=30, seq=32, vocab=64, log=print):
    import mimir_b200.tensor as T
    from mimir_b200 import nn, optim
    from mimir_b200.data import datasets
    nn.manual_seed(0)
    dim, heads, layers = 64, 4, 2

    class GPT(nn.Module):
        def __init__(self):
            self.wte, self.wpe = nn.Embedding(vocab, dim), nn.Embedding(seq, dim)
            self.blocks = [nn.DecoderBlock(dim, heads) for _ in range(layers)]
            self.norm = nn.LayerNorm(dim)

        def forward(self, tok):
            x = self.wte(tok) + self.wpe(T.arange(tok.shape[1], dtype=torch.int64))
            for b in self.blocks:
                x = b(x)
            return T.matmul_t(self.norm(x), self.wte.weight.value())     # tied output matrix
    model = GPT()
    opt = optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, clip_norm=1.0)
    ds = datasets.synthetic_tokens(rows=64, seq=seq, vocab=vocab, batch_size=8)
    losses, step = [], 0
    while step < steps:
        for batch in ds:
            opt.lr = schedule(step, 3e-3, 5, steps)
            logits = model(batch.x)
            loss = nn.loss.cross_entropy(T.reshape(logits, (-1, vocab)), T.reshape(batch.y, (-1,)))
            loss.backward()
            losses.append(float(loss.item()))
            opt.step()
            opt.zero_grad()
            step += 1
            if step % 10 == 0:
                log(f"step {step} loss {losses[-1]:.3f} lr {opt.lr:.2e}")
            if step >= steps:
                break
    return losses


def gpu_main(steps=100, log=print):
    from mimir_b200.models.gpt2 import GPT2Config, GPT2Engine
    from mimir_b200.train import FusedTrainer
    cfg = GPT2Config(n_layer=4, n_head=4, d_model=256, vocab=512, ctx=256)
    eng = GPT2Engine(cfg, batch=8, seq=256)
    tr = FusedTrainer(eng, lr=1e-3, schedule=lambda s: schedule(s, 1e-3, 10, steps))
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 512, (8, 257), generator=g)
    tok, tgt = base[:, :-1].contiguous().pin_memory(), base[:, 1:].contiguous().pin_memory()
    losses = []
    for s in range(steps):
        losses.append(tr.step(tok, tgt))
        if (s + 1) % 20 == 0:
            log(f"step {s + 1} loss {losses[-1]:.3f}")
    return losses


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=["cpu", "gpu"])
    ap.add_argument("--steps", type=int, default=30)
    a = ap.parse_args()
    out = gpu_main(a.steps) if a.device == "gpu" else cpu_main(a.steps)
    print(f"first loss {out[0]:.3f}, last loss {out[-1]:.3f}")
