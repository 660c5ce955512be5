"""Library baselines: the same five workloads as the native benchmarks, written in plain PyTorch.

Nothing here imports this repository's kernels, engines or native library: products go to cuBLAS
(``torch.nn.functional.linear`` in bf16), attention to ``scaled_dot_product_attention`` (flash),
normalisation / activation / loss to PyTorch's own kernels, the optimizer to the fused
``torch.optim.AdamW`` over fp32 master weights, and every collective to NCCL (DDP, FSDP, or
explicit all-reduces for tensor parallelism).  This is the "cuBLAS + NCCL only" execution mode the
reference's own CUDA backend corresponds to (cublasSgemm + ncclAllReduce), at bf16 instead of fp32,
i.e. a stronger baseline than the reference itself.  The benchmark drivers time it with the same
steps, warm-up, barriers and CUDA events as the native arm.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

F = torch.nn.functional


# ------------------------------------------------------------------------------- GPT-2
class _Block(torch.nn.Module):
    def __init__(self, C, H):
        super().__init__()
        self.H = H
        self.ln1, self.ln2 = torch.nn.LayerNorm(C), torch.nn.LayerNorm(C)
        self.qkv, self.o = torch.nn.Linear(C, 3 * C), torch.nn.Linear(C, C)
        self.fc, self.proj = torch.nn.Linear(C, 4 * C), torch.nn.Linear(4 * C, C)

    def forward(self, x):
        B, T, C = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.H, C // self.H).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)
        x = x + self.o(a)
        return x + self.proj(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT2(torch.nn.Module):
    """GPT-2 with a tied embedding / output matrix, vocabulary padded to a multiple of 128."""

    def __init__(self, n_layer=12, n_head=12, d_model=768, vocab=50257, ctx=1024):
        super().__init__()
        self.vocab = vocab
        vp = (vocab + 127) // 128 * 128
        self.wte, self.wpe = torch.nn.Embedding(vp, d_model), torch.nn.Embedding(ctx, d_model)
        self.h = torch.nn.ModuleList(_Block(d_model, n_head) for _ in range(n_layer))
        self.lnf = torch.nn.LayerNorm(d_model)
        for n, p in self.named_parameters():
            if p.dim() == 2:
                torch.nn.init.normal_(p, 0.0, 0.02 / math.sqrt(2 * n_layer) if n.endswith(("o.weight", "proj.weight")) else 0.02)

    def forward(self, tok, tgt):
        B, T = tok.shape
        x = self.wte(tok) + self.wpe.weight[:T]
        for b in self.h:
            x = b(x)
        logits = F.linear(self.lnf(x), self.wte.weight)      # padded vocabulary columns take part, like the native arm
        return F.cross_entropy(logits.view(B * T, -1).float(), tgt.reshape(-1))


class MasterAdamW:
    """bf16 parameters, fp32 master copies stepped by the fused ``torch.optim.AdamW``."""

    def __init__(self, params, lr, betas, weight_decay):
        self.params = [p for p in params if p.requires_grad]
        self.master = [p.detach().float().clone().requires_grad_(True) for p in self.params]
        self.opt = torch.optim.AdamW(self.master, lr=lr, betas=betas, weight_decay=weight_decay, fused=True,
                                     capturable=True)

    def step(self, grad_scale: float = 1.0):
        grads = [p.grad for p in self.params]
        for m, g in zip(self.master, grads):
            m.grad = g.float() if grad_scale == 1.0 else g.float() * grad_scale
        self.opt.step()
        with torch.no_grad():
            torch._foreach_copy_(self.params, self.master)
        for p in self.params:
            p.grad = None


class TorchTrainer:
    """One training step of a model whose ``forward(tok, tgt)`` returns the loss; captured into a CUDA
    graph on one GPU (as the native arm is), eager under DDP / FSDP."""

    def __init__(self, model, lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1, graph=True, ddp=False, local_rank=0):
        self.model = model
        self.net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True) \
            if ddp else model
        self.opt = MasterAdamW(model.parameters(), lr, betas, weight_decay)
        self.graph, self.use_graph = None, graph and not ddp
        self.tok = self.tgt = None
        self.loss = torch.zeros((), device="cuda")

    def _device_step(self):
        loss = self.net(self.tok, self.tgt)
        loss.backward()
        self.opt.step()
        self.loss.copy_(loss.detach())

    def run_device_step(self):
        if not self.use_graph:
            return self._device_step()
        if self.graph is None:
            # whole-step capture as PyTorch documents it: warm up on a side stream, then capture
            import sys
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(3):
                    self._device_step()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(g):
                    self._device_step()
                self.graph = g
            except Exception as exc:  # noqa: BLE001 - a baseline that cannot be captured runs eagerly
                sys.stderr.write(f"[baseline] CUDA graph capture failed, running eagerly: {exc}\n")
                self.use_graph = False
                torch.cuda.synchronize()
                return self._device_step()
        self.graph.replay()

    def set_batch(self, tok, tgt):
        if self.tok is None:
            self.tok = torch.empty(tok.shape, dtype=torch.int64, device="cuda")
            self.tgt = torch.empty(tgt.shape, dtype=torch.int64, device="cuda")
        self.tok.copy_(tok, non_blocking=True)
        self.tgt.copy_(tgt, non_blocking=True)

    def step(self, tok, tgt) -> float:
        """Host batch in (pinned memory), loss out: the end-to-end call."""
        self.set_batch(tok, tgt)
        self.run_device_step()
        return float(self.loss.item())


# ------------------------------------------------------------------------------- Llama
class _RMSNorm(torch.nn.Module):
    def __init__(self, C, eps=1e-5):
        super().__init__()
        self.weight, self.eps = torch.nn.Parameter(torch.ones(C)), eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def _rope(x, cos, sin):
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)


class _LlamaBlock(torch.nn.Module):
    """One decoder block; with ``tp`` > 1 the heads and the hidden units are split over a process group
    (column-parallel qkv / gate / up, row-parallel o / down + all-reduce: Megatron)."""

    def __init__(self, C, H, ffn, tp=1, group=None):
        super().__init__()
        self.H, self.D, self.tp, self.group = H // tp, C // H, tp, group
        self.n1, self.n2 = _RMSNorm(C), _RMSNorm(C)
        self.qkv = torch.nn.Linear(C, 3 * C // tp, bias=False)
        self.o = torch.nn.Linear(C // tp, C, bias=False)
        self.gu = torch.nn.Linear(C, 2 * ffn // tp, bias=False)
        self.down = torch.nn.Linear(ffn // tp, C, bias=False)

    def _reduce(self, x):
        if self.tp > 1:
            x = _AllReduce.apply(x, self.group)
        return x

    def forward(self, x, cos, sin):
        B, T, C = x.shape
        h = _copy_to_tp(self.n1(x), self.group) if self.tp > 1 else self.n1(x)
        q, k, v = self.qkv(h).view(B, T, 3, self.H, self.D).permute(2, 0, 3, 1, 4)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, -1)
        x = x + self._reduce(self.o(a))
        h = _copy_to_tp(self.n2(x), self.group) if self.tp > 1 else self.n2(x)
        g, u = self.gu(h).chunk(2, -1)
        return x + self._reduce(self.down(F.silu(g) * u))


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def _copy_to_tp(x, group):
    return _CopyToTP.apply(x, group)


class Llama(torch.nn.Module):
    def __init__(self, n_layer, d_model, n_head, ffn, vocab, seq, tp=1, group=None):
        super().__init__()
        self.emb = torch.nn.Embedding(vocab, d_model)
        self.blocks = torch.nn.ModuleList(_LlamaBlock(d_model, n_head, ffn, tp, group) for _ in range(n_layer))
        self.norm = _RMSNorm(d_model)
        self.head = torch.nn.Linear(d_model, vocab, bias=False)
        D = d_model // n_head
        ang = torch.arange(seq)[:, None].float() * (1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D)))[None]
        self.register_buffer("cos", ang.cos().to(torch.bfloat16), persistent=False)
        self.register_buffer("sin", ang.sin().to(torch.bfloat16), persistent=False)
        for p in self.parameters():
            if p.dim() == 2:
                torch.nn.init.normal_(p, 0.0, 0.02)

    def forward(self, tok, tgt):
        B, T = tok.shape
        x = self.emb(tok)
        for b in self.blocks:
            x = b(x, self.cos[:T], self.sin[:T])
        logits = self.head(self.norm(x))
        return F.cross_entropy(logits.view(B * T, -1).float(), tgt.reshape(-1))


LLAMA_SHAPES = {
    "tiny": dict(n_layer=2, d_model=256, n_head=4, ffn=512, vocab=1024),
    "1b3": dict(n_layer=24, d_model=2048, n_head=16, ffn=5504, vocab=32000),
    "7b": dict(n_layer=32, d_model=4096, n_head=32, ffn=11008, vocab=32000),
}


# ------------------------------------------------------------------------------- quantised decode
def q4_0_roundtrip(w: torch.Tensor) -> torch.Tensor:
    """Weights rounded to Q4_0 (32-value blocks, fp16 scale) and expanded again to bf16: what a
    library path that cannot multiply in 4 bits keeps in memory."""
    shape = w.shape
    b = w.float().reshape(-1, 32)
    amax = b.abs().amax(1, keepdim=True)
    idx = b.abs().argmax(1, keepdim=True)
    d = (b.gather(1, idx) / -8.0).half().float()
    q = torch.where(d == 0, torch.zeros_like(b), b / torch.where(d == 0, torch.ones_like(d), d))
    q = (q + 8.5).floor().clamp(0, 15) - 8
    del amax
    return (q * d).reshape(shape).to(torch.bfloat16)


class DecodeLlama:
    """Tensor-parallel Llama decode on dequantised bf16 weights: cuBLAS products, SDPA over an fp16 KV
    cache, NCCL all-reduce after the two row-parallel products of every layer."""

    def __init__(self, n_layer, d_model, n_head, n_kv, ffn, vocab, max_len, batch, rank=0, world=1, seed=0):
        self.L, self.C, self.H, self.Hk, self.D = n_layer, d_model, n_head // world, max(n_kv // world, 1), d_model // n_head
        self.world, self.batch, self.max_len = world, batch, max_len
        g = torch.Generator(device="cuda").manual_seed(seed)
        mk = lambda o, i: q4_0_roundtrip(torch.randn(o, i, generator=g, device="cuda") * 0.02)  # noqa: E731
        self.emb = (torch.randn(vocab, d_model, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.layers = []
        for _ in range(n_layer):
            self.layers.append(dict(
                n1=torch.ones(d_model, device="cuda", dtype=torch.bfloat16), n2=torch.ones(d_model, device="cuda", dtype=torch.bfloat16),
                qkv=mk((self.H + 2 * self.Hk) * self.D, d_model), o=mk(d_model, self.H * self.D),
                gu=mk(2 * ffn // world, d_model), down=mk(d_model, ffn // world)))
        self.norm = torch.ones(d_model, device="cuda", dtype=torch.bfloat16)
        self.head = mk(vocab // world, d_model)
        self.kc = torch.zeros(n_layer, batch, self.Hk, max_len, self.D, device="cuda", dtype=torch.float16)
        self.vc = torch.zeros_like(self.kc)
        inv = 1.0 / (500000.0 ** (torch.arange(0, self.D, 2, device="cuda").float() / self.D))
        ang = torch.arange(max_len, device="cuda")[:, None].float() * inv[None]
        self.cos, self.sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        self.pos = 0

    def _sum(self, x):
        if self.world > 1:
            dist.all_reduce(x)
        return x

    @torch.no_grad()
    def forward(self, tok):
        """tok [B, T] -> logits of the last position [B, vocab / world] (this rank's columns)."""
        B, T = tok.shape
        p0, p1 = self.pos, self.pos + T
        x = self.emb[tok]
        cos, sin = self.cos[p0:p1], self.sin[p0:p1]
        for l, w in enumerate(self.layers):
            h = F.rms_norm(x, (self.C,), w["n1"], 1e-5)
            qkv = F.linear(h, w["qkv"]).view(B, T, self.H + 2 * self.Hk, self.D).transpose(1, 2)
            q, k, v = qkv[:, : self.H], qkv[:, self.H: self.H + self.Hk], qkv[:, self.H + self.Hk:]
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
            self.kc[l, :, :, p0:p1] = k.to(torch.float16)
            self.vc[l, :, :, p0:p1] = v.to(torch.float16)
            kk, vv = self.kc[l, :, :, :p1].to(torch.bfloat16), self.vc[l, :, :, :p1].to(torch.bfloat16)
            a = F.scaled_dot_product_attention(q, kk, vv, is_causal=T > 1, enable_gqa=self.H != self.Hk)
            x = x + self._sum(F.linear(a.transpose(1, 2).reshape(B, T, -1), w["o"]))
            h = F.rms_norm(x, (self.C,), w["n2"], 1e-5)
            g, u = F.linear(h, w["gu"]).chunk(2, -1)
            x = x + self._sum(F.linear(F.silu(g) * u, w["down"]))
        self.pos = p1
        return F.linear(F.rms_norm(x[:, -1], (self.C,), self.norm, 1e-5), self.head)

    @torch.no_grad()
    def step_static(self, tok, pos):
        """One decode step with static shapes (``tok`` [B, 1] and ``pos`` a 0-d device tensor), so
        that the whole step, NCCL all-reduces included, can be captured in a CUDA graph: the new key
        and value are written with ``index_copy_`` and attention runs over the whole cache under a
        mask of the positions filled so far."""
        B = tok.shape[0]
        x = self.emb[tok]
        cos, sin = self.cos.index_select(0, pos.view(1)), self.sin.index_select(0, pos.view(1))
        mask = (torch.arange(self.max_len, device=tok.device) <= pos).view(1, 1, 1, -1)
        for l, w in enumerate(self.layers):
            h = F.rms_norm(x, (self.C,), w["n1"], 1e-5)
            qkv = F.linear(h, w["qkv"]).view(B, 1, self.H + 2 * self.Hk, self.D).transpose(1, 2)
            q, k, v = qkv[:, : self.H], qkv[:, self.H: self.H + self.Hk], qkv[:, self.H + self.Hk:]
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
            self.kc[l].index_copy_(2, pos.view(1), k.to(torch.float16))
            self.vc[l].index_copy_(2, pos.view(1), v.to(torch.float16))
            a = F.scaled_dot_product_attention(q, self.kc[l].to(torch.bfloat16), self.vc[l].to(torch.bfloat16),
                                               attn_mask=mask, enable_gqa=self.H != self.Hk)
            x = x + self._sum(F.linear(a.transpose(1, 2).reshape(B, 1, -1), w["o"]))
            h = F.rms_norm(x, (self.C,), w["n2"], 1e-5)
            g, u = F.linear(h, w["gu"]).chunk(2, -1)
            x = x + self._sum(F.linear(F.silu(g) * u, w["down"]))
        return F.linear(F.rms_norm(x[:, -1], (self.C,), self.norm, 1e-5), self.head)

    def next_token(self, logits):
        """Greedy over the vocabulary split across ranks."""
        val, idx = logits.float().max(-1)
        if self.world > 1:
            vals = [torch.empty_like(val) for _ in range(self.world)]
            idxs = [torch.empty_like(idx) for _ in range(self.world)]
            dist.all_gather(vals, val)
            dist.all_gather(idxs, idx)
            best = torch.stack(vals).argmax(0)
            idx = torch.stack(idxs).gather(0, best[None])[0] + best * logits.shape[-1]
        return idx[:, None]


# ------------------------------------------------------------------------------- MNIST CNN
class MnistCNN(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.c1, self.c2 = torch.nn.Conv2d(1, 32, 3, padding=1), torch.nn.Conv2d(32, 64, 3, padding=1)
        self.f1, self.f2 = torch.nn.Linear(3136, 128), torch.nn.Linear(128, 10)

    def forward(self, x, y):
        x = F.max_pool2d(F.relu(self.c1(x)), 2)
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        return F.cross_entropy(self.f2(F.relu(self.f1(x.flatten(1)))), y)
