"""GPT-2 training engine on the sm_100a kernels.

The whole step (embedding, 12 blocks forward, fused softmax-cross-entropy,
backward, AdamW) is an explicit kernel sequence over preallocated buffers, so it
captures into one CUDA graph and replays with no host work (the reference gets
the same effect from its plan cache and CUDA-graph batches:
internal/sched/cache.go:22-104, backend/cuda/batch_linux.go:116-320).

Model definition follows the reference example (examples/gpt2/model.go: pre-LN
decoder blocks, fused QKV laid out [all Q heads | all K heads | all V heads]
(nn/transformer.go:485-522), GELU-tanh MLP, tied embedding / output matrix) with
the real GPT-2 vocabulary (50257, padded to a multiple of 128 for the GEMM).

Parameters live in flat buffers (bf16 value, bf16 gradient, fp32 master, fp32
exp_avg / exp_avg_sq -- optimizer state names as in optim/optim.go:455-671),
grouped in buckets ordered the way backward produces gradients, each bucket laid
out [weight-decayed | not decayed]; the data-parallel trainer reduces and
updates one bucket at a time while backward continues.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import kernels as K
from ..ops.gemm import gemm


@dataclass
class GPT2Config:
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    vocab: int = 50257
    ctx: int = 1024
    eps: float = 1e-5

    @property
    def padded_vocab(self) -> int:
        return (self.vocab + 127) // 128 * 128

    @staticmethod
    def small() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(n_layer=2, n_head=2, d_model=128, vocab=1000, ctx=128)


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class ParamLayout:
    """Flat-buffer layout: buckets of [decayed | not decayed] parameters."""

    def __init__(self, cfg: GPT2Config, align: int = 1024):
        C, Vp = cfg.d_model, cfg.padded_vocab
        self.buckets = []  # (name, start, decay_elems, total_elems)
        self.entries = {}  # name -> (offset, shape)
        off = 0

        def bucket(name, decay, nodecay):
            nonlocal off
            start = off
            for pname, shape in decay:
                self.entries[pname] = (off, shape)
                off += math.prod(shape)
            off = _round_up(off, 8)
            decay_n = off - start
            for pname, shape in nodecay:
                self.entries[pname] = (off, shape)
                off += math.prod(shape)
            off = _round_up(off, align)
            self.buckets.append((name, start, decay_n, off - start))

        bucket("emb", [("wte", (Vp, C)), ("wpe", (cfg.ctx, C))], [])
        for l in range(cfg.n_layer):
            p = f"h.{l}."
            bucket(f"h.{l}",
                   [(p + "qkv_w", (3 * C, C)), (p + "o_w", (C, C)), (p + "fc_w", (4 * C, C)),
                    (p + "proj_w", (C, 4 * C))],
                   [(p + "ln1_g", (C,)), (p + "ln1_b", (C,)), (p + "qkv_b", (3 * C,)),
                    (p + "o_b", (C,)), (p + "ln2_g", (C,)), (p + "ln2_b", (C,)),
                    (p + "fc_b", (4 * C,)), (p + "proj_b", (C,))])
        bucket("lnf", [], [("lnf_g", (C,)), ("lnf_b", (C,))])
        self.total = off

    def views(self, flat: torch.Tensor) -> dict:
        return {n: flat.narrow(0, o, math.prod(s)).view(s) for n, (o, s) in self.entries.items()}


class GPT2Engine:
    """Owns parameters, optimizer state and activations of one replica."""

    def __init__(self, cfg: GPT2Config, batch: int, seq: int, device="cuda", seed: int = 0,
                 flat_alloc=None, attention: str = "native"):
        self.cfg, self.B, self.T = cfg, batch, seq
        self.M = batch * seq
        self.device = torch.device(device)
        self.attention = attention
        self.layout = ParamLayout(cfg)
        n = self.layout.total
        alloc = flat_alloc or (lambda numel, dtype: torch.zeros(numel, dtype=dtype, device=self.device))
        self.params = alloc(n, torch.bfloat16)
        self.grads = alloc(n, torch.bfloat16)
        self.master = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.p = self.layout.views(self.params)
        self.g = self.layout.views(self.grads)
        self._init_weights(seed)
        self._alloc_activations()
        self.step_count = 0
        self._dp = None
        self.hyper = torch.zeros(4, dtype=torch.float32, device=self.device)
        from ..ops._util import PinnedRing
        self._hyper_ring = PinnedRing(4)

    # ------------------------------------------------------------------ init
    def _init_weights(self, seed: int) -> None:
        cfg = self.cfg
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        mv = self.layout.views(self.master)
        for name, w in mv.items():
            leaf = name.split(".")[-1]
            if leaf in ("ln1_g", "ln2_g", "lnf_g"):
                w.fill_(1.0)
            elif leaf.endswith("_b"):
                w.zero_()
            elif leaf == "wte":
                w.zero_()
                w[: cfg.vocab].normal_(0.0, 0.02, generator=gen)
            else:
                std = 0.02 / math.sqrt(2 * cfg.n_layer) if leaf in ("o_w", "proj_w") else 0.02
                w.normal_(0.0, std, generator=gen)
        self.params.copy_(self.master)

    def _alloc_activations(self) -> None:
        cfg, M, dev = self.cfg, self.M, self.device
        C, L, Vp = cfg.d_model, cfg.n_layer, cfg.padded_vocab
        bf = dict(dtype=torch.bfloat16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.tokens = torch.zeros(M, dtype=torch.int64, device=dev)
        self.targets = torch.zeros(M, dtype=torch.int64, device=dev)
        self.x = torch.empty(L + 1, M, C, **bf)       # residual stream entering each block (+ final)
        self.ln1 = torch.empty(L, M, C, **bf)
        self.qkv = torch.empty(L, M, 3 * C, **bf)
        self.att = torch.empty(L, M, C, **bf)
        self.lse = torch.empty(L, self.B * cfg.n_head * self.T, **f32)
        self.xmid = torch.empty(L, M, C, **bf)
        self.ln2 = torch.empty(L, M, C, **bf)
        self.pre = torch.empty(L, M, 4 * C, **bf)
        self.h = torch.empty(L, M, 4 * C, **bf)
        self.stats = torch.empty(2 * L + 1, 2, M, **f32)  # mean, rstd of every LayerNorm
        self.lnf = torch.empty(M, C, **bf)
        self.logits = torch.empty(M, Vp, **bf)
        self.loss_rows = torch.empty(M, **f32)
        self.loss = torch.zeros(1, **f32)
        # backward scratch
        self.dx = torch.empty(M, C, **bf)
        self.dx2 = torch.empty(M, C, **bf)
        self.dtmp = torch.empty(M, C, **bf)
        self.dqkv = torch.empty(M, 3 * C, **bf)
        self.dh = torch.empty(M, 4 * C, **bf)
        self.dsum = torch.empty(self.B * cfg.n_head * self.T, **f32)
        self.norm_scratch = K.norm_bwd_scratch(C, dev) if dev.type == "cuda" else None
        self.col_scratch = torch.empty(64 * 4 * C, **f32)

    # --------------------------------------------------------------- forward
    def forward(self) -> None:
        cfg, p = self.cfg, self.p
        L = cfg.n_layer
        K.embedding_fwd(self.tokens, p["wte"], p["wpe"], self.x[0], self.T)
        for l in range(L):
            n = f"h.{l}."
            K.layernorm_fwd(self.x[l], p[n + "ln1_g"], p[n + "ln1_b"], self.ln1[l],
                            self.stats[2 * l, 0], self.stats[2 * l, 1], cfg.eps)
            gemm(self.ln1[l], p[n + "qkv_w"], bias=p[n + "qkv_b"], out=self.qkv[l])
            self._attn_fwd(l)
            gemm(self.att[l], p[n + "o_w"], bias=p[n + "o_b"], residual=True, aux=self.x[l],
                 out=self.xmid[l])
            K.layernorm_fwd(self.xmid[l], p[n + "ln2_g"], p[n + "ln2_b"], self.ln2[l],
                            self.stats[2 * l + 1, 0], self.stats[2 * l + 1, 1], cfg.eps)
            gemm(self.ln2[l], p[n + "fc_w"], bias=p[n + "fc_b"], gelu=True, aux_out=self.pre[l],
                 out=self.h[l])
            gemm(self.h[l], p[n + "proj_w"], bias=p[n + "proj_b"], residual=True, aux=self.xmid[l],
                 out=self.x[l + 1])
        K.layernorm_fwd(self.x[L], p["lnf_g"], p["lnf_b"], self.lnf, self.stats[2 * L, 0],
                        self.stats[2 * L, 1], cfg.eps)
        gemm(self.lnf, p["wte"], out=self.logits)

    def loss_and_dlogits(self, grad_scale: float = 1.0) -> None:
        """Mean cross-entropy into ``self.loss``; logits become d(loss)/d(logits) in place."""
        K.cross_entropy(self.logits, self.targets, self.loss_rows, self.logits, self.loss,
                        self.cfg.vocab, grad_scale / self.M, 1.0 / self.M)

    # -------------------------------------------------------------- backward
    def backward(self, on_bucket_ready=None) -> None:
        cfg, p, g = self.cfg, self.p, self.g
        L, C = cfg.n_layer, cfg.d_model
        dlogits = self.logits
        # tied output matrix: its gradient starts with the head's contribution
        gemm(dlogits, self.lnf, a_mn=True, b_mn=True, out=g["wte"])
        gemm(dlogits, p["wte"], b_mn=True, out=self.dtmp)
        K.layernorm_bwd(self.dtmp, self.x[L], p["lnf_g"], self.stats[2 * L, 0], self.stats[2 * L, 1],
                        None, self.dx, g["lnf_g"], g["lnf_b"], self.norm_scratch)
        if on_bucket_ready:
            on_bucket_ready("lnf")
        dx, dx2 = self.dx, self.dx2
        for l in reversed(range(L)):
            n = f"h.{l}."
            # MLP
            gemm(dx, p[n + "proj_w"], b_mn=True, mul_dgelu=True, aux=self.pre[l], out=self.dh)
            gemm(dx, self.h[l], a_mn=True, b_mn=True, out=g[n + "proj_w"])
            K.colsum(dx, g[n + "proj_b"], self.col_scratch)
            gemm(self.dh, p[n + "fc_w"], b_mn=True, out=self.dtmp)
            gemm(self.dh, self.ln2[l], a_mn=True, b_mn=True, out=g[n + "fc_w"])
            K.colsum(self.dh, g[n + "fc_b"], self.col_scratch)
            K.layernorm_bwd(self.dtmp, self.xmid[l], p[n + "ln2_g"], self.stats[2 * l + 1, 0],
                            self.stats[2 * l + 1, 1], dx, dx2, g[n + "ln2_g"], g[n + "ln2_b"],
                            self.norm_scratch)
            dx, dx2 = dx2, dx
            # attention
            gemm(dx, p[n + "o_w"], b_mn=True, out=self.dtmp)
            gemm(dx, self.att[l], a_mn=True, b_mn=True, out=g[n + "o_w"])
            K.colsum(dx, g[n + "o_b"], self.col_scratch)
            self._attn_bwd(l, self.dtmp)
            gemm(self.dqkv, p[n + "qkv_w"], b_mn=True, out=self.dtmp)
            gemm(self.dqkv, self.ln1[l], a_mn=True, b_mn=True, out=g[n + "qkv_w"])
            K.colsum(self.dqkv, g[n + "qkv_b"], self.col_scratch)
            K.layernorm_bwd(self.dtmp, self.x[l], p[n + "ln1_g"], self.stats[2 * l, 0],
                            self.stats[2 * l, 1], dx, dx2, g[n + "ln1_g"], g[n + "ln1_b"],
                            self.norm_scratch)
            dx, dx2 = dx2, dx
            if on_bucket_ready:
                on_bucket_ready(f"h.{l}")
        K.embedding_bwd(self.tokens, dx, g["wte"], g["wpe"], self.B, self.T)
        if on_bucket_ready:
            on_bucket_ready("emb")

    # ------------------------------------------------------------- attention
    def _attn_fwd(self, l: int) -> None:
        cfg = self.cfg
        if self.attention == "native":
            from ..ops.attention import attention_fwd_packed
            attention_fwd_packed(self.qkv[l], self.att[l], self.lse[l], self.B, self.T, cfg.n_head,
                                 cfg.n_head, cfg.d_model // cfg.n_head, causal=True)
            return
        B, T, H, D = self.B, self.T, cfg.n_head, cfg.d_model // cfg.n_head
        q, k, v = self.qkv[l].view(B, T, 3, H, D).permute(2, 0, 3, 1, 4)
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        self.att[l].view(B, T, H, D).copy_(o.transpose(1, 2))

    def _attn_bwd(self, l: int, datt: torch.Tensor) -> None:
        cfg = self.cfg
        if self.attention == "native":
            from ..ops.attention import attention_bwd_packed
            attention_bwd_packed(self.qkv[l], self.att[l], datt, self.lse[l], self.dsum, self.dqkv,
                                 self.B, self.T, cfg.n_head, cfg.n_head,
                                 cfg.d_model // cfg.n_head, causal=True)
            return
        B, T, H, D = self.B, self.T, cfg.n_head, cfg.d_model // cfg.n_head
        with torch.enable_grad():
            leaf = self.qkv[l].detach().requires_grad_(True)
            q, k, v = leaf.view(B, T, 3, H, D).permute(2, 0, 3, 1, 4)
            o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            (gq,) = torch.autograd.grad(o, leaf, datt.view(B, T, H, D).transpose(1, 2))
        self.dqkv.copy_(gq)

    # ------------------------------------------------------------- optimizer
    def set_hyper(self, lr: float, beta1: float, beta2: float, grad_scale: float = 1.0) -> None:
        """Stages lr and the step's bias corrections for the device-side AdamW arguments."""
        self.step_count += 1
        t = self.step_count
        self._hyper_ring.stage((lr, 1.0 - beta1 ** t, math.sqrt(1.0 - beta2 ** t), grad_scale), self.hyper)

    def adamw(self, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1) -> None:
        """One fused launch per bucket; lr / bias corrections come from ``self.hyper``."""
        for _, start, decay_n, total in self.layout.buckets:
            sl = slice(start, start + total)
            K.adamw_flat(self.master[sl], self.params[sl], self.grads[sl], self.exp_avg[sl],
                         self.exp_avg_sq[sl], decay_n=decay_n, lr=0.0, beta1=beta1, beta2=beta2,
                         eps=eps, wd=wd, step=1, hyper=self.hyper)

    # --------------------------------------------------------------- helpers
    def named_parameters(self):
        cfg = self.cfg
        if getattr(self, "_dp", None) is not None:      # masters are sharded over the ranks: gather them
            for k, w in self._dp.state_dict().items():
                if k.startswith("model."):
                    name = k[len("model."):]
                    yield name, (w[: cfg.vocab] if name == "wte" else w)
            return
        for name, w in self.layout.views(self.master).items():
            yield name, (w[: cfg.vocab] if name == "wte" else w)

    def state_dict(self) -> dict:
        """Tensors named like the reference checkpoint: model.* and optim.<i>.<state>.  Under fused data
        parallelism the optimizer state lives sharded in the ``FusedDataParallel`` object, which
        gathers it (every rank must call)."""
        if getattr(self, "_dp", None) is not None:
            return self._dp.state_dict()
        out = {}
        mv = self.layout.views(self.master)
        m = self.layout.views(self.exp_avg)
        v = self.layout.views(self.exp_avg_sq)
        for i, name in enumerate(mv):
            out[f"model.{name}"] = mv[name]
            out[f"optim.{i}.exp_avg"] = m[name]
            out[f"optim.{i}.exp_avg_sq"] = v[name]
        return out

    def load_state_dict(self, sd: dict) -> None:
        if getattr(self, "_dp", None) is not None:
            return self._dp.load_state_dict(sd)
        mv = self.layout.views(self.master)
        m = self.layout.views(self.exp_avg)
        v = self.layout.views(self.exp_avg_sq)
        for i, name in enumerate(mv):
            mv[name].copy_(sd[f"model.{name}"])
            m[name].copy_(sd[f"optim.{i}.exp_avg"])
            v[name].copy_(sd[f"optim.{i}.exp_avg_sq"])
        self.params.copy_(self.master)


def reference_forward_loss(engine: GPT2Engine, tokens: torch.Tensor, targets: torch.Tensor,
                           dtype=torch.float32):
    """Plain PyTorch restatement of the model (fp32), for numerics tests.

    Returns (loss, {name: grad}) computed by autograd from the engine's master weights.
    """
    cfg = engine.cfg
    C, H = cfg.d_model, cfg.n_head
    B, T = tokens.shape
    w = {n: t.detach().to(dtype).clone().requires_grad_(True)
         for n, t in engine.layout.views(engine.master).items()}
    F = torch.nn.functional
    x = w["wte"][tokens] + w["wpe"][:T]
    for l in range(cfg.n_layer):
        n = f"h.{l}."
        a = F.layer_norm(x, (C,), w[n + "ln1_g"], w[n + "ln1_b"], cfg.eps)
        qkv = a @ w[n + "qkv_w"].t() + w[n + "qkv_b"]
        q, k, v = qkv.view(B, T, 3, H, C // H).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + o.transpose(1, 2).reshape(B, T, C) @ w[n + "o_w"].t() + w[n + "o_b"]
        a = F.layer_norm(x, (C,), w[n + "ln2_g"], w[n + "ln2_b"], cfg.eps)
        hdn = F.gelu(a @ w[n + "fc_w"].t() + w[n + "fc_b"], approximate="tanh")
        x = x + hdn @ w[n + "proj_w"].t() + w[n + "proj_b"]
    x = F.layer_norm(x, (C,), w["lnf_g"], w["lnf_b"], cfg.eps)
    logits = x @ w["wte"][: cfg.vocab].t()
    loss = F.cross_entropy(logits.view(-1, cfg.vocab), targets.view(-1))
    loss.backward()
    return loss.detach(), {n: t.grad for n, t in w.items()}
