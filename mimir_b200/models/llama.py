"""Llama-style training engine on the sm_100a kernels: RMSNorm, rotary positions, grouped-query
causal attention, SwiGLU MLP, untied output matrix, AdamW on fp32 master weights.

Like the GPT-2 engine, a step is an explicit kernel sequence over preallocated buffers (it
captures into one CUDA graph).  Two placements of the parameters:

``mode="single"``   every parameter lives on this GPU.

``mode="fsdp"``     fully sharded data parallel over the ranks of a process group (reference:
    nn.FullyShard + the matmul layout rule, nn/shard.go:74-89, tensor/layout.go:621-714,
    tensor/reshard.go:175-184): every 2-D weight is split by rows; each rank keeps master
    weights, AdamW state and gradients for its rows only.  The forward product gathers the
    remote rows inside the GEMM kernel (all-gather -> GEMM over peer memory); the gathered
    copy stays in the rank's full-size buffer and serves the input-gradient product of the
    backward pass; the weight-gradient product reduce-scatters its tiles to the owning ranks
    from the GEMM epilogue (GEMM -> reduce-scatter), so each rank ends up with the summed
    gradient of its rows.  Norm gains are replicated and their gradients all-reduced once per
    step.  Every rank works on its own micro-batch (data parallel).

``mode="tp"``       Megatron tensor parallelism over the ranks of ``group`` (reference:
    nn.TensorParallel, nn/shard.go:102-158): QKV and gate|up are split by output rows (heads and
    hidden features), the attention output and down projections by input columns; attention runs
    on the local heads.  A row-parallel product is the fused GEMM -> reduce-scatter kernel (each
    rank receives its rows of the sum while the rest is still being computed), the residual is
    added on those rows, and a peer all-gather rebuilds the full activation: together one
    all-reduce per row-parallel layer, forward and backward.  ``dp_group`` adds data parallelism
    across tensor-parallel groups (gradients all-reduced once per step).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import kernels as K
from ..ops.attention import attention_bwd_packed, attention_fwd_packed
from ..ops.gemm import gemm


@dataclass
class LlamaTrainConfig:
    n_layer: int = 24
    d_model: int = 2048
    n_head: int = 16
    n_kv_head: int = 16
    ffn: int = 5504
    vocab: int = 32000
    ctx: int = 2048
    rope_base: float = 10000.0
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    @property
    def padded_vocab(self) -> int:
        return (self.vocab + 127) // 128 * 128

    @staticmethod
    def llama_1b3() -> "LlamaTrainConfig":
        return LlamaTrainConfig()

    @staticmethod
    def llama_7b() -> "LlamaTrainConfig":
        return LlamaTrainConfig(n_layer=32, d_model=4096, n_head=32, n_kv_head=32, ffn=11008, vocab=32000, ctx=4096)

    @staticmethod
    def tiny() -> "LlamaTrainConfig":
        return LlamaTrainConfig(n_layer=2, d_model=256, n_head=4, n_kv_head=2, ffn=512, vocab=1000, ctx=128)

    def param_count(self) -> int:
        C, D = self.d_model, self.head_dim
        per = (self.n_head + 2 * self.n_kv_head) * D * C + C * self.n_head * D + 3 * self.ffn * C + 2 * C
        return self.n_layer * per + 2 * self.vocab * C + C


class LlamaEngine:
    def __init__(self, cfg: LlamaTrainConfig, batch: int, seq: int, device="cuda", seed: int = 0, mode: str = "single",
                 rank: int = 0, world: int = 1, group=None, dp_group=None, dp_world: int = 1):
        if mode not in ("single", "fsdp", "tp"):
            raise ValueError(f"unknown mode {mode!r}")
        if mode == "single":
            rank, world = 0, 1
        self.cfg, self.B, self.T, self.M = cfg, batch, seq, batch * seq
        self.mode, self.rank, self.world, self.group = mode, rank, world, group
        self.dp_group, self.dp_world = dp_group, dp_world
        self.device = torch.device(device)
        C, D = cfg.d_model, cfg.head_dim
        tp = world if mode == "tp" else 1
        if cfg.n_head % tp or cfg.n_kv_head % tp or cfg.ffn % (tp * 8):
            raise ValueError("heads, KV heads and ffn / 8 must divide by the tensor-parallel size")
        # local (per tensor-parallel rank) head and feature counts
        self.Hq, self.Hk, self.F = cfg.n_head // tp, cfg.n_kv_head // tp, cfg.ffn // tp
        self.qkv_n = (self.Hq + 2 * self.Hk) * D
        # 2-D weights [rows, cols] as this rank multiplies with them, in the order backward finishes their gradients
        self.shapes = {"lm_head": (cfg.padded_vocab, C)}
        for l in reversed(range(cfg.n_layer)):
            self.shapes[f"h.{l}.wd"] = (C, self.F)
            self.shapes[f"h.{l}.wgu"] = (2 * self.F, C)
            self.shapes[f"h.{l}.wo"] = (C, self.Hq * D)
            self.shapes[f"h.{l}.wqkv"] = (self.qkv_n, C)
        self.shapes["wte"] = (cfg.padded_vocab, C)
        self.shard_rows = world if mode == "fsdp" else 1     # fsdp keeps 1 / world of the rows of every matrix
        for name, (r, _) in self.shapes.items():
            if r % self.shard_rows:
                raise ValueError(f"{name}: {r} rows do not divide over {world} ranks")
        self.gain_names = [f"h.{l}.{n}" for l in range(cfg.n_layer) for n in ("attn_norm", "ffn_norm")] + ["out_norm"]
        self._alloc_params(seed)
        self._alloc_activations()
        self.step_count = 0
        self.hyper = torch.zeros(4, dtype=torch.float32, device=self.device)
        from ..ops._util import PinnedRing
        self._hyper_ring = PinnedRing(4)

    # ------------------------------------------------------------------ parameters
    def _alloc_params(self, seed: int) -> None:
        cfg, dev, W = self.cfg, self.device, self.shard_rows
        bf, f32 = dict(dtype=torch.bfloat16, device=dev), dict(dtype=torch.float32, device=dev)
        align = 1024
        # local (owned) elements: this rank's rows of every matrix, then the gains (replicated)
        self.own = {}      # name -> (offset, (rows_own, cols))
        off = 0
        for name, (r, c) in self.shapes.items():
            self.own[name] = (off, (r // W, c))
            off = (off + (r // W) * c + align - 1) // align * align
        self.decay_n = off
        for name in self.gain_names:
            self.own[name] = (off, (cfg.d_model,))
            off += cfg.d_model
        self.n_own = (off + align - 1) // align * align
        self.master = torch.zeros(self.n_own, **f32)
        self.exp_avg = torch.zeros(self.n_own, **f32)
        self.exp_avg_sq = torch.zeros(self.n_own, **f32)
        self.grads = torch.zeros(self.n_own, **bf)
        view = lambda flat, n: flat.narrow(0, self.own[n][0], math.prod(self.own[n][1])).view(self.own[n][1])  # noqa: E731
        self.g = {n: view(self.grads, n) for n in self.own}
        self.mv = {n: view(self.master, n) for n in self.own}
        if self.mode == "fsdp":
            from ..parallel.fused_gemm import ReduceScatterGemm, ShardedWeight
            from ..parallel.peer import SymmetricBuffer
            # one symmetric arena holds the full-size copy of every matrix; rank r's rows are
            # authoritative in rank r's arena, the rest is filled by the gathers
            full_off, total = {}, 0
            for name, (r, c) in self.shapes.items():
                full_off[name] = total
                total = (total + r * c * 2 + 4095) // 4096 * 4096
            self.arena = SymmetricBuffer(total, self.rank, W, self.group)
            self.sw = {name: ShardedWeight(r, c, self.rank, W, arena=self.arena, offset=full_off[name])
                       for name, (r, c) in self.shapes.items()}
            self.p = {n: s.shard for n, s in self.sw.items()}          # owned rows (bf16), live in the arena
            self.full = {n: s.full for n, s in self.sw.items()}
            self.gains = torch.zeros(len(self.gain_names) * cfg.d_model, **bf)
            uniq = sorted({(r, c) for n, (r, c) in self.shapes.items()})
            self.rs = {shape: ReduceScatterGemm(shape[0], shape[1], self.rank, W, self.group, slot=i)
                       for i, shape in enumerate(uniq)}
            self.ag_sig = SymmetricBuffer(1024 * 4, self.rank, W, self.group)
            self.ag_state = torch.zeros(4, dtype=torch.int32, device=dev)
        else:
            self.params = torch.zeros(self.n_own, **bf)
            self.p = {n: view(self.params, n) for n in self.shapes}
            self.full = self.p
            self.gains = self.params.narrow(0, self.decay_n, len(self.gain_names) * cfg.d_model)
        for i, n in enumerate(self.gain_names):
            self.p[n] = self.gains.narrow(0, i * cfg.d_model, cfg.d_model)
        # every rank draws the full matrices from the same seed and keeps its rows
        gen = torch.Generator(device=dev).manual_seed(seed)
        for name, (r, c) in self.shapes.items():
            leaf = name.split(".")[-1]
            std = 0.02 / math.sqrt(2 * cfg.n_layer) if leaf in ("wo", "wd") else 0.02
            if self.mode == "tp":
                full = self._tp_slice(leaf, gen, std)
            else:
                full = torch.randn(r, c, generator=gen, device=dev) * std
            if leaf in ("wte", "lm_head"):
                full[cfg.vocab:] = 0
            rows = r // W
            own_rank = self.rank if self.mode == "fsdp" else 0
            self.mv[name].copy_(full[own_rank * rows: (own_rank + 1) * rows])
            del full
        for n in self.gain_names:
            self.mv[n].fill_(1.0)
        self._publish_params()

    def _tp_slice(self, leaf: str, gen, std: float) -> torch.Tensor:
        """Draws the full matrix (so that every tensor-parallel size sees the same model) and cuts this rank's part."""
        cfg, dev, r, tp = self.cfg, self.device, self.rank, self.world
        C, D = cfg.d_model, cfg.head_dim
        if leaf == "wqkv":
            full = torch.randn((cfg.n_head + 2 * cfg.n_kv_head) * D, C, generator=gen, device=dev) * std
            q, k, v = full.split([cfg.n_head * D, cfg.n_kv_head * D, cfg.n_kv_head * D], 0)
            cut = lambda t, n: t[r * n * D: (r + 1) * n * D]  # noqa: E731
            return torch.cat([cut(q, self.Hq), cut(k, self.Hk), cut(v, self.Hk)], 0)
        if leaf == "wo":
            return (torch.randn(C, cfg.n_head * D, generator=gen, device=dev) * std)[:, r * self.Hq * D: (r + 1) * self.Hq * D].contiguous()
        if leaf == "wgu":
            full = torch.randn(2 * cfg.ffn, C, generator=gen, device=dev) * std
            return torch.cat([full[r * self.F: (r + 1) * self.F], full[cfg.ffn + r * self.F: cfg.ffn + (r + 1) * self.F]], 0)
        if leaf == "wd":
            return (torch.randn(C, cfg.ffn, generator=gen, device=dev) * std)[:, r * self.F: (r + 1) * self.F].contiguous()
        return torch.randn(cfg.padded_vocab, C, generator=gen, device=dev) * std

    def _publish_params(self) -> None:
        """bf16 working copies from the fp32 masters (the optimizer kernel keeps them in step afterwards)."""
        for n in self.own:
            self.p[n].copy_(self.mv[n])

    def _alloc_activations(self) -> None:
        cfg, M, dev, L = self.cfg, self.M, self.device, self.cfg.n_layer
        C, F, D = cfg.d_model, self.F, cfg.head_dim
        bf, f32 = dict(dtype=torch.bfloat16, device=dev), dict(dtype=torch.float32, device=dev)
        self.tokens = torch.zeros(M, dtype=torch.int64, device=dev)
        self.targets = torch.zeros(M, dtype=torch.int64, device=dev)
        self.pos = torch.arange(self.T, dtype=torch.int32, device=dev).repeat(self.B)
        inv = 1.0 / (cfg.rope_base ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        self.freqs = inv.float().to(dev)
        if self.mode == "tp":
            # activations that an all-gather writes into on every rank live in symmetric memory
            from ..parallel.fused_gemm import ReduceScatterGemm
            from ..parallel.peer import SymmetricBuffer
            n = M * C
            self.act_arena = SymmetricBuffer((2 * L + 2) * n * 2, self.rank, self.world, self.group)
            flat = self.act_arena.view(torch.bfloat16, 0, (2 * L + 2) * n)
            self.x = flat[: (L + 1) * n].view(L + 1, M, C)
            self.xmid = flat[(L + 1) * n: (2 * L + 1) * n].view(L, M, C)
            self.dtmp = flat[(2 * L + 1) * n:].view(M, C)
            self.rs_act = ReduceScatterGemm(M, C, self.rank, self.world, self.group)
            self.shard = torch.empty(M // self.world, C, **bf)
            self.head_dx = torch.empty(M // self.world, C, **bf)
            self.ag_sig = SymmetricBuffer(1024 * 4, self.rank, self.world, self.group)
            self.ag_state = torch.zeros(4, dtype=torch.int32, device=dev)
        else:
            self.x = torch.empty(L + 1, M, C, **bf)
            self.xmid = torch.empty(L, M, C, **bf)
            self.dtmp = torch.empty(M, C, **bf)
        self.h1 = torch.empty(L, M, C, **bf)
        self.qkv = torch.empty(L, M, self.qkv_n, **bf)
        self.att = torch.empty(L, M, self.Hq * D, **bf)
        self.lse = torch.empty(L, self.B * self.Hq * self.T, **f32)
        self.h2 = torch.empty(L, M, C, **bf)
        self.gu = torch.empty(L, M, 2 * F, **bf)
        self.act = torch.empty(L, M, F, **bf)
        self.rstd = torch.empty(2 * L + 1, M, **f32)
        self.hf = torch.empty(M, C, **bf)
        # tensor parallel: each rank computes the logits and the loss of its M / tp rows only
        self.head_rows = M // self.world if self.mode == "tp" else M
        self.logits = torch.empty(self.head_rows, cfg.padded_vocab, **bf)
        self.loss_rows = torch.empty(self.head_rows, **f32)
        self.loss = torch.zeros(1, **f32)
        self.dx = torch.empty(M, C, **bf)
        self.dx2 = torch.empty(M, C, **bf)
        self.datt = torch.empty(M, self.Hq * D, **bf)
        self.dqkv = torch.empty(M, self.qkv_n, **bf)
        self.dgu = torch.empty(M, 2 * F, **bf)
        self.dact = torch.empty(M, F, **bf)
        self.dsum = torch.empty(self.B * self.Hq * self.T, **f32)
        self.norm_scratch = K.norm_bwd_scratch(C, dev)
        if self.mode == "fsdp":
            self.dwte_full = torch.zeros(cfg.padded_vocab, C, **bf)

    # --------------------------------------------------------------------- linears
    def _fwd(self, x, name, out, **epi):
        if self.mode == "fsdp":
            from ..parallel.fused_gemm import gemm_allgather
            return gemm_allgather(x, self.sw[name], out=out, **epi)
        return gemm(x, self.p[name], out=out, **epi)

    def _dgrad(self, dy, name, out):
        # fsdp: the forward pass of this step left every rank's rows in the local full-size copy
        return gemm(dy, self.full[name], b_mn=True, out=out)

    # tensor parallel: products whose contraction is split over the ranks
    def _allgather_rows(self, shard, out) -> None:
        """Pushes ``shard`` [M / tp, C] into rows ``rank * M / tp`` of ``out`` on every rank (``out`` lives in
        the symmetric activation arena) and waits, bounded, until every rank's rows have arrived."""
        from .. import _native
        from ..ops._util import ptr, stream_ptr
        from ..ops.quant_cuda import _L
        off = out.data_ptr() - self.act_arena.local_ptr
        rc = _L().mimir_peer_allgather(ptr(shard), self.act_arena.ptr_array(off), self.ag_sig.ptr_array(),
                                       self.ag_state.data_ptr(), self.ag_state[1:].data_ptr(), shard.numel() * 2,
                                       self.rank, self.world, 0, stream_ptr())
        _native.check(rc, "allgather_rows")

    def _row_parallel_fwd(self, a, name, resid, out) -> None:
        """out = resid + sum over ranks of a_local @ w_local^T."""
        if self.mode != "tp":
            self._fwd(a, name, out, residual=True, aux=resid)
            return
        rows = self.M // self.world
        self.rs_act(a, self.p[name], out=self.shard)
        K.axpby(self.shard, resid[self.rank * rows: (self.rank + 1) * rows], self.shard)
        self._allgather_rows(self.shard, out)

    def _col_parallel_dgrad(self, dy, name, out) -> None:
        """out = sum over ranks of dy_local @ w_local (input gradient of a column-parallel layer)."""
        if self.mode != "tp":
            self._dgrad(dy, name, out)
            return
        self.rs_act(dy, self.p[name], b_mn=True, out=self.shard)
        self._allgather_rows(self.shard, out)

    def _wgrad(self, dy, x, name):
        if self.mode == "fsdp":
            self.rs[self.shapes[name]](dy, x, transposed=True, out=self.g[name])
        else:
            gemm(dy, x, a_mn=True, b_mn=True, out=self.g[name])

    # --------------------------------------------------------------------- forward
    def forward(self) -> None:
        cfg, p, L = self.cfg, self.p, self.cfg.n_layer
        Hq, Hk, D = self.Hq, self.Hk, cfg.head_dim
        if self.mode == "fsdp":
            self._gather_rows("wte")     # also the step's barrier: every rank's optimizer has finished
        K.embedding_fwd(self.tokens, self.full["wte"], None, self.x[0], self.T)
        for l in range(L):
            n = f"h.{l}."
            K.rmsnorm_fwd(self.x[l], p[n + "attn_norm"], self.h1[l], self.rstd[2 * l], cfg.eps)
            self._fwd(self.h1[l], n + "wqkv", self.qkv[l])
            K.rope_(self.qkv[l], self.pos, self.freqs, 0, Hq + Hk, D, interleaved=True)
            attention_fwd_packed(self.qkv[l], self.att[l], self.lse[l], self.B, self.T, Hq, Hk, D, causal=True)
            self._row_parallel_fwd(self.att[l], n + "wo", self.x[l], self.xmid[l])
            K.rmsnorm_fwd(self.xmid[l], p[n + "ffn_norm"], self.h2[l], self.rstd[2 * l + 1], cfg.eps)
            self._fwd(self.h2[l], n + "wgu", self.gu[l])
            K.swiglu_fwd(self.gu[l], self.act[l])
            self._row_parallel_fwd(self.act[l], n + "wd", self.xmid[l], self.x[l + 1])
        K.rmsnorm_fwd(self.x[L], p["out_norm"], self.hf, self.rstd[2 * L], cfg.eps)
        self._fwd(self._head_slice(self.hf), "lm_head", self.logits)

    def _head_slice(self, t):
        """Rows of a [M, ...] tensor this rank's output head works on (all of them unless tensor parallel)."""
        if self.mode != "tp":
            return t
        return t[self.rank * self.head_rows: (self.rank + 1) * self.head_rows]

    def loss_and_dlogits(self, grad_scale: float = 1.0) -> None:
        """Mean cross-entropy of this rank's tokens into ``self.loss``; logits become the gradient in
        place, scaled by 1 / (tokens on all ranks) so that the summed gradients are the global mean's."""
        K.cross_entropy(self.logits, self._head_slice(self.targets), self.loss_rows, self.logits, self.loss, self.cfg.vocab,
                        grad_scale / (self.M * (self.world if self.mode == "fsdp" else 1) * self.dp_world), 1.0 / self.M)
        if self.mode == "tp" and self.world > 1:
            torch.distributed.all_reduce(self.loss, group=self.group)     # the ranks hold partial sums over their rows

    # -------------------------------------------------------------------- backward
    def backward(self, on_bucket_ready=None) -> None:
        cfg, p, g, L = self.cfg, self.p, self.g, self.cfg.n_layer
        Hq, Hk, D = self.Hq, self.Hk, cfg.head_dim
        dlogits = self.logits
        self._wgrad(dlogits, self._head_slice(self.hf), "lm_head")
        if self.mode == "tp" and self.world > 1:
            torch.distributed.all_reduce(g["lm_head"], group=self.group)  # each rank saw M / tp of the rows
            self._dgrad(dlogits, "lm_head", self.head_dx)
            self._allgather_rows(self.head_dx, self.dtmp)
        else:
            self._dgrad(dlogits, "lm_head", self.dtmp)
        K.rmsnorm_bwd(self.dtmp, self.x[L], p["out_norm"], self.rstd[2 * L], None, self.dx, g["out_norm"], self.norm_scratch)
        dx, dx2 = self.dx, self.dx2
        for l in reversed(range(L)):
            n = f"h.{l}."
            self._dgrad(dx, n + "wd", self.dact)
            self._wgrad(dx, self.act[l], n + "wd")
            K.swiglu_bwd(self.gu[l], self.dact, self.dgu)
            self._col_parallel_dgrad(self.dgu, n + "wgu", self.dtmp)
            self._wgrad(self.dgu, self.h2[l], n + "wgu")
            K.rmsnorm_bwd(self.dtmp, self.xmid[l], p[n + "ffn_norm"], self.rstd[2 * l + 1], dx, dx2, g[n + "ffn_norm"],
                          self.norm_scratch)
            dx, dx2 = dx2, dx
            self._dgrad(dx, n + "wo", self.datt)
            self._wgrad(dx, self.att[l], n + "wo")
            attention_bwd_packed(self.qkv[l], self.att[l], self.datt, self.lse[l], self.dsum, self.dqkv, self.B, self.T,
                                 Hq, Hk, D, causal=True)
            K.rope_(self.dqkv, self.pos, self.freqs, 0, Hq + Hk, D, interleaved=True, inverse=True)
            self._col_parallel_dgrad(self.dqkv, n + "wqkv", self.dtmp)
            self._wgrad(self.dqkv, self.h1[l], n + "wqkv")
            K.rmsnorm_bwd(self.dtmp, self.x[l], p[n + "attn_norm"], self.rstd[2 * l], dx, dx2, g[n + "attn_norm"],
                          self.norm_scratch)
            dx, dx2 = dx2, dx
        if self.mode == "fsdp":
            self.dwte_full.zero_()
            K.embedding_bwd(self.tokens, dx, self.dwte_full, None, self.B, self.T)
            torch.distributed.reduce_scatter_tensor(self.g["wte"], self.dwte_full, group=self.group)
            gg = self.grads.narrow(0, self.decay_n, len(self.gain_names) * cfg.d_model)
            torch.distributed.all_reduce(gg, group=self.group)
        else:
            g["wte"].zero_()
            K.embedding_bwd(self.tokens, dx, g["wte"], None, self.B, self.T)
        if self.dp_group is not None and self.dp_world > 1:
            torch.distributed.all_reduce(self.grads, group=self.dp_group)     # replicas of this shard see other data

    def _gather_rows(self, name: str) -> None:
        """Pushes this rank's rows of a sharded matrix into every rank's full-size copy and waits
        (bounded) until all ranks have done the same."""
        from .. import _native
        from ..ops._util import ptr, stream_ptr
        from ..ops.quant_cuda import _L
        sw = self.sw[name]
        nbytes = sw.shard.numel() * 2
        rc = _L().mimir_peer_allgather(ptr(sw.shard), sw._arr, self.ag_sig.ptr_array(), self.ag_state.data_ptr(),
                                       self.ag_state[1:].data_ptr(), nbytes, self.rank, self.world, 0, stream_ptr())
        _native.check(rc, "gather_rows")

    # ------------------------------------------------------------------- optimizer
    def set_hyper(self, lr: float, beta1: float, beta2: float, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        t = self.step_count
        # grad scale 1: the loss gradient already carries 1 / world
        self._hyper_ring.stage((lr, 1.0 - beta1 ** t, math.sqrt(1.0 - beta2 ** t), 1.0), self.hyper)

    def adamw(self, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1) -> None:
        """AdamW on the owned rows: decayed matrices first, then the gains (not decayed)."""
        if self.mode == "single":
            K.adamw_flat(self.master, self.params, self.grads, self.exp_avg, self.exp_avg_sq, decay_n=self.decay_n,
                         lr=0.0, beta1=beta1, beta2=beta2, eps=eps, wd=wd, step=1, hyper=self.hyper)
            return
        for name in self.own:      # the working copies are scattered over the arena: one launch per tensor
            o, shape = self.own[name]
            n = math.prod(shape)
            sl = slice(o, o + n)
            K.adamw_flat(self.master[sl], self.p[name].reshape(-1), self.grads[sl], self.exp_avg[sl], self.exp_avg_sq[sl],
                         decay_n=n if name in self.shapes else 0, lr=0.0, beta1=beta1, beta2=beta2, eps=eps, wd=wd,
                         step=1, hyper=self.hyper)

    def close(self) -> None:
        if self.mode == "tp":
            torch.cuda.synchronize()
            self.rs_act.close()
            self.ag_sig.close()
            self.act_arena.close()
        if self.mode == "fsdp":
            torch.cuda.synchronize()
            for r in self.rs.values():
                r.close()
            self.ag_sig.close()
            self.arena.close()


def reference_forward_loss(cfg: LlamaTrainConfig, weights: dict, tokens: torch.Tensor, targets: torch.Tensor):
    """Plain fp32 PyTorch restatement; ``weights`` name -> full fp32 tensor.  Returns (loss, grads)."""
    F_ = torch.nn.functional
    w = {n: t.detach().float().clone().requires_grad_(True) for n, t in weights.items()}
    B, T = tokens.shape
    Hq, Hk, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
    inv = 1.0 / (cfg.rope_base ** (torch.arange(0, D, 2, device=tokens.device).double() / D))
    ang = (torch.arange(T, device=tokens.device).double()[:, None] * inv[None]).float()

    def rope(t):   # [B, H, T, D], pairs (2i, 2i+1)
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack([a * ang.cos() - b * ang.sin(), a * ang.sin() + b * ang.cos()], -1).flatten(-2)

    def rms(v, gname):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * w[gname]
    x = w["wte"][tokens]
    for l in range(cfg.n_layer):
        n = f"h.{l}."
        q, k, v = (rms(x, n + "attn_norm") @ w[n + "wqkv"].t()).split([Hq * D, Hk * D, Hk * D], -1)
        q = rope(q.view(B, T, Hq, D).transpose(1, 2))
        k = rope(k.view(B, T, Hk, D).transpose(1, 2)).repeat_interleave(Hq // Hk, 1)
        v = v.view(B, T, Hk, D).transpose(1, 2).repeat_interleave(Hq // Hk, 1)
        o = F_.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + o.transpose(1, 2).reshape(B, T, Hq * D) @ w[n + "wo"].t()
        gate, up = (rms(x, n + "ffn_norm") @ w[n + "wgu"].t()).chunk(2, -1)
        x = x + (F_.silu(gate) * up) @ w[n + "wd"].t()
    logits = rms(x, "out_norm") @ w["lm_head"][: cfg.vocab].t()
    loss = F_.cross_entropy(logits.view(-1, cfg.vocab), targets.view(-1))
    loss.backward()
    return loss.detach(), {n: t.grad for n, t in w.items()}
