"""Tensor-parallel quantized Llama decoding (W4A8: Q4_0 weights, Q8_0 activations,
fp16 KV cache), one process per GPU.

The reference decodes on one device with a recorded CPU step (llm/decode.go:79-160)
and may only replicate quantized tensors on a mesh (tensor/mesh.go:389-391); this
engine shards every block Megatron-style (nn/shard.go:102-158: QKV and gate/up
split by output rows, attention-out and down split by input columns) and runs the
whole decode step as one CUDA graph of native kernels:

  RMSNorm+quantise -> W4A8 GEMV (QKV) -> RoPE -> KV write -> decode attention ->
  quantise -> W4A8 GEMV fused with the all-reduce (+residual) -> RMSNorm+quantise ->
  W4A8 GEMV (gate|up) -> SwiGLU+quantise -> W4A8 GEMV fused with the all-reduce.

The all-reduce inside the GEMV kernel is one-shot over NVLink peer memory
(``csrc/quant_sm100.cu``); positions live in device memory so the same graph serves
every step.  Prompts run through bf16 tcgen05 GEMMs on dequantised weights.
"""
from __future__ import annotations

import os

import ctypes
import math
from dataclasses import dataclass

import torch

from .. import _native
from ..ops import kernels as K
from ..ops import quant_cuda as Q
from ..ops._util import ptr, stream_ptr
from ..parallel.peer import SymmetricBuffer


@dataclass
class LlamaConfig:
    n_layer: int = 32
    d_model: int = 4096
    n_head: int = 32
    n_kv_head: int = 8
    ffn: int = 14336
    vocab: int = 128256
    head_dim: int = 128
    rope_base: float = 500000.0
    eps: float = 1e-5
    ctx: int = 8192

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(n_layer=2, d_model=256, n_head=4, n_kv_head=2, ffn=512, vocab=1024, head_dim=64, ctx=256)


class TPDecoder:
    def __init__(self, cfg: LlamaConfig, rank: int, world: int, batch: int, cap: int, seed: int = 0,
                 device=None, weights: dict | None = None, engine: str = "auto", sampler=None,
                 keep_expanded: bool = True):
        """``engine``: "tc" runs every projection on the tensor cores (Q4_0 tiles expanded to bf16 in
        shared memory, activations rounded to Q8_0 and kept as bf16); "dp4a" is the integer
        dot-product path (one warp per weight row), whose time grows with the batch; "auto" takes
        dp4a up to 4 rows and the tensor cores above (the measured crossover).  ``sampler`` (an
        ``llm.generate.Sampler`` with a temperature above 0) draws the next tokens with the fused
        sampling kernel inside the step; every rank holds the same gathered logits, seed and step
        counter, so every rank draws the same tokens.  Without one the step is greedy."""
        if engine not in ("auto", "tc", "dp4a"):
            raise ValueError(f"unknown decode engine {engine!r}")
        # Prompt processing multiplies hundreds of tokens at once: compute bound, so it runs as bf16
        # GEMMs on expanded weights.  ``keep_expanded`` keeps the expanded copy of every matrix after
        # the first prompt (2 bytes per weight on top of the 4.5 bits decode reads); without it each
        # matrix is expanded into one scratch buffer every time it is used.
        self.keep_expanded = keep_expanded
        self._expanded: dict = {}
        if engine == "auto":
            engine = "tc" if batch > 4 else "dp4a"
        if engine == "tc" and (batch > 32 or cfg.d_model % 64 or (cfg.ffn // world) % 64 or (cfg.n_head // world * cfg.head_dim) % 64):
            engine = "dp4a"
        self.engine = engine
        self.sampler = sampler if sampler is not None and sampler.temperature > 0 else None
        self.cfg, self.rank, self.world, self.B, self.cap = cfg, rank, world, batch, cap
        self.dev = torch.device(device or f"cuda:{torch.cuda.current_device()}")
        d, D = cfg.d_model, cfg.head_dim
        if cfg.n_head % world or cfg.n_kv_head % world or cfg.ffn % (world * 32) or cfg.vocab % (world * 8):
            raise ValueError("heads, kv heads, ffn/32 and vocab/8 must divide by the tensor-parallel size")
        self.Hq, self.Hk, self.F = cfg.n_head // world, cfg.n_kv_head // world, cfg.ffn // world
        self.Vl = cfg.vocab // world
        self.qkv_n = (self.Hq + 2 * self.Hk) * D
        self._init_weights(seed, weights)
        B = batch
        bf, f32 = dict(dtype=torch.bfloat16, device=self.dev), dict(dtype=torch.float32, device=self.dev)
        self.h = torch.zeros(B, d, **bf)
        self.h1 = torch.zeros(B, d, **bf)
        self.qkv = torch.zeros(B, self.qkv_n, **bf)
        self.att = torch.zeros(B, self.Hq * D, **bf)
        self.gu = torch.zeros(B, 2 * self.F, **bf)
        kmax = max(d, self.F, self.Hq * D)
        self.xq = torch.zeros(B, kmax, dtype=torch.int8, device=self.dev)
        self.xs = torch.zeros(B, kmax // 32, **f32)
        self.kc = torch.zeros(cfg.n_layer, B, self.Hk, cap, D, dtype=torch.float16, device=self.dev)
        self.vc = torch.zeros_like(self.kc)
        # decode attention splits the keys over enough blocks to fill the GPU (about 4 per SM)
        sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        self.attn_splits = max(1, min((cap + 63) // 64, (4 * sms) // max(1, B * self.Hk), 64))
        self.attn_ws = torch.zeros(B * self.Hq * self.attn_splits * (D + 2), **f32)
        self.attn_cnt = torch.zeros(B * self.Hk, dtype=torch.int32, device=self.dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=self.dev)      # write position
        self.len = torch.ones(1, dtype=torch.int32, device=self.dev)       # keys visible = pos + 1
        self.pos_rows = torch.zeros(B, dtype=torch.int32, device=self.dev)
        self.tokens = torch.zeros(B, dtype=torch.int64, device=self.dev)
        self.logits_local = torch.zeros(B, self.Vl, **f32)
        inv = 1.0 / (cfg.rope_base ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        self.freqs = inv.float().to(self.dev)
        # symmetric memory: two rotating partial buffers, gathered logits, signal pad
        self.ar_splits = 4 if B <= 8 else 2   # k-splits of the row-parallel products (their partials cross NVLink)
        self.part = [SymmetricBuffer(self.ar_splits * B * d * 4, rank, world) for _ in range(2)]
        self.xdq = torch.zeros(B, kmax, **bf)  # activations rounded to Q8_0, as bf16 (tensor-core engine)
        self.tc_scratch = Q.TcScratch(B * max(self.qkv_n, 2 * self.F, self.Vl), self.dev) if engine == "tc" else None
        self.logits_all = SymmetricBuffer(world * B * self.Vl * 4, rank, world)
        self.sig = SymmetricBuffer(4096 * 4, rank, world)
        self.epochs = torch.zeros(8, dtype=torch.int32, device=self.dev)
        self.counters = torch.zeros(8, dtype=torch.int32, device=self.dev)
        self._part_arr = [p.ptr_array() for p in self.part]
        self._sig_arr = self.sig.ptr_array()
        self._logits_arr = self.logits_all.ptr_array()
        self.graph = None
        self.launches_per_step = 0
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ weights
    def _init_weights(self, seed: int, weights):
        cfg, d, D = self.cfg, self.cfg.d_model, self.cfg.head_dim
        g = torch.Generator(device=self.dev).manual_seed(seed)

        def rnd(n, k, std):
            return torch.randn(n, k, generator=g, device=self.dev) * std

        def shard_rows(full, parts, sizes):
            """Rows of a [sum(sizes) * world... ] matrix that belong to this rank, per logical part."""
            out, off = [], 0
            for size in sizes:
                per = size // self.world
                out.append(full[off + self.rank * per: off + (self.rank + 1) * per])
                off += size
            return torch.cat(out, 0)

        self.layers = []
        std = 0.02
        for l in range(cfg.n_layer):
            if weights is not None:
                wqkv, wo, wgu, wd = (weights[f"blk.{l}.{n}"] for n in ("qkv", "o", "gate_up", "down"))
                an, fn = weights[f"blk.{l}.attn_norm"], weights[f"blk.{l}.ffn_norm"]
            else:  # every rank draws the same full matrices from the seed, then keeps its shard
                wqkv = rnd((cfg.n_head + 2 * cfg.n_kv_head) * D, d, std)
                wo = rnd(d, cfg.n_head * D, std / math.sqrt(2 * cfg.n_layer))
                wgu = rnd(2 * cfg.ffn, d, std)
                wd = rnd(d, cfg.ffn, std / math.sqrt(2 * cfg.n_layer))
                an = torch.ones(d, device=self.dev)
                fn = torch.ones(d, device=self.dev)
            qkv_l = shard_rows(wqkv, 3, [cfg.n_head * D, cfg.n_kv_head * D, cfg.n_kv_head * D])
            gu_l = shard_rows(wgu, 2, [cfg.ffn, cfg.ffn])
            o_l = wo[:, self.rank * self.Hq * D: (self.rank + 1) * self.Hq * D]
            d_l = wd[:, self.rank * self.F: (self.rank + 1) * self.F]
            self.layers.append(dict(qkv=Q.PlanarQ4.quantize(qkv_l), o=Q.PlanarQ4.quantize(o_l.contiguous()),
                                    gate_up=Q.PlanarQ4.quantize(gu_l), down=Q.PlanarQ4.quantize(d_l.contiguous()),
                                    attn_norm=an.bfloat16(), ffn_norm=fn.bfloat16()))
            del wqkv, wo, wgu, wd
        if weights is not None:
            emb, head, onorm = weights["token_embd"], weights["output"], weights["output_norm"]
        else:
            emb = rnd(cfg.vocab, d, std)
            head = rnd(cfg.vocab, d, std)
            onorm = torch.ones(d, device=self.dev)
        self.embed = emb.bfloat16()
        self.head = Q.PlanarQ4.quantize(head[self.rank * self.Vl: (self.rank + 1) * self.Vl])
        if self.engine == "tc":
            for w in self.layers:
                for k in ("qkv", "o", "gate_up", "down"):
                    w[k + "_t"] = Q.TiledQ4.from_planar(w[k])
            self.head_t = Q.TiledQ4.from_planar(self.head)
        self.out_norm = onorm.bfloat16()

    # ------------------------------------------------------------- primitives
    def _gemv_allreduce(self, w: Q.PlanarQ4, k: int, residual, out, slot: int):
        lib = Q._L()
        rc = lib.mimir_q4_gemv_allreduce(ptr(w.scales), ptr(w.quants), ptr(self.xq), ptr(self.xs),
                                         self._part_arr[slot], self._sig_arr, self.epochs[slot:].data_ptr(),
                                         self.counters[slot:].data_ptr(), ptr(residual), ptr(out), w.N, k, self.B,
                                         self.rank, self.world, slot, stream_ptr())
        _native.check(rc, "q4_gemv_allreduce")

    def _tc_allreduce(self, w: Q.TiledQ4, x, residual, out, slot: int):
        lib = Q._L()
        rc = lib.mimir_q4_tc(ptr(w.blob), ptr(x), x.stride(0), self._part_arr[slot], self._sig_arr,
                             self.epochs[slot:].data_ptr(), self.counters[slot:].data_ptr(), ptr(residual), ptr(out), 0,
                             out.stride(0), w.N, w.K, self.B, 0, self.ar_splits, self.rank, self.world, slot, stream_ptr())
        _native.check(rc, "q4_tc(all-reduce)")

    def _attention_step(self, l: int, scale: float):
        cfg, D, B = self.cfg, self.cfg.head_dim, self.B
        lib = Q._L()
        _native.check(lib.mimir_rope_kv_write(ptr(self.qkv), self.qkv_n, ptr(self.pos_rows), ptr(self.freqs),
                                              ptr(self.kc[l]), ptr(self.vc[l]), B, self.Hq, self.Hk, D, self.cap,
                                              ptr(self.pos), stream_ptr()), "rope_kv_write")
        _native.check(lib.mimir_attn_decode(ptr(self.qkv), ptr(self.kc[l]), ptr(self.vc[l]), ptr(self.att), B,
                                            self.Hq, self.Hk, D, self.cap, ptr(self.len), scale, self.qkv_n,
                                            ptr(self.attn_ws), ptr(self.attn_cnt), self.attn_splits, stream_ptr()),
                      "attn_decode")

    def _decode_layers_tc(self):
        cfg, d, D, B = self.cfg, self.cfg.d_model, self.cfg.head_dim, self.B
        scale = 1.0 / math.sqrt(D)
        xd, xa, xf = self.xdq[:, :d], self.xdq[:, : self.Hq * D], self.xdq[:, : self.F]
        for l, w in enumerate(self.layers):
            Q.round_act_q8(self.h, xd, d, 1, w["attn_norm"], cfg.eps)
            Q.q4_tc(w["qkv_t"], xd, self.qkv, self.tc_scratch)
            self._attention_step(l, scale)
            Q.round_act_q8(self.att, xa, self.Hq * D, 0)
            self._tc_allreduce(w["o_t"], xa, self.h, self.h1, 0)
            Q.round_act_q8(self.h1, xd, d, 1, w["ffn_norm"], cfg.eps)
            Q.q4_tc(w["gate_up_t"], xd, self.gu, self.tc_scratch)
            Q.round_act_q8(self.gu, xf, self.F, 2)
            self._tc_allreduce(w["down_t"], xf, self.h1, self.h, 1)

    def _decode_layers(self):
        if self.engine == "tc":
            return self._decode_layers_tc()
        cfg, d, D, B = self.cfg, self.cfg.d_model, self.cfg.head_dim, self.B
        scale = 1.0 / math.sqrt(D)
        lib = Q._L()
        for l, w in enumerate(self.layers):
            Q.quantize_act(self.h, self.xq, self.xs, d, mode=1, gamma=w["attn_norm"], eps=cfg.eps)
            Q.q4_gemv(w["qkv"], self.xq, self.xs, self.qkv)
            self._attention_step(l, scale)
            Q.quantize_act(self.att, self.xq, self.xs, self.Hq * D, mode=0)
            self._gemv_allreduce(w["o"], self.Hq * D, self.h, self.h1, 0)
            Q.quantize_act(self.h1, self.xq, self.xs, d, mode=1, gamma=w["ffn_norm"], eps=cfg.eps)
            Q.q4_gemv(w["gate_up"], self.xq, self.xs, self.gu)
            Q.quantize_act(self.gu, self.xq, self.xs, self.F, mode=2)
            self._gemv_allreduce(w["down"], self.F, self.h1, self.h, 1)

    def _device_step(self):
        """One decode step for the tokens in ``self.tokens``; leaves the next tokens there."""
        cfg, d = self.cfg, self.cfg.d_model
        lib = Q._L()
        K.embedding_fwd(self.tokens, self.embed, None, self.h, 1)
        self._decode_layers()
        if self.engine == "tc":
            Q.round_act_q8(self.h, self.xdq[:, :d], d, 1, self.out_norm, cfg.eps)
            Q.q4_tc(self.head_t, self.xdq[:, :d], self.logits_local, self.tc_scratch)
        else:
            Q.quantize_act(self.h, self.xq, self.xs, d, mode=1, gamma=self.out_norm, eps=cfg.eps)
            Q.q4_gemv(self.head, self.xq, self.xs, self.logits_local)
        _native.check(lib.mimir_peer_allgather(ptr(self.logits_local), self._logits_arr, self._sig_arr,
                                               self.epochs[2:].data_ptr(), self.counters[2:].data_ptr(),
                                               self.logits_local.numel() * 4, self.rank, self.world, 2, stream_ptr()),
                      "allgather")
        full = self.logits_all.view(torch.float32).view(self.world, self.B, self.Vl)
        flat = full.permute(1, 0, 2).reshape(self.B, -1)
        if self.sampler is None:
            self.tokens.copy_(flat.argmax(-1))  # greedy, on the device
        else:
            from ..ops.sampling import sample
            sm = self.sampler
            if getattr(self, "_sampled", None) is None:
                self._sampled = torch.empty(self.B, dtype=torch.int32, device=self.dev)
            sample(flat, sm.temperature, sm.top_k, sm.top_p, sm.min_p, sm.seed, draw_dev=self.pos, out=self._sampled)
            self.tokens.copy_(self._sampled)
        self.pos.add_(1)
        self.len.add_(1)
        self.pos_rows.add_(1)

    # ------------------------------------------------------------------ public
    def reset(self):
        self.pos.zero_()
        self.len.fill_(1)
        self.pos_rows.zero_()

    def step(self) -> None:
        """Runs (or replays) one decode step; no host synchronisation."""
        lib = _native.lib()
        if self.graph is None:
            if getattr(self, "_warm", 0) < 2 or os.environ.get("MIMIR_CUDA_GRAPHS", "1") == "0":
                self._warm = getattr(self, "_warm", 0) + 1
                before = lib.mimir_launch_count()
                self._device_step()
                self.launches_per_step = lib.mimir_launch_count() - before
                return
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = lib.mimir_launch_count()
            with torch.cuda.graph(g):
                self._device_step()
            self.launches_per_step = lib.mimir_launch_count() - before
            self.graph = g
        self.graph.replay()
        lib.mimir_launch_count_add(self.launches_per_step)

    def prefill(self, prompt: torch.Tensor) -> None:
        """Feeds ``prompt`` [B, T] token by token through the decode path (fills the cache and
        leaves the first generated token in ``self.tokens``)."""
        for t in range(prompt.shape[1]):
            self.tokens.copy_(prompt[:, t].to(self.dev))
            self.step()

    def prefill_batched(self, prompt: torch.Tensor, rows_per_chunk: int = 16384) -> None:
        """Prompt processing as GEMMs: all but the last prompt token go through the layers as
        one [B*(T-1), d] bf16 activation matrix (tcgen05 GEMMs on weights expanded from Q4_0 to
        bf16 one matrix at a time, the causal flash-attention kernel, one NCCL all-reduce per
        row-parallel projection), filling the fp16 KV cache; the last token then takes the
        ordinary decode step, which leaves the first generated token in ``self.tokens``.
        Activations stay bf16 here (the decode step rounds them to Q8_0)."""
        from ..ops.attention import attention_fwd
        from ..ops.gemm import gemm
        cfg, d, D, B = self.cfg, self.cfg.d_model, self.cfg.head_dim, self.B
        T = prompt.shape[1]
        if prompt.shape[0] != B:
            raise ValueError(f"prompt batch {prompt.shape[0]} != decoder batch {B}")
        if T + 1 > self.cap:
            raise ValueError(f"prompt of {T} tokens does not fit a cache of {self.cap}")
        Tm = T - 1
        if Tm >= 1:
            bf, f32 = dict(dtype=torch.bfloat16, device=self.dev), dict(dtype=torch.float32, device=self.dev)
            M = B * Tm
            tok = prompt[:, :Tm].reshape(-1).to(self.dev, torch.int64)
            h = torch.empty(M, d, **bf)
            K.embedding_fwd(tok, self.embed, None, h, Tm)
            pos = torch.arange(Tm, dtype=torch.int32, device=self.dev).repeat(B)
            x, rstd = torch.empty(M, d, **bf), torch.empty(M, **f32)
            qkv, att = torch.empty(M, self.qkv_n, **bf), torch.empty(M, self.Hq * D, **bf)
            lse = torch.empty(B * self.Hq * Tm, **f32)
            part = torch.empty(M, d, **bf)
            chunk = max(128, min(M, rows_per_chunk))
            gu = torch.empty(chunk, 2 * self.F, **bf)
            act = torch.empty(chunk, self.F, **bf)
            wmax = max(self.qkv_n * d, d * self.Hq * D, 3 * self.F * d)
            wbuf = torch.empty(wmax, **bf)

            def expand(w, key=None, into=None):
                if self.keep_expanded and key is not None:
                    full = self._expanded.get(key)
                    if full is None:
                        full = self._expanded[key] = w.to_bf16(torch.empty(w.N, w.K, **bf))
                    return full
                return w.to_bf16((wbuf if into is None else into)[: w.N * w.K].view(w.N, w.K))

            def allreduce_residual(partial, resid):
                if self.world > 1:
                    torch.distributed.all_reduce(partial)
                resid.add_(partial)

            q4 = qkv.view(B, Tm, self.qkv_n)
            qv = q4[:, :, : self.Hq * D].unflatten(2, (self.Hq, D))
            kv = q4[:, :, self.Hq * D: (self.Hq + self.Hk) * D].unflatten(2, (self.Hk, D))
            vv = q4[:, :, (self.Hq + self.Hk) * D:].unflatten(2, (self.Hk, D))
            for l, w in enumerate(self.layers):
                K.rmsnorm_fwd(h, w["attn_norm"], x, rstd, cfg.eps)
                gemm(x, expand(w["qkv"], (l, "qkv")), out=qkv)
                K.rope_(qkv, pos, self.freqs, 0, self.Hq + self.Hk, D, interleaved=True)
                self.kc[l][:, :, :Tm].copy_(kv.permute(0, 2, 1, 3))
                self.vc[l][:, :, :Tm].copy_(vv.permute(0, 2, 1, 3))
                attention_fwd(qv, kv, vv, att.view(B, Tm, self.Hq, D), lse, causal=True)
                gemm(att, expand(w["o"], (l, "o")), out=part)
                allreduce_residual(part, h)
                K.rmsnorm_fwd(h, w["ffn_norm"], x, rstd, cfg.eps)
                wgu = expand(w["gate_up"], (l, "gate_up"))
                wd = expand(w["down"], (l, "down"), into=wbuf[2 * self.F * d:])
                for r0 in range(0, M, chunk):
                    r1 = min(M, r0 + chunk)
                    gemm(x[r0:r1], wgu, out=gu[: r1 - r0])
                    K.swiglu_fwd(gu[: r1 - r0], act[: r1 - r0])
                    gemm(act[: r1 - r0], wd, out=part[r0:r1])
                allreduce_residual(part, h)
            self.pos.fill_(Tm)
            self.len.fill_(Tm + 1)
            self.pos_rows.fill_(Tm)
        self.tokens.copy_(prompt[:, T - 1].to(self.dev))
        self.step()

    def generate(self, prompt: torch.Tensor, n: int, batched_prefill: bool = True) -> torch.Tensor:
        self.reset()
        (self.prefill_batched if batched_prefill else self.prefill)(prompt)
        out = [self.tokens.clone()]
        for _ in range(n - 1):
            self.step()
            out.append(self.tokens.clone())
        return torch.stack(out, 1)

    def primitive_times(self, iters: int = 50) -> dict:
        """Device time in microseconds of each kernel of a decode step, measured by queueing
        ``iters`` back-to-back calls of it (layer 0's weights) between two CUDA events.  Every
        rank makes the same calls, so the collective kernels meet their peers."""
        cfg, d, D, B = self.cfg, self.cfg.d_model, self.cfg.head_dim, self.B
        lib, w = Q._L(), self.layers[0]
        scale = 1.0 / math.sqrt(D)
        full = self.logits_all.view(torch.float32).view(self.world, self.B, self.Vl)
        common = {
            "embedding": lambda: K.embedding_fwd(self.tokens, self.embed, None, self.h, 1),
            "rope_kv_write": lambda: _native.check(lib.mimir_rope_kv_write(
                ptr(self.qkv), self.qkv_n, ptr(self.pos_rows), ptr(self.freqs), ptr(self.kc[0]), ptr(self.vc[0]), B,
                self.Hq, self.Hk, D, self.cap, ptr(self.pos), stream_ptr()), "rope_kv_write"),
            "attn_decode": lambda: _native.check(lib.mimir_attn_decode(
                ptr(self.qkv), ptr(self.kc[0]), ptr(self.vc[0]), ptr(self.att), B, self.Hq, self.Hk, D, self.cap,
                ptr(self.len), scale, self.qkv_n, ptr(self.attn_ws), ptr(self.attn_cnt), self.attn_splits,
                stream_ptr()), "attn_decode"),
            "logits_allgather": lambda: _native.check(lib.mimir_peer_allgather(
                ptr(self.logits_local), self._logits_arr, self._sig_arr, self.epochs[2:].data_ptr(),
                self.counters[2:].data_ptr(), self.logits_local.numel() * 4, self.rank, self.world, 2, stream_ptr()),
                "allgather"),
            "argmax": lambda: full.permute(1, 0, 2).reshape(self.B, -1).argmax(-1),
        }
        if self.engine == "tc":
            xd, xa, xf = self.xdq[:, :d], self.xdq[:, : self.Hq * D], self.xdq[:, : self.F]
            cases = dict(common, **{
                "rmsnorm_round": lambda: Q.round_act_q8(self.h, xd, d, 1, w["attn_norm"], cfg.eps),
                "tc_qkv": lambda: Q.q4_tc(w["qkv_t"], xd, self.qkv, self.tc_scratch),
                "round_att": lambda: Q.round_act_q8(self.att, xa, self.Hq * D, 0),
                "tc_o_allreduce": lambda: self._tc_allreduce(w["o_t"], xa, self.h, self.h1, 0),
                "tc_gate_up": lambda: Q.q4_tc(w["gate_up_t"], xd, self.gu, self.tc_scratch),
                "swiglu_round": lambda: Q.round_act_q8(self.gu, xf, self.F, 2),
                "tc_down_allreduce": lambda: self._tc_allreduce(w["down_t"], xf, self.h1, self.h, 1),
                "tc_head": lambda: Q.q4_tc(self.head_t, xd, self.logits_local, self.tc_scratch),
            })
        else:
            cases = dict(common, **{
                "rmsnorm_quantize": lambda: Q.quantize_act(self.h, self.xq, self.xs, d, mode=1, gamma=w["attn_norm"], eps=cfg.eps),
                "gemv_qkv": lambda: Q.q4_gemv(w["qkv"], self.xq, self.xs, self.qkv),
                "quantize_att": lambda: Q.quantize_act(self.att, self.xq, self.xs, self.Hq * D, mode=0),
                "gemv_o_allreduce": lambda: self._gemv_allreduce(w["o"], self.Hq * D, self.h, self.h1, 0),
                "gemv_gate_up": lambda: Q.q4_gemv(w["gate_up"], self.xq, self.xs, self.gu),
                "swiglu_quantize": lambda: Q.quantize_act(self.gu, self.xq, self.xs, self.F, mode=2),
                "gemv_down_allreduce": lambda: self._gemv_allreduce(w["down"], self.F, self.h1, self.h, 1),
                "gemv_head": lambda: Q.q4_gemv(self.head, self.xq, self.xs, self.logits_local),
            })
        out = {}
        for name, fn in cases.items():
            for _ in range(3):
                fn()
            if self.world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            out[name] = round(e0.elapsed_time(e1) * 1e3 / iters, 2)
        return out

    def close(self):
        torch.cuda.synchronize()
        if self.world > 1:
            torch.distributed.barrier()
        for b in (*self.part, self.logits_all, self.sig):
            b.close()
