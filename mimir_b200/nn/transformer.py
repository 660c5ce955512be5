"""Transformer building blocks (reference: nn/transformer.go:31-730).

``SelfAttention`` keeps the fused QKV projection laid out as [all Q heads | all K
heads | all V heads] (nn/transformer.go:485-522), supports grouped-query heads,
rotary embeddings (interleaved pairs for "llama", halves for "qwen2",
llm/model.go:315-321) and a ``KVCache`` for incremental decoding.
"""
from __future__ import annotations

import math

import torch

from .. import tensor as T
from ..tensor.autograd import Param
from .module import LayerNorm, Linear, Module, RMSNorm


class RotaryEmbedding:
    """Rotary position embedding with optional Llama-3 frequency scaling (nn/transformer.go:110,191-259)."""

    def __init__(self, dim: int, base: float = 10000.0, interleaved: bool = True, scaling: dict | None = None):
        self.dim, self.base, self.interleaved = dim, base, interleaved
        inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        if scaling:
            kind = scaling.get("type", "linear")
            if kind == "linear":
                inv = inv / scaling.get("factor", 1.0)
            elif kind == "llama3":
                factor, lo, hi = scaling.get("factor", 8.0), scaling.get("low_freq_factor", 1.0), scaling.get("high_freq_factor", 4.0)
                old = scaling.get("original_context", 8192)
                wl = 2 * math.pi / inv
                smooth = ((old / wl) - lo) / (hi - lo)
                inv = torch.where(wl > old / lo, inv / factor,
                                  torch.where(wl < old / hi, inv, (1 - smooth) * inv / factor + smooth * inv))
        self.inv_freq = inv.float()

    def apply(self, x, positions):
        """``x`` [B, H, T, D]; ``positions`` an int tensor [T] (lazy or torch)."""
        inv, inter, d = self.inv_freq, self.interleaved, self.dim
        pos = positions if isinstance(positions, T.Tensor) else T.tensor(positions, dtype=torch.int32, device=x.device)

        def run(v, p):
            ang = p.float()[:, None] * inv.to(v.device)[None]
            cos, sin = ang.cos().to(v.dtype), ang.sin().to(v.dtype)
            rot, rest = v[..., :d], v[..., d:]
            if inter:
                a, b = rot[..., 0::2], rot[..., 1::2]
                out = torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)
            else:
                a, b = rot[..., : d // 2], rot[..., d // 2:]
                out = torch.cat([a * cos - b * sin, a * sin + b * cos], -1)
            return torch.cat([out, rest], -1) if rest.shape[-1] else out
        return T.core._node(run, (x, pos), {}, "rope")


class KVCache:
    """Preallocated key/value buffers for incremental decoding (nn/transformer.go:348-476)."""

    def __init__(self, batch: int, heads: int, cap: int, dim: int, dtype=torch.float32, device="cpu"):
        self.k = torch.zeros(batch, heads, cap, dim, dtype=dtype, device=device)
        self.v = torch.zeros(batch, heads, cap, dim, dtype=dtype, device=device)
        self.len, self.cap = 0, cap

    def reset(self):
        self.len = 0

    def truncate(self, n: int):
        self.len = min(self.len, n)

    def positions(self, t: int):
        return torch.arange(self.len, self.len + t, dtype=torch.int32, device=self.k.device)

    def append(self, k: torch.Tensor, v: torch.Tensor):
        t = k.shape[2]
        if self.len + t > self.cap:
            raise T.ErrShape(f"KV cache overflow: {self.len} + {t} > {self.cap}")
        self.k[:, :, self.len: self.len + t] = k.to(self.k.dtype)
        self.v[:, :, self.len: self.len + t] = v.to(self.v.dtype)
        self.len += t
        return self.k[:, :, : self.len], self.v[:, :, : self.len]

    def buffers(self):
        return self.k, self.v

    def write(self, k: torch.Tensor, v: torch.Tensor, at: int | None = None) -> None:
        """Stores keys / values at position ``at`` (default: the current length) without moving the
        length: a recorded decode step writes first and calls ``advance`` afterwards."""
        at = self.len if at is None else at
        t = k.shape[2]
        if at + t > self.cap:
            raise T.ErrShape(f"KV cache overflow: {at} + {t} > {self.cap}")
        self.k[:, :, at: at + t] = k.to(self.k.dtype)
        self.v[:, :, at: at + t] = v.to(self.v.dtype)

    def advance(self, t: int = 1) -> None:
        if self.len + t > self.cap:
            raise T.ErrShape(f"KV cache overflow: {self.len} + {t} > {self.cap}")
        self.len += t


class SelfAttention(Module):
    def __init__(self, dim: int, heads: int, kv_heads: int | None = None, bias: bool = True, causal: bool = True,
                 rope: RotaryEmbedding | None = None, head_dim: int | None = None, dtype=torch.float32):
        self.heads, self.kv_heads = heads, kv_heads or heads
        self.head_dim = head_dim or dim // heads
        self.causal, self.rope = causal, rope
        self.qkv = Linear(dim, (self.heads + 2 * self.kv_heads) * self.head_dim, bias, dtype)
        # rows are [all Q heads | all K heads | all V heads]: a tensor-parallel split cuts each section
        self.qkv._qkv_sections = (self.heads * self.head_dim, self.kv_heads * self.head_dim,
                                  self.kv_heads * self.head_dim)
        self.out = Linear(self.heads * self.head_dim, dim, bias, dtype)

    def forward(self, x, cache: KVCache | None = None, mask=None):
        B, Tq, _ = x.shape
        H, Hk, D = self.heads, self.kv_heads, self.head_dim
        qkv = self.qkv(x)
        q, k, v = T.split(qkv, [H * D, Hk * D, Hk * D], dim=-1)
        q = T.permute(T.reshape(q, (B, Tq, H, D)), (0, 2, 1, 3))
        k = T.permute(T.reshape(k, (B, Tq, Hk, D)), (0, 2, 1, 3))
        v = T.permute(T.reshape(v, (B, Tq, Hk, D)), (0, 2, 1, 3))
        past = cache.len if cache is not None else 0
        if self.rope is not None:
            pos = torch.arange(past, past + Tq, dtype=torch.int32)
            q, k = self.rope.apply(q, pos), self.rope.apply(k, pos)
        if cache is not None:
            T.realize(k, v)
            kk, vv = cache.append(k.data(), v.data())
            k, v = T.from_torch(kk.to(q.dtype)), T.from_torch(vv.to(q.dtype))
        o = T.attention(q, k, v, causal=self.causal, causal_offset=past if self.causal else None, mask=mask)
        o = T.reshape(T.permute(o, (0, 2, 1, 3)), (B, Tq, H * D))
        return self.out(o)


class MultiheadAttention(Module):
    """Separate query / key / value inputs (cross attention)."""

    def __init__(self, dim: int, heads: int, bias: bool = True, dtype=torch.float32):
        self.heads, self.head_dim = heads, dim // heads
        self.q, self.k, self.v, self.out = (Linear(dim, dim, bias, dtype) for _ in range(4))

    def forward(self, query, key, value, mask=None, causal=False):
        B, Tq, C = query.shape
        Tk = key.shape[1]
        sp = lambda t, n: T.permute(T.reshape(t, (B, n, self.heads, self.head_dim)), (0, 2, 1, 3))  # noqa: E731
        o = T.attention(sp(self.q(query), Tq), sp(self.k(key), Tk), sp(self.v(value), Tk), causal=causal, mask=mask)
        return self.out(T.reshape(T.permute(o, (0, 2, 1, 3)), (B, Tq, C)))


class MLP(Module):
    def __init__(self, dim: int, hidden: int, bias: bool = True, dtype=torch.float32):
        self.up, self.down = Linear(dim, hidden, bias, dtype), Linear(hidden, dim, bias, dtype)

    def forward(self, x):
        return self.down(T.gelu(self.up(x)))


class GatedMLP(Module):
    """SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``."""

    def __init__(self, dim: int, hidden: int, bias: bool = False, dtype=torch.float32):
        self.gate, self.up, self.down = Linear(dim, hidden, bias, dtype), Linear(dim, hidden, bias, dtype), Linear(hidden, dim, bias, dtype)

    def forward(self, x):
        return self.down(T.swiglu(self.gate(x), self.up(x)))


class DecoderBlock(Module):
    """Pre-norm decoder block; ``style="gpt2"`` = LayerNorm + GELU MLP with biases,
    ``style="llama"`` = RMSNorm + SwiGLU without biases."""

    def __init__(self, dim: int, heads: int, hidden: int | None = None, kv_heads: int | None = None, style: str = "gpt2",
                 rope: RotaryEmbedding | None = None, eps: float = 1e-5, dtype=torch.float32):
        llama = style == "llama"
        norm = (lambda: RMSNorm(dim, eps, dtype)) if llama else (lambda: LayerNorm(dim, eps, dtype))
        self.norm1, self.norm2 = norm(), norm()
        self.attn = SelfAttention(dim, heads, kv_heads, bias=not llama, causal=True, rope=rope, dtype=dtype)
        self.mlp = GatedMLP(dim, hidden or 4 * dim, False, dtype) if llama else MLP(dim, hidden or 4 * dim, True, dtype)

    def forward(self, x, cache: KVCache | None = None):
        x = x + self.attn(self.norm1(x), cache)
        return x + self.mlp(self.norm2(x))


class TransformerEncoderLayer(Module):
    """Post-norm encoder layer (BERT style)."""

    def __init__(self, dim: int, heads: int, hidden: int, eps: float = 1e-12, dtype=torch.float32):
        self.attn = SelfAttention(dim, heads, causal=False, dtype=dtype)
        self.norm1, self.norm2 = LayerNorm(dim, eps, dtype), LayerNorm(dim, eps, dtype)
        self.mlp = MLP(dim, hidden, True, dtype)

    def forward(self, x, mask=None):
        x = self.norm1(x + self.attn(x, mask=mask))
        return self.norm2(x + self.mlp(x))
