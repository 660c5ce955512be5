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
from .module import Dropout, LayerNorm, Linear, Module, RMSNorm, uniform_init


class RotaryEmbedding:
    """Rotary position embedding with optional Llama-3 frequency scaling (nn/transformer.go:110,191-259)."""

    def __init__(self, dim: int, base: float = 10000.0, interleaved: bool = False, scaling: dict | None = None):
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

    def apply(self, x, positions=0):
        """``x`` [B, H, T, D]; ``positions`` an int tensor [T] (lazy or torch), or the position of the
        first row (the reference's ``Apply(x, offset)``).  The default pairs column i with column
        i + dim/2 (GPT-NeoX, Hugging Face Llama); ``interleaved`` pairs (2i, 2i+1) (GPT-J, Meta's Llama)."""
        inv, inter, d = self.inv_freq, self.interleaved, self.dim
        if isinstance(positions, int):
            positions = torch.arange(positions, positions + x.shape[-2], dtype=torch.int32)
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
    """Attention over separate query / key / value inputs ``[B, T, dim]`` with the three input
    projections stored as one ``in_proj_weight [3 dim, dim]`` (rows: query, key, value) and
    ``in_proj_bias [3 dim]``, then ``out_proj`` (nn/transformer_layers.go: MultiheadAttention).  When
    the three inputs are one tensor the projection is a single product."""

    def __init__(self, dim: int, heads: int, bias: bool = True, dtype=torch.float32):
        if dim % heads:
            raise ValueError(f"MultiheadAttention: {dim} features do not split into {heads} heads")
        self.dim, self.heads, self.head_dim = dim, heads, dim // heads
        bound = math.sqrt(6.0 / (dim + 3 * dim))            # Xavier uniform over the fused matrix
        self.in_proj_weight = Param(uniform_init((3 * dim, dim), bound, dtype), "in_proj_weight")
        self.in_proj_bias = Param(torch.zeros(3 * dim, dtype=dtype), "in_proj_bias") if bias else None
        self.out_proj = Linear(dim, dim, bias, dtype)

    def _project(self, query, key, value):
        w = self.in_proj_weight.value()
        b = self.in_proj_bias.value() if self.in_proj_bias is not None else None
        E = self.dim
        if query is key and key is value:
            return T.split(T.matmul_t(query, w, b), [E, E, E], dim=-1)
        out = []
        for i, x in enumerate((query, key, value)):
            wi = T.shrink(w, ((i * E, (i + 1) * E), (0, E)))
            bi = T.shrink(b, ((i * E, (i + 1) * E),)) if b is not None else None
            out.append(T.matmul_t(x, wi, bi))
        return out

    def forward(self, query, key=None, value=None, mask=None, causal=False):
        key = query if key is None else key
        value = key if value is None else value
        B, Tq, C = query.shape
        Tk = key.shape[1]
        q, k, v = self._project(query, key, value)
        sp = lambda t, n: T.permute(T.reshape(t, (B, n, self.heads, self.head_dim)), (0, 2, 1, 3))  # noqa: E731
        o = T.attention(sp(q, Tq), sp(k, Tk), sp(v, Tk), causal=causal, mask=mask)
        return self.out_proj(T.reshape(T.permute(o, (0, 2, 1, 3)), (B, Tq, C)))


_ACTIVATIONS = {"gelu": lambda x: T.gelu(x), "gelu_exact": lambda x: T.gelu(x, "none"), "relu": lambda x: T.relu(x),
                "silu": lambda x: T.silu(x), "tanh": lambda x: T.tanh(x)}


class MLP(Module):
    """``down(act(up(x)))``; ``activation`` is a name ("gelu", the tanh form; "gelu_exact"; "relu"; "silu";
    "tanh") or a function of one tensor."""

    def __init__(self, dim: int, hidden: int, bias: bool = True, dtype=torch.float32, activation="gelu"):
        self.up, self.down = Linear(dim, hidden, bias, dtype), Linear(hidden, dim, bias, dtype)
        self.act = _ACTIVATIONS[activation] if isinstance(activation, str) else activation

    def forward(self, x):
        return self.down(self.act(self.up(x)))


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
    """Self-attention and a two-layer feed-forward, each with a residual and a LayerNorm
    (nn/transformer_layers.go: NewTransformerEncoderLayer).  The defaults are the reference's and
    PyTorch's: ReLU, LayerNorm epsilon 1e-5, dropout 0.1 (active only while training), the norm after
    each residual; ``norm_first`` moves it in front of each sub-layer, ``activation`` names another
    function.  The attention's projections are one ``attn.qkv`` matrix ``[3 dim, dim]`` (rows: query,
    key, value)."""

    def __init__(self, dim: int, heads: int, hidden: int, eps: float = 1e-5, dtype=torch.float32,
                 activation="relu", dropout: float = 0.1, norm_first: bool = False):
        self.attn = SelfAttention(dim, heads, causal=False, dtype=dtype)
        self.norm1, self.norm2 = LayerNorm(dim, eps, dtype), LayerNorm(dim, eps, dtype)
        self.mlp = MLP(dim, hidden, True, dtype, activation)
        self.drop1, self.drop2, self.norm_first = Dropout(dropout), Dropout(dropout), norm_first

    def forward(self, x, mask=None):
        if self.norm_first:
            x = x + self.drop1(self.attn(self.norm1(x), mask=mask))
            return x + self.drop2(self.mlp(self.norm2(x)))
        x = self.norm1(x + self.drop1(self.attn(x, mask=mask)))
        return self.norm2(x + self.drop2(self.mlp(x)))
