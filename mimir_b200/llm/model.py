"""Llama / Qwen2 language models loaded from ``.mim`` files with GGUF-style metadata
(reference: llm/model.go:52-168 config, :216-313 load, :391-437 logits with KV caches;
llm/train.go loss / score / embedding / hidden; llm/lora.go adapters)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn
from .. import tensor as T
from ..io import mim

MAX_LAYERS, MAX_DIM = 1 << 10, 1 << 20


@dataclass
class Config:
    arch: str = "llama"
    vocab: int = 0
    context: int = 2048
    embed: int = 0
    hidden: int = 0
    layers: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    rope_dim: int = 0
    rope_base: float = 10000.0
    rope_scale: float = 1.0
    eps: float = 1e-5

    @staticmethod
    def from_metadata(md: dict, arch: str | None = None) -> "Config":
        arch = arch or md.get("general.architecture")
        if arch not in ("llama", "qwen2"):
            raise T.ErrUnsupported(f"llm: architecture {arch!r}, want llama or qwen2")
        errs = []

        def integer(key, default, required):
            v = md.get(f"{arch}.{key}")
            if v is None:
                if required:
                    errs.append(f"no {arch}.{key}")
                return default
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0 or v > MAX_DIM:
                errs.append(f"{arch}.{key} = {v!r}")
                return default
            return v

        def number(key, default):
            v = md.get(f"{arch}.{key}")
            if v is None:
                return default
            if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0 or math.isinf(v):
                errs.append(f"{arch}.{key} = {v!r}")
                return default
            return float(v)
        c = Config(arch=arch, context=integer("context_length", 2048, False), embed=integer("embedding_length", 0, True),
                   hidden=integer("feed_forward_length", 0, True), layers=integer("block_count", 0, True),
                   heads=integer("attention.head_count", 0, True), rope_base=number("rope.freq_base", 10000.0),
                   eps=number("attention.layer_norm_rms_epsilon", 1e-5))
        c.kv_heads = integer("attention.head_count_kv", c.heads, False)
        c.head_dim = integer("attention.key_length", c.embed // max(c.heads, 1), False)
        c.rope_dim = integer("rope.dimension_count", c.head_dim, False)
        scaling = md.get(f"{arch}.rope.scaling.type", "none")
        if scaling == "none":
            c.rope_scale = number("rope.scale_linear", 1.0)
        elif scaling == "linear":
            c.rope_scale = number("rope.scaling.factor", 1.0)
        else:
            errs.append(f"rope scaling {scaling!r}")
        if integer("attention.value_length", c.head_dim, False) != c.head_dim:
            errs.append(f"values of other than {c.head_dim} features")
        if not c.rope_base > 1:
            errs.append(f"rope base {c.rope_base}")
        if c.layers > MAX_LAYERS or c.heads % max(c.kv_heads, 1) or c.rope_dim > c.head_dim or c.rope_dim % 2:
            errs.append(f"{c.layers} layers, {c.heads} heads and {c.kv_heads} key heads of {c.head_dim} features, {c.rope_dim} rotated")
        if errs:
            raise T.ErrShape("llm: model hyperparameters: " + "; ".join(errs))
        return c

    def metadata(self) -> dict:
        a = self.arch
        return {"general.architecture": a, f"{a}.context_length": self.context, f"{a}.embedding_length": self.embed,
                f"{a}.feed_forward_length": self.hidden, f"{a}.block_count": self.layers,
                f"{a}.attention.head_count": self.heads, f"{a}.attention.head_count_kv": self.kv_heads,
                f"{a}.attention.key_length": self.head_dim, f"{a}.rope.dimension_count": self.rope_dim,
                f"{a}.rope.freq_base": float(self.rope_base), f"{a}.attention.layer_norm_rms_epsilon": float(self.eps)}


class Block(nn.Module):
    def __init__(self, c: Config):
        bias = c.arch == "qwen2"
        q, kv = c.heads * c.head_dim, c.kv_heads * c.head_dim
        self.attn_norm, self.mlp_norm = nn.RMSNorm(c.embed, c.eps), nn.RMSNorm(c.embed, c.eps)
        self.q, self.k, self.v = nn.Linear(c.embed, q, bias), nn.Linear(c.embed, kv, bias), nn.Linear(c.embed, kv, bias)
        self.o = nn.Linear(q, c.embed, False)
        self.gate, self.up = nn.Linear(c.embed, c.hidden, False), nn.Linear(c.embed, c.hidden, False)
        self.down = nn.Linear(c.hidden, c.embed, False)

    def forward(self, x, rope, c: Config, cache=None):
        B, Tn, _ = x.shape
        H, Hk, D = c.heads, c.kv_heads, c.head_dim
        h = self.attn_norm(x)
        sp = lambda t, n: T.permute(T.reshape(t, (B, Tn, n, D)), (0, 2, 1, 3))  # noqa: E731
        q, k, v = sp(self.q(h), H), sp(self.k(h), Hk), sp(self.v(h), Hk)
        past = cache.len if cache is not None else 0
        pos = torch.arange(past, past + Tn, dtype=torch.int32)
        q, k = rope.apply(q, pos), rope.apply(k, pos)
        if cache is not None:
            T.realize(k, v)
            kk, vv = cache.append(k.data(), v.data())
            k, v = T.from_torch(kk.to(q.dtype)), T.from_torch(vv.to(q.dtype))
        o = T.attention(q, k, v, causal=True, causal_offset=past)
        x = x + self.o(T.reshape(T.permute(o, (0, 2, 1, 3)), (B, Tn, H * D)))
        h = self.mlp_norm(x)
        return x + self.down(T.swiglu(self.gate(h), self.up(h)))


class Model(nn.Module):
    def __init__(self, c: Config, rope_freqs: torch.Tensor | None = None):
        self.cfg = c
        self.embed = nn.Embedding(c.vocab, c.embed)
        self.embed.weight.set(nn.normal_init((c.vocab, c.embed), 0.02))
        self.blocks = [Block(c) for _ in range(c.layers)]
        self.norm = nn.RMSNorm(c.embed, c.eps)
        self.output = None                      # tied to the embedding unless the file has output.weight
        # llama.cpp rotates pairs (2i, 2i+1) for "llama" and halves for "qwen2"
        scaling = {"type": "linear", "factor": c.rope_scale} if c.rope_scale != 1.0 else None
        self._nn_skip_rope = nn.RotaryEmbedding(c.rope_dim, c.rope_base, interleaved=c.arch == "llama", scaling=scaling)
        if rope_freqs is not None:              # Llama 3.1+: a stored divisor of every frequency
            self._nn_skip_rope.inv_freq = self._nn_skip_rope.inv_freq / rope_freqs.float()

    # ------------------------------------------------------------------ file I/O
    NAMES = (("attn_norm", "attn_norm"), ("q", "attn_q"), ("k", "attn_k"), ("v", "attn_v"), ("o", "attn_output"),
             ("mlp_norm", "ffn_norm"), ("gate", "ffn_gate"), ("up", "ffn_up"), ("down", "ffn_down"))

    def _file_tensors(self):
        yield "token_embd.weight", self.embed.weight
        yield "output_norm.weight", self.norm.weight
        if self.output is not None:
            yield "output.weight", self.output.weight
        for i, b in enumerate(self.blocks):
            for attr, stem in self.NAMES:
                m = getattr(b, attr)
                m = m.base if isinstance(m, nn.LoRALinear) else m
                yield f"blk.{i}.{stem}.weight", m.weight
                if getattr(m, "bias", None) is not None and stem in ("attn_q", "attn_k", "attn_v"):
                    yield f"blk.{i}.{stem}.bias", m.bias

    @staticmethod
    def load(src, dtype=torch.float32) -> "Model":
        """``src``: a path or an open ``mim.Model``.  Quantized tensors are dequantized to ``dtype``."""
        f = mim.open(src) if isinstance(src, (str, bytes)) or hasattr(src, "__fspath__") else src
        md = f.metadata
        c = Config.from_metadata(md)
        if "token_embd.weight" not in f:
            raise T.ErrShape("llm: no token_embd.weight")
        c.vocab = int(f.info("token_embd.weight")[1][0])
        m = Model(c, f.tensor("rope_freqs.weight") if "rope_freqs.weight" in f else None)
        if "output.weight" in f:
            m.output = nn.Linear(c.embed, c.vocab, False)
        for name, p in m._file_tensors():
            if name not in f:
                raise T.ErrShape(f"llm: no tensor {name}")
            t = f.tensor(name)
            t = t.dequantize(dtype) if isinstance(t, mim.QuantizedTensor) else t.to(dtype)
            if tuple(t.shape) != tuple(p.shape):
                raise T.ErrShape(f"llm: {name} of shape {tuple(t.shape)}, want {tuple(p.shape)}")
            p.set(t.clone())
        m.tokenizer_metadata = {k: v for k, v in md.items() if k.startswith("tokenizer.")}
        return m

    def save(self, path: str, extra_metadata: dict | None = None) -> None:
        md = dict(self.cfg.metadata(), **(extra_metadata or {}))
        mim.write_tensors(path, {n: p._data for n, p in self._file_tensors()}, metadata=md)

    # ------------------------------------------------------------------- compute
    def new_caches(self, batch: int = 1, cap: int | None = None, dtype=torch.float32):
        c = self.cfg
        return [nn.KVCache(batch, c.kv_heads, cap or c.context, c.head_dim, dtype) for _ in self.blocks]

    def hidden(self, tokens, caches=None):
        """tokens [B, T] -> final normalised hidden states [B, T, embed]."""
        x = self.embed(tokens)
        for i, b in enumerate(self.blocks):
            x = b(x, self._nn_skip_rope, self.cfg, caches[i] if caches is not None else None)
        return self.norm(x)

    def logits(self, tokens, caches=None):
        h = self.hidden(tokens, caches)
        w = self.output.weight.value() if self.output is not None else self.embed.weight.value()
        return T.matmul_t(h, w)

    forward = logits

    def _check(self, seqs):
        for s in seqs:
            if len(s) < 2:
                raise T.ErrShape("llm: a sequence needs at least two tokens")
            if len(s) > self.cfg.context:
                raise T.ErrShape(f"llm: sequence of {len(s)} tokens, context {self.cfg.context}")
            if min(s) < 0 or max(s) >= self.cfg.vocab:
                raise T.ErrIndex("llm: token outside the vocabulary")

    def _batch(self, seqs, learn):
        """Right-padded inputs, next tokens and per-position weights (``learn`` masks what counts)."""
        self._check(seqs)
        n = max(len(s) for s in seqs) - 1
        inp = torch.zeros(len(seqs), n, dtype=torch.int64)
        nxt = torch.zeros(len(seqs), n, dtype=torch.int64)
        w = torch.zeros(len(seqs), n)
        for i, s in enumerate(seqs):
            inp[i, : len(s) - 1] = torch.tensor(s[:-1])
            nxt[i, : len(s) - 1] = torch.tensor(s[1:])
            w[i, : len(s) - 1] = 1.0 if learn is None else torch.tensor([float(b) for b in learn[i][1:]])
        return inp, nxt, w

    def loss(self, seqs, learn=None):
        """Mean next-token cross entropy over the positions that ``learn`` selects (all if None)."""
        inp, nxt, w = self._batch(seqs, learn)
        logp = T.log_softmax(self.logits(T.from_torch(inp)), -1)
        picked = T.reshape(T.gather(logp, 2, T.from_torch(nxt[..., None])), tuple(nxt.shape))
        return -T.sum_(picked * T.from_torch(w)) / max(float(w.sum()), 1.0)

    def score(self, seqs, learn=None):
        """``(mean loss, tokens predicted right, tokens counted)`` without building gradients."""
        inp, nxt, w = self._batch(seqs, learn)
        with torch.no_grad():
            lg = self.logits(T.from_torch(inp)).data().float()
        logp = torch.log_softmax(lg, -1).gather(2, nxt[..., None]).squeeze(-1)
        total = int(w.sum())
        right = int(((lg.argmax(-1) == nxt).float() * w).sum())
        return float(-(logp * w).sum() / max(total, 1)), right, total

    def embedding(self, tokens) -> torch.Tensor:
        """Mean of the final hidden states of one sequence, L2-normalised."""
        with torch.no_grad():
            h = self.hidden(T.from_torch(torch.tensor([list(tokens)]))).data()[0].float().mean(0)
        return h / h.norm().clamp_min(1e-12)

    # ---------------------------------------------------------------------- LoRA
    TARGETS = ("q", "k", "v", "o", "gate", "up", "down")

    def add_lora(self, rank: int = 8, alpha: float = 16.0, targets=("q", "v")) -> None:
        for t in targets:
            if t not in self.TARGETS:
                raise T.ErrUnsupported(f"llm: no projection {t!r}")
        for p in self.parameters():
            p.freeze()
        for b in self.blocks:
            for t in targets:
                m = getattr(b, t)
                if not isinstance(m, nn.LoRALinear):
                    setattr(b, t, nn.LoRALinear(m, rank, alpha))
        self.lora = {"rank": rank, "alpha": alpha, "targets": list(targets)}

    def _pairs(self):
        stems = dict(self.NAMES)
        for i, b in enumerate(self.blocks):
            for t in self.TARGETS:
                m = getattr(b, t)
                if isinstance(m, nn.LoRALinear):
                    yield f"blk.{i}.{stems[t]}", m

    def adapters(self) -> list:
        return [p for _, m in self._pairs() for p in (m.lora_a, m.lora_b)]

    def write_adapter(self, path: str, base: str = "", name: str = "") -> None:
        tensors = {}
        for stem, m in self._pairs():
            tensors[stem + ".lora_a"] = m.lora_a._data
            tensors[stem + ".lora_b"] = m.lora_b._data
        md = {"general.type": "adapter", "adapter.type": "lora", "adapter.lora.alpha": float(self.lora["alpha"]),
              "adapter.lora.rank": int(self.lora["rank"]), "adapter.base": base, "general.name": name,
              "general.architecture": self.cfg.arch}
        mim.write_tensors(path, tensors, metadata=md)

    def read_adapter(self, src) -> None:
        f = mim.open(src) if isinstance(src, (str, bytes)) else src
        md = f.metadata
        if md.get("adapter.type") != "lora":
            raise T.ErrUnsupported("llm: not a LoRA adapter file")
        rank, alpha = int(md["adapter.lora.rank"]), float(md["adapter.lora.alpha"])
        stems = {v: k for k, v in self.NAMES}
        targets = sorted({stems[n.split(".")[2]] for n in f.names() if n.endswith(".lora_a")})
        self.add_lora(rank, alpha, targets)
        for stem, m in self._pairs():
            for which in ("lora_a", "lora_b"):
                t = f.tensor(f"{stem}.{which}")
                p = getattr(m, which)
                if tuple(t.shape) != tuple(p.shape):
                    raise T.ErrShape(f"llm: adapter tensor {stem}.{which} of shape {tuple(t.shape)}, want {tuple(p.shape)}")
                p.set(t.clone().to(p.dtype))

    # -------------------------------------------------- tensor-parallel decoding
    def tp_weights(self) -> dict:
        """Weights in the fused layout ``TPDecoder`` takes (qkv and gate|up rows concatenated)."""
        out = {"token_embd": self.embed.weight._data, "output_norm": self.norm.weight._data,
               "output": (self.output.weight if self.output is not None else self.embed.weight)._data}
        for i, b in enumerate(self.blocks):
            w = lambda m: (m.merged_weight() if isinstance(m, nn.LoRALinear) else m.weight._data)  # noqa: E731
            out[f"blk.{i}.qkv"] = torch.cat([w(b.q), w(b.k), w(b.v)], 0)
            out[f"blk.{i}.o"] = w(b.o)
            out[f"blk.{i}.gate_up"] = torch.cat([w(b.gate), w(b.up)], 0)
            out[f"blk.{i}.down"] = w(b.down)
            out[f"blk.{i}.attn_norm"] = b.attn_norm.weight._data
            out[f"blk.{i}.ffn_norm"] = b.mlp_norm.weight._data
        return out
