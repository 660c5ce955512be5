"""Decoding on the host with the weights kept in their block encoding (reference:
llm/decode.go:79-160 recorded CPU decode step with fused QKV and gate / up rows, :188-227 the
products over quantized rows, :330-371 the cache; llm/model.go:216-313 the loader).

``CPUDecoder`` reads a language-model ``.mim`` file (or takes weights directly), leaves every
quantized matrix as the ggml blocks the file holds (Q8_0 / Q4_0 / Q4_K / Q6_K, 0.56 to 1.06 bytes per
weight instead of 4) and runs one token at a time: RMSNorm, the q / k / v rows as ONE product when
their encodings agree (their blocks are simply stacked), rotary embedding in the file's pair or
halves order, attention over a preallocated cache, the gate and up rows as one product, SwiGLU, the
down product and the residuals.  Every product is the native CPU kernel of ``csrc/cpu_quant.cc``
(``mode="int8"``: activations rounded to int8 blocks, VNNI dot products; ``"exact"``: float
activations); matrices a file stores in float take the same path as Q8_0 after one rounding at load
(``float_as="q8_0"``) or stay float (``"f32"``).  The token embedding row is decoded from its blocks;
a tied output head multiplies with the embedding's blocks.
"""
from __future__ import annotations

import math

import threading

import torch

from ..io import mim
from ..ops import quant as Q
from ..ops import quant_cpu
from .model import Config


WIDE_ROWS = 32            # activation rows from which a product expands the weight and runs in bfloat16
_LOCAL = threading.local()


def _scratch(values: int) -> torch.Tensor:
    """This thread's bfloat16 buffer of at least ``values`` elements (it only grows)."""
    buf = getattr(_LOCAL, "buf", None)
    if buf is None or buf.numel() < values:
        buf = _LOCAL.buf = torch.empty(values, dtype=torch.bfloat16)
    return buf


class _Mat:
    """A weight matrix [N, K]: ggml blocks (``code`` != 0) or a float tensor."""

    def __init__(self, code: int, n: int, k: int, data: torch.Tensor):
        self.code, self.n, self.k, self.data = code, n, k, data

    @staticmethod
    def of(t, float_as: str) -> "_Mat":
        if isinstance(t, mim.QuantizedTensor):
            n, k = t.shape
            return _Mat(t.code, n, k, t.raw.reshape(-1).contiguous())
        t = t.float()
        n, k = t.shape
        if float_as == "q8_0" and k % 32 == 0:
            return _Mat(Q.Q8_0, n, k, Q.quantize_q8_0(t).reshape(-1).contiguous())
        return _Mat(0, n, k, t.contiguous())

    def row_bytes(self) -> int:
        vals, nbytes = Q.BLOCK[self.code]
        return self.k // vals * nbytes

    def rows(self, idx: torch.Tensor) -> torch.Tensor:
        """Float rows ``idx`` (the embedding lookup)."""
        if self.code == 0:
            return self.data[idx]
        rb = self.row_bytes()
        raw = self.data.view(self.n, rb)[idx].reshape(-1)
        return Q.dequantize_raw(self.code, raw, idx.numel() * self.k).view(idx.numel(), self.k)

    def mul(self, x: torch.Tensor, mode: str) -> torch.Tensor:
        """``x [B, K] -> [B, N]``.  A few rows (decoding) multiply the blocks as they are; a prompt's many rows
        (``WIDE_ROWS`` or more, unless ``mode`` is "exact") expand the matrix to bfloat16 once into a scratch
        buffer and run one bfloat16 matrix product, which the CPU's matrix units serve: the expansion is paid
        once per chunk of the prompt instead of the blocks being unpacked again for every eight rows."""
        if self.code == 0:
            return x @ self.data.t()
        if x.shape[0] >= WIDE_ROWS and mode != "exact":
            w = quant_cpu.dequant_bf16(self.code, self.data, self.n, self.k, _scratch(self.n * self.k))
            return (x.to(torch.bfloat16) @ w.t()).float()
        return quant_cpu.qgemv(self.code, self.data, self.n, self.k, x, mode)

    @staticmethod
    def stack(mats) -> "_Mat | None":
        """One matrix whose rows are the rows of ``mats``, when they share encoding and width."""
        if len({(m.code, m.k) for m in mats}) != 1:
            return None
        m0 = mats[0]
        data = torch.cat([m.data for m in mats]) if m0.code else torch.cat([m.data for m in mats], 0)
        return _Mat(m0.code, sum(m.n for m in mats), m0.k, data.contiguous())

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()


class CPUDecoder:
    def __init__(self, cfg: Config, tensors: dict, batch: int = 1, cap: int | None = None, mode: str = "auto",
                 float_as: str = "q8_0", rope_freqs: torch.Tensor | None = None, fused_layers: bool = True):
        """``tensors``: file names (``token_embd.weight``, ``blk.N.attn_q.weight`` ...) -> float tensors
        or ``QuantizedTensor``s.  ``fused_layers=False`` keeps single-token steps on the tensor-op path that
        prompts use (the native layer routine is checked against it)."""
        if mode not in ("auto", "int8", "exact"):
            raise ValueError("mode is 'auto', 'int8' or 'exact'")
        self.cfg, self.batch, self.cap = cfg, batch, cap or cfg.context
        self.mode = "exact" if mode == "auto" and not quant_cpu.has_int8() else ("int8" if mode == "auto" else mode)
        c = cfg
        mat = lambda name: _Mat.of(tensors[name], float_as)  # noqa: E731
        self.embed = _Mat.of(tensors["token_embd.weight"], "f32" if not isinstance(tensors["token_embd.weight"], mim.QuantizedTensor) else float_as)
        self.out_norm = tensors["output_norm.weight"].float()
        self.head = mat("output.weight") if "output.weight" in tensors else (
            self.embed if self.embed.code else _Mat.of(tensors["token_embd.weight"], float_as))
        self.layers = []
        for i in range(c.layers):
            p = f"blk.{i}."
            q, k, v = mat(p + "attn_q.weight"), mat(p + "attn_k.weight"), mat(p + "attn_v.weight")
            gate, up = mat(p + "ffn_gate.weight"), mat(p + "ffn_up.weight")
            bias = None
            if p + "attn_q.bias" in tensors:
                bias = torch.cat([tensors[p + f"attn_{s}.bias"].float() for s in "qkv"])
            self.layers.append(dict(
                attn_norm=tensors[p + "attn_norm.weight"].float(), ffn_norm=tensors[p + "ffn_norm.weight"].float(),
                qkv=_Mat.stack([q, k, v]), q=q, k=k, v=v, qkv_bias=bias, o=mat(p + "attn_output.weight"),
                gate_up=_Mat.stack([gate, up]), gate=gate, up=up, down=mat(p + "ffn_down.weight")))
        d = c.rope_dim
        inv = 1.0 / (c.rope_base ** (torch.arange(0, d, 2).float() / d))
        if c.rope_scale != 1.0:
            inv = inv / c.rope_scale
        if rope_freqs is not None:
            inv = inv / rope_freqs.float()
        self.inv_freq = inv
        self.interleaved = c.arch == "llama"
        # products of block-encoded matrices run on the native worker pool; float matrices use PyTorch's
        self.own_threads = all(l[k].code != 0 for l in self.layers for k in ("q", "k", "v", "o", "gate", "up", "down"))
        self.kc = torch.zeros(c.layers, batch, c.kv_heads, self.cap, c.head_dim)
        self.vc = torch.zeros_like(self.kc)
        self.len = 0
        # one native call per layer when every product reads blocks and the q / k / v and gate / up rows are fused
        self.fused_layers = fused_layers and self.own_threads and batch <= quant_cpu.MAX_ROWS and all(
            l["qkv"] is not None and l["gate_up"] is not None for l in self.layers)
        self._args = None

    # ------------------------------------------------------------------ construction
    @staticmethod
    def load(src, **kw) -> "CPUDecoder":
        """From a ``.mim`` language-model file; quantized tensors stay as the file has them."""
        f = mim.open(src) if isinstance(src, (str, bytes)) or hasattr(src, "__fspath__") else src
        cfg = Config.from_metadata(f.metadata)
        cfg.vocab = int(f.info("token_embd.weight")[1][0])
        tensors = {}
        for name in f.names():
            t = f.tensor(name)
            tensors[name] = mim.QuantizedTensor(t.code, t.shape, t.raw.clone()) if isinstance(t, mim.QuantizedTensor) else t.clone()
        return CPUDecoder(cfg, tensors, rope_freqs=tensors.get("rope_freqs.weight"), **kw)

    @staticmethod
    def from_model(model, **kw) -> "CPUDecoder":
        """From an ``llm.Model`` (float weights)."""
        return CPUDecoder(model.cfg, {n: p._data for n, p in model._file_tensors()}, **kw)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for m in [self.embed, self.head] + [l[k] for l in self.layers for k in ("q", "k", "v", "o", "gate", "up", "down")]:
            if id(m) not in seen:
                seen.add(id(m))
                total += m.nbytes()
        return total

    # ------------------------------------------------------------------ one step
    def reset(self) -> None:
        self.len = 0

    def _rope(self, x: torch.Tensor, pos: int) -> torch.Tensor:
        """``x [B, T, H, D]`` rotated for positions ``pos .. pos + T - 1``."""
        d = self.cfg.rope_dim
        ang = (torch.arange(pos, pos + x.shape[1], dtype=torch.float32)[:, None] * self.inv_freq[None])[None, :, None, :]
        cos, sin = ang.cos(), ang.sin()
        rot, rest = x[..., :d], x[..., d:]
        if self.interleaved:
            a, b = rot[..., 0::2], rot[..., 1::2]
            out = torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)
        else:
            a, b = rot[..., : d // 2], rot[..., d // 2:]
            out = torch.cat([a * cos - b * sin, a * sin + b * cos], -1)
        return torch.cat([out, rest], -1) if rest.shape[-1] else out

    def _norm(self, x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * g

    def _own_thread(self, fn, *a):
        """Runs ``fn`` with PyTorch's thread pool set to one thread: the small tensor ops between the
        products run on the calling thread, because PyTorch's workers would compete with the product
        workers for the same cores."""
        if not self.own_threads:
            return fn(*a)
        had = torch.get_num_threads()
        torch.set_num_threads(1)
        try:
            return fn(*a)
        finally:
            torch.set_num_threads(had)

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """One token per sequence: ``tokens [B]`` -> logits ``[B, vocab]``; the cache grows by one."""
        if self.fused_layers:
            return self._step_native(tokens.reshape(self.batch))
        return self._own_thread(self._forward, tokens.reshape(self.batch, 1))

    def _layer_args(self):
        """The argument block of each layer (addresses of weights and caches do not change between steps)."""
        if self._args is None:
            c, B = self.cfg, self.batch
            self._x = torch.empty(B, c.embed)
            self._work = torch.empty(quant_cpu.decode_scratch(B, c.embed, c.heads, c.kv_heads, c.head_dim, c.hidden, self.cap))
            self._args = []
            for li, l in enumerate(self.layers):
                a = quant_cpu.DecodeLayer(
                    B=B, E=c.embed, H=c.heads, Hk=c.kv_heads, D=c.head_dim, hidden=c.hidden, rope_dim=c.rope_dim,
                    interleaved=int(self.interleaved), pos=0, cap=self.cap, mode=quant_cpu._MODES[self.mode],
                    qkv_code=l["qkv"].code, o_code=l["o"].code, gate_up_code=l["gate_up"].code, down_code=l["down"].code,
                    eps=float(c.eps), attn_norm=l["attn_norm"].data_ptr(), ffn_norm=l["ffn_norm"].data_ptr(),
                    qkv_bias=l["qkv_bias"].data_ptr() if l["qkv_bias"] is not None else None,
                    inv_freq=self.inv_freq.data_ptr(), qkv=l["qkv"].data.data_ptr(), o=l["o"].data.data_ptr(),
                    gate_up=l["gate_up"].data.data_ptr(), down=l["down"].data.data_ptr(),
                    k_cache=self.kc[li].data_ptr(), v_cache=self.vc[li].data_ptr(), x=self._x.data_ptr(),
                    scratch=self._work.data_ptr())
                self._args.append(a)
        return self._args

    def _step_native(self, tokens: torch.Tensor) -> torch.Tensor:
        pos = self.len
        if pos + 1 > self.cap:
            raise IndexError(f"KV cache overflow: {pos} + 1 > {self.cap}")
        args = self._layer_args()
        self._x.copy_(self.embed.rows(tokens.long()))
        for a in args:
            a.pos = pos
            quant_cpu.decode_layer(a)
        self.len = pos + 1
        return self.head.mul(self._own_thread(self._norm, self._x, self.out_norm), self.mode)

    def _forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """``tokens [B, T]`` at positions ``len .. len + T - 1`` -> logits of the last one ``[B, vocab]``.
        The products see ``B * T`` activation rows, eight per pass over a weight matrix."""
        c, B, pos = self.cfg, self.batch, self.len
        Tn = tokens.shape[1]
        if pos + Tn > self.cap:
            raise IndexError(f"KV cache overflow: {pos} + {Tn} > {self.cap}")
        H, Hk, D = c.heads, c.kv_heads, c.head_dim
        x = self.embed.rows(tokens.reshape(-1).long())                       # [B * T, embed]
        scale = 1.0 / math.sqrt(D)
        mask = None
        if Tn > 1:
            i, j = torch.arange(Tn)[:, None], torch.arange(pos + Tn)[None]
            mask = torch.zeros(Tn, pos + Tn).masked_fill(j > i + pos, float("-inf"))
        for li, l in enumerate(self.layers):
            h = self._norm(x, l["attn_norm"])
            if l["qkv"] is not None:
                qkv = l["qkv"].mul(h, self.mode)
            else:
                qkv = torch.cat([l["q"].mul(h, self.mode), l["k"].mul(h, self.mode), l["v"].mul(h, self.mode)], 1)
            if l["qkv_bias"] is not None:
                qkv = qkv + l["qkv_bias"]
            q, k, v = qkv.split([H * D, Hk * D, Hk * D], 1)
            q = self._rope(q.view(B, Tn, H, D), pos)
            k = self._rope(k.view(B, Tn, Hk, D), pos)
            self.kc[li, :, :, pos: pos + Tn] = k.transpose(1, 2)
            self.vc[li, :, :, pos: pos + Tn] = v.view(B, Tn, Hk, D).transpose(1, 2)
            keys, vals = self.kc[li, :, :, : pos + Tn], self.vc[li, :, :, : pos + Tn]     # [B, Hk, S, D]
            qg = q.permute(0, 2, 1, 3).reshape(B, Hk, (H // Hk) * Tn, D)                # the heads of a group side by side
            att = torch.matmul(qg, keys.transpose(-1, -2)) * scale                       # [B, Hk, G * T, S]
            if mask is not None:
                att = att.view(B, Hk, H // Hk, Tn, pos + Tn) + mask
            att = torch.softmax(att, -1).view(B, Hk, (H // Hk) * Tn, pos + Tn)
            o = torch.matmul(att, vals).view(B, H, Tn, D).permute(0, 2, 1, 3).reshape(B * Tn, H * D)
            x = x + l["o"].mul(o, self.mode)
            h = self._norm(x, l["ffn_norm"])
            if l["gate_up"] is not None:
                g, u = l["gate_up"].mul(h, self.mode).split([c.hidden, c.hidden], 1)
            else:
                g, u = l["gate"].mul(h, self.mode), l["up"].mul(h, self.mode)
            x = x + l["down"].mul(torch.nn.functional.silu(g) * u, self.mode)
        self.len = pos + Tn
        last = x.view(B, Tn, -1)[:, -1]
        return self.head.mul(self._norm(last, self.out_norm), self.mode)

    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor, chunk: int = 256) -> torch.Tensor:
        """Feeds ``prompt [B, T]`` in chunks of ``chunk`` positions (a chunk of 32 rows or more expands each
        weight matrix once and multiplies in bfloat16; smaller ones read the blocks once per eight rows);
        returns the logits after the last token."""
        logits = None
        for t0 in range(0, prompt.shape[1], chunk):
            part = prompt[:, t0: t0 + chunk]
            if part.shape[0] * part.shape[1] >= WIDE_ROWS and self.mode != "exact":
                logits = self._forward(part)          # wide products are PyTorch's: they need its threads
            else:
                logits = self._own_thread(self._forward, part)
        return logits

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n: int, sampler=None) -> torch.Tensor:
        """``prompt [B, T]`` -> ``[B, n]`` new tokens (greedy, or drawn by ``sampler``)."""
        logits = self.prefill(prompt)
        out = []
        for _ in range(n):
            if sampler is None:
                nxt = logits.argmax(-1)
            else:
                nxt = torch.tensor([int(sampler.sample(logits[b], [int(o[b]) for o in out])) for b in range(logits.shape[0])])
            out.append(nxt)
            logits = self.step(nxt)
        return torch.stack(out, 1) if out else torch.zeros(prompt.shape[0], 0, dtype=torch.int64)
