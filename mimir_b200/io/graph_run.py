"""Interpreter of ``io.graph`` programs: the 33 primitives, the standard-library composites and
sessions with variables (reference: io/mim/ops.go:282-392, io/mim/stdlib.go:33-640,
io/mim/session.go:48-252).

A run binds the symbolic dimensions from the inputs (one size per symbol, at most its bound),
walks the main program in order and checks every output of every op against its declared
shape and dtype.  Float composites compute in fp32 and cast to the declared type.  Nothing is
recorded for autograd: a run is inference.
"""
from __future__ import annotations

import math
import os
import threading

import torch
import torch.nn.functional as F

from ..tensor import errors as E
from . import graph as G

_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def _is_float(dt) -> bool:
    return dt in _FLOATS


class _Call:
    """One op being run: its inputs, its attributes and the declared types of its outputs."""

    def __init__(self, run: "_Run", op: G.Op, ins):
        self.run, self.op, self.ins = run, op, ins

    def attr(self, key, default=None):
        return self.op.attrs.get(key, default)

    def int(self, key, default=0) -> int:
        v = self.op.attrs.get(key, default)
        if isinstance(v, bool) or not isinstance(v, int):
            raise G.FormatError(f"{self.name}: attribute {key!r} is not an integer")
        return v

    def ints(self, key, default=None):
        v = self.op.attrs.get(key, default)
        if v is None:
            return None
        if isinstance(v, list) and any(isinstance(i, G.Sym) for i in v):
            # a symbolic dimension in an integer list (the end of a shrink over a sequence axis):
            # takes the size the symbol was bound to by this run's inputs
            out = []
            for i in v:
                if isinstance(i, G.Sym):
                    if i.name not in self.run.syms:
                        raise G.FormatError(f"{self.name}: attribute {key!r} uses symbol {i.name!r} before it is known")
                    i = self.run.syms[i.name]
                out.append(i)
            v = out
        if not isinstance(v, list) or any(isinstance(i, bool) or not isinstance(i, int) for i in v):
            raise G.FormatError(f"{self.name}: attribute {key!r} is not a list of integers")
        return v

    def float(self, key, default=0.0) -> float:
        v = self.op.attrs.get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise G.FormatError(f"{self.name}: attribute {key!r} is not a number")
        return float(v)

    def bool(self, key, default=False) -> bool:
        v = self.op.attrs.get(key, default)
        if isinstance(v, int) and v in (0, 1):      # the binary encoding stores flags as integers
            return bool(v)
        if not isinstance(v, bool):
            raise G.FormatError(f"{self.name}: attribute {key!r} is not a bool")
        return v

    def str(self, key, default="") -> str:
        v = self.op.attrs.get(key, default)
        if not isinstance(v, str):
            raise G.FormatError(f"{self.name}: attribute {key!r} is not a string")
        return v

    @property
    def name(self) -> str:
        return f"call {self.op.attrs.get('name')}" if self.op.opcode == "call" else self.op.opcode

    def axis(self, key, default, rank) -> int:
        a = self.int(key, default)
        if not -rank <= a < max(rank, 1):
            raise G.FormatError(f"{self.name}: axis {a} of rank {rank}")
        return a % max(rank, 1)

    def out_dtype(self, i=0):
        return G.DTYPES[self.run.g.values[self.op.outputs[i]].dtype]

    def out_shape(self, i=0, like=None):
        return self.run.declared(self.op.outputs[i], like)

    def f32(self, i):
        t = self.ins[i]
        return t.float() if _is_float(t.dtype) and t.dtype != torch.float64 else t

    def need(self, lo, hi):
        if not lo <= len(self.ins) <= hi:
            raise G.FormatError(f"{self.name}: {len(self.ins)} inputs, want {lo} to {hi}")


# =============================================================================================
# primitives
# =============================================================================================

def _trunc(t):
    return torch.trunc(t) if _is_float(t.dtype) else t


def _cast(t, to):
    if to == torch.bool:
        return t != 0
    if _is_float(t.dtype) and not _is_float(to):
        t = torch.trunc(torch.nan_to_num(t, nan=0.0))    # float -> int rounds toward zero, NaN -> 0
        info = torch.iinfo(to)
        return t.clamp(info.min, info.max).to(to)
    return t.to(to)


def _idiv(a, b, rem):
    if _is_float(a.dtype):
        q = torch.trunc(a / b)
        return a - q * b if rem else q
    if bool((b == 0).any()):
        raise E.ErrDivideByZero("graph: integer division by zero")
    q = torch.div(a, b, rounding_mode="trunc")
    return a - q * b if rem else q


def _gather(c, data, idx, axis):
    n = data.shape[axis]
    flat = idx.reshape(-1).long().clamp(0, max(n - 1, 0))
    out = data.index_select(axis, flat)
    return out.reshape(*data.shape[:axis], *idx.shape, *data.shape[axis + 1:])


def _scatter(c, data, idx, updates, axis):
    n = data.shape[axis]
    flat = idx.reshape(-1).long().clamp(0, max(n - 1, 0))
    shape = list(data.shape)
    shape[axis] = flat.numel()
    upd = updates.reshape(shape).to(data.dtype)
    if c.run.may_overwrite(c.op.inputs[0]):
        out, c.run.wrote = data, True
    else:
        out = data.clone()
    n_pos = flat.numel()
    if 1 < n_pos <= 4096:
        # repeated positions: every copy of a position writes the slice of its LAST occurrence, so the
        # result does not depend on the order of the writes (and nothing is read back on the host)
        same = flat[:, None] == flat[None, :]
        order = torch.arange(n_pos, device=flat.device)
        winner = torch.where(same, order[None, :], order.new_zeros(())).amax(1)
        return out.index_copy_(axis, flat, upd.index_select(axis, winner))
    if n_pos > 1:
        if torch.cuda.is_available() and flat.is_cuda and torch.cuda.is_current_stream_capturing():
            raise E.ErrUnsupported("graph: a scatter of more than 4096 positions is not recorded")
        if flat.unique().numel() != n_pos:
            for j in range(n_pos):             # repeated positions: the last one wins, in order
                out.index_copy_(axis, flat[j:j + 1], upd.narrow(axis, j, 1))
            return out
    return out.index_copy_(axis, flat, upd)


def _reduce(c, x):
    axes = c.ints("axes", []) or []
    if not axes:
        return x
    for a in axes:
        if not 0 <= a < x.dim():
            raise G.FormatError(f"reduce over axis {a} of rank {x.dim()}")
    mode = c.str("mode")
    if mode == "add":
        return x.sum(dim=axes, keepdim=True, dtype=x.dtype if x.dtype != torch.bool else torch.int32)
    if mode == "max":
        return x.amax(dim=axes, keepdim=True)
    if mode == "mul":
        for a in axes:
            x = x.prod(dim=a, keepdim=True, dtype=x.dtype)
        return x
    raise G.FormatError(f"reduce mode {mode!r}")


def _pow(a, b):
    if not _is_float(a.dtype) and bool((b < 0).any()):
        raise E.ErrUnsupported("graph: integer power with a negative exponent")
    return torch.pow(a, b)


def _eval_primitive(c: _Call):
    i, code = c.ins, c.op.opcode
    if code == "neg":
        return [-i[0]]
    if code == "recip":
        return [torch.reciprocal(i[0])]
    if code == "sqrt":
        return [torch.sqrt(i[0])]
    if code == "exp2":
        return [torch.exp2(i[0])]
    if code == "log2":
        return [torch.log2(i[0])]
    if code == "sin":
        return [torch.sin(i[0])]
    if code == "trunc":
        return [_trunc(i[0])]
    if code == "cast":
        to = c.attr("to")
        if not isinstance(to, torch.dtype):
            raise G.FormatError("cast without a dtype to cast to")
        return [_cast(i[0], to)]
    if code == "add":
        return [i[0] + i[1]]
    if code in ("mul", "and"):
        return [i[0] * i[1]]
    if code in ("max", "or"):
        return [torch.maximum(*torch.broadcast_tensors(i[0], i[1]))]
    if code == "pow":
        return [_pow(i[0], i[1])]
    if code in ("idiv", "imod"):
        return [_idiv(i[0], i[1], code == "imod")]
    if code in ("shl", "shr"):
        if _is_float(i[0].dtype) or i[0].dtype == torch.bool:
            raise E.ErrDType(f"graph: {code} of {i[0].dtype}")
        sh = i[1].to(i[0].dtype)
        return [torch.bitwise_left_shift(i[0], sh) if code == "shl" else torch.bitwise_right_shift(i[0], sh)]
    if code == "bitcast":
        to = c.attr("to")
        if not isinstance(to, torch.dtype) or to == torch.bool or i[0].dtype == torch.bool:
            raise G.FormatError("bitcast without a numeric dtype to reinterpret as")
        if torch.empty((), dtype=to).element_size() != i[0].element_size():
            raise E.ErrDType(f"graph: bitcast from {i[0].dtype} to {to} changes the width")
        return [i[0].contiguous().view(to)]
    if code == "xor":
        return [(i[0] != i[1]).to(i[0].dtype)]
    if code == "cmplt":
        return [(i[0] < i[1]).to(torch.int32)]
    if code == "cmpeq":
        return [(i[0] == i[1]).to(torch.int32)]
    if code == "where":
        return [torch.where(i[0] != 0, i[1], i[2])]
    if code == "reduce":
        return [_reduce(c, i[0])]
    if code == "reshape":
        return [i[0].reshape(c.out_shape(0, like=i[0]))]
    if code == "expand":
        return [i[0].expand(c.out_shape(0, like=i[0]))]
    if code == "permute":
        perm = c.ints("perm")
        if perm is None or sorted(perm) != list(range(i[0].dim())):
            raise G.FormatError(f"permute {perm} of rank {i[0].dim()}")
        return [i[0].permute(perm)]
    if code == "pad":
        pads = c.ints("pads")
        if pads is None or len(pads) != 2 * i[0].dim():
            raise G.FormatError(f"{0 if pads is None else len(pads)} pads for rank {i[0].dim()}")
        flat = []
        for d in reversed(range(i[0].dim())):
            flat += [pads[2 * d], pads[2 * d + 1]]
        x = i[0]
        if x.dtype == torch.bool:
            return [F.pad(x.to(torch.uint8), flat, value=c.float("value", 0.0)).bool()]
        return [F.pad(x, flat, value=c.float("value", 0.0))]
    if code == "shrink":
        begin, end = c.ints("begin"), c.ints("end")
        x = i[0]
        if begin is None or end is None or len(begin) != x.dim() or len(end) != x.dim():
            raise G.FormatError(f"shrink begins / ends do not match rank {x.dim()}")
        for d, (lo, hi) in enumerate(zip(begin, end)):
            hi = x.shape[d] if hi == -1 else hi
            if not 0 <= lo <= hi <= x.shape[d]:
                raise E.ErrShape(f"graph: shrink [{lo}, {hi}) of a dimension of {x.shape[d]}")
            x = x.narrow(d, lo, hi - lo)
        return [x]
    if code == "gather":
        return [_gather(c, i[0], i[1], c.axis("axis", 0, i[0].dim()))]
    if code == "scatter":
        return [_scatter(c, i[0], i[1], i[2], c.axis("axis", 0, i[0].dim()))]
    if code == "const":
        v = c.attr("value")
        if v is None or isinstance(v, (str, list, dict)):
            raise G.FormatError("const without a value")
        dt = c.out_dtype(0)
        if not _is_float(dt) and dt != torch.bool and isinstance(v, int):
            info = torch.iinfo(dt)
            if not info.min <= v <= info.max:
                raise E.ErrUnsupported(f"graph: const {v} does not fit in {dt}")
        return [torch.full(c.out_shape(0), v, dtype=dt, device=c.run.device)]
    if code == "dequantize":
        return [i[0].float()]
    if code == "call":
        return _composite(c)
    if code == "while":
        return _while(c)
    if code == "if":
        return _if(c)
    raise E.ErrUnsupported(f"graph: opcode {code!r}")


def _sub(c: _Call, key) -> G.Subgraph:
    ref = c.attr(key)
    if not isinstance(ref, G.SubgraphRef):
        raise G.FormatError(f"{c.name}: no subgraph {key}")
    return c.run.g.subgraphs[ref.index]


def _truth(c, sg, vals) -> bool:
    out = c.run.subgraph(sg, vals)
    if len(out) != 1 or out[0].numel() != 1:
        raise G.FormatError("a condition must have one scalar output")
    return bool(out[0].reshape(()).item() != 0)


def _while(c):
    cond, body = _sub(c, "cond"), _sub(c, "body")
    vals = list(c.ins)
    limit = c.int("max_iterations", 1 << 31)
    n = 0
    while _truth(c, cond, vals):
        vals = c.run.subgraph(body, vals)
        n += 1
        if n >= limit:
            raise E.ErrUnsupported(f"graph: while ran its limit of {limit} iterations")
        c.run.check_cancel()
    return vals


def _if(c):
    then, other = _sub(c, "then"), _sub(c, "else")
    pred = c.ins[0]
    if pred.numel() != 1:
        raise G.FormatError("if: the predicate is not a scalar")
    return c.run.subgraph(then if pred.reshape(()).item() != 0 else other, list(c.ins[1:]))


# =============================================================================================
# standard library
# =============================================================================================

def _composite(c: _Call):
    name = c.str("name")
    own = c.run.g.composites.get(name)
    if own is not None:
        return c.run.subgraph(c.run.g.subgraphs[own], list(c.ins))
    fn = G.STDLIB.get(name)
    if fn is None:
        raise E.ErrUnsupported(f"graph: call of {name!r}")
    return fn(c)


def _unary(f):
    def run(c):
        c.need(1, 1)
        return [f(c.f32(0))]
    return run


def _matmul(c):
    c.need(2, 2)
    return [torch.matmul(c.f32(0), c.f32(1))]


def _bias(c, y, i):
    return y + c.f32(i) if len(c.ins) > i else y


def _linear(c):
    c.need(2, 3)
    return [_bias(c, torch.matmul(c.f32(0), c.f32(1).transpose(-1, -2)), 2)]


def _round_q8_blocks(x):
    """Rounds activations the way a W4A8 / W8A8 product does: blocks of 32 along the last axis, one
    fp16 scale per block, 8-bit values."""
    k = x.shape[-1]
    if k % 32:
        raise E.ErrShape(f"graph: dequant_matmul_a8 over an inner dimension of {k}, not a multiple of 32")
    b = x.reshape(*x.shape[:-1], k // 32, 32)
    amax = b.abs().amax(-1, keepdim=True)
    d = (amax / 127.0).half().float()
    q = torch.where(d > 0, torch.round(b / torch.where(d > 0, d, torch.ones_like(d))), torch.zeros_like(b))
    return (q.clamp(-127, 127) * d).reshape(x.shape)


def _dequant_matmul(a8):
    def run(c):
        c.need(2, 3)
        x, w = c.f32(0), c.f32(1)     # the environment hands block-quantized weights over dequantized
        if a8:
            x = _round_q8_blocks(x)
        return [_bias(c, torch.matmul(x, w.transpose(-1, -2)), 2)]
    return run


def _conv2d(c):
    c.need(2, 3)
    stride = c.ints("strides", [1, 1])
    dil = c.ints("dilations", [1, 1])
    pads = c.ints("pads", [0, 0, 0, 0])          # top, bottom, left, right (io/mim/stdlib.go:208)
    groups = c.int("groups", 1)
    x, w = c.f32(0), c.f32(1)
    if len(pads) != 4 or len(stride) != 2 or len(dil) != 2:
        raise G.FormatError("conv2d: strides / dilations of 2 and pads of 4 values")
    top, bottom, left, right = pads
    if top != bottom or left != right:
        x = F.pad(x, [left, right, top, bottom])
        pad = (0, 0)
    else:
        pad = (top, left)
    b = c.f32(2) if len(c.ins) > 2 else None
    return [F.conv2d(x, w, b, stride=tuple(stride), padding=pad, dilation=tuple(dil), groups=groups)]


def _swiglu(c):
    c.need(2, 2)
    return [F.silu(c.f32(0)) * c.f32(1)]


def _geglu(c):
    c.need(2, 2)
    approx = "tanh" if c.str("approximate", "tanh") == "tanh" else "none"
    return [F.gelu(c.f32(0), approximate=approx) * c.f32(1)]


def _softmax(log):
    def run(c):
        c.need(1, 1)
        x = c.f32(0)
        a = c.axis("axis", -1, x.dim())
        return [F.log_softmax(x, a) if log else F.softmax(x, a)]
    return run


def _axes_of(c, rank):
    axes = c.ints("axes", None)
    if axes is None:
        return [rank - 1]
    out = []
    for a in axes:
        if not -rank <= a < rank:
            raise G.FormatError(f"{c.name}: axis {a} of rank {rank}")
        out.append(a % rank)
    return out


def _layer_norm(c):
    c.need(1, 3)
    x = c.f32(0)
    axes = _axes_of(c, x.dim())
    mu = x.mean(dim=axes, keepdim=True)
    var = (x - mu).pow(2).mean(dim=axes, keepdim=True)
    y = (x - mu) * torch.rsqrt(var + c.float("eps", 1e-5))
    if len(c.ins) > 1:
        y = y * c.f32(1)
    if len(c.ins) > 2:
        y = y + c.f32(2)
    return [y]


def _rms_norm(c):
    c.need(1, 2)
    x = c.f32(0)
    axes = _axes_of(c, x.dim())
    y = x * torch.rsqrt(x.pow(2).mean(dim=axes, keepdim=True) + c.float("eps", 1e-6))
    if c.bool("round_before_scale", False):
        y = y.to(c.ins[0].dtype).float()
    if len(c.ins) > 1:
        y = y * c.f32(1)
    return [y]


def _mean(c):
    c.need(1, 1)
    x = c.f32(0)
    return [x.mean(dim=_axes_of(c, x.dim()), keepdim=c.bool("keepdims", True))]


def _variance(c):
    c.need(1, 1)
    x = c.f32(0)
    return [x.var(dim=_axes_of(c, x.dim()), keepdim=c.bool("keepdims", True), correction=c.int("correction", 0))]


def _cumsum(c):
    c.need(1, 1)
    x = c.ins[0]
    a = c.axis("axis", -1, x.dim())
    rev, excl = c.bool("reverse", False), c.bool("exclusive", False)
    if rev:
        x = x.flip(a)
    y = torch.cumsum(x, a, dtype=x.dtype)
    if excl:
        y = y - x
    return [y.flip(a) if rev else y]


def _rope(c):
    """x [..., T, D], positions [T] or broadcastable to x's leading axes + [T]."""
    c.need(2, 2)
    x, pos = c.f32(0), c.ins[1]
    d = x.shape[-1]
    rot = c.int("rotary_dim", d)
    if rot % 2 or rot > d:
        raise G.FormatError(f"rope: rotary_dim {rot} of a head of {d}")
    base = c.float("base", 10000.0)
    inv = base ** (-torch.arange(0, rot, 2, device=x.device, dtype=torch.float32) / rot)
    ang = pos.float().unsqueeze(-1) * inv * c.float("scale", 1.0)
    cos, sin = torch.cos(ang), torch.sin(ang)
    xr, rest = x[..., :rot], x[..., rot:]
    if c.bool("interleaved", False):
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
    else:
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return [torch.cat([out, rest], dim=-1) if rot < d else out]


def _attention(v2):
    def run(c):
        """q [B, Hq, Tq, D], k / v [B, Hkv, Tk, D] (Hq a multiple of Hkv), optional additive or 0-1 mask
        broadcastable to [B, Hq, Tq, Tk]; version 2 adds ``softcap`` and per-head ``sinks``."""
        c.need(3, 5 if v2 else 4)
        q, k, v = c.f32(0), c.f32(1), c.f32(2)
        mask = c.ins[3] if len(c.ins) > 3 else None
        sinks = c.f32(4) if v2 and len(c.ins) > 4 else None
        hq, hkv = q.shape[-3], k.shape[-3]
        if hq % hkv:
            raise E.ErrShape(f"graph: attention with {hq} query heads over {hkv} key heads")
        if hq != hkv:
            k = k.repeat_interleave(hq // hkv, dim=-3)
            v = v.repeat_interleave(hq // hkv, dim=-3)
        scale = c.float("scale", 0.0) or 1.0 / math.sqrt(q.shape[-1])
        s = torch.matmul(q, k.transpose(-1, -2)) * scale
        cap = c.float("softcap", 0.0) if v2 else 0.0
        if cap > 0:
            s = torch.tanh(s / cap) * cap
        tq, tk = s.shape[-2], s.shape[-1]
        if c.bool("causal", False):
            keep = torch.ones(tq, tk, dtype=torch.bool, device=s.device).tril(tk - tq)
            s = s.masked_fill(~keep, float("-inf"))
        if mask is not None:
            if _is_float(mask.dtype):
                s = s + mask.float()
            else:
                s = s.masked_fill(mask == 0, float("-inf"))
        if sinks is not None:
            sink = sinks.reshape(1, hq, 1, 1).expand(s.shape[0], hq, tq, 1)
            p = torch.softmax(torch.cat([s, sink], dim=-1), dim=-1)[..., :tk]
        else:
            p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)      # a fully masked row attends to nothing
        return [torch.matmul(p, v)]
    return run


def _embedding(c):
    c.need(2, 2)
    table, idx = c.ins[0], c.ins[1]
    return [_gather(c, table, idx, 0)]


def _top_k(c):
    c.need(1, 1)
    x = c.ins[0]
    a = c.axis("axis", -1, x.dim())
    k = c.int("k", 1)
    if not 0 < k <= x.shape[a]:
        raise E.ErrShape(f"graph: top_k of {k} along a dimension of {x.shape[a]}")
    vals, idx = torch.topk(x, k, dim=a, largest=c.bool("largest", True), sorted=True)
    return [vals, idx]


def _argsort(c):
    c.need(1, 1)
    x = c.ins[0]
    return [torch.argsort(x, dim=c.axis("axis", -1, x.dim()), descending=c.bool("descending", False), stable=True)]


def _gelu_erf(x):
    return F.gelu(x, approximate="none")


G.STDLIB.update({
    "matmul.v1": _matmul,
    "linear.v1": _linear,
    "dequant_matmul.v1": _dequant_matmul(False),
    "dequant_matmul_a8.v1": _dequant_matmul(True),
    "dequant_matmul_a8.v2": _dequant_matmul(True),
    "conv2d.v1": _conv2d,
    "sigmoid.v1": _unary(torch.sigmoid),
    "tanh.v1": _unary(torch.tanh),
    "erf.v1": _unary(torch.erf),
    "exp.v1": _unary(torch.exp),
    "log.v1": _unary(torch.log),
    "cos.v1": _unary(torch.cos),
    "rsqrt.v1": _unary(torch.rsqrt),
    "silu.v1": _unary(F.silu),
    "gelu_erf.v1": _unary(_gelu_erf),
    "gelu_tanh.v1": _unary(lambda x: F.gelu(x, approximate="tanh")),
    "swiglu.v1": _swiglu,
    "geglu.v1": _geglu,
    "softmax.v1": _softmax(False),
    "log_softmax.v1": _softmax(True),
    "layer_norm.v1": _layer_norm,
    "rms_norm.v1": _rms_norm,
    "mean.v1": _mean,
    "variance.v1": _variance,
    "cumsum.v1": _cumsum,
    "rope.v1": _rope,
    "attention.v1": _attention(False),
    "attention.v2": _attention(True),
    "embedding.v1": _embedding,
    "top_k.v1": _top_k,
    "argsort.v1": _argsort,
})


# =============================================================================================
# runs and sessions
# =============================================================================================

class _Run:
    def __init__(self, program: "Program", device, cancel=None):
        self.p, self.g, self.device = program, program.g, device
        self.env = [None] * len(self.g.values)
        self.syms: dict = {}
        self.cancel = cancel
        self.owned: set = set()      # variable values this run may overwrite in place
        self.wrote = False           # set once a variable's memory was written

    def check_cancel(self):
        if self.cancel is not None and self.cancel():
            raise E.MimirError("graph: run cancelled")

    def may_overwrite(self, vi: int) -> bool:
        return vi in self.owned

    def bind(self, vi: int, shape) -> None:
        v = self.g.values[vi]
        if len(shape) != len(v.dims):
            raise E.ErrShape(f"graph: {v.name!r} has rank {len(shape)}, declared {len(v.dims)}")
        for d, s in zip(v.dims, shape):
            if isinstance(d, int):
                if d != s:
                    raise E.ErrShape(f"graph: {v.name!r} has shape {tuple(shape)}, declared {self._show(v)}")
            else:
                if s > d.bound:
                    raise E.ErrShape(f"graph: {v.name!r}: dimension {d.name} = {s} is above its bound {d.bound}")
                if self.syms.setdefault(d.name, s) != s:
                    raise E.ErrShape(f"graph: {v.name!r}: dimension {d.name} = {s}, bound to "
                                     f"{self.syms[d.name]} earlier in the run")

    @staticmethod
    def _show(v):
        return "[" + ", ".join(str(d) if isinstance(d, int) else d.name for d in v.dims) + "]"

    def declared(self, vi: int, like=None):
        """The declared shape with its symbols resolved; one unresolved symbol of a reshape target is
        inferred from the element count of ``like``."""
        v = self.g.values[vi]
        out, unknown = [], []
        for i, d in enumerate(v.dims):
            if isinstance(d, int):
                out.append(d)
            elif d.name in self.syms:
                out.append(self.syms[d.name])
            else:
                out.append(-1)
                unknown.append(i)
        if unknown:
            if like is None or len(unknown) > 1:
                raise E.ErrShape(f"graph: {v.name!r}: dimension(s) of {self._show(v)} are not bound")
            known = math.prod(d for d in out if d != -1)
            if known == 0 or like.numel() % known:
                raise E.ErrShape(f"graph: {v.name!r}: {like.numel()} elements do not fill {self._show(v)}")
            out[unknown[0]] = like.numel() // known
        return out

    def subgraph(self, sg: G.Subgraph, ins):
        if len(ins) != len(sg.inputs):
            raise G.FormatError(f"subgraph of {len(sg.inputs)} inputs called with {len(ins)}")
        saved = [(vi, self.env[vi]) for vi in sg.inputs]
        for vi, t in zip(sg.inputs, ins):
            self.env[vi] = t
        try:
            self.body(sg)
            return [self._get(vi, "a subgraph output") for vi in sg.outputs]
        finally:
            for vi, t in saved:
                self.env[vi] = t

    def _get(self, vi, what):
        t = self.env[vi]
        if t is None:
            raise G.FormatError(f"{what} reads {self.g.values[vi].name!r} before it is computed")
        return t

    def body(self, sg: G.Subgraph) -> None:
        for op in sg.ops:
            self.check_cancel()
            c = _Call(self, op, [self._get(vi, op.opcode) for vi in op.inputs])
            try:
                outs = _eval_primitive(c)
            except E.MimirError:
                raise
            except (RuntimeError, ValueError, IndexError, TypeError) as exc:
                raise E.classify(exc) from None
            if len(outs) != len(op.outputs):
                raise G.FormatError(f"{c.name}: {len(outs)} outputs, declared {len(op.outputs)}")
            for vi, t in zip(op.outputs, outs):
                v = self.g.values[vi]
                want = G.DTYPES.get(v.dtype)
                if want is None:
                    raise G.FormatError(f"{c.name}: output {v.name!r} declared with the stored-only type {v.dtype}")
                if t.dtype != want:
                    t = _cast(t, want)
                self.bind(vi, tuple(t.shape))
                self.env[vi] = t


class Program:
    """A parsed graph plus its stored tensors; shared by the sessions of a model."""

    def __init__(self, g: G.Graph, fetch):
        """``fetch(name)`` returns a stored tensor (torch tensor or ``QuantizedTensor``)."""
        self.g, self._fetch = g, fetch
        self._consts: dict = {}      # device -> {value index: tensor}
        self._lock = threading.Lock()
        self.inputs = [g.values[i] for i in g.main.inputs]
        self.outputs = [(n, g.values[i]) for n, i in zip(g.output_names, g.main.outputs)]
        if len(g.output_names) != len(g.main.outputs):
            raise G.FormatError("graph: the main program's outputs and their names differ in number")
        self.replayable = not self._data_dependent()

    def _data_dependent(self) -> bool:
        """True when a run's kernel sequence depends on tensor values (``while`` / ``if``) or an op has to
        look at values on the host (integer division and powers check their operands): such programs
        are never recorded."""
        ints = ("i8", "i16", "i32", "i64", "u8", "bool")
        for sg in self.g.subgraphs:
            for op in sg.ops:
                if op.opcode in ("while", "if"):
                    return True
                if op.opcode in ("idiv", "imod", "pow") and any(self.g.values[i].dtype in ints for i in op.inputs):
                    return True
        return False

    def stored(self, v: G.Value, device):
        from .mim import QuantizedTensor
        t = self._fetch(v.store)
        if isinstance(t, QuantizedTensor):
            return t.dequantize().to(device)     # consumers (dequantize, dequant_matmul, gather) see fp32 values
        return t.to(device)

    def consts_on(self, device):
        with self._lock:
            got = self._consts.get(device)
            if got is None:
                got = {}
                for i, v in enumerate(self.g.values):
                    if v.kind in ("weight", "const"):
                        t = self.stored(v, device)
                        if v.dtype in G.DTYPES and tuple(t.shape) != tuple(d for d in v.dims):
                            raise G.FormatError(f"graph: stored tensor {v.store!r} has shape {tuple(t.shape)}, "
                                                f"declared {v.dims}")
                        got[i] = t
                self._consts[device] = got
            return got

    def new_session(self) -> "Session":
        return Session(self)

    def run(self, inputs: dict, cancel=None) -> dict:
        """One run on fresh variables (reference: Model.Run).  A program without variables keeps one
        session for these calls, so repeated shapes are replayed from their recording."""
        if any(v.kind == "variable" for v in self.g.values):
            return Session(self).run(inputs, cancel=cancel)
        with self._lock:
            if getattr(self, "_stateless", None) is None:
                self._stateless = Session(self)
        return self._stateless.run(inputs, cancel=cancel)


def _to_torch(x):
    from ..tensor.core import Tensor
    if isinstance(x, Tensor):
        if x.err is not None:
            raise x.err
        return x.data()
    if torch.is_tensor(x):
        return x
    raise E.ErrDType(f"graph: an input of type {type(x).__name__} is not a tensor")


class Session:
    """Variables that live from run to run (reference: Session, io/mim/session.go:31-75).

    A run reads the values the previous run left and, once outputs and new values are computed,
    the variables take them.  A run that fails before computing changes nothing.  ``reset`` puts
    the variables back to their initial values.  One run at a time per session.
    """

    def __init__(self, program: Program):
        self.p = program
        self._vars: dict = {}
        self._lock = threading.Lock()
        self._broken = None
        self._recs: dict = {}        # (device, input shapes) -> run count, False, or (graph, inputs, outputs)
        # False (or MIMIR_CUDA_GRAPHS=0) runs every pass plainly on the GPU too
        self.replay = os.environ.get("MIMIR_CUDA_GRAPHS", "1") != "0"

    def reset(self) -> None:
        """Puts the variables back to their initial values (in their buffers, which recordings keep)."""
        with self._lock:
            self._broken = None
            with torch.no_grad():
                for i, cur in self._vars.items():
                    v = self.p.g.values[i]
                    if v.store:
                        cur.copy_(self.p.stored(v, cur.device))
                    else:
                        cur.zero_()

    def run(self, inputs: dict, cancel=None) -> dict:
        from ..tensor.core import from_torch
        with self._lock:
            if self._broken is not None:
                raise E.MimirError(f"graph: the session's variables are unreadable after a failed run "
                                   f"({self._broken}); call reset()")
            ins, device = self._prepare(inputs)
            outs = None
            if device.type == "cuda" and self.replay and cancel is None and self.p.replayable:
                outs = self._run_recorded(ins, device)
            if outs is None:
                outs = self._execute(ins, device, cancel)
            return {n: from_torch(t) for n, t in outs.items()}

    def _prepare(self, inputs: dict):
        p = self.p
        ins = {}
        device = None
        for v in p.inputs:
            if v.name not in inputs:
                raise E.ErrShape(f"graph: input {v.name!r} is missing")
            t = _to_torch(inputs[v.name])
            want = G.DTYPES[v.dtype]
            ints = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)
            if t.dtype != want and t.dtype in ints and want in ints:
                t = t.to(want)      # the reference has one integer type: any integer input fits an integer slot
            if t.dtype != want:
                raise E.ErrDType(f"graph: input {v.name!r} is {t.dtype}, declared {v.dtype}")
            if device is None:
                device = t.device
            elif t.device != device:
                raise E.ErrDevice(f"graph: input {v.name!r} on {t.device}, others on {device}")
            ins[v.name] = t.detach()
        for name in inputs:
            if all(v.name != name for v in p.inputs):
                raise E.ErrShape(f"graph: the model has no input {name!r}")
        if device is None:
            from ..tensor.core import default_device
            device = default_device().torch
        return ins, device

    def _execute(self, ins: dict, device, cancel=None) -> dict:
        """One pass over the main program.  The variables live in buffers that stay where they are for
        the life of the session (a recorded run replays kernels that read and write those addresses):
        a new value is copied into its variable's buffer unless the run computed it there."""
        p, g = self.p, self.p.g
        r = _Run(p, device, cancel)
        for vi, v in zip(g.main.inputs, p.inputs):
            r.bind(vi, tuple(ins[v.name].shape))
            r.env[vi] = ins[v.name]
        for i, t in p.consts_on(device).items():
            r.env[i] = t
        outs_set = set(g.main.outputs)
        for i, v in enumerate(g.values):
            if v.kind != "variable":
                continue
            cur = self._vars.get(i)
            if cur is None or cur.device != device:
                if cur is not None:
                    cur = cur.to(device)
                    self._recs.clear()        # recordings hold the old buffers
                elif v.store:
                    cur = p.stored(v, device).clone()
                else:
                    cur = torch.zeros(r.declared(i), dtype=G.DTYPES[v.dtype], device=device)
                self._vars[i] = cur
            r.bind(i, tuple(cur.shape))
            r.env[i] = cur
            # the old contents may be overwritten when the variable is replaced by a value that is
            # not also an output (a KV cache that a run writes a few rows of)
            nxt = g.updates.get(i)
            if nxt is not None and i not in outs_set and nxt not in outs_set:
                r.owned.add(i)
        try:
            with torch.no_grad():
                r.body(g.main)
                outs = {n: r._get(vi, "an output") for n, vi in zip(g.output_names, g.main.outputs)}
                new = {var: r._get(nxt, "a variable update") for var, nxt in g.updates.items()}
        except BaseException as exc:
            if r.wrote:
                self._broken = type(exc).__name__
            raise
        for var, t in new.items():
            want = self._vars[var]
            if t.shape != want.shape or t.dtype != want.dtype:
                raise E.ErrShape(f"graph: variable {g.values[var].name!r} would change from "
                                 f"{tuple(want.shape)} {want.dtype} to {tuple(t.shape)} {t.dtype}")
        with torch.no_grad():
            var_ptrs = {v.untyped_storage().data_ptr() for v in self._vars.values()}
            # outputs and new values that live in a variable's memory are detached from it first
            outs = {n: (t.clone() if t.untyped_storage().data_ptr() in var_ptrs else t) for n, t in outs.items()}
            staged = {var: (None if t is self._vars[var] else
                            t.clone() if t.untyped_storage().data_ptr() in var_ptrs else t) for var, t in new.items()}
            for var, t in staged.items():
                if t is not None:
                    self._vars[var].copy_(t)
        return outs

    def _run_recorded(self, ins: dict, device):
        """Recording and replay per input shape (reference: io/mim/replay.go:60-130).  The first run of a
        shape is a plain pass; the second is captured into a CUDA graph over fixed input, output and
        variable buffers; later runs copy the inputs in, replay, and copy the outputs out.  Returns None
        when this shape is run plainly."""
        key = (str(device), tuple((n, tuple(t.shape)) for n, t in ins.items()))
        rec = self._recs.get(key, 0)
        if rec is False:
            return None
        if isinstance(rec, int):
            if rec < 1:
                self._recs[key] = rec + 1
                return None
            static_in = {n: t.clone() for n, t in ins.items()}
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph):
                    static_out = self._execute(static_in, device)
            except Exception:  # noqa: BLE001 - this shape cannot be captured: run it plainly from now on
                self._recs[key] = False
                torch.cuda.synchronize(device)
                return None
            rec = self._recs[key] = (graph, static_in, static_out)
        graph, static_in, static_out = rec
        for n, t in ins.items():
            static_in[n].copy_(t)
        graph.replay()
        return {n: t.clone() for n, t in static_out.items()}

    def variable(self, name: str):
        """Current contents of a variable (a copy), or None before the first run."""
        for i, v in enumerate(self.p.g.values):
            if v.kind == "variable" and v.name == name:
                t = self._vars.get(i)
                return None if t is None else t.clone()
        raise KeyError(name)
